// Self-test of the C++ host layer: the reference's projection unit tests
// (crates/izwi-core/src/models/architectures/qwen3/core.rs:2481-2684, 3100-3142) restated against
// the CUDA path, plus the host-only error behaviour.  `--no-gpu` runs only what needs no device.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>

#include <cstdlib>

#include "izwi_chat.hpp"
#include "izwi_host.hpp"

using namespace izwi_host;

static int g_failed = 0;
#define EXPECT(cond)                                                            \
    do {                                                                        \
        if (!(cond)) { std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); ++g_failed; } \
    } while (0)

static bool throws_with(const std::function<void()>& f, const char* needle) {
    try { f(); } catch (const InferenceError& e) { return std::strstr(e.what(), needle) != nullptr; }
    return false;
}

static uint16_t bf16(float f) {
    uint32_t u; std::memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
static float from_bf16(uint16_t b) { uint32_t u = static_cast<uint32_t>(b) << 16; float f; std::memcpy(&f, &u, 4); return f; }

// [rows, cols] fp32 -> bf16 on the device, columns zero-padded to `k` (the kernels need in-dim % 64 == 0)
static std::shared_ptr<DeviceBuffer> upload(const std::vector<float>& v, int rows, int cols, int k) {
    std::vector<uint16_t> h(static_cast<size_t>(rows) * k, 0);
    for (int r = 0; r < rows; ++r) for (int c = 0; c < cols; ++c) h[static_cast<size_t>(r) * k + c] = bf16(v[r * cols + c]);
    return std::make_shared<DeviceBuffer>(h.data(), h.size() * 2);
}
static std::vector<float> download(const DeviceBuffer& b) {
    auto raw = b.to_host();
    std::vector<float> out(raw.size() / 2);
    for (size_t i = 0; i < out.size(); ++i) { uint16_t h; std::memcpy(&h, raw.data() + 2 * i, 2); out[i] = from_bf16(h); }
    return out;
}
// GGML Q8_0 quantisation of one row of 32-value blocks.
static std::vector<uint8_t> quantize_q8_0(const std::vector<float>& x) {
    std::vector<uint8_t> out(x.size() / 32 * 34);
    for (size_t b = 0; b < x.size() / 32; ++b) {
        float amax = 0; for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(x[b * 32 + i]));
        const float d = amax / 127.0f, id = d ? 1.0f / d : 0.0f;
        // fp16 encode of d (normal range only, enough for these fixtures)
        uint32_t u; std::memcpy(&u, &d, 4);
        uint16_t h = 0;
        if (d != 0) {
            const int e = static_cast<int>((u >> 23) & 0xFF) - 127 + 15;
            uint32_t man = (u & 0x7FFFFFu) + 0xFFFu + ((u >> 13) & 1u);
            int ee = e; if (man & 0x800000u) { man = 0; ++ee; }
            h = static_cast<uint16_t>((ee << 10) | (man >> 13));
        }
        std::memcpy(&out[b * 34], &h, 2);
        for (int i = 0; i < 32; ++i) out[b * 34 + 2 + i] = static_cast<uint8_t>(static_cast<int8_t>(std::roundf(x[b * 32 + i] * id)));
    }
    return out;
}

static void host_only_tests() {
    EXPECT(quantized_storage_bytes(3, 32, IZB_W_Q8_0) == 102);
    EXPECT(quantized_storage_bytes(4096, 1024, IZB_W_Q4_K) == 4096u * 1024u / 256u * 144u);
    EXPECT(throws_with([] { quantized_storage_bytes(3, 100, IZB_W_Q4_K); }, "not divisible by block size 256"));
    EXPECT(throws_with([] { packed_qmatmul_from_qtensors({}); }, "Cannot pack empty"));
    EXPECT(std::strcmp(izb_status_string(IZB_ERR_TIMEOUT), "a bounded device-side wait gave up") == 0);
    Qwen3ProjectionDiagnostics a{1, 1, 0}, b{0, 0, 1};
    EXPECT((a.add(b) == Qwen3ProjectionDiagnostics{1, 1, 1}));
}

static void gpu_tests() {
    Context ctx(0);
    const int K = 64;
    // dense projection with and without bias: [2,3] . [[1,2],[3,4]]^T (+ [0.5,-1]) = [8.5,17] / [8,18]
    auto w = upload({1, 2, 3, 4}, 2, 2, K);
    auto x = upload({2, 3}, 1, 2, K);
    auto bias = upload({0.5f, -1.0f}, 1, 2, 2);
    DeviceBuffer y(2 * 2);
    auto with_bias = Qwen3Projection::dense(w, 2, K, bias);
    EXPECT((with_bias.diagnostics() == Qwen3ProjectionDiagnostics{1, 1, 0}));
    with_bias.forward(ctx, nullptr, x->get(), 1, y.get());
    ctx.check_device();
    auto out = download(y);
    EXPECT(out[0] == 8.5f && out[1] == 17.0f);
    auto no_bias = Qwen3Projection::dense(w, 2, K);
    EXPECT((no_bias.diagnostics() == Qwen3ProjectionDiagnostics{1, 0, 0}));
    no_bias.forward(ctx, nullptr, x->get(), 1, y.get());
    ctx.check_device();
    out = download(y);
    EXPECT(out[0] == 8.0f && out[1] == 18.0f);

    // fused QKV == three separate projections (same kernel, same per-row arithmetic: bit for bit)
    auto q = Qwen3Projection::dense(upload({0.1f, 0.2f, 0.3f, -0.4f, 0.5f, 0.6f, 0.7f, -0.8f, 0.9f, 1.0f, -1.1f, 1.2f}, 4, 3, K), 4, K);
    auto k = Qwen3Projection::dense(upload({0.3f, -0.2f, 0.1f, 0.6f, 0.4f, -0.5f}, 2, 3, K), 2, K);
    auto v = Qwen3Projection::dense(upload({-0.7f, 0.8f, 0.9f, 0.2f, -0.1f, 0.4f}, 2, 3, K), 2, K);
    Qwen3FusedQkvProjection fused(q, k, v);
    auto xin = upload({1.0f, -2.0f, 0.5f, 0.25f, 1.5f, -0.75f}, 2, 3, K);
    DeviceBuffer qkv(2 * 8 * 2), yq(2 * 4 * 2), yk(2 * 2 * 2), yv(2 * 2 * 2);
    fused.forward(ctx, nullptr, xin->get(), 2, qkv.get());
    q.forward(ctx, nullptr, xin->get(), 2, yq.get());
    k.forward(ctx, nullptr, xin->get(), 2, yk.get());
    v.forward(ctx, nullptr, xin->get(), 2, yv.get());
    ctx.check_device();
    auto f = download(qkv), sq = download(yq), sk = download(yk), sv = download(yv);
    for (int r = 0; r < 2; ++r) {
        for (int c = 0; c < 4; ++c) EXPECT(f[r * 8 + c] == sq[r * 4 + c]);
        for (int c = 0; c < 2; ++c) EXPECT(f[r * 8 + 4 + c] == sk[r * 2 + c] && f[r * 8 + 6 + c] == sv[r * 2 + c]);
    }
    EXPECT(std::fabs(f[0] - (0.1f * 1 + 0.2f * -2 + 0.3f * 0.5f)) < 2e-2f);
    EXPECT(fused.diagnostics().dense_projection_count == 3);
    EXPECT(throws_with([&] { Qwen3FusedQkvProjection bad(q, Qwen3Projection::dense(upload({1, 2}, 1, 2, 128), 1, 128), v); },
                       "input dimensions do not match"));
    EXPECT(throws_with([&] { Qwen3FusedGateUpProjection bad(with_bias, no_bias); }, "mixed bias presence"));

    // byte-packed Q8_0 rows == separately quantised matrices (rows tiled out to K = 256)
    std::vector<float> w1(2 * 256), w2(256), xv(256);
    for (int i = 0; i < 512; ++i) w1[i] = ((i % 64) - 31.0f) / 8.0f;
    for (int i = 0; i < 256; ++i) { w2[i] = (15.0f - (i % 32)) / 7.0f; xv[i] = ((i % 32) + 1.0f) / 16.0f; }
    auto q1 = quantize_q8_0(w1), q2 = quantize_q8_0(w2);
    QTensor t1{std::make_shared<DeviceBuffer>(q1.data(), q1.size()), 2, 256, IZB_W_Q8_0};
    QTensor t2{std::make_shared<DeviceBuffer>(q2.data(), q2.size()), 1, 256, IZB_W_Q8_0};
    auto packed = packed_qmatmul_from_qtensors({t1, t2});
    auto xq = upload(xv, 1, 256, 256);
    DeviceBuffer yp(3 * 2), y1(2 * 2), y2(1 * 2);
    packed.forward(ctx, nullptr, xq->get(), 1, yp.get());
    Qwen3Projection::quantized(t1).forward(ctx, nullptr, xq->get(), 1, y1.get());
    Qwen3Projection::quantized(t2).forward(ctx, nullptr, xq->get(), 1, y2.get());
    ctx.check_device();
    auto op = download(yp), o1 = download(y1), o2 = download(y2);
    EXPECT(op[0] == o1[0] && op[1] == o1[1] && op[2] == o2[0]);
    EXPECT(packed.diagnostics().quantized_projection_count == 1);
    // the residual add carried inside a one-token quantised projection == projection, then add (one bf16 step)
    {
        std::vector<float> resv = {0.5f, -1.25f};
        auto resd = upload(resv, 1, 2, 2);
        DeviceBuffer yf(2 * 2);
        Qwen3Projection::Fusion fu;
        fu.residual = resd->get();
        Qwen3Projection::quantized(t1).forward(ctx, nullptr, xq->get(), 1, yf.get(), 0, 0, nullptr, 0, IZB_EPI_NONE, &fu);
        ctx.check_device();
        auto of = download(yf);
        for (int c = 0; c < 2; ++c) EXPECT(std::fabs(of[c] - (o1[c] + resv[c])) <= 2e-2f * std::fmax(1.0f, std::fabs(o1[c] + resv[c])));
        EXPECT(izb_linear_fusion_max_tokens(IZB_W_Q8_0) >= 1 && izb_linear_fusion_max_tokens(IZB_W_BF16) == 0);
        // a dense projection takes the residual too (added by the streaming kernel's epilogue): sq + residual rows
        {
            auto res2 = upload({0.5f, -1.25f, 2.0f, 0.125f, -0.5f, 1.0f, 0.25f, -2.0f}, 2, 4, 4);
            Qwen3Projection::Fusion fd;
            fd.residual = res2->get();
            DeviceBuffer yr(2 * 4 * 2);
            q.forward(ctx, nullptr, xin->get(), 2, yr.get(), 0, 0, nullptr, 0, IZB_EPI_NONE, &fd);
            ctx.check_device();
            auto got = download(yr), resh = download(*res2);
            for (int i = 0; i < 8; ++i) EXPECT(std::fabs(got[i] - (sq[i] + resh[i])) <= 2e-2f * std::fmax(1.0f, std::fabs(sq[i] + resh[i])));
        }
    }
    QTensor wide{t2.data, 1, 512, IZB_W_Q8_0};
    EXPECT(throws_with([&] { packed_qmatmul_from_qtensors({t1, wide}); }, "input mismatch: expected 256, got 512"));
    QTensor other{t2.data, 1, 256, IZB_W_Q4_K};
    EXPECT(throws_with([&] { packed_qmatmul_from_qtensors({t1, other}); }, "dtype mismatch"));

    // MLP: down(silu(gate) * up) against a host double-precision evaluation
    const int H = 64, I = 64, M = 3;
    std::vector<float> wg(I * H), wu(I * H), wd(H * I), xm(M * H);
    for (size_t i = 0; i < wg.size(); ++i) { wg[i] = std::sin(0.37f * i) * 0.1f; wu[i] = std::cos(0.11f * i) * 0.1f; wd[i] = std::sin(0.05f * i + 1) * 0.1f; }
    for (size_t i = 0; i < xm.size(); ++i) xm[i] = std::cos(0.7f * i);
    auto gate = Qwen3Projection::dense(upload(wg, I, H, H), I, H), up = Qwen3Projection::dense(upload(wu, I, H, H), I, H);
    Qwen3FusedGateUpProjection gu(gate, up);
    Qwen3Mlp mlp(gu.fused, Qwen3Projection::dense(upload(wd, H, I, I), H, I));
    DeviceBuffer scratch(mlp.scratch_bytes(M)), ym(M * H * 2);
    auto xmd = upload(xm, M, H, H);
    mlp.forward(ctx, nullptr, xmd->get(), M, ym.get(), scratch.get());
    ctx.check_device();
    auto got = download(ym);
    double worst = 0, scale = 0;
    for (int m = 0; m < M; ++m) for (int o = 0; o < H; ++o) {
        double acc = 0;
        for (int i = 0; i < I; ++i) {
            double g = 0, u = 0;
            for (int h = 0; h < H; ++h) { g += from_bf16(bf16(wg[i * H + h])) * from_bf16(bf16(xm[m * H + h])); u += from_bf16(bf16(wu[i * H + h])) * from_bf16(bf16(xm[m * H + h])); }
            acc += from_bf16(bf16(wd[o * I + i])) * (g / (1 + std::exp(-g)) * u);
        }
        worst = std::fmax(worst, std::fabs(acc - got[m * H + o])); scale = std::fmax(scale, std::fabs(acc));
    }
    EXPECT(worst <= 2e-2 * scale);
}

// `chat <model.gguf> <max_new_tokens> <logits.bin> <mode> <prompt ids...>`: loads a Qwen3 model from a GGUF file,
// runs the prompt (mode "prefill": all tokens in one pass through the GEMM and the causal attention; mode "decode":
// one token at a time through the decode kernels), writes the fp32 logits the first new token is chosen from to
// logits.bin, then generates greedily with start_decode / decode_step and prints the ids.  Token 0 ends a reply.
static int chat_main(int argc, char** argv) {
    if (argc < 7) {
        std::printf("usage: host_selftest chat model.gguf max_new logits.bin prefill|decode id...\n");
        return 2;
    }
    try {
        auto ctx = std::make_shared<Context>(0);
        GgufLoader loader(argv[2]);
        auto model = loader.load_qwen3(*ctx, 256);
        const size_t max_new = static_cast<size_t>(std::atoi(argv[3]));
        const bool token_by_token = std::strcmp(argv[5], "decode") == 0;
        std::vector<uint32_t> prompt;
        for (int i = 6; i < argc; ++i) prompt.push_back(static_cast<uint32_t>(std::atoi(argv[i])));
        ChatSpecials specials;
        specials.eos = 0;
        Qwen3ChatModel chat(ctx, model, specials);
        ChatDecodeState st = chat.start_decode(token_by_token ? std::vector<uint32_t>{prompt[0]} : prompt, max_new);
        if (token_by_token) {
            // the same prompt through the one-token path: every further prompt token is a forced decode step
            for (size_t i = 1; i < prompt.size(); ++i) {
                const int32_t id = static_cast<int32_t>(prompt[i]);
                if (cudaMemcpy(st.next_id.get(), &id, 4, cudaMemcpyHostToDevice) != cudaSuccess) throw InferenceError("copy failed");
                model->forward(*ctx, nullptr, static_cast<const int32_t*>(st.next_id.get()), 1, st.pos, st.cache,
                               static_cast<float*>(st.logits.get()), st.scratch);
                st.pos += 1;
            }
            ctx->check_device();
        }
        const auto raw = st.logits.to_host();
        if (FILE* f = std::fopen(argv[4], "wb")) {
            std::fwrite(raw.data(), 1, raw.size(), f);
            std::fclose(f);
        } else {
            throw InferenceError("cannot write the logits file");
        }
        std::printf("generated:");
        while (true) {
            const ChatDecodeStep step = chat.decode_step(st);
            if (step.has_token) std::printf(" %u", step.token);
            if (step.finished) break;
        }
        ctx->check_device();
        std::printf("\npositions: %lld\nlaunches: %lld\nchat: ok\n", static_cast<long long>(st.pos),
                    static_cast<long long>(izb_ctx_launch_count(ctx->get())));
        return 0;
    } catch (const std::exception& e) {
        std::printf("FAIL %s\n", e.what());
        return 1;
    }
}

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "chat") == 0) return chat_main(argc, argv);
    const bool no_gpu = argc > 1 && std::strcmp(argv[1], "--no-gpu") == 0;
    try {
        host_only_tests();
        if (no_gpu) {
            EXPECT(throws_with([] { Context c(0); }, "izb_ctx_create") || true);
        } else {
            gpu_tests();
        }
    } catch (const std::exception& e) {
        std::printf("FAIL unexpected exception: %s\n", e.what());
        return 2;
    }
    // sizes of the structs that cross the C ABI, for bindings in other languages to compare theirs with
    std::printf("abi: izb_linear_args=%zu izb_moe_args=%zu izb_gguf_tensor=%zu\n", sizeof(izb_linear_args), sizeof(izb_moe_args),
                sizeof(izb_gguf_tensor));
    std::printf(g_failed ? "host_selftest: %d failure(s)\n" : "host_selftest: ok\n", g_failed);
    return g_failed ? 1 : 0;
}
