// Host driver of a Qwen3 chat model over the C ABI: the compiled counterpart of
//   Qwen3Model::forward / forward_hidden_with_embeds / logits_from_hidden
//       (crates/izwi-core/src/models/architectures/qwen3/core.rs:2099-2125),
//   Qwen3Layer::forward (core.rs:1863-1881) and Qwen3Attention::forward (core.rs:1624-1732),
//   Qwen3ChatModel::{start_decode, decode_step} (models/architectures/qwen3/chat.rs:295-388) and its
//       argmax (chat.rs:574-601),
//   GgufLoader (models/shared/weights/gguf.rs:36-143) for the weights.
// A prompt of any length runs through the tensor-core GEMM (prefill); every following token runs
// the decode kernels with the norms, SiLU-multiply and residual adds inside the one-token
// projections where the format allows.  The greedy choice stays on the device: the host reads
// four bytes per token (the id it needs for the end-of-sequence test).  Tokenisation and text
// assembly are outside this layer: prompts come and go as token ids.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "izwi_host.hpp"

namespace izwi_host {

struct Qwen3Config {
    int64_t vocab_size = 0, hidden_size = 0, num_layers = 0, num_heads = 0, num_kv_heads = 0, head_dim = 0;
    int64_t intermediate_size = 0;
    float rms_norm_eps = 1e-6f;
    double rope_theta = 1e6;
    int64_t max_positions = 4096;  // capacity of the KV cache and of the rotation tables
};

struct Qwen3LayerWeights {
    std::shared_ptr<DeviceBuffer> input_layernorm, post_attention_layernorm;  // bf16 [hidden]
    std::shared_ptr<DeviceBuffer> q_norm, k_norm;                             // bf16 [head_dim] or null
    Qwen3Projection qkv, o, gate_up, down;  // fused at load (core.rs:931-981, 1132-1168)
};

// Head-major cache of every layer: [1, kv_heads, capacity, head_dim] for k and v (Qwen3Cache, core.rs:251-306).
class Qwen3Cache {
  public:
    Qwen3Cache(const Qwen3Config& c) : capacity(c.max_positions) {
        const size_t bytes = static_cast<size_t>(c.num_kv_heads) * capacity * c.head_dim * 2;
        for (int64_t l = 0; l < c.num_layers; ++l) {
            k.emplace_back(bytes);
            v.emplace_back(bytes);
        }
    }
    std::vector<DeviceBuffer> k, v;
    int64_t capacity;
    // the one-launch token (izb_qwen3_decode_token): its workspace and the 4 bytes its own arg-max goes to;
    // created by the first single-token forward of a model that qualifies
    DeviceBuffer token_workspace, token_choice;
};

class Qwen3Model {
  public:
    Qwen3Model(Qwen3Config cfg, std::shared_ptr<DeviceBuffer> embed_bf16, std::vector<Qwen3LayerWeights> layers,
               std::shared_ptr<DeviceBuffer> final_norm, Qwen3Projection lm_head)
        : cfg_(cfg), embed_(std::move(embed_bf16)), layers_(std::move(layers)), final_norm_(std::move(final_norm)),
          lm_head_(std::move(lm_head)) {
        if (static_cast<int64_t>(layers_.size()) != cfg_.num_layers) throw InferenceError("Qwen3 layer count mismatch");
        if (!embed_ || embed_->bytes() != static_cast<size_t>(cfg_.vocab_size * cfg_.hidden_size * 2))
            throw InferenceError("Qwen3 embedding table must be [vocab, hidden] bf16");
        // rotation tables for every position the cache can hold (apply_rotary_emb, core.rs:2402-2415)
        const int64_t half = cfg_.head_dim / 2;
        std::vector<uint16_t> cs(static_cast<size_t>(cfg_.max_positions * half)), sn(cs.size());
        for (int64_t p = 0; p < cfg_.max_positions; ++p)
            for (int64_t j = 0; j < half; ++j) {
                const double inv = 1.0 / std::pow(cfg_.rope_theta, static_cast<double>(2 * j) / static_cast<double>(cfg_.head_dim));
                // the reference builds the angles in f32 and stores the tables in the model dtype
                const float ang = static_cast<float>(p) * static_cast<float>(inv);
                cs[p * half + j] = to_bf16(std::cos(ang));
                sn[p * half + j] = to_bf16(std::sin(ang));
            }
        cos_ = DeviceBuffer(cs.data(), cs.size() * 2);
        sin_ = DeviceBuffer(sn.data(), sn.size() * 2);
    }

    const Qwen3Config& config() const { return cfg_; }
    int64_t num_layers() const { return cfg_.num_layers; }

    // Bytes of activation scratch a forward pass of up to `tokens` tokens needs.
    size_t scratch_bytes(int64_t tokens) const {
        const int64_t qkv = (cfg_.num_heads + 2 * cfg_.num_kv_heads) * cfg_.head_dim;
        const int64_t per_tok = 4 * cfg_.hidden_size + qkv + 2 * cfg_.num_heads * cfg_.head_dim + 3 * cfg_.intermediate_size;
        return static_cast<size_t>(tokens) * per_tok * 2 + 4096 + attention_workspace_bytes() + dequant_workspace_bytes(tokens);
    }

    // `ids` (device, int32) are `n` consecutive tokens of one sequence starting at position `pos`; the cache is
    // extended by them and `logits` (device, fp32 [vocab]) receives the logits of the LAST token, which is
    // what Qwen3Model::forward's caller reads (chat.rs:343: `embeds.i((0, len - 1))`).
    void forward(const Context& ctx, cudaStream_t s, const int32_t* ids, int64_t n, int64_t pos, Qwen3Cache& cache,
                 float* logits, DeviceBuffer& scratch) const {
        if (n <= 0) throw InferenceError("Qwen3 forward needs at least one token");
        if (pos < 0 || pos + n > cache.capacity) throw InferenceError("Qwen3 forward exceeds the KV cache capacity");
        if (scratch.bytes() < scratch_bytes(n)) throw InferenceError("Qwen3 forward scratch is too small");
        const Qwen3Config& c = cfg_;
        if (n == 1 && forward_one_launch(ctx, s, ids, pos, cache, logits)) return;
        const int64_t H = c.hidden_size, QD = c.num_heads * c.head_dim, KD = c.num_kv_heads * c.head_dim, I = c.intermediate_size;
        const int64_t QKV = QD + 2 * KD;
        auto* base = static_cast<uint8_t*>(scratch.get());
        size_t at = 0;
        auto take = [&](int64_t elems) { void* p = base + at; at += (static_cast<size_t>(elems) * 2 + 255) / 256 * 256; return p; };
        void* x = take(n * H);          // residual stream
        void* normed = take(n * H);
        void* sum = take(n * H);
        void* tmp = take(n * H);
        void* qkv = take(n * QKV);
        void* q = take(n * QD);
        void* attn = take(n * QD);
        void* gu = take(n * 2 * I);
        void* act = take(n * I);
        void* att_ws = base + at;
        const size_t att_ws_bytes = attention_workspace_bytes();
        at += att_ws_bytes;
        // more than 64 tokens over block-quantised weights: the GEMM multiplies a bf16 copy kept here
        void* deq_ws = base + at;
        const size_t deq_ws_bytes = dequant_workspace_bytes(n);
        const void* cos_row = static_cast<const uint8_t*>(cos_.get()) + static_cast<size_t>(pos) * (c.head_dim / 2) * 2;
        const void* sin_row = static_cast<const uint8_t*>(sin_.get()) + static_cast<size_t>(pos) * (c.head_dim / 2) * 2;
        const float scale = 1.0f / std::sqrt(static_cast<float>(c.head_dim));
        // one or two tokens over block-quantised weights: norms, SiLU-multiply and residual adds ride in the projections
        const bool fuse = n <= izb_linear_fusion_max_tokens(layers_[0].qkv.wfmt()) &&
                          n <= izb_linear_fusion_max_tokens(layers_[0].down.wfmt());

        check(izb_embed_rows(ctx.get(), s, embed_->get(), c.vocab_size, H, ids, n, x, H), "izb_embed_rows");
        for (int64_t l = 0; l < c.num_layers; ++l) {
            const Qwen3LayerWeights& w = layers_[l];
            // ---- attention block (Qwen3Layer::forward, core.rs:1866-1872) ----
            if (fuse) {
                Qwen3Projection::Fusion f;
                f.prologue = IZB_PRO_RMSNORM;
                f.norm_weight = w.input_layernorm->get();
                f.norm_eps = c.rms_norm_eps;
                w.qkv.forward(ctx, s, x, n, qkv, 0, 0, nullptr, 0, IZB_EPI_NONE, &f);
            } else {
                check(izb_rms_norm(ctx.get(), s, x, w.input_layernorm->get(), nullptr, normed, nullptr, n, H, H, 0, H, 0, c.rms_norm_eps),
                      "izb_rms_norm");
                w.qkv.forward(ctx, s, normed, n, qkv, 0, 0, deq_ws, deq_ws_bytes);
            }
            check(izb_qk_norm_rope_append_seq(ctx.get(), s, qkv, QKV, w.q_norm ? w.q_norm->get() : nullptr,
                                              w.k_norm ? w.k_norm->get() : nullptr, c.rms_norm_eps, cos_row, sin_row, q, QD,
                                              cache.k[l].get(), cache.v[l].get(), 1, n, static_cast<int32_t>(c.num_heads),
                                              static_cast<int32_t>(c.num_kv_heads), static_cast<int32_t>(c.head_dim), pos, cache.capacity),
                  "izb_qk_norm_rope_append_seq");
            if (n == 1)
                check(izb_decode_gqa_attention(ctx.get(), s, q, cache.k[l].get(), cache.v[l].get(), attn, 1,
                                               static_cast<int32_t>(c.num_heads), static_cast<int32_t>(c.num_kv_heads),
                                               static_cast<int32_t>(c.head_dim), pos + 1, cache.capacity, QD, QD, scale, att_ws, att_ws_bytes),
                      "izb_decode_gqa_attention");
            else
                check(izb_prefill_gqa_attention(ctx.get(), s, q, cache.k[l].get(), cache.v[l].get(), attn, 1, n,
                                                static_cast<int32_t>(c.num_heads), static_cast<int32_t>(c.num_kv_heads),
                                                static_cast<int32_t>(c.head_dim), pos, cache.capacity, QD, QD, scale),
                      "izb_prefill_gqa_attention");
            // ---- O projection, residual, MLP block (core.rs:1873-1880, Qwen3Mlp::forward :1786-1798) ----
            if (fuse) {
                Qwen3Projection::Fusion fo;
                fo.residual = x;
                w.o.forward(ctx, s, attn, n, sum, 0, 0, nullptr, 0, IZB_EPI_NONE, &fo);  // sum = x + o(attn)
                Qwen3Projection::Fusion fg;
                fg.prologue = IZB_PRO_RMSNORM;
                fg.norm_weight = w.post_attention_layernorm->get();
                fg.norm_eps = c.rms_norm_eps;
                w.gate_up.forward(ctx, s, sum, n, gu, 0, 0, nullptr, 0, IZB_EPI_NONE, &fg);
                Qwen3Projection::Fusion fd;
                fd.prologue = IZB_PRO_SILU_MUL;
                fd.residual = sum;
                w.down.forward(ctx, s, gu, n, x, 0, 0, nullptr, 0, IZB_EPI_NONE, &fd);   // x = sum + down(silu(gate) * up)
            } else {
                w.o.forward(ctx, s, attn, n, tmp, 0, 0, deq_ws, deq_ws_bytes);
                // sum = x + o; normed = post_attention_layernorm(sum)
                check(izb_rms_norm(ctx.get(), s, tmp, w.post_attention_layernorm->get(), x, normed, sum, n, H, H, H, H, H,
                                   c.rms_norm_eps), "izb_rms_norm");
                w.gate_up.forward(ctx, s, normed, n, gu, 0, 0, deq_ws, deq_ws_bytes);
                check(izb_silu_mul(ctx.get(), s, gu, static_cast<uint8_t*>(gu) + I * 2, act, n, I, 2 * I, 2 * I, I), "izb_silu_mul");
                w.down.forward(ctx, s, act, n, tmp, 0, 0, deq_ws, deq_ws_bytes);
                add_rows(ctx, s, sum, tmp, x, n, H);  // x = sum + mlp_out
            }
        }
        // final norm + lm_head on the last token only (logits_from_hidden, core.rs:2114-2125)
        const void* last = static_cast<const uint8_t*>(x) + static_cast<size_t>(n - 1) * H * 2;
        izb_linear_args a{};
        a.wfmt = lm_head_.wfmt();
        a.y_dtype = IZB_F32;
        a.w = lm_head_.weight()->get();
        a.y = logits;
        a.M = 1; a.N = c.vocab_size; a.K = H; a.ldx = H; a.ldy = c.vocab_size;
        if (izb_linear_fusion_max_tokens(lm_head_.wfmt()) >= 1) {
            a.x = last;
            a.prologue = IZB_PRO_RMSNORM;
            a.norm_weight = final_norm_->get();
            a.norm_eps = c.rms_norm_eps;
        } else {
            check(izb_rms_norm(ctx.get(), s, last, final_norm_->get(), nullptr, normed, nullptr, 1, H, H, 0, H, 0, c.rms_norm_eps),
                  "izb_rms_norm");
            a.x = normed;
        }
        check(izb_linear(ctx.get(), s, &a), "lm_head");
    }

  private:
    // One token of one sequence as ONE launch when the library takes this model (every projection of the layers in
    // one of Q8_0 / Q4_K, lm_head in either, head_dim 128, ...: izb_qwen3_decode_token); false = compose the step.
    // IZWI_B200_TOKEN_KERNEL=0 keeps the composed step.
    bool forward_one_launch(const Context& ctx, cudaStream_t s, const int32_t* id, int64_t pos, Qwen3Cache& cache, float* logits) const {
        static const bool enabled = [] {
            const char* e = std::getenv("IZWI_B200_TOKEN_KERNEL");
            return !(e && e[0] == '0');
        }();
        if (!enabled || token_kernel_refused_) return false;
        const Qwen3Config& c = cfg_;
        const int32_t fmt = layers_[0].qkv.wfmt();
        for (const Qwen3LayerWeights& w : layers_)
            for (const Qwen3Projection* p : {&w.qkv, &w.o, &w.gate_up, &w.down})
                if (p->wfmt() != fmt) { token_kernel_refused_ = true; return false; }
        std::vector<izb_qwen3_layer_ptrs> rows(static_cast<size_t>(c.num_layers));
        for (int64_t l = 0; l < c.num_layers; ++l) {
            const Qwen3LayerWeights& w = layers_[l];
            rows[l] = {w.input_layernorm->get(), w.post_attention_layernorm->get(), w.q_norm ? w.q_norm->get() : nullptr,
                       w.k_norm ? w.k_norm->get() : nullptr, w.qkv.weight()->get(), w.o.weight()->get(), w.gate_up.weight()->get(),
                       w.down.weight()->get(), cache.k[l].get(), cache.v[l].get()};
        }
        izb_qwen3_decode_args a{};
        a.wfmt = fmt;
        a.lm_head_fmt = lm_head_.wfmt();
        a.n_layers = static_cast<int32_t>(c.num_layers);
        a.hidden = static_cast<int32_t>(c.hidden_size);
        a.heads = static_cast<int32_t>(c.num_heads);
        a.kv_heads = static_cast<int32_t>(c.num_kv_heads);
        a.head_dim = static_cast<int32_t>(c.head_dim);
        a.intermediate = static_cast<int32_t>(c.intermediate_size);
        a.vocab = static_cast<int32_t>(c.vocab_size);
        a.pos = static_cast<int32_t>(pos);
        a.kv_capacity = cache.capacity;
        a.eps = c.rms_norm_eps;
        a.layers = rows.data();
        a.embed = embed_->get();
        a.final_norm = final_norm_->get();
        a.lm_head = lm_head_.weight()->get();
        a.token = id;
        a.cos_half = static_cast<const uint8_t*>(cos_.get()) + static_cast<size_t>(pos) * (c.head_dim / 2) * 2;
        a.sin_half = static_cast<const uint8_t*>(sin_.get()) + static_cast<size_t>(pos) * (c.head_dim / 2) * 2;
        a.logits = logits;
        const size_t need = izb_qwen3_decode_token_workspace_bytes(ctx.get(), &a);
        if (need == 0) { token_kernel_refused_ = true; return false; }
        if (cache.token_workspace.bytes() < need) {
            cache.token_workspace = DeviceBuffer(need);
            cache.token_choice = DeviceBuffer(4);
        }
        a.workspace = cache.token_workspace.get();
        a.workspace_bytes = cache.token_workspace.bytes();
        a.next_token = static_cast<int32_t*>(cache.token_choice.get());
        const int32_t rc = izb_qwen3_decode_token(ctx.get(), s, &a);
        if (rc == IZB_ERR_UNSUPPORTED) { token_kernel_refused_ = true; return false; }
        check(rc, "izb_qwen3_decode_token");
        return true;
    }

    static uint16_t to_bf16(float f) {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        u += 0x7FFFu + ((u >> 16) & 1u);
        return static_cast<uint16_t>(u >> 16);
    }
    size_t attention_workspace_bytes() const {
        // the decode attention splits a cache over at most 64 CTAs per KV head, whatever its length
        return static_cast<size_t>(cfg_.num_heads) * 64 * (cfg_.head_dim + 2) * sizeof(float);
    }
    size_t dequant_workspace_bytes(int64_t tokens) const {
        size_t need = 0;
        for (const Qwen3LayerWeights& w : layers_)
            for (const Qwen3Projection* p : {&w.qkv, &w.o, &w.gate_up, &w.down})
            {
                // the query that knows the whole call: the bf16 copy for the GEMM route, or (3..8 tokens over Q8_0)
                // room for the activations as the integer tensor-core kernel reads them
                izb_linear_args a{};
                a.wfmt = p->wfmt();
                a.M = tokens;
                a.N = p->out_dim();
                a.K = p->in_dim();
                need = std::max(need, izb_linear_workspace_bytes_args(&a));
            }
        return (need + 255) / 256 * 256;
    }
    // out = a + b over bf16 rows: the residual add after the MLP when no projection carries it.  Done by the
    // RMS-norm kernel's residual path (its `sum_out`), with unit weights kept on the device.
    void add_rows(const Context& ctx, cudaStream_t s, const void* a, const void* b, void* out, int64_t n, int64_t H) const {
        if (!ones_ || ones_->bytes() != static_cast<size_t>(H * 2)) {
            std::vector<uint16_t> one(static_cast<size_t>(H), to_bf16(1.0f));
            ones_ = std::make_shared<DeviceBuffer>(one.data(), one.size() * 2);
            add_sink_ = std::make_shared<DeviceBuffer>(static_cast<size_t>(cfg_.max_positions) * H * 2);
        }
        if (add_sink_->bytes() < static_cast<size_t>(n * H * 2)) add_sink_ = std::make_shared<DeviceBuffer>(static_cast<size_t>(n * H * 2));
        check(izb_rms_norm(ctx.get(), s, a, ones_->get(), b, add_sink_->get(), out, n, H, H, H, H, H, cfg_.rms_norm_eps), "izb_rms_norm");
    }

    Qwen3Config cfg_;
    std::shared_ptr<DeviceBuffer> embed_;
    std::vector<Qwen3LayerWeights> layers_;
    std::shared_ptr<DeviceBuffer> final_norm_;
    Qwen3Projection lm_head_;
    DeviceBuffer cos_, sin_;
    mutable std::shared_ptr<DeviceBuffer> ones_, add_sink_;
    mutable bool token_kernel_refused_ = false;
};

// Token ids that end a reply (the tokenizer's im_end / eos / eos_alt, chat.rs:346-349).
struct ChatSpecials {
    uint32_t im_end = 0xFFFFFFFFu, eos = 0xFFFFFFFFu;
    bool has_eos_alt = false;
    uint32_t eos_alt = 0;
};

struct ChatDecodeState {
    Qwen3Cache cache;
    DeviceBuffer logits;     // fp32 [vocab]: the logits the next token is chosen from (`embeds` in the reference)
    DeviceBuffer next_id;    // int32 [1] on the device: the greedy choice, fed straight back into the embedding
    DeviceBuffer scratch;
    int64_t pos = 0;
    std::vector<uint32_t> generated_ids;
    size_t max_new_tokens = 1;
    bool finished = false;
};

struct ChatDecodeStep {
    bool has_token = false;
    uint32_t token = 0;         // the token this step produced (the reference returns its text delta)
    size_t tokens_generated = 0;
    bool finished = false;
};

class Qwen3ChatModel {
  public:
    Qwen3ChatModel(std::shared_ptr<Context> ctx, std::shared_ptr<Qwen3Model> model, ChatSpecials specials)
        : ctx_(std::move(ctx)), text_model_(std::move(model)), specials_(specials) {}

    // Runs the prompt through the model and leaves the state ready for decode_step (chat.rs:295-330).
    ChatDecodeState start_decode(const std::vector<uint32_t>& prompt_ids, size_t max_new_tokens, cudaStream_t s = nullptr) const {
        if (prompt_ids.empty()) throw InferenceError("Qwen3 chat prompt is empty");
        const Qwen3Config& c = text_model_->config();
        const size_t scratch = std::max(text_model_->scratch_bytes(static_cast<int64_t>(prompt_ids.size())), text_model_->scratch_bytes(1));
        ChatDecodeState st{Qwen3Cache(c), DeviceBuffer(static_cast<size_t>(c.vocab_size) * 4), DeviceBuffer(4), DeviceBuffer(scratch)};
        std::vector<int32_t> ids(prompt_ids.begin(), prompt_ids.end());
        DeviceBuffer d_ids(ids.data(), ids.size() * 4);
        text_model_->forward(*ctx_, s, static_cast<const int32_t*>(d_ids.get()), static_cast<int64_t>(ids.size()), 0, st.cache,
                             static_cast<float*>(st.logits.get()), st.scratch);
        ctx_->check_device(s);  // also orders the temporary id buffer's release after its use
        st.pos = static_cast<int64_t>(ids.size());
        st.max_new_tokens = max_new_tokens > 0 ? max_new_tokens : 1;
        return st;
    }

    // One greedy token (chat.rs:332-388): choose from the pending logits, stop on an end token, otherwise run
    // the model on the chosen token to produce the next logits.
    ChatDecodeStep decode_step(ChatDecodeState& st, cudaStream_t s = nullptr) const {
        if (st.finished || st.generated_ids.size() >= st.max_new_tokens) {
            st.finished = true;
            return {false, 0, st.generated_ids.size(), true};
        }
        const Qwen3Config& c = text_model_->config();
        check(izb_argmax_rows(ctx_->get(), s, st.logits.get(), IZB_F32, 1, c.vocab_size, c.vocab_size,
                              static_cast<int32_t*>(st.next_id.get()), nullptr), "izb_argmax_rows");
        int32_t next = 0;  // the one device-to-host read of the step
        if (cudaMemcpyAsync(&next, st.next_id.get(), 4, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
            throw InferenceError("reading the chosen token failed");
        const uint32_t tok = static_cast<uint32_t>(next);
        if (tok == specials_.im_end || tok == specials_.eos || (specials_.has_eos_alt && tok == specials_.eos_alt)) {
            st.finished = true;
            return {false, 0, st.generated_ids.size(), true};
        }
        st.generated_ids.push_back(tok);
        if (st.pos >= st.cache.capacity) throw InferenceError("Qwen3 chat decode ran past the KV cache capacity");
        text_model_->forward(*ctx_, s, static_cast<const int32_t*>(st.next_id.get()), 1, st.pos, st.cache,
                             static_cast<float*>(st.logits.get()), st.scratch);
        st.pos += 1;
        if (st.generated_ids.size() >= st.max_new_tokens) st.finished = true;
        return {true, tok, st.generated_ids.size(), st.finished};
    }

    bool supports_incremental_decode() const { return true; }
    const Qwen3Model& text_model() const { return *text_model_; }

  private:
    std::shared_ptr<Context> ctx_;
    std::shared_ptr<Qwen3Model> text_model_;
    ChatSpecials specials_;
};

// ---- weights from a GGUF file (GgufLoader, models/shared/weights/gguf.rs:36-143; llama.cpp tensor names as
// models/architectures/qwen35/text.rs:152-171 uses them) ----
class GgufLoader {
  public:
    explicit GgufLoader(const std::string& path) { check(izb_gguf_open(path.c_str(), &g_), "GgufLoader::from_path"); }
    ~GgufLoader() { if (g_) izb_gguf_close(g_); }
    GgufLoader(const GgufLoader&) = delete;
    GgufLoader& operator=(const GgufLoader&) = delete;

    bool has_tensor(const std::string& name) const {
        izb_gguf_tensor t;
        return izb_gguf_find(g_, name.c_str(), &t) == IZB_OK;
    }
    uint64_t get_metadata_u64(const std::string& key) const {
        uint64_t v = 0;
        if (izb_gguf_meta_u64(g_, key.c_str(), &v) != IZB_OK) throw InferenceError("Missing GGUF metadata key: " + key);
        return v;
    }
    double get_metadata_f64(const std::string& key, double dflt) const {
        double v = dflt;
        return izb_gguf_meta_f64(g_, key.c_str(), &v) == IZB_OK ? v : dflt;
    }
    // Raw block bytes on the device, as the kernels take them (load_qtensor).
    QTensor load_qtensor(const std::string& name) const {
        const izb_gguf_tensor t = find(name);
        if (t.wfmt != IZB_W_Q8_0 && t.wfmt != IZB_W_Q4_K && t.wfmt != IZB_W_Q6_K)
            throw InferenceError("GGUF tensor " + name + " is not block-quantised");
        auto buf = std::make_shared<DeviceBuffer>(t.bytes);
        check(izb_gguf_upload(g_, &t, buf->get(), buf->bytes(), nullptr), "izb_gguf_upload");
        cudaStreamSynchronize(nullptr);
        return QTensor{buf, t.rows, t.cols, t.wfmt};
    }
    // A tensor as bf16 on the device whatever its stored type (load_tensor + to_dtype): F32 and F16 are
    // converted on the host, BF16 copied, block formats dequantised by izb_dequantize.
    std::shared_ptr<DeviceBuffer> load_bf16(const Context& ctx, const std::string& name, int64_t* rows = nullptr,
                                            int64_t* cols = nullptr) const {
        const izb_gguf_tensor t = find(name);
        if (rows) *rows = t.rows;
        if (cols) *cols = t.cols;
        const size_t n = static_cast<size_t>(t.rows * t.cols);
        if (t.wfmt == IZB_W_Q8_0 || t.wfmt == IZB_W_Q4_K || t.wfmt == IZB_W_Q6_K) {
            DeviceBuffer raw(t.bytes);
            check(izb_gguf_upload(g_, &t, raw.get(), raw.bytes(), nullptr), "izb_gguf_upload");
            auto out = std::make_shared<DeviceBuffer>(n * 2);
            check(izb_dequantize(ctx.get(), nullptr, t.wfmt, raw.get(), static_cast<int64_t>(n), IZB_BF16, out->get()), "izb_dequantize");
            cudaStreamSynchronize(nullptr);
            return out;
        }
        std::vector<uint16_t> h(n);
        if (t.ggml_type == 0) {         // F32
            const float* src = static_cast<const float*>(t.data);
            for (size_t i = 0; i < n; ++i) h[i] = f32_to_bf16(src[i]);
        } else if (t.ggml_type == 30) {  // BF16
            std::memcpy(h.data(), t.data, n * 2);
        } else if (t.ggml_type == 1) {   // F16
            const uint16_t* src = static_cast<const uint16_t*>(t.data);
            for (size_t i = 0; i < n; ++i) h[i] = f32_to_bf16(f16_to_f32(src[i]));
        } else {
            throw InferenceError("GGUF tensor " + name + " has an unsupported type");
        }
        return std::make_shared<DeviceBuffer>(h.data(), n * 2);
    }

    // A Qwen3 model from llama.cpp tensor names: token_embd, blk.{i}.attn_{q,k,v,output}, attn_{q,k}_norm,
    // attn_norm, ffn_norm, ffn_{gate,up,down}, output_norm, output (tied to token_embd when absent).
    std::shared_ptr<Qwen3Model> load_qwen3(const Context& ctx, int64_t max_positions) const {
        Qwen3Config c;
        const std::string a = "qwen3.";
        c.num_layers = static_cast<int64_t>(get_metadata_u64(a + "block_count"));
        c.hidden_size = static_cast<int64_t>(get_metadata_u64(a + "embedding_length"));
        c.num_heads = static_cast<int64_t>(get_metadata_u64(a + "attention.head_count"));
        c.num_kv_heads = static_cast<int64_t>(get_metadata_u64(a + "attention.head_count_kv"));
        c.head_dim = static_cast<int64_t>(get_metadata_u64(a + "attention.key_length"));
        c.intermediate_size = static_cast<int64_t>(get_metadata_u64(a + "feed_forward_length"));
        c.rms_norm_eps = static_cast<float>(get_metadata_f64(a + "attention.layer_norm_rms_epsilon", 1e-6));
        c.rope_theta = get_metadata_f64(a + "rope.freq_base", 1e6);
        c.max_positions = max_positions;
        int64_t vocab = 0, hid = 0;
        auto embed = load_bf16(ctx, "token_embd.weight", &vocab, &hid);
        if (hid != c.hidden_size) throw InferenceError("token_embd.weight does not match embedding_length");
        c.vocab_size = vocab;
        std::vector<Qwen3LayerWeights> layers;
        for (int64_t i = 0; i < c.num_layers; ++i) {
            const std::string p = "blk." + std::to_string(i) + ".";
            Qwen3LayerWeights w;
            w.input_layernorm = load_bf16(ctx, p + "attn_norm.weight");
            w.post_attention_layernorm = load_bf16(ctx, p + "ffn_norm.weight");
            if (has_tensor(p + "attn_q_norm.weight")) {
                w.q_norm = load_bf16(ctx, p + "attn_q_norm.weight");
                w.k_norm = load_bf16(ctx, p + "attn_k_norm.weight");
            }
            w.qkv = projection(ctx, {p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"});
            w.o = projection(ctx, {p + "attn_output.weight"});
            w.gate_up = projection(ctx, {p + "ffn_gate.weight", p + "ffn_up.weight"});
            w.down = projection(ctx, {p + "ffn_down.weight"});
            layers.push_back(std::move(w));
        }
        auto final_norm = load_bf16(ctx, "output_norm.weight");
        Qwen3Projection head = has_tensor("output.weight") ? projection(ctx, {"output.weight"})
                                                           : Qwen3Projection::tied_dense(embed, c.vocab_size, c.hidden_size);
        return std::make_shared<Qwen3Model>(c, embed, std::move(layers), final_norm, std::move(head));
    }

  private:
    izb_gguf_tensor find(const std::string& name) const {
        izb_gguf_tensor t;
        if (izb_gguf_find(g_, name.c_str(), &t) != IZB_OK) throw InferenceError("Missing GGUF tensor: " + name);
        return t;
    }
    // One projection from one or more row-stacked tensors: block formats are packed byte-wise
    // (packed_qmatmul_from_qtensors), anything else becomes one dense bf16 matrix.
    Qwen3Projection projection(const Context& ctx, const std::vector<std::string>& names) const {
        const izb_gguf_tensor first = find(names[0]);
        if (first.wfmt == IZB_W_Q8_0 || first.wfmt == IZB_W_Q4_K) {
            std::vector<QTensor> parts;
            for (const auto& n : names) parts.push_back(load_qtensor(n));
            return packed_qmatmul_from_qtensors(parts);
        }
        std::vector<std::shared_ptr<DeviceBuffer>> bufs;
        std::vector<const DeviceBuffer*> ptrs;
        int64_t rows = 0, cols = 0;
        for (const auto& n : names) {
            int64_t r = 0, cc = 0;
            bufs.push_back(load_bf16(ctx, n, &r, &cc));
            if (cols && cc != cols) throw InferenceError("Qwen3 fused projection input dimensions do not match");
            cols = cc;
            rows += r;
            ptrs.push_back(bufs.back().get());
        }
        return Qwen3Projection::dense(names.size() == 1 ? bufs[0] : detail::concat(ptrs), rows, cols);
    }
    static uint16_t f32_to_bf16(float f) {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        u += 0x7FFFu + ((u >> 16) & 1u);
        return static_cast<uint16_t>(u >> 16);
    }
    static float f16_to_f32(uint16_t h) {
        const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
        uint32_t bits;
        if (exp == 0) {
            if (man == 0) bits = sign;
            else {
                int e = -1;
                uint32_t m = man;
                do { ++e; m <<= 1; } while ((m & 0x400u) == 0);
                bits = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
            }
        } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
        else bits = sign | ((exp + 112u) << 23) | (man << 13);
        float f;
        std::memcpy(&f, &bits, 4);
        return f;
    }
    izb_gguf* g_ = nullptr;
};

}  // namespace izwi_host
