// Host-side C++ mirror of the reference's projection types over the C ABI of libizwi_b200.so.
//
// Same names, argument meaning and error behaviour as
// crates/izwi-core/src/models/architectures/qwen3/core.rs:
//   Qwen3Projection               :671-728, forward :791-832
//   Qwen3FusedQkvProjection       :931-981
//   Qwen3FusedGateUpProjection    :1132-1168
//   packed_qmatmul_from_qtensors  :846-885, quantized_storage_bytes :891-909
//   Qwen3Mlp                      :1786-1798
// Errors are thrown as InferenceError (the counterpart of izwi_core::Error::InferenceError);
// nothing here computes on the host: every forward() is a launch through the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/izwi_b200.h"

namespace izwi_host {

struct InferenceError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

// The IZWI_B200_KERNELS gate (default on; the rule of `use_fused_kernels`, kernels/mod.rs:46-57), read once per
// process.  Off means "take the caller's own path": a Rust shim would run Candle's ops; this layer has no other
// path and refuses.
inline bool use_b200_kernels() { return izb_kernels_enabled() != 0; }

inline void check(int32_t status, const char* where) {
    if (status != IZB_OK) throw InferenceError(std::string(where) + ": " + izb_status_string(status));
}

// Owning device allocation (model-load time only; forward passes never allocate weights).
class DeviceBuffer {
  public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes) : bytes_(bytes) {
        if (bytes && cudaMalloc(&ptr_, bytes) != cudaSuccess) throw InferenceError("device allocation failed");
    }
    DeviceBuffer(const void* host, size_t bytes) : DeviceBuffer(bytes) {
        if (bytes && cudaMemcpy(ptr_, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess)
            throw InferenceError("host to device copy failed");
    }
    DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { release(); ptr_ = o.ptr_; bytes_ = o.bytes_; o.ptr_ = nullptr; o.bytes_ = 0; }
        return *this;
    }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { release(); }
    void* get() const { return ptr_; }
    size_t bytes() const { return bytes_; }
    std::vector<uint8_t> to_host() const {
        std::vector<uint8_t> out(bytes_);
        if (bytes_ && cudaMemcpy(out.data(), ptr_, bytes_, cudaMemcpyDeviceToHost) != cudaSuccess)
            throw InferenceError("device to host copy failed");
        return out;
    }

  private:
    void release() { if (ptr_) cudaFree(ptr_); ptr_ = nullptr; }
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

class Context {
  public:
    explicit Context(int device = 0) { check(izb_ctx_create(device, &ctx_), "izb_ctx_create"); }
    ~Context() { if (ctx_) izb_ctx_destroy(ctx_); }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    izb_ctx* get() const { return ctx_; }
    void check_device(cudaStream_t s = nullptr) const { check(izb_ctx_check(ctx_, s), "izb_ctx_check"); }

  private:
    izb_ctx* ctx_ = nullptr;
};

inline const char* wfmt_name(int32_t f) {
    return f == IZB_W_Q8_0 ? "Q8_0" : f == IZB_W_Q4_K ? "Q4K" : f == IZB_W_Q6_K ? "Q6K" : "BF16";
}
inline int64_t wfmt_block(int32_t f) { return f == IZB_W_Q8_0 ? 32 : (f == IZB_W_Q4_K || f == IZB_W_Q6_K) ? 256 : 1; }

inline size_t quantized_storage_bytes(int64_t rows, int64_t cols, int32_t dtype) {
    size_t out = 0;
    if (izb_quantized_storage_bytes(dtype, rows, cols, &out) != IZB_OK)
        throw InferenceError("Qwen3 quantized projection element count " + std::to_string(rows * cols) +
                             " is not divisible by block size " + std::to_string(wfmt_block(dtype)));
    return out;
}

// Raw GGML block bytes of a [rows, cols] matrix on the device (Candle's QTensor).
struct QTensor {
    std::shared_ptr<DeviceBuffer> data;
    int64_t rows = 0, cols = 0;
    int32_t dtype = IZB_W_Q8_0;
};

struct Qwen3ProjectionDiagnostics {
    size_t dense_projection_count = 0, dense_bias_projection_count = 0, quantized_projection_count = 0;
    Qwen3ProjectionDiagnostics add(const Qwen3ProjectionDiagnostics& o) const {
        return {dense_projection_count + o.dense_projection_count,
                dense_bias_projection_count + o.dense_bias_projection_count,
                quantized_projection_count + o.quantized_projection_count};
    }
    bool operator==(const Qwen3ProjectionDiagnostics& o) const {
        return dense_projection_count == o.dense_projection_count &&
               dense_bias_projection_count == o.dense_bias_projection_count &&
               quantized_projection_count == o.quantized_projection_count;
    }
};

// One linear layer: Dense (bf16 [out, in] weight, optional bf16 bias) or Quantized (GGML blocks).
class Qwen3Projection {
  public:
    enum class Kind { Dense, Quantized };

    static Qwen3Projection dense(std::shared_ptr<DeviceBuffer> weight_bf16, int64_t out_dim, int64_t in_dim,
                                 std::shared_ptr<DeviceBuffer> bias_bf16 = nullptr) {
        if (!weight_bf16 || weight_bf16->bytes() != static_cast<size_t>(out_dim * in_dim * 2))
            throw InferenceError("dense projection weight must be [out, in] bf16");
        if (bias_bf16 && bias_bf16->bytes() != static_cast<size_t>(out_dim * 2))
            throw InferenceError("dense projection bias must be [out] bf16");
        Qwen3Projection p;
        p.kind_ = Kind::Dense;
        p.weight_ = std::move(weight_bf16);
        p.bias_ = std::move(bias_bf16);
        p.out_ = out_dim;
        p.in_ = in_dim;
        p.wfmt_ = IZB_W_BF16;
        return p;
    }
    static Qwen3Projection tied_dense(std::shared_ptr<DeviceBuffer> weight_bf16, int64_t out_dim, int64_t in_dim) {
        return dense(std::move(weight_bf16), out_dim, in_dim, nullptr);
    }
    static Qwen3Projection quantized(const QTensor& q) {
        if (!q.data || q.data->bytes() != quantized_storage_bytes(q.rows, q.cols, q.dtype))
            throw InferenceError("quantized projection storage does not match its shape");
        Qwen3Projection p;
        p.kind_ = Kind::Quantized;
        p.weight_ = q.data;
        p.out_ = q.rows;
        p.in_ = q.cols;
        p.wfmt_ = q.dtype;
        return p;
    }

    Kind kind() const { return kind_; }
    int64_t out_dim() const { return out_; }
    int64_t in_dim() const { return in_; }
    int32_t wfmt() const { return wfmt_; }
    const std::shared_ptr<DeviceBuffer>& weight() const { return weight_; }
    const std::shared_ptr<DeviceBuffer>& bias() const { return bias_; }

    Qwen3ProjectionDiagnostics diagnostics() const {
        if (kind_ == Kind::Dense) return {1, bias_ ? size_t(1) : size_t(0), 0};
        return {0, 0, 1};
    }

    // What a decode layer does around a projection, carried inside it (one or two tokens over Q8_0 / Q4_K
    // weights: m <= izb_linear_fusion_max_tokens(wfmt); any other shape throws "unsupported").
    struct Fusion {
        int32_t prologue = IZB_PRO_NONE;     // IZB_PRO_RMSNORM: x is the un-normalised stream; IZB_PRO_SILU_MUL: x is [m, 2 in] = gate | up
        const void* norm_weight = nullptr;   // bf16 [in]
        float norm_eps = 0.f;
        const void* residual = nullptr;      // bf16 [m, ld_residual], added to y
        int64_t ld_residual = 0;             // 0: out
    };

    // y[M, out] = x[M, in] . W^T (+ bias); x and y are bf16 device pointers with row strides ldx / ldy.
    void forward(const Context& ctx, cudaStream_t stream, const void* x, int64_t m, void* y, int64_t ldx = 0,
                 int64_t ldy = 0, void* workspace = nullptr, size_t workspace_bytes = 0,
                 int32_t epilogue = IZB_EPI_NONE, const Fusion* fusion = nullptr) const {
        if (!use_b200_kernels())
            throw InferenceError("IZWI_B200_KERNELS is off: the B200 projection kernels are disabled");
        izb_linear_args a{};
        if (fusion) {
            a.prologue = fusion->prologue;
            a.norm_weight = fusion->norm_weight;
            a.norm_eps = fusion->norm_eps;
            a.residual = fusion->residual;
            a.ld_residual = fusion->residual ? (fusion->ld_residual ? fusion->ld_residual : out_) : 0;
            if (!ldx && fusion->prologue == IZB_PRO_SILU_MUL) ldx = 2 * in_;
        }
        a.wfmt = wfmt_;
        a.y_dtype = IZB_BF16;
        a.x = x;
        a.w = weight_->get();
        a.bias = bias_ ? bias_->get() : nullptr;
        a.y = y;
        a.M = m; a.N = out_; a.K = in_;
        a.ldx = ldx ? ldx : in_;
        a.ldy = ldy ? ldy : (epilogue == IZB_EPI_SWIGLU ? out_ / 2 : out_);
        a.workspace = workspace;
        a.workspace_bytes = workspace_bytes;
        a.epilogue = epilogue;
        check(izb_linear(ctx.get(), stream, &a), "Qwen3Projection::forward");
    }

  private:
    Kind kind_ = Kind::Dense;
    std::shared_ptr<DeviceBuffer> weight_, bias_;
    int64_t out_ = 0, in_ = 0;
    int32_t wfmt_ = IZB_W_BF16;
};

namespace detail {
inline std::shared_ptr<DeviceBuffer> concat(const std::vector<const DeviceBuffer*>& parts) {
    size_t total = 0;
    for (auto* p : parts) total += p->bytes();
    auto out = std::make_shared<DeviceBuffer>(total);
    size_t at = 0;
    for (auto* p : parts) {
        if (p->bytes() && cudaMemcpy(static_cast<uint8_t*>(out->get()) + at, p->get(), p->bytes(),
                                     cudaMemcpyDeviceToDevice) != cudaSuccess)
            throw InferenceError("device to device copy failed");
        at += p->bytes();
    }
    return out;
}
inline std::shared_ptr<DeviceBuffer> concat_biases(const char* name, const std::vector<const Qwen3Projection*>& ps) {
    size_t have = 0;
    for (auto* p : ps) have += p->bias() ? 1 : 0;
    if (have == 0) return nullptr;
    if (have != ps.size()) throw InferenceError(std::string(name) + " cannot fuse projections with mixed bias presence");
    std::vector<const DeviceBuffer*> parts;
    for (auto* p : ps) parts.push_back(p->bias().get());
    return concat(parts);
}
}  // namespace detail

// Row-wise concatenation of raw GGML bytes into one quantized projection.
inline Qwen3Projection packed_qmatmul_from_qtensors(const std::vector<QTensor>& tensors) {
    if (tensors.empty()) throw InferenceError("Cannot pack empty Qwen3 quantized projection group");
    const int32_t dtype = tensors[0].dtype;
    const int64_t cols = tensors[0].cols;
    int64_t rows = 0;
    std::vector<const DeviceBuffer*> parts;
    for (const auto& t : tensors) {
        if (t.cols != cols)
            throw InferenceError("Qwen3 quantized projection group input mismatch: expected " + std::to_string(cols) +
                                 ", got " + std::to_string(t.cols));
        if (t.dtype != dtype)
            throw InferenceError(std::string("Qwen3 quantized projection group dtype mismatch: expected ") +
                                 wfmt_name(dtype) + ", got " + wfmt_name(t.dtype));
        rows += t.rows;
        parts.push_back(t.data.get());
    }
    size_t raw = 0;
    for (auto* p : parts) raw += p->bytes();
    const size_t expected = quantized_storage_bytes(rows, cols, dtype);
    if (raw != expected)
        throw InferenceError("Qwen3 packed quantized projection has " + std::to_string(raw) + " bytes, expected " +
                             std::to_string(expected));
    return Qwen3Projection::quantized(QTensor{detail::concat(parts), rows, cols, dtype});
}

class Qwen3FusedQkvProjection {
  public:
    Qwen3FusedQkvProjection(const Qwen3Projection& q, const Qwen3Projection& k, const Qwen3Projection& v)
        : q_out(q.out_dim()), k_out(k.out_dim()), v_out(v.out_dim()),
          bias_count((q.bias() ? 1 : 0) + (k.bias() ? 1 : 0) + (v.bias() ? 1 : 0)),
          fused(make(q, k, v)) {}
    // qkv[M, q_out + k_out + v_out]; q | k | v are column ranges of it (views, no copies).
    void forward(const Context& ctx, cudaStream_t s, const void* x, int64_t m, void* qkv) const {
        fused.forward(ctx, s, x, m, qkv);
    }
    Qwen3ProjectionDiagnostics diagnostics() const { return {3, bias_count, 0}; }
    const int64_t q_out, k_out, v_out;
    const size_t bias_count;
    const Qwen3Projection fused;

  private:
    static Qwen3Projection make(const Qwen3Projection& q, const Qwen3Projection& k, const Qwen3Projection& v) {
        if (k.in_dim() != q.in_dim() || v.in_dim() != q.in_dim())
            throw InferenceError("Qwen3 fused QKV projection input dimensions do not match");
        auto w = detail::concat({q.weight().get(), k.weight().get(), v.weight().get()});
        auto b = detail::concat_biases("Qwen3 fused QKV projection", {&q, &k, &v});
        return Qwen3Projection::dense(w, q.out_dim() + k.out_dim() + v.out_dim(), q.in_dim(), b);
    }
};

class Qwen3FusedGateUpProjection {
  public:
    Qwen3FusedGateUpProjection(const Qwen3Projection& gate, const Qwen3Projection& up)
        : intermediate_size(gate.out_dim()), bias_count((gate.bias() ? 1 : 0) + (up.bias() ? 1 : 0)),
          fused(make(gate, up)) {}
    void forward(const Context& ctx, cudaStream_t s, const void* x, int64_t m, void* gate_up) const {
        fused.forward(ctx, s, x, m, gate_up);
    }
    Qwen3ProjectionDiagnostics diagnostics() const { return {2, bias_count, 0}; }
    const int64_t intermediate_size;
    const size_t bias_count;
    const Qwen3Projection fused;

  private:
    static Qwen3Projection make(const Qwen3Projection& gate, const Qwen3Projection& up) {
        if (up.out_dim() != gate.out_dim() || up.in_dim() != gate.in_dim())
            throw InferenceError("Qwen3 fused MLP projection dimensions do not match");
        auto w = detail::concat({gate.weight().get(), up.weight().get()});
        auto b = detail::concat_biases("Qwen3 fused MLP projection", {&gate, &up});
        return Qwen3Projection::dense(w, 2 * gate.out_dim(), gate.in_dim(), b);
    }
};

// down( silu(gate) * up ): fused gate/up projection, fused SiLU-multiply on the two halves in
// place, down projection.  `scratch` holds [M, 2I + I] bf16 values.
class Qwen3Mlp {
  public:
    Qwen3Mlp(Qwen3Projection gate_up, Qwen3Projection down)
        : gate_up_proj(std::move(gate_up)), down_proj(std::move(down)), inter_(gate_up_proj.out_dim() / 2) {}
    size_t scratch_bytes(int64_t m) const { return static_cast<size_t>(m) * inter_ * 3 * 2; }
    void forward(const Context& ctx, cudaStream_t s, const void* x, int64_t m, void* y, void* scratch) const {
        auto* gu = static_cast<uint8_t*>(scratch);
        auto* hidden = gu + static_cast<size_t>(m) * inter_ * 2 * 2;
        gate_up_proj.forward(ctx, s, x, m, gu);
        check(izb_silu_mul(ctx.get(), s, gu, gu + inter_ * 2, hidden, m, inter_, 2 * inter_, 2 * inter_, inter_),
              "izb_silu_mul");
        down_proj.forward(ctx, s, hidden, m, y);
    }
    const Qwen3Projection gate_up_proj, down_proj;

  private:
    int64_t inter_;
};

}  // namespace izwi_host
