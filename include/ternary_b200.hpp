// Header-only C++17 shim over the C ABI of ternary_b200.h, for a C++ host such as the NSOS runtime.
//
// It gives the C entry points the reference's calling conventions: errors become the exception types
// the reference throws (OXN/nsos/src/bitnet_gpu_dispatch.cpp:70-116: std::invalid_argument for bad
// arguments, std::overflow_error for K > INT_MAX/254 or M*N > INT_MAX, std::runtime_error for the rest),
// and `bitnet_gemm_158bit_gpu` has the argument list of nsos::bitnet_gemm_158bit_gpu
// (OXN/nsos/include/bitnet_gpu_dispatch.h:46-51) with raw device pointers in place of nsos::Tensor
// (a Tensor-typed wrapper passes raw_data() of each tensor).  Nothing here allocates device memory
// or synchronises: the caller owns the output and the scratch, and orders the stream.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

extern "C" {
#include "ternary_b200.h"
}

namespace ternary_b200 {

// Status code of the C ABI -> the exception the reference would have thrown at the same place.
inline void throw_on_status(int status, const char* where) {
    if (status == TBL_OK) return;
    const std::string what = std::string(where) + ": " + tbl_status_string(status);
    switch (status) {
        case TBL_ERR_OVERFLOW: throw std::overflow_error(what);
        case TBL_ERR_INVALID_ARG:
        case TBL_ERR_SCALE:
        case TBL_ERR_BITS:
        case TBL_ERR_SHAPE: throw std::invalid_argument(what);
        default: throw std::runtime_error(what);
    }
}

// What BitLinear keeps on the device for one layer (OXN/nsos/include/bitlinear.h:304 holds the first of
// these today; the other two are derived from it once, where the packed words are uploaded).
struct DeviceWeights {
    const std::uint32_t* words = nullptr;   // canonical 2-bit words (the reference's device format)
    const void* strips = nullptr;           // tbl_relayout_strips(words): decode path, K % 256 == 0
    const std::int8_t* w_i8 = nullptr;      // tbl_expand_weights_i8(words): prefill path, M > 64
    float weight_scale = 0.0f;
    int out_features = 0, in_features = 0;
};

// Scratch bytes one call needs; the reference reserves its equivalent from ExecutionContext workspace
// slots (OXN/nsos/src/bitnet_gpu_dispatch.cpp:118-123).
inline std::size_t workspace_bytes(int M, int K, int N) { return tbl_linear_workspace_bytes(M, K, N); }

// nsos::bitnet_gemm_158bit_gpu with raw pointers: y[M,N] = epilogue(quantise(x[M,K]) x ternary[N,K]^T).
// `rms_mode` is TBL_RMS_NONE when the caller has already normalised x, as BitLinear::forward does.
inline void bitnet_gemm_158bit_gpu(const float* x_gpu, const DeviceWeights& w, int M, int precision_bits,
                                   const float* magnitude, const float* bias, float* y_gpu, void* scratch,
                                   std::size_t scratch_bytes, void* stream, int rms_mode = TBL_RMS_NONE) {
    throw_on_status(tbl_linear_forward(x_gpu, w.words, w.strips, w.w_i8, w.weight_scale, M, w.in_features,
                                       w.out_features, precision_bits, rms_mode, magnitude, bias, y_gpu, scratch,
                                       scratch_bytes, stream),
                    "bitnet_gemm_158bit_gpu");
}

// BitLinear::pack_weights (OXN/nsos/src/bitlinear.cpp:152-193) on the host: canonical words + weight_scale.
inline float pack_weights(const float* w, int N, int K, std::uint32_t* words) {
    float scale = 0.0f;
    throw_on_status(tbl_pack_weights(w, N, K, words, &scale), "pack_weights");
    return scale;
}

// The checks of BitLinear::prepare_packed_state (OXN/nsos/src/bitlinear.cpp:834-900) before a pack is installed.
inline void validate_packed(const std::uint32_t* words, long long nwords, int N, int K, float weight_scale,
                            const float* magnitude = nullptr, const float* bias = nullptr) {
    throw_on_status(tbl_validate_packed(words, nwords, N, K, weight_scale, magnitude, bias), "import_packed_state");
}

// cuda::launch_mamba_gated_rmsnorm (OXN/nsos/include/cuda/mamba_kernels.cuh:383) with its argument list plus the
// stream: output = rmsnorm(y * silu(z), epsilon) * weight, one launch.  Throws std::invalid_argument where the
// reference does ("Invalid Mamba RMS geometry": rows < 1, dim < 1, epsilon <= 0).
inline void mamba_gated_rmsnorm(const float* y, const float* z, const float* weight, float* output, int rows,
                                int dim, float epsilon, void* stream) {
    throw_on_status(tbl_row_norm(y, z, weight, rows, dim, epsilon, output, 8, nullptr, nullptr, nullptr, stream),
                    "mamba_gated_rmsnorm");
}

// Tensor::rmsnorm(eps).mul(weight) of the block norm (OXN/nsos/src/jamba.cpp:3175-3179); weight may be null.
inline void rmsnorm_weight(const float* x, const float* weight, float* output, int rows, int dim, float eps,
                           void* stream) {
    throw_on_status(tbl_row_norm(x, nullptr, weight, rows, dim, eps, output, 8, nullptr, nullptr, nullptr, stream),
                    "rmsnorm");
}

// ---- the layer object ------------------------------------------------------------------------------------------

// nsos::BitLinearPackedState (OXN/nsos/include/bitlinear.h:37-47), field for field: the interchange form of a layer.
struct PackedState {
    int in_features = 0;
    int out_features = 0;
    bool use_bias = true;
    float weight_scale = 1.0f;
    std::vector<std::uint32_t> packed_weights;
    std::vector<float> magnitude;
    std::vector<float> bias;
    std::vector<float> flat_alpha;
    std::vector<float> flat_beta;
};

// How the host runtime hands out device memory.  The C ABI never allocates; the layer object asks its owner.
// (The reference draws from its tensor pool, OXN/nsos/include/tensor.h:89-152.)  `upload` enqueues a host-to-device
// copy on `stream`; the source stays alive until the caller has synchronised.
struct DeviceMemory {
    std::function<void*(std::size_t bytes)> allocate;
    std::function<void(void* ptr)> release;
    std::function<void(void* dst, const void* src, std::size_t bytes, void* stream)> upload;
};

// The packed-inference surface of nsos::BitLinear (OXN/nsos/include/bitlinear.h:77-212) over the C ABI:
// import_packed_state / export_packed_state / forward / prepare_gpu_decode_view, with the reference's transactional
// import -- prepare_packed_state validates and fills freshly allocated buffers and may throw without touching the
// layer, commit_prepared_packed_state only swaps owned buffers (OXN/nsos/src/bitlinear.cpp:834-1028).
class TernaryLinear {
public:
    TernaryLinear(int in_features, int out_features, bool bias, DeviceMemory memory)
        : in_(in_features), out_(out_features), use_bias_(bias), mem_(std::move(memory)) {
        if (in_features <= 0 || out_features <= 0) throw std::invalid_argument("BitLinear feature counts must be positive");
        if (!mem_.allocate || !mem_.release || !mem_.upload) throw std::invalid_argument("DeviceMemory callbacks are required");
    }
    TernaryLinear(const TernaryLinear&) = delete;
    TernaryLinear& operator=(const TernaryLinear&) = delete;
    ~TernaryLinear() { release(live_); }

    // Device buffers of one validated state, owned until committed or destroyed.
    class Prepared {
    public:
        Prepared(Prepared&& o) noexcept : owner_(o.owner_), dev_(o.dev_), host_(std::move(o.host_)) { o.dev_ = Buffers{}; }
        Prepared& operator=(Prepared&&) = delete;
        Prepared(const Prepared&) = delete;
        ~Prepared() { if (owner_) owner_->release(dev_); }
    private:
        friend class TernaryLinear;
        struct Buffers { void *words = nullptr, *strips = nullptr, *w_i8 = nullptr, *magnitude = nullptr, *bias = nullptr; };
        Prepared(const TernaryLinear* owner, PackedState host) : owner_(owner), host_(std::move(host)) {}
        const TernaryLinear* owner_;
        Buffers dev_;
        PackedState host_;
    };

    // Validation (shape, lengths, finite positive scale, no reserved code, finite affine; with `retained_fp32` the
    // codes and the scale must equal a fresh packing of those weights, OXN/nsos/src/bitlinear.cpp:957-973), then
    // upload into new buffers and derivation of the device layouts.  Throws std::runtime_error like the reference;
    // the live layer is untouched.  `with_int8` also keeps the int8 expansion the prefill GEMM (M > 64) reads.
    Prepared prepare_packed_state(const PackedState& state, void* stream, bool with_int8 = true,
                                  const float* retained_fp32 = nullptr) const {
        if (state.in_features != in_ || state.out_features != out_ || state.use_bias != use_bias_)
            throw std::runtime_error("BitLinear packed state shape mismatch");
        const std::size_t total = static_cast<std::size_t>(out_) * static_cast<std::size_t>(in_);
        if (state.packed_weights.size() != (total + 15) / 16 || state.magnitude.size() != static_cast<std::size_t>(out_) ||
            state.bias.size() != (use_bias_ ? static_cast<std::size_t>(out_) : 0u) ||
            state.flat_alpha.size() != static_cast<std::size_t>(in_) || state.flat_beta.size() != static_cast<std::size_t>(in_))
            throw std::runtime_error("BitLinear packed state buffer length mismatch");
        const int rc = tbl_validate_packed(state.packed_weights.data(), static_cast<long long>(state.packed_weights.size()), out_,
                                           in_, state.weight_scale, state.magnitude.data(), use_bias_ ? state.bias.data() : nullptr);
        if (rc != TBL_OK) throw std::runtime_error(std::string("BitLinear packed state rejected: ") + tbl_status_string(rc));
        for (const std::vector<float>* v : {&state.flat_alpha, &state.flat_beta})
            for (float f : *v)
                if (!(f - f == 0.0f)) throw std::runtime_error("BitLinear packed state contains non-finite values");
        if (retained_fp32) {
            std::vector<std::uint32_t> words(state.packed_weights.size());
            float scale = 0.0f;
            throw_on_status(tbl_pack_weights(retained_fp32, out_, in_, words.data(), &scale), "prepare_packed_state");
            if (std::memcmp(&scale, &state.weight_scale, sizeof(float)) != 0 || words != state.packed_weights)
                throw std::runtime_error("BitLinear packed state does not match the retained full-precision weights");
        }
        Prepared p(this, state);
        const std::size_t word_bytes = state.packed_weights.size() * sizeof(std::uint32_t);
        p.dev_.words = take(word_bytes);
        mem_.upload(p.dev_.words, p.host_.packed_weights.data(), word_bytes, stream);
        p.dev_.magnitude = take(sizeof(float) * out_);
        mem_.upload(p.dev_.magnitude, p.host_.magnitude.data(), sizeof(float) * out_, stream);
        if (use_bias_) {
            p.dev_.bias = take(sizeof(float) * out_);
            mem_.upload(p.dev_.bias, p.host_.bias.data(), sizeof(float) * out_, stream);
        }
        if (in_ % 16 == 0) {
            const std::size_t strip_bytes = tbl_strip_bytes(out_, in_);
            if (strip_bytes) {
                p.dev_.strips = take(strip_bytes);
                throw_on_status(tbl_relayout_strips(static_cast<const std::uint32_t*>(p.dev_.words), out_, in_, p.dev_.strips, stream),
                                "prepare_packed_state");
            }
            if (with_int8) {
                p.dev_.w_i8 = take(total);
                throw_on_status(tbl_expand_weights_i8(static_cast<const std::uint32_t*>(p.dev_.words), out_, in_,
                                                      static_cast<std::int8_t*>(p.dev_.w_i8), stream),
                                "prepare_packed_state");
            }
        }
        return p;
    }

    // Installs a prepared state: swaps owned pointers, frees the previous buffers, cannot fail.
    void commit_prepared_packed_state(Prepared&& p) noexcept {
        std::swap(live_, p.dev_);
        std::swap(host_, p.host_);
        loaded_ = true;
    }

    void import_packed_state(const PackedState& state, void* stream, bool with_int8 = true) {
        commit_prepared_packed_state(prepare_packed_state(state, stream, with_int8));
    }

    // BitLinear::export_packed_state (OXN/nsos/src/bitlinear.cpp:764-799).
    PackedState export_packed_state() const {
        if (!loaded_) throw std::runtime_error("BitLinear has no packed state to export");
        return host_;
    }

    void set_exact_linear_mode(bool enabled) { exact_ = enabled; }    // no input RMSNorm, no magnitude (bitlinear.h:99-108)
    bool exact_linear_mode() const { return exact_; }
    void set_precision_mode(int bits) {
        if (bits < 2 || bits > 8) throw std::invalid_argument("activation bits must be in [2,8]");
        bits_ = bits;
    }
    int input_features() const { return in_; }
    int output_features() const { return out_; }
    bool uses_bias() const { return use_bias_; }

    std::size_t workspace_bytes(int rows) const { return tbl_linear_workspace_bytes(rows, in_, out_); }

    // BitLinear::forward, packed branch: x fp32 [rows, in] -> y fp32 [rows, out], enqueued on `stream`.
    // rms_mode applies in default mode only: TBL_RMS_FAST, or TBL_RMS_REFERENCE_ORDER for the CPU path's sum order.
    void forward(const float* x_dev, int rows, float* y_dev, void* scratch, std::size_t scratch_bytes, void* stream,
                 int rms_mode = TBL_RMS_FAST) const {
        if (!loaded_) throw std::runtime_error("BitLinear::forward before import_packed_state");
        throw_on_status(tbl_linear_forward(x_dev, static_cast<const std::uint32_t*>(live_.words), live_.strips,
                                           static_cast<const std::int8_t*>(live_.w_i8), host_.weight_scale, rows, in_, out_,
                                           bits_, exact_ ? TBL_RMS_NONE : rms_mode,
                                           exact_ ? nullptr : static_cast<const float*>(live_.magnitude),
                                           static_cast<const float*>(live_.bias), y_dev, scratch, scratch_bytes, stream),
                        "BitLinear::forward");
    }

    // BitLinear::prepare_gpu_decode_view (OXN/nsos/src/bitlinear.cpp:335-389): a borrowed descriptor for the grouped
    // entry points; false when the layer has nothing packed to show.
    bool prepare_gpu_decode_view(tbl_linear_view& view) const {
        if (!loaded_ || in_ % 16 != 0) return false;
        view = tbl_linear_view{};
        view.packed = static_cast<const std::uint32_t*>(live_.words);
        view.magnitude = exact_ ? nullptr : static_cast<const float*>(live_.magnitude);
        view.bias = static_cast<const float*>(live_.bias);
        view.inputs = in_;
        view.outputs = out_;
        view.activation_bits = bits_;
        view.rms_input = exact_ ? 0 : 1;
        view.weight_scale = host_.weight_scale;
        view.strips = live_.strips;
        view.w_i8 = static_cast<const std::int8_t*>(live_.w_i8);
        return true;
    }

private:
    void* take(std::size_t bytes) const {
        void* p = mem_.allocate(bytes ? bytes : 16);
        if (!p) throw std::runtime_error("BitLinear: device allocation failed");
        return p;
    }
    void release(Prepared::Buffers& b) const {
        for (void** p : {&b.words, &b.strips, &b.w_i8, &b.magnitude, &b.bias}) {
            if (*p) mem_.release(*p);
            *p = nullptr;
        }
    }
    int in_, out_;
    bool use_bias_;
    bool exact_ = false, loaded_ = false;
    int bits_ = 8;
    DeviceMemory mem_;
    mutable Prepared::Buffers live_;
    PackedState host_;
};

// launch_grouped_decode_projections with the reference's argument list (OXN/nsos/include/cuda/kernels.cuh:27-29,
// OXN/nsos/src/cuda/moe_kernels.cu:779-784): `groups` linears on ONE input row, view g writing output + g*output_stride.
// Differences a caller has to know: the descriptors are read on the HOST -- pass the host vector that
// GpuProjectionGroup::forward fills before it uploads a device copy (OXN/nsos/src/gpu_projection_group.cpp:15-29) --
// and `prepared` / `scales`, the caller's two ExecutionContext slots (float [groups*inputs] and float [groups],
// gpu_projection_group.cpp:33-36), serve as this library's scratch: `prepared_floats` says how large the first is.
// All views must share inputs, activation_bits and rms_input (the row is quantised once; the reference's own
// callers satisfy this: Q/KV, Mamba x/z/B/C/dt).  Throws std::invalid_argument / std::runtime_error like the shim above.
inline void launch_grouped_decode_projections(const tbl_linear_view* views_host, const float* input, float* prepared,
                                              std::size_t prepared_floats, float* scales, float* output, int groups,
                                              int output_stride, void* stream, int rms_mode = TBL_RMS_FAST) {
    (void)scales;     // the per-row scale lives inside `prepared` here
    if (!views_host || groups <= 0) throw std::invalid_argument("launch_grouped_decode_projections: no descriptors");
    const std::size_t need = tbl_grouped_workspace_bytes(groups, views_host[0].inputs);
    if (prepared_floats * sizeof(float) < need)
        throw std::invalid_argument("launch_grouped_decode_projections: the GroupedPrepared slot is smaller than " +
                                    std::to_string(need) + " bytes");
    throw_on_status(tbl_grouped_forward(views_host, groups, input, output, output_stride, rms_mode, prepared,
                                        prepared_floats * sizeof(float), stream),
                    "launch_grouped_decode_projections");
}

// Sticky device status (bounded waits that gave up, MoE route overflow); synchronises the stream.
inline void check_device(void* stream) {
    const int status = tbl_device_status(stream);
    if (status < 0) throw std::runtime_error("tbl_device_status: CUDA error");
    if (status & TBL_DEV_WAIT_TIMEOUT) throw std::runtime_error("ternary_b200: a device-side wait timed out");
    if (status & TBL_DEV_ROUTE_OVERFLOW) throw std::runtime_error("ternary_b200: more routes per row than allowed");
}

}  // namespace ternary_b200
