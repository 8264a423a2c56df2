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
#include <stdexcept>
#include <string>

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

// Sticky device status (bounded waits that gave up, MoE route overflow); synchronises the stream.
inline void check_device(void* stream) {
    const int status = tbl_device_status(stream);
    if (status < 0) throw std::runtime_error("tbl_device_status: CUDA error");
    if (status & TBL_DEV_WAIT_TIMEOUT) throw std::runtime_error("ternary_b200: a device-side wait timed out");
    if (status & TBL_DEV_ROUTE_OVERFLOW) throw std::runtime_error("ternary_b200: more routes per row than allowed");
}

}  // namespace ternary_b200
