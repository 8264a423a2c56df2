// Correctness fallback for shapes the streamed kernels do not take (K % 64 != 0, very long
// rows): one warp per output row, 32-bit word loads, dp4a on byte-spread codes.  Any M.
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

constexpr int kRowsPerBlock = 4;
constexpr int kMTile = 8;

// four 2-bit codes in the low byte -> four signed bytes (code - 1)
__device__ __forceinline__ int spread_codes(uint32_t b) {
    const uint32_t s = (b & 0x03u) | ((b & 0x0cu) << 6) | ((b & 0x30u) << 12) | ((b & 0xc0u) << 18);
    return static_cast<int>(__vsub4(s, 0x01010101u));
}

__global__ void __launch_bounds__(kRowsPerBlock * 32)
gemv_generic_kernel(const int8_t* __restrict__ q, const float* __restrict__ act_scales,
                    const uint32_t* __restrict__ words, float weight_scale,
                    const float* __restrict__ magnitude, const float* __restrict__ bias, int M, int K,
                    int N, float* __restrict__ y, int32_t* __restrict__ acc_debug, int squared_relu,
                    const int32_t* __restrict__ rows_dev, const int32_t* __restrict__ offset_dev) {
    const int n = blockIdx.x * kRowsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    if (rows_dev) M = min(M, *rows_dev);
    if (offset_dev) {
        const int off = *offset_dev;
        q += static_cast<size_t>(off) * K;
        act_scales += off;
        y += static_cast<size_t>(off) * N;
        if (acc_debug) acc_debug += static_cast<size_t>(off) * N;
    }
    const int wpr = K >> 4;  // words per row
    const uint32_t* wrow = words + static_cast<size_t>(n) * wpr;
    for (int m0 = 0; m0 < M; m0 += kMTile) {
        int acc[kMTile];
#pragma unroll
        for (int i = 0; i < kMTile; ++i) acc[i] = 0;
        for (int w = lane; w < wpr; w += 32) {
            const uint32_t word = __ldg(wrow + w);
            const int t0 = spread_codes(word & 0xffu), t1 = spread_codes((word >> 8) & 0xffu);
            const int t2 = spread_codes((word >> 16) & 0xffu), t3 = spread_codes(word >> 24);
#pragma unroll
            for (int i = 0; i < kMTile; ++i) {
                if (m0 + i < M) {
                    const int4 a = __ldg(reinterpret_cast<const int4*>(q + static_cast<size_t>(m0 + i) * K + w * 16));
                    acc[i] = dp4a_ss(a.x, t0, acc[i]);
                    acc[i] = dp4a_ss(a.y, t1, acc[i]);
                    acc[i] = dp4a_ss(a.z, t2, acc[i]);
                    acc[i] = dp4a_ss(a.w, t3, acc[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kMTile; ++i) {
            int t = acc[i];
#pragma unroll
            for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0 && m0 + i < M) {
                const int m = m0 + i;
                if (acc_debug) acc_debug[static_cast<size_t>(m) * N + n] = t;
                float v = epilogue(t, __fmul_rn(act_scales[m], weight_scale), magnitude, bias, n);
                if (squared_relu) { v = fmaxf(v, 0.0f); v = __fmul_rn(v, v); }
                y[static_cast<size_t>(m) * N + n] = v;
            }
        }
    }
}

}  // namespace

cudaError_t launch_gemv_generic(const int8_t* q, const float* act_scales, const uint32_t* words,
                                float weight_scale, const float* magnitude, const float* bias, int M,
                                int K, int N, float* y, int32_t* acc_debug, int squared_relu,
                                const int32_t* rows_dev, const int32_t* offset_dev, cudaStream_t stream) {
    const int blocks = (N + kRowsPerBlock - 1) / kRowsPerBlock;
    gemv_generic_kernel<<<blocks, kRowsPerBlock * 32, 0, stream>>>(q, act_scales, words, weight_scale,
                                                                   magnitude, bias, M, K, N, y, acc_debug,
                                                                   squared_relu, rows_dev, offset_dev);
    note_launch();
    return cudaGetLastError();
}

}  // namespace tbl
