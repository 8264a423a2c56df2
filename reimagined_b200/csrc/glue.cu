// Row norms that sit either side of a ternary linear in the hybrid's decode / prefill step, fused with the
// gate that precedes them and, optionally, with the activation quantiser that follows them.
//
//   gate == null : block norm            out = (x * inv_rms(x)) * weight          (OXN/nsos/src/jamba.cpp:3175-3179)
//   gate != null : Mamba-2 epilogue      v = y * silu(z); out = (v * inv_rms(v)) * weight
//                  (OXN/nsos/src/mamba2.cpp:4011; the reference's device form is
//                   OXN/nsos/src/cuda/mamba_kernels.cu:3421-3441, which writes v to global memory and reads
//                   it back for the second pass)
//
// One CTA per row, the row held in shared memory between the passes, so global traffic is the algorithmic
// minimum: one read of each input and one write of each requested output.  With q != null the int8 codes, the
// per-row activation scale and the code sum of the normalised row are produced in the same launch (the
// arithmetic of the per-token quantiser, OXN/nsos/src/bitlinear.cpp:240-291, applied to the fp32 values this
// kernel would have stored), which removes the fp32 round trip between the norm and the next linear.
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;

// x * sigmoid(x) with the two-sided sigmoid of Tensor::silu (OXN/nsos/src/tensor.cpp:3273-3280).
__device__ __forceinline__ float silu(float g) {
    const float sig = g >= 0.0f ? __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)))
                                : __fdiv_rn(expf(g), __fadd_rn(1.0f, expf(g)));
    return __fmul_rn(g, sig);
}

__device__ __forceinline__ float norm_block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormWarps; ++w) r += scratch[w];   // fixed order: the same sum in every thread
    __syncthreads();
    return r;
}

__device__ __forceinline__ float norm_block_max(float v, float* scratch) {
    // non-negative floats order like their bit patterns
    const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(v));
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = __uint_as_float(m);
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormWarps; ++w) r = fmaxf(r, scratch[w]);
    __syncthreads();
    return r;
}

// In the vector passes every thread touches the same elements of `row` each time (j = tid*4 + i*1024); the
// scalar passes (dim % 4 != 0 or unaligned pointers) index differently from the code pass, and the block
// reductions between the passes plus the barrier that ends a quantised row order those.
template <bool GATED>
__global__ void __launch_bounds__(kNormThreads)
row_norm_kernel(const float* __restrict__ value, const float* __restrict__ gate, const float* __restrict__ weight,
                int rows, int dim, float eps, float q_max, bool vec, float* __restrict__ out,
                int8_t* __restrict__ q, float* __restrict__ act_scales, int32_t* __restrict__ q_sums) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[kNormWarps];
    __shared__ int sum_scratch[kNormWarps];
    const float fdim = static_cast<float>(dim);

    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const size_t base = static_cast<size_t>(r) * dim;
        const float* v = value + base;
        const float* z = GATED ? gate + base : nullptr;

        // pass 1: gate, cache, sum of squares
        float ss = 0.0f;
        if (vec) {
            for (int j = threadIdx.x * 4; j < dim; j += kNormThreads * 4) {
                float4 a = __ldg(reinterpret_cast<const float4*>(v + j));
                if (GATED) {
                    const float4 g = __ldg(reinterpret_cast<const float4*>(z + j));
                    a.x = __fmul_rn(a.x, silu(g.x)); a.y = __fmul_rn(a.y, silu(g.y));
                    a.z = __fmul_rn(a.z, silu(g.z)); a.w = __fmul_rn(a.w, silu(g.w));
                }
                *reinterpret_cast<float4*>(row + j) = a;
                ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        } else {
            for (int j = threadIdx.x; j < dim; j += kNormThreads) {
                float a = v[j];
                if (GATED) a = __fmul_rn(a, silu(z[j]));
                row[j] = a;
                ss += a * a;
            }
        }
        ss = norm_block_sum(ss, scratch);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, fdim), eps)));

        // pass 2: normalise, weight, store fp32; track the absmax when codes are wanted
        float mx = 0.0f;
        if (vec) {
            for (int j = threadIdx.x * 4; j < dim; j += kNormThreads * 4) {
                float4 a = *reinterpret_cast<const float4*>(row + j);
                a.x = __fmul_rn(a.x, inv); a.y = __fmul_rn(a.y, inv);
                a.z = __fmul_rn(a.z, inv); a.w = __fmul_rn(a.w, inv);
                if (weight) {
                    const float4 w = __ldg(reinterpret_cast<const float4*>(weight + j));
                    a.x = __fmul_rn(a.x, w.x); a.y = __fmul_rn(a.y, w.y);
                    a.z = __fmul_rn(a.z, w.z); a.w = __fmul_rn(a.w, w.w);
                }
                if (out) *reinterpret_cast<float4*>(out + base + j) = a;
                if (q) {
                    *reinterpret_cast<float4*>(row + j) = a;
                    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
                }
            }
        } else {
            for (int j = threadIdx.x; j < dim; j += kNormThreads) {
                float a = __fmul_rn(row[j], inv);
                if (weight) a = __fmul_rn(a, weight[j]);
                if (out) out[base + j] = a;
                if (q) {
                    row[j] = a;
                    mx = fmaxf(mx, fabsf(a));
                }
            }
        }
        if (!q) continue;     // uniform across the block

        // pass 3 (dim % 16 == 0, checked by the launcher): the per-token quantiser on the cached row
        mx = norm_block_max(mx, scratch);
        const float denom = __fadd_rn(mx, 1e-8f);
        const float scale = __fdiv_rn(q_max, denom);
        if (threadIdx.x == 0) act_scales[r] = __fdiv_rn(denom, q_max);
        int local_sum = 0;
        for (int j = threadIdx.x * 4; j < dim; j += kNormThreads * 4) {
            const float4 a = *reinterpret_cast<const float4*>(row + j);
            const int c0 = round_code(__fmul_rn(a.x, scale), false);
            const int c1 = round_code(__fmul_rn(a.y, scale), false);
            const int c2 = round_code(__fmul_rn(a.z, scale), false);
            const int c3 = round_code(__fmul_rn(a.w, scale), false);
            const uint32_t word = (c0 & 0xff) | ((c1 & 0xff) << 8) | ((c2 & 0xff) << 16) |
                                  (static_cast<uint32_t>(c3 & 0xff) << 24);
            local_sum = dp4a_ss(static_cast<int>(word), 0x01010101, local_sum);
            *reinterpret_cast<uint32_t*>(q + base + j) = word;
        }
        if (q_sums) {
            local_sum = __reduce_add_sync(0xffffffffu, local_sum);
            if ((threadIdx.x & 31) == 0) sum_scratch[threadIdx.x >> 5] = local_sum;
            __syncthreads();
            if (threadIdx.x == 0) {
                int total = 0;
#pragma unroll
                for (int w = 0; w < kNormWarps; ++w) total += sum_scratch[w];
                q_sums[r] = total;
            }
        }
        __syncthreads();      // the scalar passes and this one index the row differently: order them across rows
    }
}

template <bool GATED>
cudaError_t launch_one(const float* value, const float* gate, const float* weight, int rows, int dim, float eps,
                       float q_max, float* out, int8_t* q, float* act_scales, int32_t* q_sums,
                       cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(dim) * sizeof(float);
    static size_t configured = 0;      // one per instantiation
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(row_norm_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kRowNormMaxDim * sizeof(float)));
        if (e != cudaSuccess) return e;
        configured = kRowNormMaxDim * sizeof(float);
    }
    // one CTA per row while the rows fit one wave of resident CTAs, else a grid-stride over rows
    int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm);
    const int grid = rows < 148 * per_sm ? rows : 148 * per_sm;
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = dim % 4 == 0 && aligned16(value) && aligned16(gate) && aligned16(weight) && aligned16(out);
    row_norm_kernel<GATED><<<grid, kNormThreads, smem, stream>>>(value, gate, weight, rows, dim, eps, q_max, vec, out,
                                                                q, act_scales, q_sums);
    note_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_row_norm(const float* value, const float* gate, const float* weight, int rows, int dim, float eps,
                            int bits, float* out, int8_t* q, float* act_scales, int32_t* q_sums,
                            cudaStream_t stream) {
    if (dim < 1 || dim > kRowNormMaxDim || rows < 1) return cudaErrorInvalidValue;
    if (q && (dim % 16 || (reinterpret_cast<uintptr_t>(q) & 3))) return cudaErrorInvalidValue;
    const float q_max = q ? qmax_for_bits(bits) : 0.0f;
    return gate ? launch_one<true>(value, gate, weight, rows, dim, eps, q_max, out, q, act_scales, q_sums, stream)
                : launch_one<false>(value, gate, weight, rows, dim, eps, q_max, out, q, act_scales, q_sums, stream);
}

}  // namespace tbl
