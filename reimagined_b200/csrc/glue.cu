// Row norms that sit either side of a ternary linear in the hybrid's decode / prefill step, fused with the
// gate that precedes them and, optionally, with the activation quantiser that follows them.
//
//   gate == null : block norm            out = (x * inv_rms(x)) * weight          (OXN/nsos/src/jamba.cpp:3175-3179)
//   gate != null : Mamba-2 epilogue      v = y * silu(z); out = (v * inv_rms(v)) * weight
//                  (OXN/nsos/src/mamba2.cpp:4011; the reference's device form is
//                   OXN/nsos/src/cuda/mamba_kernels.cu:3421-3441, which writes v to global memory and reads
//                   it back for the second pass)
//
// One CTA per row with the row held in shared memory between the passes (or, for many short rows, one warp
// per row with the row in registers), so global traffic is the algorithmic minimum: one read of each input and one write of each requested output.  With q != null the int8 codes, the
// per-row activation scale and the code sum of the normalised row are produced in the same launch (the
// arithmetic of the per-token quantiser, OXN/nsos/src/bitlinear.cpp:240-291, applied to the fp32 values this
// kernel would have stored), which removes the fp32 round trip between the norm and the next linear.
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {

namespace {

constexpr int kNormMaxThreads = 1024;
constexpr int kNormMaxWarps = kNormMaxThreads / 32;

// x * sigmoid(x) with the two-sided sigmoid of Tensor::silu (OXN/nsos/src/tensor.cpp:3273-3280):
// 1 / (1 + exp(-g)) for g >= 0, exp(g) / (1 + exp(g)) below; both need only e = exp(-|g|).
__device__ __forceinline__ float silu(float g) {
    const float e = expf(-fabsf(g));
    const float sig = __fdiv_rn(g >= 0.0f ? 1.0f : e, __fadd_rn(1.0f, e));
    return __fmul_rn(g, sig);
}

__device__ __forceinline__ float norm_block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) r += scratch[w];   // fixed order: the same sum in every thread
    __syncthreads();
    return r;
}

__device__ __forceinline__ float norm_block_max(float v, float* scratch) {
    // non-negative floats order like their bit patterns
    const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(v));
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = __uint_as_float(m);
    __syncthreads();
    float r = 0.0f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) r = fmaxf(r, scratch[w]);
    __syncthreads();
    return r;
}

// In the vector passes every thread touches the same elements of `row` each time (j = 4 * tid + 4 * i * blockDim.x); the
// scalar passes (dim % 4 != 0 or unaligned pointers) index differently from the code pass, and the block
// reductions between the passes plus the barrier that ends a quantised row order those.
template <bool GATED>
__global__ void __launch_bounds__(kNormMaxThreads)
row_norm_kernel(const float* __restrict__ value, const float* __restrict__ gate, const float* __restrict__ weight,
                int rows, int dim, float eps, float q_max, bool vec, float* __restrict__ out,
                int8_t* __restrict__ q, float* __restrict__ act_scales, int32_t* __restrict__ q_sums) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[kNormMaxWarps];
    __shared__ int sum_scratch[kNormMaxWarps];
    const int nthreads = blockDim.x;
    const float fdim = static_cast<float>(dim);

    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const size_t base = static_cast<size_t>(r) * dim;
        const float* v = value + base;
        const float* z = GATED ? gate + base : nullptr;

        // pass 1: gate, cache, sum of squares
        float ss = 0.0f;
        if (vec) {
            for (int j = threadIdx.x * 4; j < dim; j += nthreads * 4) {
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
            for (int j = threadIdx.x; j < dim; j += nthreads) {
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
            for (int j = threadIdx.x * 4; j < dim; j += nthreads * 4) {
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
            for (int j = threadIdx.x; j < dim; j += nthreads) {
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
        for (int j = threadIdx.x * 4; j < dim; j += nthreads * 4) {
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
                for (int w = 0; w < (nthreads >> 5); ++w) total += sum_scratch[w];
                q_sums[r] = total;
            }
        }
        __syncthreads();      // the scalar passes and this one index the row differently: order them across rows
    }
}

// Many short rows: one warp per row, the row held in registers (NV float4 per lane, dim <= 128 * NV), no block
// barrier anywhere, and every load of a row issued before the first use -- with 16 warps or more resident per
// SM that keeps enough bytes in flight to follow HBM, which one CTA per 3 KB row cannot.
template <bool GATED, int NV>
__global__ void __launch_bounds__(256, 2)
row_norm_warp_kernel(const float* __restrict__ value, const float* __restrict__ gate,
                     const float* __restrict__ weight, int rows, int dim, float eps, float q_max,
                     float* __restrict__ out, int8_t* __restrict__ q, float* __restrict__ act_scales,
                     int32_t* __restrict__ q_sums) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const float fdim = static_cast<float>(dim);
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const size_t base = static_cast<size_t>(r) * dim;
        float4 a[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int j = (i * 32 + lane) * 4;
            a[i] = j < dim ? __ldcs(reinterpret_cast<const float4*>(value + base + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (GATED) {
            // up to 12 vectors per lane the whole gate is loaded up front beside the row (every load of the row
            // in flight at once); beyond that it goes through registers four vectors at a time, since holding
            // all of it would halve the warps an SM can keep resident
            constexpr int CH = NV <= 12 ? NV : 4;
#pragma unroll
            for (int c = 0; c < NV; c += CH) {
                float4 g[CH];
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    const int j = ((c + i) * 32 + lane) * 4;
                    g[i] = j < dim ? __ldcs(reinterpret_cast<const float4*>(gate + base + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < CH; ++i) {
                    float4& v = a[c + i];
                    v.x = __fmul_rn(v.x, silu(g[i].x)); v.y = __fmul_rn(v.y, silu(g[i].y));
                    v.z = __fmul_rn(v.z, silu(g[i].z)); v.w = __fmul_rn(v.w, silu(g[i].w));
                }
            }
        }
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) ss += a[i].x * a[i].x + a[i].y * a[i].y + a[i].z * a[i].z + a[i].w * a[i].w;
#pragma unroll
        for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);    // the same bits in every lane
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, fdim), eps)));

        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int j = (i * 32 + lane) * 4;
            if (j < dim) {
                a[i].x = __fmul_rn(a[i].x, inv); a[i].y = __fmul_rn(a[i].y, inv);
                a[i].z = __fmul_rn(a[i].z, inv); a[i].w = __fmul_rn(a[i].w, inv);
                if (weight) {
                    const float4 w = __ldg(reinterpret_cast<const float4*>(weight + j));
                    a[i].x = __fmul_rn(a[i].x, w.x); a[i].y = __fmul_rn(a[i].y, w.y);
                    a[i].z = __fmul_rn(a[i].z, w.z); a[i].w = __fmul_rn(a[i].w, w.w);
                }
                if (out) __stcs(reinterpret_cast<float4*>(out + base + j), a[i]);
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a[i].x), fabsf(a[i].y)), fmaxf(fabsf(a[i].z), fabsf(a[i].w))));
            }
        }
        if (!q) continue;     // uniform
        mx = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(mx)));
        const float denom = __fadd_rn(mx, 1e-8f);
        const float scale = __fdiv_rn(q_max, denom);
        if (lane == 0) act_scales[r] = __fdiv_rn(denom, q_max);
        int local_sum = 0;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int j = (i * 32 + lane) * 4;
            if (j < dim) {
                const int c0 = round_code(__fmul_rn(a[i].x, scale), false);
                const int c1 = round_code(__fmul_rn(a[i].y, scale), false);
                const int c2 = round_code(__fmul_rn(a[i].z, scale), false);
                const int c3 = round_code(__fmul_rn(a[i].w, scale), false);
                const uint32_t word = (c0 & 0xff) | ((c1 & 0xff) << 8) | ((c2 & 0xff) << 16) |
                                      (static_cast<uint32_t>(c3 & 0xff) << 24);
                local_sum = dp4a_ss(static_cast<int>(word), 0x01010101, local_sum);
                *reinterpret_cast<uint32_t*>(q + base + j) = word;
            }
        }
        if (q_sums) {
            local_sum = __reduce_add_sync(0xffffffffu, local_sum);
            if (lane == 0) q_sums[r] = local_sum;
        }
    }
}

template <bool GATED, int NV>
cudaError_t launch_warp_rows(const float* value, const float* gate, const float* weight, int rows, int dim, float eps,
                             float q_max, float* out, int8_t* q, float* act_scales, int32_t* q_sums,
                             cudaStream_t stream) {
    static int per_sm = 0;      // one per instantiation
    if (!per_sm) {
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, row_norm_warp_kernel<GATED, NV>, 256, 0);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) per_sm = 1;
    }
    const int ctas = (rows + 7) / 8;                       // 8 warps per CTA
    const int resident = 148 * per_sm;                     // one wave of CTAs; a warp strides over rows
    const int grid = ctas < resident ? ctas : resident;
    row_norm_warp_kernel<GATED, NV><<<grid, 256, 0, stream>>>(value, gate, weight, rows, dim, eps, q_max, out, q,
                                                             act_scales, q_sums);
    note_launch();
    return cudaGetLastError();
}

template <bool GATED>
cudaError_t launch_one(const float* value, const float* gate, const float* weight, int rows, int dim, float eps,
                       float q_max, float* out, int8_t* q, float* act_scales, int32_t* q_sums,
                       cudaStream_t stream) {
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool vec = dim % 4 == 0 && aligned16(value) && aligned16(gate) && aligned16(weight) && aligned16(out);
    if (vec && dim <= 2048 && rows >= 512) {
        if (dim <= 512)
            return launch_warp_rows<GATED, 4>(value, gate, weight, rows, dim, eps, q_max, out, q, act_scales, q_sums, stream);
        if (dim <= 1024)
            return launch_warp_rows<GATED, 8>(value, gate, weight, rows, dim, eps, q_max, out, q, act_scales, q_sums, stream);
        if (dim <= 1536)
            return launch_warp_rows<GATED, 12>(value, gate, weight, rows, dim, eps, q_max, out, q, act_scales, q_sums, stream);
        return launch_warp_rows<GATED, 16>(value, gate, weight, rows, dim, eps, q_max, out, q, act_scales, q_sums, stream);
    }
    const size_t smem = static_cast<size_t>(dim) * sizeof(float);
    if (smem > 48 * 1024) {
        // the opt-in is a per-device attribute of the kernel: remember it per device (one flag set per instantiation)
        static bool configured[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            cudaError_t e = cudaFuncSetAttribute(row_norm_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kRowNormMaxDim * sizeof(float)));
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    // Few rows (decode): one CTA per row, as many threads as the row has 4-element groups, up to 1024, so the
    // row is one load per thread.  Many rows: 256 threads, several CTAs per SM, a grid-stride over rows.
    int threads = 256;
    if (rows <= 296) {
        threads = ((dim + 3) / 4 + 31) / 32 * 32;
        threads = threads < 128 ? 128 : (threads > kNormMaxThreads ? kNormMaxThreads : threads);
    }
    int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
    const int by_threads = 2048 / threads;
    per_sm = per_sm > by_threads ? by_threads : per_sm;
    per_sm = per_sm < 1 ? 1 : per_sm;
    const int grid = rows < 148 * per_sm ? rows : 148 * per_sm;
    row_norm_kernel<GATED><<<grid, threads, smem, stream>>>(value, gate, weight, rows, dim, eps, q_max, vec, out, q,
                                                           act_scales, q_sums);
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

namespace {
// max(x,0)^2 in place (Tensor::squared_relu); the product is rounded on its own like the host form.
__global__ void __launch_bounds__(256) squared_relu_kernel(float* __restrict__ x, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = fmaxf(x[i], 0.0f);
        x[i] = __fmul_rn(v, v);
    }
}
}  // namespace

namespace {
// gathered [parts][rows][cols] -> out [rows][parts*cols]; 128-bit accesses when cols % 4 == 0.
template <typename V>
__global__ void __launch_bounds__(256) retile_columns_kernel(const V* __restrict__ src, int parts, int rows, int cols,
                                                             V* __restrict__ dst) {
    const int64_t n = static_cast<int64_t>(parts) * rows * cols;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < n; o += stride) {
        const int c = static_cast<int>(o % cols);
        const int64_t rp = o / cols;
        const int p = static_cast<int>(rp % parts);
        const int64_t r = rp / parts;
        dst[o] = src[(static_cast<int64_t>(p) * rows + r) * cols + c];
    }
}
}  // namespace

cudaError_t launch_retile_columns(const float* gathered, int parts, int rows, int cols, float* out, cudaStream_t stream) {
    if (parts < 1 || rows < 1 || cols < 1) return cudaErrorInvalidValue;
    const bool vec = cols % 4 == 0 && (reinterpret_cast<uintptr_t>(gathered) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    const int64_t n = static_cast<int64_t>(parts) * rows * (vec ? cols / 4 : cols);
    const int64_t want = (n + 255) / 256;
    const int grid = static_cast<int>(want < 148 * 16 ? want : 148 * 16);
    if (vec)
        retile_columns_kernel<float4><<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(gathered), parts, rows, cols / 4,
                                                               reinterpret_cast<float4*>(out));
    else
        retile_columns_kernel<float><<<grid, 256, 0, stream>>>(gathered, parts, rows, cols, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_squared_relu(float* x, int64_t n, cudaStream_t stream) {
    if (n < 1) return cudaErrorInvalidValue;
    const int64_t want = (n + 255) / 256;
    const int grid = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
    squared_relu_kernel<<<grid, 256, 0, stream>>>(x, n);
    note_launch();
    return cudaGetLastError();
}

}  // namespace tbl
