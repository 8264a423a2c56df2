// Per-row absmax int8 activation quantiser (optionally preceded by the input RMSNorm), and the
// 2-bit -> int8 weight expansion that feeds the tensor-core GEMM.  Both are pure HBM/L2
// streaming kernels.
#include <type_traits>

#include "common.cuh"
#include "kernels.cuh"

namespace tbl {

__device__ int g_device_status = 0;

int* device_status_ptr() {
    static int* cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        cached[dev] = static_cast<int*>(p);
    }
    return cached[dev];
}

int read_and_clear_device_status(int* out) {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (status != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    *out = status;
    return 0;
}

namespace {

constexpr int kQuantThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide reductions over kQuantThreads threads; every thread gets the result.
__device__ float block_max(float v, float* scratch) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch[0];
#pragma unroll
    for (int w = 1; w < kQuantThreads / 32; ++w) r = fmaxf(r, scratch[w]);
    __syncthreads();
    return r;
}
__device__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kQuantThreads / 32; ++w) r += scratch[w];
    __syncthreads();
    return r;
}

// Reference-order RMS factor: one thread per row walks the row left to right with a
// separately rounded multiply and add per element, exactly like the CPU loop it mirrors
// (sum_sq += v*v; inv = 1/sqrt(sum_sq/K + eps)).  Latency-bound by design; rows run in parallel.
__global__ void rms_reference_order_kernel(const float* __restrict__ x,
                                           const int32_t* __restrict__ row_index, int M, int K,
                                           float eps, float* __restrict__ inv_norm,
                                           const int32_t* __restrict__ active_rows) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= M) return;
    if (active_rows && row >= *active_rows) return;
    const int src = row_index ? row_index[row] : row;
    const float* p = x + static_cast<size_t>(src) * K;
    float sum_sq = 0.0f;
    for (int j = 0; j < K; ++j) {
        const float v = p[j];
        sum_sq = __fadd_rn(sum_sq, __fmul_rn(v, v));
    }
    const float mean = __fdiv_rn(sum_sq, static_cast<float>(K > 1 ? K : 1));
    inv_norm[row] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

// One CTA per output row.  VEC16: K % 16 == 0 and 16-byte aligned rows -> 128-bit loads and
// stores, optional second output in the strip GEMV's interleaved order (qp).
template <bool VEC16>
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ row_index, int K,
                     float q_max, int rms_mode, bool tie_away, const float* __restrict__ inv_norm_in,
                     int8_t* __restrict__ q, int8_t* __restrict__ qp, float* __restrict__ act_scales,
                     int32_t* __restrict__ q_sums, const int32_t* __restrict__ active_rows,
                     int qp_rows, QuantSegments seg) {
    __shared__ float scratch[kQuantThreads / 32];
    __shared__ int sum_scratch[kQuantThreads / 32];
    const int row = blockIdx.x;
    if (active_rows && row >= *active_rows) return;
    const int src = row_index ? row_index[row] : row;
    const float* xr = x + static_cast<size_t>(src) * K;
    // position of this row inside its problem (for the interleaved copy)
    int prow = row, prows = qp_rows;
    size_t pbase = 0;
    if (VEC16 && qp && seg.offsets) {
        for (int e = 0; e < seg.segs; ++e) {
            const int o = seg.offsets[e], c = seg.counts[e];
            if (row >= o && row < o + c) { prow = row - o; prows = c; pbase = static_cast<size_t>(o) * K; break; }
        }
    }

    float inv = 1.0f;
    if (rms_mode == TBL_RMS_REFERENCE_ORDER) {
        inv = inv_norm_in[row];
    } else if (rms_mode == TBL_RMS_FAST) {
        float ss = 0.0f;
        if (VEC16) {
            for (int j = threadIdx.x * 4; j < K; j += kQuantThreads * 4) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(xr + j));
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        } else {
            for (int j = threadIdx.x; j < K; j += kQuantThreads) ss += xr[j] * xr[j];
        }
        ss = block_sum(ss, scratch);
        inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), 1e-6f)));
    }
    const bool normed = rms_mode != TBL_RMS_NONE;

    float mx = 0.0f;
    if (VEC16) {
        for (int j = threadIdx.x * 4; j < K; j += kQuantThreads * 4) {
            float4 v = __ldg(reinterpret_cast<const float4*>(xr + j));
            if (normed) {
                v.x = __fmul_rn(v.x, inv); v.y = __fmul_rn(v.y, inv);
                v.z = __fmul_rn(v.z, inv); v.w = __fmul_rn(v.w, inv);
            }
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int j = threadIdx.x; j < K; j += kQuantThreads) {
            float v = xr[j];
            if (normed) v = __fmul_rn(v, inv);
            mx = fmaxf(mx, fabsf(v));
        }
    }
    mx = block_max(mx, scratch);
    const float denom = __fadd_rn(mx, 1e-8f);
    const float scale = __fdiv_rn(q_max, denom);
    if (threadIdx.x == 0) act_scales[row] = __fdiv_rn(denom, q_max);

    int local_sum = 0;
    if (VEC16) {
        // each thread turns 16 consecutive elements into one 128-bit store
        for (int j = threadIdx.x * 16; j < K; j += kQuantThreads * 16) {
            uint32_t words[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float4 v = __ldg(reinterpret_cast<const float4*>(xr + j + 4 * e));
                if (normed) {
                    v.x = __fmul_rn(v.x, inv); v.y = __fmul_rn(v.y, inv);
                    v.z = __fmul_rn(v.z, inv); v.w = __fmul_rn(v.w, inv);
                }
                const int a = round_code(__fmul_rn(v.x, scale), tie_away);
                const int b = round_code(__fmul_rn(v.y, scale), tie_away);
                const int c = round_code(__fmul_rn(v.z, scale), tie_away);
                const int d = round_code(__fmul_rn(v.w, scale), tie_away);
                words[e] = (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | (static_cast<uint32_t>(d & 0xff) << 24);
                local_sum = dp4a_ss(static_cast<int>(words[e]), 0x01010101, local_sum);   // the sum of the stored codes
            }
            const uint4 natural = make_uint4(words[0], words[1], words[2], words[3]);
            if (q) *reinterpret_cast<uint4*>(q + static_cast<size_t>(row) * K + j) = natural;
            if (qp) {
                *reinterpret_cast<uint4*>(qp + pbase + qp_offset(prow, prows, K, j)) =
                    transpose4x4_bytes(natural);
            }
        }
    } else {
        // general K: the reference's AVX2 quantiser rounds the 8-wide body half-to-even and the
        // K % 8 tail with std::round
        const int body = tie_away ? 0 : (K / 8) * 8;
        for (int j = threadIdx.x; j < K; j += kQuantThreads) {
            float v = xr[j];
            if (normed) v = __fmul_rn(v, inv);
            const float r = round_tie(__fmul_rn(v, scale), j >= body);
            const int a = static_cast<int>(fminf(127.0f, fmaxf(-127.0f, r)));
            local_sum += a;
            if (q) q[static_cast<size_t>(row) * K + j] = static_cast<int8_t>(a);
        }
    }
    if (q_sums) {
        local_sum = warp_sum_i(local_sum);
        if ((threadIdx.x & 31) == 0) sum_scratch[threadIdx.x >> 5] = local_sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            int s = 0;
            for (int w = 0; w < kQuantThreads / 32; ++w) s += sum_scratch[w];
            q_sums[row] = s;
        }
    }
}

// Plane-major codes for the widening tensor-core kernel (gemm_widen.cu): inside each block of 512 elements of a
// row (leading dimension plane_ld, a multiple of 512), byte 4g + e of plane p (128 bytes per plane) is element
// 16g + 4e + p.  `t` is the 4x4 byte transpose of the 16-element group at element j: its four words go to the four planes.
__device__ __forceinline__ void store_planes(int8_t* planes, int row, int plane_ld, int j, uint4 t) {
    const int gg = j >> 4;
    uint32_t* dst = reinterpret_cast<uint32_t*>(planes + static_cast<size_t>(row) * plane_ld + (gg >> 5) * 512) + (gg & 31);
    dst[0] = t.x;
    dst[32] = t.y;
    dst[64] = t.z;
    dst[96] = t.w;
}

// Register-resident variant for K % 16 == 0 and K <= 16 * G * blockDim (G <= 2, so K <= 32768): every thread keeps its
// G groups of 16 elements in registers, so the row is read from memory exactly once and the kernel
// is a single load -> reduce -> quantise -> store chain (what matters at decode batch sizes, where
// one row per CTA is pure latency).
template <int G>
__global__ void __launch_bounds__(1024)
quantize_rows_reg_kernel(const float* __restrict__ x, const int32_t* __restrict__ row_index, int K,
                         float q_max, int rms_mode, bool tie_away, const float* __restrict__ inv_norm_in,
                         int8_t* __restrict__ q, int8_t* __restrict__ qp, float* __restrict__ act_scales,
                         int32_t* __restrict__ q_sums, const int32_t* __restrict__ active_rows,
                         int qp_rows, QuantSegments seg, int plane_ld) {
    __shared__ float scratch[32];
    __shared__ int sum_scratch[32];
    // a dependent launch (the widening GEMM) may start its prologue and its weight stream now; it waits for this
    // kernel's completion before it reads the codes
    pdl_launch_dependents();
    const int row = blockIdx.x;
    if (active_rows && row >= *active_rows) return;
    const int src = row_index ? row_index[row] : row;
    const float* xr = x + static_cast<size_t>(src) * K;
    const int nwarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int prow = row, prows = qp_rows;
    size_t pbase = 0;
    if (qp && seg.offsets) {
        for (int e = 0; e < seg.segs; ++e) {
            const int o = seg.offsets[e], c = seg.counts[e];
            if (row >= o && row < o + c) { prow = row - o; prows = c; pbase = static_cast<size_t>(o) * K; break; }
        }
    }

    float4 v[G][4];
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int j = (threadIdx.x + i * blockDim.x) * 16;
#pragma unroll
        for (int e = 0; e < 4; ++e)
            v[i][e] = j < K ? __ldg(reinterpret_cast<const float4*>(xr + j + 4 * e)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }

    auto reduce = [&](float val, bool is_max) -> float {
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, val, o);
            val = is_max ? fmaxf(val, other) : val + other;
        }
        __syncthreads();
        if (lane == 0) scratch[warp] = val;
        __syncthreads();
        float r = scratch[0];
        for (int w = 1; w < nwarps; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
        return r;
    };

    float inv = 1.0f;
    if (rms_mode == TBL_RMS_REFERENCE_ORDER) {
        inv = inv_norm_in[row];
    } else if (rms_mode == TBL_RMS_FAST) {
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < G; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                ss += v[i][e].x * v[i][e].x + v[i][e].y * v[i][e].y + v[i][e].z * v[i][e].z + v[i][e].w * v[i][e].w;
        ss = reduce(ss, false);
        inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), 1e-6f)));
    }
    float mx = 0.0f;
#pragma unroll
    for (int i = 0; i < G; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (rms_mode != TBL_RMS_NONE) {
                v[i][e].x = __fmul_rn(v[i][e].x, inv); v[i][e].y = __fmul_rn(v[i][e].y, inv);
                v[i][e].z = __fmul_rn(v[i][e].z, inv); v[i][e].w = __fmul_rn(v[i][e].w, inv);
            }
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[i][e].x), fabsf(v[i][e].y)), fmaxf(fabsf(v[i][e].z), fabsf(v[i][e].w))));
        }
    mx = reduce(mx, true);
    const float denom = __fadd_rn(mx, 1e-8f);
    const float scale = __fdiv_rn(q_max, denom);
    if (threadIdx.x == 0) act_scales[row] = __fdiv_rn(denom, q_max);

    int local_sum = 0;
    auto round_and_store = [&](auto away) {
#pragma unroll
    for (int i = 0; i < G; ++i) {
        const int j = (threadIdx.x + i * blockDim.x) * 16;
        if (j < K) {
            uint32_t words[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int a = round_code(__fmul_rn(v[i][e].x, scale), decltype(away)::value);
                const int b = round_code(__fmul_rn(v[i][e].y, scale), decltype(away)::value);
                const int c = round_code(__fmul_rn(v[i][e].z, scale), decltype(away)::value);
                const int d = round_code(__fmul_rn(v[i][e].w, scale), decltype(away)::value);
                words[e] = (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | (static_cast<uint32_t>(d & 0xff) << 24);
                local_sum = dp4a_ss(static_cast<int>(words[e]), 0x01010101, local_sum);   // the sum of the stored codes
            }
            const uint4 natural = make_uint4(words[0], words[1], words[2], words[3]);
            if (q) *reinterpret_cast<uint4*>(q + static_cast<size_t>(row) * K + j) = natural;
            if (qp && !plane_ld) *reinterpret_cast<uint4*>(qp + pbase + qp_offset(prow, prows, K, j)) = transpose4x4_bytes(natural);
            if (qp && plane_ld) store_planes(qp, row, plane_ld, j, transpose4x4_bytes(natural));
        } else if (qp && j < plane_ld) {
            store_planes(qp, row, plane_ld, j, make_uint4(0u, 0u, 0u, 0u));     // the padding up to the row's leading dimension
        }
    }
    };
    // one uniform branch: the half-away path converts on the XU pipe
    if (tie_away) round_and_store(std::true_type{}); else round_and_store(std::false_type{});
    if (q_sums) {
        local_sum = warp_sum_i(local_sum);
        if (lane == 0) sum_scratch[warp] = local_sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < nwarps; ++w) t += sum_scratch[w];
            q_sums[row] = t;
        }
    }
}

// Prefill-sized quantiser (many rows, natural-order codes only): persistent CTAs, one producer warp that
// streams whole rows into a shared-memory ring with 1-D bulk (TMA) copies, sixteen consumer warps.  The
// one-CTA-per-row kernels above keep a row in registers, which caps the bytes in flight per SM at what the
// register file holds (measured 3.75 TB/s at 8192 x 8192); here the ring holds up to 208 KB per SM.
// The consumer warps form `groups` independent teams (16384 / K of them, so a thread always holds up to
// eight float4): team g takes the CTA's rows g, g + groups, ... so that several per-row chains
// (wait -> load -> reduce -> barrier -> round -> store, ~1 us each) run side by side.
// A thread takes float4 number lane + 32*e of its warp's span (conflict-free shared loads, coalesced
// 32-bit stores of four codes) and hands the stage back as soon as the row is in registers.
constexpr int kStreamConsumers = 16;
constexpr int kStreamThreads = (kStreamConsumers + 1) * 32;
constexpr int kStreamMaxStages = 16;
constexpr int kStreamVec = 8;      // float4 per consumer thread per row

__global__ void __launch_bounds__(kStreamThreads, 1)
quantize_rows_stream_kernel(const float* __restrict__ x, const int32_t* __restrict__ row_index, int M, int K,
                            float q_max, int rms_mode, bool tie_away, const float* __restrict__ inv_norm_in,
                            int8_t* __restrict__ q, float* __restrict__ act_scales, int32_t* __restrict__ q_sums,
                            const int32_t* __restrict__ active_rows, int stages, int groups, int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kStreamMaxStages;
    uint32_t* s_amax = reinterpret_cast<uint32_t*>(smem + 256);   // [8 teams][4] row absmax bit patterns
    int* s_sum = reinterpret_cast<int*>(smem + 384);              // [8 teams][4] row code sums
    uint8_t* ring = smem + 512;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = static_cast<uint32_t>(K) * 4u;
    const int rows = active_rows ? min(M, __ldg(active_rows)) : M;
    const int wpg = kStreamConsumers / groups;       // warps per team

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], wpg); }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (threadIdx.x < 32) { s_amax[threadIdx.x] = 0u; s_sum[threadIdx.x] = 0; }
    __syncthreads();

    if (warp == kStreamConsumers) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int it = 0;
            for (int row = blockIdx.x; row < rows; row += gridDim.x, ++it) {
                const int st = it % stages;
                if (it >= stages && !mbar_wait_bounded(&empty[st], ((it / stages) - 1) & 1, status)) break;
                const int src = row_index ? __ldg(row_index + row) : row;
                mbar_arrive_expect_tx(&full[st], row_bytes);
                bulk_g2s(ring + static_cast<size_t>(st) * row_bytes, x + static_cast<size_t>(src) * K, row_bytes, &full[st]);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int team = warp / wpg, tw = warp % wpg;
    const int team_threads = wpg * 32;
    const bool leader = tw == 0 && lane == 0;
    uint32_t* amax = s_amax + team * 4;
    int* sum = s_sum + team * 4;
    const int nvec = K >> 2;                       // float4 per row
    int prev_row = -1, n = 0;                      // n: rows this team has done
    bool alive = true;
    for (int it = team; alive; it += groups, ++n) {
        const int row = blockIdx.x + it * gridDim.x;
        if (row >= rows) break;
        const int st = it % stages, slot = n & 3;
        alive = mbar_wait_bounded(&full[st], (it / stages) & 1, status);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) break;
        const float4* src = reinterpret_cast<const float4*>(ring + static_cast<size_t>(st) * row_bytes);
        float4 v[kStreamVec];
        float mx = 0.0f;
        float inv = 1.0f;
        if (rms_mode == TBL_RMS_REFERENCE_ORDER) inv = __ldg(inv_norm_in + row);
#pragma unroll
        for (int e = 0; e < kStreamVec; ++e) {
            const int i = tw * 32 * kStreamVec + e * 32 + lane;     // warp tw of the team owns 256 float4
            v[e] = i < nvec ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (rms_mode != TBL_RMS_NONE) {
                v[e].x = __fmul_rn(v[e].x, inv); v[e].y = __fmul_rn(v[e].y, inv);
                v[e].z = __fmul_rn(v[e].z, inv); v[e].w = __fmul_rn(v[e].w, inv);
            }
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[e].x), fabsf(v[e].y)), fmaxf(fabsf(v[e].z), fabsf(v[e].w))));
        }
        // the row is in registers: hand the stage back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
        const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(mx));
        if (lane == 0 && wmax != 0u) atomicMax(&amax[slot], wmax);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(team_threads) : "memory");
        // behind this barrier every thread of the team has finished the previous row: publish its sum and
        // recycle its slot (next used three rows from now, behind two more barriers)
        if (leader && prev_row >= 0) {
            const int pslot = (n - 1) & 3;
            if (q_sums) q_sums[prev_row] = sum[pslot];
            sum[pslot] = 0;
            amax[pslot] = 0u;
        }
        const float denom = __fadd_rn(__uint_as_float(amax[slot]), 1e-8f);
        const float scale = __fdiv_rn(q_max, denom);
        if (leader) act_scales[row] = __fdiv_rn(denom, q_max);
        uint32_t* dst = reinterpret_cast<uint32_t*>(q + static_cast<size_t>(row) * K);
        int local_sum = 0;
        // one uniform branch per row: the half-away path converts on the XU pipe, which the compiler would
        // otherwise execute for every element and select away
        auto round_and_store = [&](auto away) {
#pragma unroll
            for (int e = 0; e < kStreamVec; ++e) {
                const int i = tw * 32 * kStreamVec + e * 32 + lane;
                if (i < nvec) {
                    const int a = round_code(__fmul_rn(v[e].x, scale), decltype(away)::value);
                    const int b = round_code(__fmul_rn(v[e].y, scale), decltype(away)::value);
                    const int c = round_code(__fmul_rn(v[e].z, scale), decltype(away)::value);
                    const int d = round_code(__fmul_rn(v[e].w, scale), decltype(away)::value);
                    const uint32_t w = (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | (static_cast<uint32_t>(d & 0xff) << 24);
                    dst[i] = w;
                    local_sum = dp4a_ss(static_cast<int>(w), 0x01010101, local_sum);
                }
            }
        };
        if (tie_away) round_and_store(std::true_type{}); else round_and_store(std::false_type{});
        if (q_sums) {
            local_sum = __reduce_add_sync(0xffffffffu, local_sum);
            if (lane == 0 && local_sum != 0) atomicAdd(&sum[slot], local_sum);
        }
        prev_row = row;
    }
    // the team's last row
    if (q_sums) {
        asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(team_threads) : "memory");
        if (leader && prev_row >= 0) q_sums[prev_row] = sum[(n - 1) & 3];
    }
}

// Each thread expands one 128-bit load (64 weights of one row) into four 128-bit stores.
__global__ void expand_i8_kernel(const uint4* __restrict__ words, int64_t n_vec, int8_t* __restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        const uint4 v = __ldg(words + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint4* dst = reinterpret_cast<uint4*>(out + i * 64);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // weights 4e..4e+3 of this word: 2-bit codes -> bytes, minus 1 per byte
                const uint32_t b = (w[x] >> (8 * e)) & 0xffu;
                const uint32_t spread = (b & 0x03u) | ((b & 0x0cu) << 6) | ((b & 0x30u) << 12) | ((b & 0xc0u) << 18);
                o[e] = __vsub4(spread, 0x01010101u);
            }
            dst[x] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// scalar tail for N*K not a multiple of 64
__global__ void expand_i8_tail_kernel(const uint32_t* __restrict__ words, int64_t first, int64_t total,
                                      int8_t* __restrict__ out) {
    const int64_t i = first + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    out[i] = static_cast<int8_t>(static_cast<int>((words[i >> 4] >> ((i & 15) << 1)) & 3u) - 1);
}

}  // namespace

cudaError_t launch_quantize_rows(const float* x, const int32_t* row_index, int M, int K, int bits,
                                 int rms_mode, int tie_mode, int8_t* q, int8_t* qp, float* act_scales,
                                 int32_t* q_sums, float* inv_norm_scratch, const int32_t* active_rows,
                                 QuantSegments segments, cudaStream_t stream, int plane_ld) {
    // plane_ld != 0: qp receives the plane-major codes (leading dimension plane_ld) instead of the interleaved copy;
    // only the register kernel writes them
    if (plane_ld && (!qp || segments.offsets || K % 16 || K > 32768 || plane_ld % 512 || plane_ld < K || plane_ld - K >= 512 ||
                     (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(qp) & 15) ||
                     (q && (reinterpret_cast<uintptr_t>(q) & 15))))
        return cudaErrorInvalidValue;
    if (rms_mode == TBL_RMS_REFERENCE_ORDER) {
        rms_reference_order_kernel<<<(M + 63) / 64, 64, 0, stream>>>(x, row_index, M, K, 1e-6f,
                                                                     inv_norm_scratch, active_rows);
        note_launch();
    }
    const bool vec = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     (!q || (reinterpret_cast<uintptr_t>(q) & 15) == 0) &&
                     (!qp || (reinterpret_cast<uintptr_t>(qp) & 15) == 0);
    const float q_max = qmax_for_bits(bits);
    const bool away = tie_mode == TBL_TIE_AWAY;
    // prefill-sized calls (natural-order codes only): the streaming kernel
    if (vec && !qp && !segments.offsets && M >= 256 && K >= 2048 && K <= 16384 && rms_mode != TBL_RMS_FAST) {
        int* status = device_status_ptr();
        if (!status) return cudaErrorUnknown;
        const size_t row_bytes = static_cast<size_t>(K) * 4;
        int stages = static_cast<int>((208 * 1024) / row_bytes);
        if (stages > kStreamMaxStages) stages = kStreamMaxStages;
        int teams = 1;                                  // largest power of two with K <= 16384 / teams
        while (teams < 8 && K * (teams * 2) <= 16384) teams *= 2;
        const size_t smem = 512 + stages * row_bytes;
        const int grid = M < 148 ? M : 148;
        static bool configured[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            cudaError_t e = cudaFuncSetAttribute(quantize_rows_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
        quantize_rows_stream_kernel<<<grid, kStreamThreads, smem, stream>>>(x, row_index, M, K, q_max, rms_mode, away,
                                                                           inv_norm_scratch, q, act_scales, q_sums,
                                                                           active_rows, stages, teams, status);
        note_launch();
        return cudaGetLastError();
    }
    if (vec && K <= 32768) {
        const int groups = K / 16;
        int threads = ((groups + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        const int g = (groups + threads - 1) / threads;
#define TBL_LAUNCH_REG(G)                                                                                  \
    quantize_rows_reg_kernel<G><<<M, threads, 0, stream>>>(x, row_index, K, q_max, rms_mode, away,         \
                                                           inv_norm_scratch, q, qp, act_scales, q_sums,    \
                                                           active_rows, M, segments, plane_ld)
        if (g <= 1) TBL_LAUNCH_REG(1);
        else TBL_LAUNCH_REG(2);
#undef TBL_LAUNCH_REG
    } else if (vec) {
        quantize_rows_kernel<true><<<M, kQuantThreads, 0, stream>>>(
            x, row_index, K, q_max, rms_mode, away, inv_norm_scratch, q, qp,
            act_scales, q_sums, active_rows, M, segments);
    } else {
        quantize_rows_kernel<false><<<M, kQuantThreads, 0, stream>>>(
            x, row_index, K, q_max, rms_mode, away, inv_norm_scratch, q, nullptr,
            act_scales, q_sums, active_rows, M, segments);
    }
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_expand_i8(const uint32_t* words, int N, int K, int8_t* out, cudaStream_t stream) {
    const int64_t total = static_cast<int64_t>(N) * K;
    const int64_t n_vec = total / 64;
    if (n_vec > 0) {
        const int threads = 256;
        int64_t blocks = (n_vec + threads - 1) / threads;
        if (blocks > 148 * 16) blocks = 148 * 16;
        expand_i8_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(
            reinterpret_cast<const uint4*>(words), n_vec, out);
        note_launch();
    }
    const int64_t done = n_vec * 64;
    if (done < total) {
        expand_i8_tail_kernel<<<1, 64, 0, stream>>>(words, done, total, out);
        note_launch();
    }
    return cudaGetLastError();
}

}  // namespace tbl
