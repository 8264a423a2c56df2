// Decode GEMV for 1 <= M <= 4 rows: HBM-bound stream of the canonical 2-bit words.
//
// Each warp owns a ring of shared-memory stages filled by 1-D bulk (TMA) copies; a stage holds a
// run of whole weight rows, which are contiguous in the canonical layout.  A 128-bit shared load
// hands a lane 64 weights of one row; the 2-bit codes are widened in registers with one AND per
// dp4a (mask 0x03030303 << 2j keeps weights {j,4+j,8+j,12+j} of each word as unsigned bytes scaled
// by 4^j; the four partial sums are recombined exactly with shifts) and the constant "-1" of the
// code is removed by subtracting the row's sum of activations.  The activations a lane needs are
// the same for every row it visits, so they live in registers (CPL > 0) or, for long rows, in
// shared memory (CPL == 0).  The per-token absmax quantiser runs in the prologue of the same
// kernel while the first weight stages are already in flight.
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

constexpr int kMaxWarps = 8;
constexpr int kStageTarget = 4096;     // bytes of packed weights per stage
constexpr int kStageMax = 8192;        // a stage must hold at least one row: K <= 32768
constexpr int kSmemBudget = 200 * 1024;
constexpr int kNumSm = 148;

struct Plan {
    int C;        // 16-byte chunks per row (K/64)
    int G;        // lanes cooperating on one row (power of two)
    int cpl;      // chunks per lane = ceil(C/G)
    int rsw;      // rows per stage
    int stage_bytes;
    int stages;
    int warps;
    int units;    // number of stages' worth of rows in the matrix
    int grid;
    size_t smem;
};

struct KParams {
    GemvSmallArgs a;
    Plan p;
    int* status;
};

__device__ __forceinline__ float blk_max(float v, float* scratch, int warps) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch[0];
    for (int w = 1; w < warps; ++w) r = fmaxf(r, scratch[w]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float blk_sum(float v, float* scratch, int warps) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
    for (int w = 0; w < warps; ++w) r += scratch[w];
    __syncthreads();
    return r;
}

// Shared-memory activation layout: act[m][x][c] is the 16-byte transposed group of elements
// 64c + 16x .. 64c + 16x + 15 of row m, so lanes with consecutive c read consecutive 16 bytes.
__device__ __forceinline__ int act_offset(int m, int x, int c, int K, int C) {
    return m * K + (x * C + c) * 16;
}

template <int M, int CPL>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) gemv_stream_kernel(const KParams kp) {
    extern __shared__ __align__(128) uint8_t smem[];
    const GemvSmallArgs& a = kp.a;
    const Plan& p = kp.p;
    const int K = a.K, N = a.N, C = p.C, G = p.G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = p.warps;

    // carve shared memory: rings | activations | barriers | small arrays
    uint8_t* ring = smem + static_cast<size_t>(warp) * p.stages * p.stage_bytes;
    uint8_t* act = smem + static_cast<size_t>(warps) * p.stages * p.stage_bytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(act + ((static_cast<size_t>(M) * K + 127) & ~size_t(127)));
    uint64_t* my_bars = bars + warp * p.stages;
    float* red = reinterpret_cast<float*>(bars + kMaxWarps * 4);
    float* s_scale = red + kMaxWarps;            // [M] act_scale
    int* s_qsum = reinterpret_cast<int*>(s_scale + 4);  // [M]

    const int gw = blockIdx.x * warps + warp;
    const int wstride = gridDim.x * warps;
    const int row_bytes = K >> 2;
    const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(a.words);

    // ---- the weight rings start as early as possible, but behind the first row's activation loads: issued
    // the other way round, those loads queue behind a ring's worth of weight copies in the memory pipeline
    if (lane == 0) {
        for (int s = 0; s < p.stages; ++s) mbar_init(&my_bars[s], 1);
        fence_mbar_init();
        fence_proxy_async();
    }
    bool ring_started = false;
    auto start_ring = [&]() {
        if (ring_started) return;
        ring_started = true;
        if (lane != 0) return;
        for (int s = 0; s < p.stages; ++s) {
            const int u = gw + s * wstride;
            if (u < p.units) {
                const int n0 = u * p.rsw;
                const int rows_u = min(p.rsw, N - n0);
                const uint32_t bytes = static_cast<uint32_t>(rows_u) * row_bytes;
                mbar_arrive_expect_tx(&my_bars[s], bytes);
                bulk_g2s(ring + s * p.stage_bytes, wbytes + static_cast<size_t>(n0) * row_bytes, bytes,
                         &my_bars[s]);
            }
        }
    };
    if (threadIdx.x < M) s_qsum[threadIdx.x] = 0;
    __syncthreads();

    // ---- prologue: quantise (fused) or load the int8 codes, into the transposed layout ------
    const int nthreads = warps * 32;
#pragma unroll
    for (int m = 0; m < M; ++m) {
        int local_sum = 0;
        if (a.x) {
            const float* xr = a.x + static_cast<size_t>(m) * K;
            float inv = 1.0f;
            if (a.rms_mode == TBL_RMS_FAST) {
                start_ring();
                float ss = 0.0f;
                for (int j = threadIdx.x * 4; j < K; j += nthreads * 4) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(xr + j));
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                ss = blk_sum(ss, red, warps);
                inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, static_cast<float>(K)), 1e-6f)));
            }
            const bool normed = a.rms_mode != TBL_RMS_NONE;
            // Rows of up to 16 * 4 * nthreads elements stay in registers between the absmax pass and the
            // rounding pass (one trip through L2 instead of two); longer rows are read again.
            constexpr int kCached = 4;                         // 16-element groups per thread
            const bool cached = K <= 16 * kCached * nthreads;
            float4 xc[kCached][4];
            float mx = 0.0f;
            if (!cached || a.rms_mode == TBL_RMS_FAST) start_ring();
            if (cached) {
#pragma unroll
                for (int i = 0; i < kCached; ++i) {
                    const int j = (threadIdx.x + i * nthreads) * 16;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float4 v = j < K ? __ldg(reinterpret_cast<const float4*>(xr + j + 4 * e)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        if (normed) {
                            v.x = __fmul_rn(v.x, inv); v.y = __fmul_rn(v.y, inv);
                            v.z = __fmul_rn(v.z, inv); v.w = __fmul_rn(v.w, inv);
                        }
                        xc[i][e] = v;
                        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                    }
                }
            } else {
                for (int j = threadIdx.x * 4; j < K; j += nthreads * 4) {
                    float4 v = __ldg(reinterpret_cast<const float4*>(xr + j));
                    if (normed) {
                        v.x = __fmul_rn(v.x, inv); v.y = __fmul_rn(v.y, inv);
                        v.z = __fmul_rn(v.z, inv); v.w = __fmul_rn(v.w, inv);
                    }
                    mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            }
            start_ring();        // this row's loads are in flight (the block reduction below waits for them)
            mx = blk_max(mx, red, warps);
            const float denom = __fadd_rn(mx, 1e-8f);
            const float scale = __fdiv_rn(a.q_max, denom);
            if (threadIdx.x == 0) {
                const float as = __fdiv_rn(denom, a.q_max);
                s_scale[m] = as;
                if (a.scales_out && blockIdx.x == 0) a.scales_out[m] = as;
            }
            // codes: ties-to-even on the FMA pipe (round_code), their sum from the stored bytes
            auto emit_group = [&](int j, const float4 (&g)[4]) {
                uint32_t wds[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int q0 = round_code(__fmul_rn(g[e].x, scale), false);
                    const int q1 = round_code(__fmul_rn(g[e].y, scale), false);
                    const int q2 = round_code(__fmul_rn(g[e].z, scale), false);
                    const int q3 = round_code(__fmul_rn(g[e].w, scale), false);
                    wds[e] = (q0 & 0xff) | ((q1 & 0xff) << 8) | ((q2 & 0xff) << 16) |
                             (static_cast<uint32_t>(q3 & 0xff) << 24);
                    local_sum = dp4a_ss(static_cast<int>(wds[e]), 0x01010101, local_sum);
                }
                const uint4 natural = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                if (a.q_out && blockIdx.x == 0)
                    *reinterpret_cast<uint4*>(a.q_out + static_cast<size_t>(m) * K + j) = natural;
                *reinterpret_cast<uint4*>(act + act_offset(m, (j >> 4) & 3, j >> 6, K, C)) =
                    transpose4x4_bytes(natural);
            };
            if (cached) {
#pragma unroll
                for (int i = 0; i < kCached; ++i) {
                    const int j = (threadIdx.x + i * nthreads) * 16;
                    if (j < K) emit_group(j, xc[i]);
                }
            } else {
                for (int j = threadIdx.x * 16; j < K; j += nthreads * 16) {
                    float4 g[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float4 v = __ldg(reinterpret_cast<const float4*>(xr + j + 4 * e));
                        if (normed) {
                            v.x = __fmul_rn(v.x, inv); v.y = __fmul_rn(v.y, inv);
                            v.z = __fmul_rn(v.z, inv); v.w = __fmul_rn(v.w, inv);
                        }
                        g[e] = v;
                    }
                    emit_group(j, g);
                }
            }
        } else {
            start_ring();
            const int8_t* qr = a.q + static_cast<size_t>(m) * K;
            if (threadIdx.x == 0) s_scale[m] = a.act_scales[m];
            for (int j = threadIdx.x * 16; j < K; j += nthreads * 16) {
                const uint4 natural = __ldg(reinterpret_cast<const uint4*>(qr + j));
                local_sum = dp4a_ss(static_cast<int>(natural.x), 0x01010101, local_sum);
                local_sum = dp4a_ss(static_cast<int>(natural.y), 0x01010101, local_sum);
                local_sum = dp4a_ss(static_cast<int>(natural.z), 0x01010101, local_sum);
                local_sum = dp4a_ss(static_cast<int>(natural.w), 0x01010101, local_sum);
                *reinterpret_cast<uint4*>(act + act_offset(m, (j >> 4) & 3, j >> 6, K, C)) =
                    transpose4x4_bytes(natural);
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) local_sum += __shfl_xor_sync(0xffffffffu, local_sum, o);
        if (lane == 0) atomicAdd(&s_qsum[m], local_sum);
    }
    __syncthreads();

    float comb[M];
    int qsum[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
        comb[m] = __fmul_rn(s_scale[m], a.weight_scale);
        qsum[m] = s_qsum[m];
    }

    const int lg = lane & (G - 1);   // position inside the lane group
    const int rl = lane / G;         // which row of the iteration this lane group takes
    const int rpi = 32 / G;

    // ---- register-resident activations ---------------------------------------------------
    constexpr int kRegChunks = CPL > 0 ? CPL : 1;
    uint32_t areg[M][kRegChunks][16];
    if (CPL > 0) {
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int c = i * G + lg;
#pragma unroll
            for (int m = 0; m < M; ++m) {
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (c < C) v = *reinterpret_cast<const uint4*>(act + act_offset(m, x, c, K, C));
                    areg[m][i][x * 4 + 0] = v.x; areg[m][i][x * 4 + 1] = v.y;
                    areg[m][i][x * 4 + 2] = v.z; areg[m][i][x * 4 + 3] = v.w;
                }
            }
        }
    }

    // ---- main loop: one stage (a run of whole rows) per iteration ---------------------------
    bool alive = true;
    int it = 0;
    for (int u = gw; u < p.units && alive; u += wstride, ++it) {
        const int s = it % p.stages;
        const uint32_t parity = (it / p.stages) & 1;
        alive = mbar_wait_bounded(&my_bars[s], parity, kp.status);
        alive = __all_sync(0xffffffffu, alive);
        if (!alive) break;
        const int n0 = u * p.rsw;
        const int rows_u = min(p.rsw, N - n0);
        const uint8_t* st = ring + s * p.stage_bytes;

        for (int rb = 0; rb < rows_u; rb += rpi) {
            const int r = rb + rl;
            const bool valid_r = r < rows_u;
            int acc[M][4];
#pragma unroll
            for (int m = 0; m < M; ++m) { acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0; }

            if (CPL > 0) {
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    const int c = i * G + lg;
                    if (valid_r && c < C) {
                        const uint4 w = *reinterpret_cast<const uint4*>(st + (static_cast<size_t>(r) * C + c) * 16);
                        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t masked = wv[x] & (0x03030303u << (2 * j));
#pragma unroll
                                for (int m = 0; m < M; ++m)
                                    acc[m][j] = dp4a_su(static_cast<int>(areg[m][i][x * 4 + j]), masked, acc[m][j]);
                            }
                        }
                    }
                }
            } else {
                for (int i = 0; i < p.cpl; ++i) {
                    const int c = i * G + lg;
                    if (valid_r && c < C) {
                        const uint4 w = *reinterpret_cast<const uint4*>(st + (static_cast<size_t>(r) * C + c) * 16);
                        const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (int x = 0; x < 4; ++x) {
#pragma unroll
                            for (int m = 0; m < M; ++m) {
                                const uint4 av = *reinterpret_cast<const uint4*>(act + act_offset(m, x, c, K, C));
                                acc[m][0] = dp4a_su(static_cast<int>(av.x), wv[x] & 0x03030303u, acc[m][0]);
                                acc[m][1] = dp4a_su(static_cast<int>(av.y), wv[x] & 0x0c0c0c0cu, acc[m][1]);
                                acc[m][2] = dp4a_su(static_cast<int>(av.z), wv[x] & 0x30303030u, acc[m][2]);
                                acc[m][3] = dp4a_su(static_cast<int>(av.w), wv[x] & 0xc0c0c0c0u, acc[m][3]);
                            }
                        }
                    }
                }
            }

#pragma unroll
            for (int m = 0; m < M; ++m) {
                // partial sums are exact multiples of 1, 4, 16, 64
                int t = acc[m][0] + (acc[m][1] >> 2) + (acc[m][2] >> 4) + (acc[m][3] >> 6);
                for (int o = G >> 1; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                if (lg == 0 && valid_r) {
                    const int n = n0 + r;
                    const int total = t - qsum[m];
                    if (a.acc_debug) a.acc_debug[static_cast<size_t>(m) * N + n] = total;
                    a.y[static_cast<size_t>(m) * N + n] = epilogue(total, comb[m], a.magnitude, a.bias, n);
                }
            }
        }

        // every lane is done reading this stage: refill it with the unit NST turns ahead
        __syncwarp();
        if (lane == 0) {
            const int nu = u + p.stages * wstride;
            if (nu < p.units) {
                const int nn0 = nu * p.rsw;
                const int nrows = min(p.rsw, N - nn0);
                const uint32_t bytes = static_cast<uint32_t>(nrows) * row_bytes;
                mbar_arrive_expect_tx(&my_bars[s], bytes);
                bulk_g2s(ring + s * p.stage_bytes, wbytes + static_cast<size_t>(nn0) * row_bytes, bytes,
                         &my_bars[s]);
            }
        }
    }

    if (!alive) {
        // a wait gave up: before leaving, give copies still in flight a bounded chance to land
        // so they do not write into shared memory of a CTA that has already exited
        for (int s = 0; s < p.stages; ++s) {
            for (uint32_t spin = 0; spin < (1u << 16); ++spin)
                if (mbar_try_wait(&my_bars[s], 0) || mbar_try_wait(&my_bars[s], 1)) break;
        }
    }
}

int pow2ceil(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

bool make_plan(int M, int K, int N, Plan& p) {
    if (M < 1 || M > 4 || K % 64 != 0 || K > 4 * kStageMax) return false;
    p.C = K / 64;
    p.G = p.C >= 32 ? 32 : pow2ceil(p.C);
    p.cpl = (p.C + p.G - 1) / p.G;
    const int rpi = 32 / p.G;
    const int row_bytes = K / 4;
    int rsw = kStageTarget / row_bytes;
    if (rsw < 1) rsw = 1;
    if (rsw > rpi) rsw -= rsw % rpi;
    // small matrices: shrink stages so every SM gets work
    const int want_units = 2 * kNumSm;
    int cap = (N + want_units - 1) / want_units;
    cap = ((cap + rpi - 1) / rpi) * rpi;
    if (cap < rpi) cap = rpi;
    if (rsw > cap) rsw = cap;
    p.rsw = rsw;
    p.stage_bytes = ((rsw * row_bytes + 127) / 128) * 128;
    p.units = (N + rsw - 1) / rsw;
    p.warps = (p.units + kNumSm - 1) / kNumSm;
    if (p.warps > kMaxWarps) p.warps = kMaxWarps;
    if (p.warps < 1) p.warps = 1;
    const size_t act_bytes = ((static_cast<size_t>(M) * K + 127) & ~size_t(127));
    const size_t fixed = act_bytes + kMaxWarps * 4 * sizeof(uint64_t) + 128;
    p.stages = 4;
    while (p.stages >= 2 && fixed + static_cast<size_t>(p.warps) * p.stages * p.stage_bytes > kSmemBudget) --p.stages;
    if (p.stages < 2) return false;
    p.smem = fixed + static_cast<size_t>(p.warps) * p.stages * p.stage_bytes;
    int ctas = (p.units + p.warps - 1) / p.warps;
    int per_sm = static_cast<int>((220 * 1024) / (p.smem + 1024));
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    if (ctas > kNumSm * per_sm) ctas = kNumSm * per_sm;
    p.grid = ctas;
    return true;
}

// smallest compiled register variant that covers `cpl` chunks per lane within the register
// budget of M rows; 0 selects the shared-memory variant
int reg_variant(int M, int cpl) {
    static const int options[] = {1, 2, 3, 4, 6, 8};
    for (int o : options)
        if (o >= cpl) return (M * o * 16 <= 128) ? o : 0;
    return 0;
}

template <int M, int CPL>
cudaError_t launch_variant(const KParams& kp, cudaStream_t stream) {
    auto kernel = gemv_stream_kernel<M, CPL>;
    static bool configured[64] = {};  // per (M,CPL) instantiation and device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kernel<<<kp.p.grid, kp.p.warps * 32, kp.p.smem, stream>>>(kp);
    note_launch();
    return cudaGetLastError();
}

template <int M>
cudaError_t dispatch_cpl(const KParams& kp, int variant, cudaStream_t stream) {
    switch (variant) {
        case 1: return launch_variant<M, 1>(kp, stream);
        case 2: return launch_variant<M, 2>(kp, stream);
        case 3: if constexpr (M <= 2) return launch_variant<M, 3>(kp, stream); break;
        case 4: if constexpr (M <= 2) return launch_variant<M, 4>(kp, stream); break;
        case 6: if constexpr (M == 1) return launch_variant<M, 6>(kp, stream); break;
        case 8: if constexpr (M == 1) return launch_variant<M, 8>(kp, stream); break;
        default: break;
    }
    return launch_variant<M, 0>(kp, stream);
}

}  // namespace

bool gemv_small_supported(int M, int K, int N) {
    Plan p;
    return N > 0 && make_plan(M, K, N, p);
}

cudaError_t launch_gemv_small(const GemvSmallArgs& a, cudaStream_t stream) {
    KParams kp;
    kp.a = a;
    if (!make_plan(a.M, a.K, a.N, kp.p)) return cudaErrorInvalidValue;
    kp.status = device_status_ptr();
    if (!kp.status) return cudaErrorUnknown;
    const int variant = reg_variant(a.M, kp.p.cpl);
    switch (a.M) {
        case 1: return dispatch_cpl<1>(kp, variant, stream);
        case 2: return dispatch_cpl<2>(kp, variant, stream);
        case 3: return dispatch_cpl<3>(kp, variant, stream);
        case 4: return dispatch_cpl<4>(kp, variant, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace tbl
