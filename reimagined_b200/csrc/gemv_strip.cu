// Decode GEMV / small-M GEMM (1 <= M <= 64 activation rows per pass) on the strip-major device
// layout of the 2-bit weights: HBM-bound streaming with int8 tensor-core MMAs ("swap-AB").
//
// Layout ("strips", produced once per matrix by relayout_strips): rows are grouped in strips of 16
// and K in blocks of 256; block (strip s, block b) is 1 KB and holds, for lane = 4g+t of a warp, the
// 16-byte chunk (64 weights, k = 256b + 64t ..) of row g at byte lane*16 and of row g+8 at
// 512 + lane*16 -- the two 128-bit shared loads of a lane are its m16n8k32 A-fragment source
// (rows g / g+8) with no bank conflicts.  Blocks are ordered slab-major: a slab is 4 consecutive
// k-blocks (1024 weights of K) of EVERY strip, [slab][strip][block in slab].  CTAs own runs of
// adjacent strips and walk the slabs in step, so at any moment the whole GPU is reading one
// contiguous window of memory (DRAM pages are swept once, front to back) and a CTA's stage is one
// contiguous bulk copy per slab (strips x 4 KB; two slabs per stage for M <= 16) plus, unless the
// quantiser ran in the prologue and left the activations resident, the matching slab of activations.
//
// Widening: for 2-bit position j, (word & (0x03030303 << 2j)) is the unsigned byte vector
// 4^j * code of weights {j,4+j,8+j,12+j} of that word.  With one accumulator set per j the four
// partial sums are exact multiples of 4^j and are recombined with shifts (SCALED variant, one AND
// per A register); the NT = 8 variant shifts instead to keep a single accumulator set.  The
// constant "-1" of the code is removed in the epilogue by subtracting sum_k q[m,k].
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

constexpr int kMaxStages = 8;
constexpr int kStripSlots = 8;     // strips processed concurrently by a CTA
constexpr int kNumSm = 148;

struct StripParams {
    StripProblem prob[TBL_MAX_GROUPS];
    int count;
    int total_strips;
    int share_base, share_rem;   // CTA b owns share_base strips, one more when b < share_rem
    int ks;       // k per stage, multiple of 256
    int stages;
    int stage_shift;   // log2(ks / 256)
    int slots;    // strips per pass (<= kStripSlots): sized to the CTA's share so no stage space idles
    int act_rows; // activation rows held per stage (<= 8*NT); 0 when the activations are resident
    int fused;    // 1: prob[0].x is quantised in the prologue into a resident shared-memory copy
    int* status;
    long long weight_bytes;   // of all problems, for the launcher
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// WPS warps share one strip: warp `part` of a strip takes the 1 KB blocks b with b % WPS == part and
// the partial sums meet in shared memory before the epilogue (more warps in flight per SM).
//
// FAST is the single-row decode case (one activation row quantised in the prologue, K a multiple of
// the 2048-deep stage): every shared-memory offset of a stage is then a compile-time constant off three
// base registers, the four blocks of a warp are fully unrolled, and all lanes read row 0's activation
// fragment (one 128-byte wavefront per load instead of four).
template <int NT, bool SCALED, int WPS, int FAST>
__global__ void __launch_bounds__((kStripSlots * WPS + 1) * 32, 1)
gemv_strip_kernel(const __grid_constant__ StripParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int MPAD = 8 * NT;
    constexpr int NJ = SCALED ? 4 : 1;
    constexpr int kConsumers = kStripSlots * WPS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk_stage = P.ks >> 8;
    const int wstage = P.slots * nblk_stage * 1024;               // weight bytes of a stage
    const int stage_bytes = wstage + nblk_stage * P.act_rows * 256;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    int* reduce_buf = reinterpret_cast<int*>(smem + 128);        // [slot][WPS-1][32 lanes][4*NT]
    constexpr int kReduceBytes = WPS > 1 ? kStripSlots * (WPS - 1) * 32 * 4 * NT * 4 : 0;
    // fused mode: [scales 8 f32 | sums 8 i32 | scratch 16 warps x 8 f32] then the resident activations
    float* s_scale = reinterpret_cast<float*>(smem + 128 + kReduceBytes);
    int* s_qsum = reinterpret_cast<int*>(s_scale + 8);
    float* s_red = s_scale + 16;
    const int fused_bytes = P.fused ? 1024 + ((P.prob[0].rows * P.prob[0].K + 127) & ~127) : 0;
    uint8_t* acts_resident = smem + 128 + kReduceBytes + 1024;
    uint8_t* stage_base = smem + 128 + kReduceBytes + fused_bytes;
    const uint32_t stage_base_addr = smem_u32(stage_base);
    const uint32_t acts_resident_addr = smem_u32(acts_resident);
    const int nstages = P.stages;

    // Programmatic dependent launch: the next kernel of the stream may be scheduled as soon as every
    // CTA of this grid has got here; it can then set up and prefetch weights while this grid drains.
    pdl_launch_dependents();

    uint32_t* s_amax = reinterpret_cast<uint32_t*>(s_red + 16 * 8);      // [8] row absmax as bit patterns

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumers);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (P.fused && threadIdx.x < 8) { s_qsum[threadIdx.x] = 0; s_amax[threadIdx.x] = 0u; }
    __syncthreads();

    if (P.fused && warp < kConsumers) {
        // ---- fused per-token absmax quantiser (consumer warps only; the producer warp is already
        // streaming weights).  Same arithmetic as the stand-alone quantiser kernel.  The rows*K <= 16384
        // inputs are read once, 16 consecutive elements per group and up to two groups per thread, and
        // stay in registers between the absmax reduction and the rounding. ----
        const StripProblem& pr = P.prob[0];
        const int K = pr.K, R = pr.rows;
        constexpr int kT = kConsumers * 32;
        constexpr int kMaxFusedRows = 8;
        constexpr int kGroups = 16384 / 16 / kT;     // 16-element groups per thread
        const int total_groups = R * K / 16;
        pdl_wait();   // x may be the output of the kernel before this one
        float4 xv[kGroups][4];
        int grow[kGroups];
#pragma unroll
        for (int i = 0; i < kGroups; ++i) {
            const int Gl = threadIdx.x + i * kT;
            grow[i] = -1;
            if (Gl < total_groups) {
                const int e = Gl * 16;
                int row = 0;
#pragma unroll
                for (int m = 1; m < kMaxFusedRows; ++m) row += e >= m * K ? 1 : 0;
                grow[i] = row;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) xv[i][q4] = __ldg(reinterpret_cast<const float4*>(pr.x + e + 4 * q4));
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) xv[i][q4] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        // optional residual add in front: x += a * ga [+ b * gb] (same operations, same order as the stand-alone
        // residual kernel, so the residual stream is bit-identical); CTA 0 stores the sum
        if (pr.pre.a) {
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                if (grow[i] >= 0) {
                    const int e = (threadIdx.x + i * kT) * 16, k0 = e - grow[i] * K;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        float4 c = __ldg(reinterpret_cast<const float4*>(pr.pre.a + e + 4 * q4));
                        if (pr.pre.ga) {
                            const float4 g4 = __ldg(reinterpret_cast<const float4*>(pr.pre.ga + k0 + 4 * q4));
                            c.x = __fmul_rn(c.x, g4.x); c.y = __fmul_rn(c.y, g4.y); c.z = __fmul_rn(c.z, g4.z); c.w = __fmul_rn(c.w, g4.w);
                        }
                        if (pr.pre.b) {
                            const float4 b4 = __ldg(reinterpret_cast<const float4*>(pr.pre.b + e + 4 * q4));
                            const float4 g4 = __ldg(reinterpret_cast<const float4*>(pr.pre.gb + k0 + 4 * q4));
                            c.x = __fadd_rn(c.x, __fmul_rn(b4.x, g4.x)); c.y = __fadd_rn(c.y, __fmul_rn(b4.y, g4.y));
                            c.z = __fadd_rn(c.z, __fmul_rn(b4.z, g4.z)); c.w = __fadd_rn(c.w, __fmul_rn(b4.w, g4.w));
                        }
                        xv[i][q4].x = __fadd_rn(xv[i][q4].x, c.x); xv[i][q4].y = __fadd_rn(xv[i][q4].y, c.y);
                        xv[i][q4].z = __fadd_rn(xv[i][q4].z, c.z); xv[i][q4].w = __fadd_rn(xv[i][q4].w, c.w);
                    }
                }
            }
        }
        // The loads above are in the memory pipeline: only now may the producer warp queue its (much
        // larger) weight copies behind them.  Issued the other way round, x waits for up to a ring of
        // weights (measured: 3.5K .. 10.5K cycles until the last x load returned, against ~2K).
        asm volatile("bar.arrive 11, %0;" ::"r"(kT + 32) : "memory");
        if (blockIdx.x == 0 && (pr.pre.hidden_out || pr.pre.trace_out)) {
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                if (grow[i] >= 0) {
                    const int e = (threadIdx.x + i * kT) * 16;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        if (pr.pre.hidden_out) *reinterpret_cast<float4*>(pr.pre.hidden_out + e + 4 * q4) = xv[i][q4];
                        if (pr.pre.trace_out) *reinterpret_cast<float4*>(pr.pre.trace_out + e + 4 * q4) = xv[i][q4];
                    }
                }
            }
        }
        if (pr.pre.norm_w) {
            // RMSNorm x weight of the rows (the norm that opens a stage of the hybrid): the same reduction as the
            // input RMSNorm below with the caller's eps, then (x * inv) * w
            float ss[kMaxFusedRows];
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) ss[m] = 0.0f;
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                float q = 0.0f;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    q += xv[i][q4].x * xv[i][q4].x + xv[i][q4].y * xv[i][q4].y + xv[i][q4].z * xv[i][q4].z + xv[i][q4].w * xv[i][q4].w;
#pragma unroll
                for (int m = 0; m < kMaxFusedRows; ++m) if (grow[i] == m) ss[m] += q;
            }
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) {
                if (m < R) {
#pragma unroll
                    for (int o = 16; o; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
                    if (lane == 0) s_red[warp * kMaxFusedRows + m] = ss[m];
                }
            }
            asm volatile("bar.sync 10, %0;" ::"r"(kT) : "memory");
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                if (grow[i] >= 0) {
                    float r = s_red[grow[i]];
                    for (int w = 1; w < kConsumers; ++w) r += s_red[w * kMaxFusedRows + grow[i]];
                    const float f = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(r, static_cast<float>(K)), pr.pre.norm_eps)));
                    const int k0 = (threadIdx.x + i * kT) * 16 - grow[i] * K;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const float4 w4 = __ldg(reinterpret_cast<const float4*>(pr.pre.norm_w + k0 + 4 * q4));
                        xv[i][q4].x = __fmul_rn(__fmul_rn(xv[i][q4].x, f), w4.x); xv[i][q4].y = __fmul_rn(__fmul_rn(xv[i][q4].y, f), w4.y);
                        xv[i][q4].z = __fmul_rn(__fmul_rn(xv[i][q4].z, f), w4.z); xv[i][q4].w = __fmul_rn(__fmul_rn(xv[i][q4].w, f), w4.w);
                    }
                }
            }
            asm volatile("bar.sync 10, %0;" ::"r"(kT) : "memory");      // s_red is reused by the input RMSNorm below
        }
        if (pr.rms_fast) {
            // per-row sum of squares: thread partials, warp shuffles, then a
            // fixed-order sum over the warps
            float ss[kMaxFusedRows];
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) ss[m] = 0.0f;
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                float q = 0.0f;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    q += xv[i][q4].x * xv[i][q4].x + xv[i][q4].y * xv[i][q4].y + xv[i][q4].z * xv[i][q4].z + xv[i][q4].w * xv[i][q4].w;
#pragma unroll
                for (int m = 0; m < kMaxFusedRows; ++m) if (grow[i] == m) ss[m] += q;
            }
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) {
                if (m < R) {
#pragma unroll
                    for (int o = 16; o; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
                    if (lane == 0) s_red[warp * kMaxFusedRows + m] = ss[m];
                }
            }
            asm volatile("bar.sync 10, %0;" ::"r"(kT) : "memory");
            float inv[kMaxFusedRows];
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) {
                inv[m] = 1.0f;
                if (m < R) {
                    float r = s_red[m];
                    for (int w = 1; w < kConsumers; ++w) r += s_red[w * kMaxFusedRows + m];
                    inv[m] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(r, static_cast<float>(K)), 1e-6f)));
                }
            }
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                float f = 1.0f;
#pragma unroll
                for (int m = 0; m < kMaxFusedRows; ++m) if (grow[i] == m) f = inv[m];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    xv[i][q4].x = __fmul_rn(xv[i][q4].x, f); xv[i][q4].y = __fmul_rn(xv[i][q4].y, f);
                    xv[i][q4].z = __fmul_rn(xv[i][q4].z, f); xv[i][q4].w = __fmul_rn(xv[i][q4].w, f);
                }
            }
        }
        // absmax: thread maxima (fmaxf drops NaNs), one redux and one shared atomic max per warp and row;
        // non-negative floats order like their bit patterns
        {
            float mx[kMaxFusedRows];
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) mx[m] = 0.0f;
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                float q = 0.0f;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    q = fmaxf(q, fmaxf(fmaxf(fabsf(xv[i][q4].x), fabsf(xv[i][q4].y)), fmaxf(fabsf(xv[i][q4].z), fabsf(xv[i][q4].w))));
#pragma unroll
                for (int m = 0; m < kMaxFusedRows; ++m) if (grow[i] == m) mx[m] = fmaxf(mx[m], q);
            }
#pragma unroll
            for (int m = 0; m < kMaxFusedRows; ++m) {
                if (m < R) {
                    const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(mx[m]));
                    if (lane == 0 && wmax != 0u) atomicMax(&s_amax[m], wmax);
                }
            }
        }
        asm volatile("bar.sync 10, %0;" ::"r"(kT) : "memory");
        // rounding: q = rint(x * scale) by adding 1.5 * 2^23 (round-to-nearest-even at integer granularity,
        // exact for |x * scale| < 2^22): the low byte of the sum's bit pattern is the int8 code
        int qsum[kMaxFusedRows];
#pragma unroll
        for (int m = 0; m < kMaxFusedRows; ++m) qsum[m] = 0;
#pragma unroll
        for (int i = 0; i < kGroups; ++i) {
            if (grow[i] >= 0) {
                const int m = grow[i];
                const float denom = __fadd_rn(__uint_as_float(s_amax[m]), 1e-8f);
                const float scale = __fdiv_rn(pr.q_max, denom);
                uint32_t wds[4];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint32_t c0 = __float_as_uint(__fadd_rn(__fmul_rn(xv[i][q4].x, scale), 12582912.0f));
                    const uint32_t c1 = __float_as_uint(__fadd_rn(__fmul_rn(xv[i][q4].y, scale), 12582912.0f));
                    const uint32_t c2 = __float_as_uint(__fadd_rn(__fmul_rn(xv[i][q4].z, scale), 12582912.0f));
                    const uint32_t c3 = __float_as_uint(__fadd_rn(__fmul_rn(xv[i][q4].w, scale), 12582912.0f));
                    wds[q4] = __byte_perm(__byte_perm(c0, c1, 0x0040), __byte_perm(c2, c3, 0x0040), 0x5410);
                    const int s4 = dp4a_ss(static_cast<int>(wds[q4]), 0x01010101, 0);
#pragma unroll
                    for (int r = 0; r < kMaxFusedRows; ++r) if (m == r) qsum[r] += s4;
                }
                const int e = (threadIdx.x + i * kT) * 16;
                const uint4 codes = transpose4x4_bytes(make_uint4(wds[0], wds[1], wds[2], wds[3]));
                *reinterpret_cast<uint4*>(acts_resident + qp_offset(m, R, K, e - m * K)) = codes;
            }
        }
#pragma unroll
        for (int m = 0; m < kMaxFusedRows; ++m) {
            if (m < R) {
                const int wsum = __reduce_add_sync(0xffffffffu, qsum[m]);
                if (lane == 0 && wsum != 0) atomicAdd(&s_qsum[m], wsum);
            }
        }
        if (static_cast<int>(threadIdx.x) < R)
            s_scale[threadIdx.x] = __fdiv_rn(__fadd_rn(__uint_as_float(s_amax[threadIdx.x]), 1e-8f), pr.q_max);
        asm volatile("bar.sync 10, %0;" ::"r"(kT) : "memory");
    }

    // contiguous, balanced share of the global strip list
    const int bid = static_cast<int>(blockIdx.x);
    const int s_begin = bid * P.share_base + min(bid, P.share_rem);
    const int s_end = s_begin + P.share_base + (bid < P.share_rem ? 1 : 0);
    const bool producer = warp == kConsumers;
    if (producer && P.fused) asm volatile("bar.sync 11, %0;" ::"r"(kConsumers * 32 + 32) : "memory");
    const int slot = warp / WPS, part = warp % WPS;
    // Everything but the weights (quantised activations, their scales and sums, row counts) may come
    // from the preceding kernel: consumers wait for it here, the producer just before its first
    // activation copy, so the first weight stage is already in flight.
    bool upstream_done = P.fused != 0;
    if (!producer && !upstream_done) { pdl_wait(); upstream_done = true; }
    const int g = lane >> 2, t = lane & 3;
    // byte offset, inside a 256-byte activation row block, of the 16-byte group (quarter x, chunk t)
    // of activation row g (row nt*8+g adds nt*2048; the XOR term is the same since 8 is even)
    int aoff[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) aoff[x] = g * 256 + ((((x ^ (g & 1)) << 2) + t) << 4);

    int it = 0;
    bool alive = true;
    int pi = 0;
    for (int s = s_begin; s < s_end && alive;) {
        while (pi + 1 < P.count && s >= P.prob[pi + 1].strip_begin) ++pi;
        const StripProblem& pr = P.prob[pi];
        const int K = pr.K, N = pr.N;
        const int nstrips = (N + 15) >> 4;
        const int local = s - pr.strip_begin;
        const int cnt = min(P.slots, min(s_end - s, nstrips - local));
        s += cnt;
        int rows = pr.rows;
        if ((pr.rows_dev || pr.offset_dev) && !upstream_done) { pdl_wait(); upstream_done = true; }
        if (pr.rows_dev) rows = min(rows, __ldg(pr.rows_dev));
        if (rows <= 0) continue;
        const int row0 = pr.offset_dev ? __ldg(pr.offset_dev) : 0;
        const int nblk = K >> 8;
        const int ksteps = (nblk + nblk_stage - 1) >> P.stage_shift;   // nblk_stage = 1 << stage_shift
        const int mtiles = (rows + MPAD - 1) / MPAD;   // > 1 only in the NT = 8 variant
        const int8_t* qsrc = pr.qp + static_cast<size_t>(row0) * K;

        for (int mt = 0; mt < mtiles && alive; ++mt) {
            const int R = min(MPAD, rows - mt * MPAD);
            const int8_t* qtile = qsrc + static_cast<size_t>(mt) * MPAD * K;

            if (producer) {
                for (int ksi = 0; ksi < ksteps; ++ksi, ++it) {
                    const int st = it % nstages;
                    if (it >= nstages) {
                        alive = mbar_wait_bounded(&empty[st], ((it / nstages) - 1) & 1, P.status);
                        alive = __all_sync(0xffffffffu, alive);
                        if (!alive) break;
                    }
                    const int b0 = ksi * nblk_stage;
                    const int nb = min(nblk_stage, nblk - b0);
                    uint8_t* wst = stage_base + static_cast<size_t>(st) * stage_bytes;
                    if (lane == 0)
                        mbar_arrive_expect_tx(&full[st], static_cast<uint32_t>(cnt) * nb * 1024 +
                                                             (P.fused ? 0u : static_cast<uint32_t>(nb) * R * 256));
                    __syncwarp();
                    // slab-major source: slab t starts at block 4*t*nstrips and gives each strip bs blocks
                    const int slab = b0 >> 2, bin = b0 & 3;
                    const int bs = min(4, nblk - 4 * slab);
                    const uint8_t* slab_src = pr.strips + ((static_cast<size_t>(4) * slab * nstrips +
                                                            static_cast<size_t>(local) * bs) << 10);
                    if (nblk_stage >= 4) {
                        // the stage is one or more whole slabs of cnt adjacent strips: one contiguous copy
                        // per slab, laid out [slab][strip][block in slab]
                        if (lane < ((nb + 3) >> 2)) {
                            const int sl = slab + lane;
                            const int sbs = min(4, nblk - 4 * sl);
                            bulk_g2s(wst + lane * cnt * 4096,
                                     pr.strips + ((static_cast<size_t>(4) * sl * nstrips + static_cast<size_t>(local) * sbs) << 10),
                                     cnt * sbs * 1024, &full[st]);
                        }
                    } else if (lane < cnt) {
                        bulk_g2s(wst + lane * nb * 1024, slab_src + ((static_cast<size_t>(lane) * bs + bin) << 10),
                                 nb * 1024, &full[st]);
                    }
                    if (!upstream_done) { pdl_wait(); upstream_done = true; }
                    if (lane == kStripSlots && !P.fused)
                        bulk_g2s(wst + wstage, qtile + static_cast<size_t>(b0) * R * 256, nb * R * 256,
                                 &full[st]);
                }
                continue;
            }

            // ---------------- consumer warps ----------------
            const bool active = slot < cnt;
            int acc[NJ][NT][4];
#pragma unroll
            for (int j = 0; j < NJ; ++j)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) acc[j][nt][0] = acc[j][nt][1] = acc[j][nt][2] = acc[j][nt][3] = 0;

            for (int ksi = 0; ksi < ksteps; ++ksi, ++it) {
                const int st = it % nstages;
                alive = mbar_wait_bounded(&full[st], (it / nstages) & 1, P.status);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;

                if (active) {
                    const int nb = min(nblk_stage, nblk - ksi * nblk_stage);
                    const uint32_t stage_addr = stage_base_addr + st * stage_bytes;
                    // activations: this stage's slab, or the resident copy at the stage's first block
                    const uint32_t ast = P.fused ? acts_resident_addr + ksi * nblk_stage * R * 256 : stage_addr + wstage;
                    // one 1 KB weight block (lane's two 16-byte chunks at wblk, wblk + 512) against the
                    // activation block at ablk.  Rows m >= R of that block are stale shared memory: their
                    // accumulator columns are never stored, so the loads need no predicate.
                    auto process_block = [&](const uint32_t wblk, const uint32_t ablk) {
                        const uint4 lo = lds128(wblk);
                        const uint4 hi = lds128(wblk + 512);
                        const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w};
                        const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
                        // Word pairs (0,1) and (2,3) of the lane's chunk feed one MMA each per 2-bit position j.
                        // Loop order keeps consecutive MMAs on different accumulators (sets j when SCALED,
                        // activation tiles nt otherwise), so none waits on the one issued just before it.
#pragma unroll
                        for (int xp = 0; xp < 2; ++xp) {
                            uint32_t bw[NT][2][4];
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    const uint4 B = lds128(ablk + nt * 2048 + aoff[2 * xp + h]);
                                    bw[nt][h][0] = B.x; bw[nt][h][1] = B.y; bw[nt][h][2] = B.z; bw[nt][h][3] = B.w;
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint32_t a0, a1, a2, a3;
                                if (SCALED) {
                                    const uint32_t mk = 0x03030303u << (2 * j);
                                    a0 = lw[2 * xp] & mk; a1 = hw[2 * xp] & mk;
                                    a2 = lw[2 * xp + 1] & mk; a3 = hw[2 * xp + 1] & mk;
                                } else {
                                    const uint32_t mk = 0x03030303u;
                                    a0 = (lw[2 * xp] >> (2 * j)) & mk; a1 = (hw[2 * xp] >> (2 * j)) & mk;
                                    a2 = (lw[2 * xp + 1] >> (2 * j)) & mk; a3 = (hw[2 * xp + 1] >> (2 * j)) & mk;
                                }
#pragma unroll
                                for (int nt = 0; nt < NT; ++nt)
                                    mma_u8s8(acc[SCALED ? j : 0][nt], a0, a1, a2, a3, bw[nt][0][j], bw[nt][1][j]);
                            }
                        }
                    };
                    if constexpr (FAST == 2) {
                        // Up to 16 rows, fused or staged activations, full 2048-deep stages: the stage's blocks of
                        // this warp unrolled with constant weight offsets and the loads of a block issued ahead
                        // of the MMAs of the block before it (as in the single-row path below); only the
                        // activation addresses depend on the row count.
                        static_assert(NT <= 2 && SCALED && 4 % WPS == 0, "pipelined few-row path");
                        constexpr int kBlocks = 8 / WPS;                       // blocks part, part + WPS, ...
                        const uint32_t w0 = stage_addr + lane * 16 + (slot * 4 + part) * 1024;
                        const uint32_t wslab = cnt * 4096;
                        const uint32_t rstride = R * 256;
                        const uint32_t a0 = (P.fused ? acts_resident_addr + ksi * 8 * rstride : stage_addr + wstage) + part * rstride;
                        struct Operands { uint4 lo, hi, b[NT][4]; };
                        auto load_block = [&](Operands& o, const int i) {
                            const int b = i * WPS;                             // relative to `part`
                            const uint32_t wblk = w0 + (b >> 2) * wslab + (b & 3) * 1024;
                            const uint32_t ablk = a0 + b * rstride;
                            o.lo = lds128(wblk);
                            o.hi = lds128(wblk + 512);
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                                for (int x = 0; x < 4; ++x) o.b[nt][x] = lds128(ablk + nt * 2048 + aoff[x]);
                        };
                        auto mma_block = [&](const Operands& o) {
                            const uint32_t lw[4] = {o.lo.x, o.lo.y, o.lo.z, o.lo.w};
                            const uint32_t hw[4] = {o.hi.x, o.hi.y, o.hi.z, o.hi.w};
#pragma unroll
                            for (int xp = 0; xp < 2; ++xp) {
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint32_t mk = 0x03030303u << (2 * j);
#pragma unroll
                                    for (int nt = 0; nt < NT; ++nt) {
                                        const uint4& B0 = o.b[nt][2 * xp];
                                        const uint4& B1 = o.b[nt][2 * xp + 1];
                                        const uint32_t b0 = j == 0 ? B0.x : (j == 1 ? B0.y : (j == 2 ? B0.z : B0.w));
                                        const uint32_t b1 = j == 0 ? B1.x : (j == 1 ? B1.y : (j == 2 ? B1.z : B1.w));
                                        mma_u8s8(acc[j][nt], lw[2 * xp] & mk, hw[2 * xp] & mk, lw[2 * xp + 1] & mk,
                                                 hw[2 * xp + 1] & mk, b0, b1);
                                    }
                                }
                            }
                        };
                        Operands ops[2];
                        load_block(ops[0], 0);
#pragma unroll
                        for (int i = 0; i < kBlocks; ++i) {
                            if (i + 1 < kBlocks) load_block(ops[(i + 1) & 1], i + 1);
                            mma_block(ops[i & 1]);
                        }
                    } else if constexpr (FAST == 1) {
                        static_assert(NT == 1 && WPS == 2 && SCALED, "single-row fast path");
                        // blocks part, part+2 of both slabs; activation block b of the resident row at b*256
                        const uint32_t w0 = stage_addr + lane * 16 + (slot * 4 + part) * 1024;
                        const uint32_t w1 = w0 + cnt * 4096;
                        const uint32_t a0 = acts_resident_addr + t * 16 + (ksi * 8 + part) * 256;
                        // software pipeline: the six shared loads of a block are issued before the MMAs of
                        // the block ahead of it (the asm statements keep this order)
                        struct Operands { uint4 lo, hi, b[4]; };
                        auto load_block = [&](const uint32_t wblk, const uint32_t ablk) {
                            Operands o;
                            o.lo = lds128(wblk);
                            o.hi = lds128(wblk + 512);
#pragma unroll
                            for (int x = 0; x < 4; ++x) o.b[x] = lds128(ablk + x * 64);
                            return o;
                        };
                        // One row: each lane takes the dot products of its own 16-byte chunks (row g and row g + 8,
                        // 64 weights each) with the matching 64 codes by dp4a, plane by plane -- seven of an MMA's
                        // eight columns would be idle; the four lanes of a row meet once, after the k-loop.
                        // acc[p][0][0] / acc[p][0][2] are the plane-p sums of row g / g + 8.
                        auto mma_block = [&](const Operands& o) {
                            const uint32_t lw[4] = {o.lo.x, o.lo.y, o.lo.z, o.lo.w};
                            const uint32_t hw[4] = {o.hi.x, o.hi.y, o.hi.z, o.hi.w};
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
                                const uint32_t a[4] = {o.b[x].x, o.b[x].y, o.b[x].z, o.b[x].w};   // word p: plane p of quarter x
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const uint32_t mk = 0x03030303u << (2 * j);
                                    acc[j][0][0] = dp4a_su(static_cast<int>(a[j]), lw[x] & mk, acc[j][0][0]);
                                    acc[j][0][2] = dp4a_su(static_cast<int>(a[j]), hw[x] & mk, acc[j][0][2]);
                                }
                            }
                        };
                        const Operands o0 = load_block(w0, a0);
                        const Operands o1 = load_block(w0 + 2048, a0 + 512);
                        mma_block(o0);
                        const Operands o2 = load_block(w1, a0 + 1024);
                        mma_block(o1);
                        const Operands o3 = load_block(w1 + 2048, a0 + 1536);
                        mma_block(o2);
                        mma_block(o3);
                    } else if (nblk_stage >= 4) {
                        // stage layout [slab][strip][block in slab]; blocks of this stage are global blocks
                        // ksi*nblk_stage + 4*sl + bin and this warp takes its residue class modulo WPS
                        static_assert(4 % WPS == 0, "a slab must split evenly over the warps of a strip");
                        const int first = (part + WPS - (ksi * nblk_stage) % WPS) % WPS;
                        const uint32_t astep = WPS * R * 256;
                        for (int sl = 0; 4 * sl < nb; ++sl) {
                            const int sbs = min(4, nb - 4 * sl);
                            const uint32_t wslab = stage_addr + lane * 16 + sl * cnt * 4096 + (slot * sbs + first) * 1024;
                            uint32_t ablk = ast + (4 * sl + first) * R * 256;
#pragma unroll
                            for (int i = 0; i < 4 / WPS; ++i) {
                                if (first + i * WPS < sbs) process_block(wslab + i * WPS * 1024, ablk);
                                ablk += astep;
                            }
                        }
                    } else {
                        // stage layout [strip][block]
                        const uint32_t wst = stage_addr + slot * nb * 1024 + lane * 16;
                        const int first = (part + WPS - (ksi * nblk_stage) % WPS) % WPS;
#pragma unroll 2
                        for (int b = first; b < nb; b += WPS) process_block(wst + b * 1024, ast + b * R * 256);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }
            if (!alive) break;

            if (active) {
                if constexpr (FAST == 1) {
                    // the four lanes of a row (t = 0..3) hold the sums of their quarters of every k-block
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            int v = acc[j][0][e];
                            v += __shfl_xor_sync(0xffffffffu, v, 1);
                            v += __shfl_xor_sync(0xffffffffu, v, 2);
                            acc[j][0][e] = v;
                        }
                    }
                }
                // exact recombination of the scaled partial sums, then the cross-warp reduction
                int tot[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (SCALED)
                            tot[nt][e] = acc[0][nt][e] + (acc[NJ > 1 ? 1 : 0][nt][e] >> 2) +
                                         (acc[NJ > 2 ? 2 : 0][nt][e] >> 4) + (acc[NJ > 3 ? 3 : 0][nt][e] >> 6);
                        else
                            tot[nt][e] = acc[0][nt][e];
                    }
                if (WPS > 1) {
                    int* mine = reduce_buf + ((slot * (WPS - 1) + (part - 1)) * 32 + lane) * 4 * NT;
                    if (part > 0) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
                            *reinterpret_cast<int4*>(mine + 4 * nt) = make_int4(tot[nt][0], tot[nt][1], tot[nt][2], tot[nt][3]);
                    }
                    asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * WPS) : "memory");
                    if (part == 0) {
#pragma unroll
                        for (int w = 0; w < WPS - 1; ++w) {
                            const int* other = reduce_buf + ((slot * (WPS - 1) + w) * 32 + lane) * 4 * NT;
#pragma unroll
                            for (int nt = 0; nt < NT; ++nt) {
                                const int4 v = *reinterpret_cast<const int4*>(other + 4 * nt);
                                tot[nt][0] += v.x; tot[nt][1] += v.y; tot[nt][2] += v.z; tot[nt][3] += v.w;
                            }
                        }
                    }
                    // the buffer is reused by the next pass: readers must be done before writers return
                    asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * WPS) : "memory");
                }
                if (part == 0) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int n = (local + slot) * 16 + g + 8 * h;
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int m = nt * 8 + 2 * t + c;
                            if (n < N && m < R) {
                                const int e = 2 * h + c;
                                int total = tot[nt][e];
                                const int gm = row0 + mt * MPAD + m;
                                total -= P.fused ? s_qsum[m] : __ldg(pr.q_sums + gm);
                                if (pr.acc_debug) pr.acc_debug[static_cast<size_t>(gm) * pr.ldy + n] = total;
                                const float a_scale = P.fused ? s_scale[m] : __ldg(pr.act_scales + gm);
                                float v = epilogue(total, __fmul_rn(a_scale, pr.weight_scale),
                                                   pr.magnitude, pr.bias, n);
                                if (pr.squared_relu) { v = fmaxf(v, 0.0f); v = __fmul_rn(v, v); }
                                pr.y[static_cast<size_t>(gm) * pr.ldy + n] = v;
                            }
                        }
                    }
                }
                }
            }
        }
    }
}

// canonical [N, K/16] words -> strip layout (slab-major); one thread per 16-byte chunk of the output.
__global__ void __launch_bounds__(256)
relayout_strips_kernel(const uint4* __restrict__ words, int N, int K, uint4* __restrict__ strips, int64_t chunks) {
    const int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (o >= chunks) return;
    const int cpr = K >> 6;               // 16-byte chunks per row
    const int nblk = K >> 8;
    const int nstrips = (N + 15) >> 4;
    const int64_t blk = o >> 6;           // 1 KB block index in the output
    const int within = static_cast<int>(o & 63);
    const int full_slabs = nblk >> 2;
    const int64_t boundary = static_cast<int64_t>(full_slabs) * 4 * nstrips;
    int s, b;
    if (blk < boundary) {
        const int64_t slab = blk / (4 * static_cast<int64_t>(nstrips));
        const int rem = static_cast<int>(blk % (4 * static_cast<int64_t>(nstrips)));
        s = rem >> 2;
        b = static_cast<int>(slab) * 4 + (rem & 3);
    } else {
        const int r = nblk & 3;           // blocks per strip in the last, partial slab
        const int rem = static_cast<int>(blk - boundary);
        s = rem / r;
        b = full_slabs * 4 + rem % r;
    }
    const int h = within >> 5, ln = within & 31;
    const int row = s * 16 + h * 8 + (ln >> 2);
    const int c = 4 * b + (ln & 3);
    uint4 v = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);  // code 1 = weight 0
    if (row < N) v = __ldg(words + static_cast<size_t>(row) * cpr + c);
    strips[o] = v;
}

// q row-major [M,K] -> tile-exact interleaved order + per-row sums; one CTA per row.
__global__ void __launch_bounds__(256) permute_q_kernel(const int8_t* __restrict__ q, int M, int K,
                                                        int8_t* __restrict__ qp, int32_t* __restrict__ q_sums) {
    __shared__ int partial[8];
    const int row = blockIdx.x;
    const int8_t* src = q + static_cast<size_t>(row) * K;
    int sum = 0;
    for (int j = threadIdx.x * 16; j < K; j += 256 * 16) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + j));
        sum = dp4a_ss(static_cast<int>(v.x), 0x01010101, sum);
        sum = dp4a_ss(static_cast<int>(v.y), 0x01010101, sum);
        sum = dp4a_ss(static_cast<int>(v.z), 0x01010101, sum);
        sum = dp4a_ss(static_cast<int>(v.w), 0x01010101, sum);
        *reinterpret_cast<uint4*>(qp + qp_offset(row, M, K, j)) = transpose4x4_bytes(v);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int w = 0; w < 8; ++w) s += partial[w];
        q_sums[row] = s;
    }
}

cudaEvent_t g_event_start = nullptr, g_event_stop = nullptr;

template <int NT, bool SCALED, int WPS, int FAST = 0>
cudaError_t launch_variant(const StripParams& P, int grid, size_t smem, cudaStream_t stream) {
    auto kernel = gemv_strip_kernel<NT, SCALED, WPS, FAST>;
    smem += WPS > 1 ? kStripSlots * (WPS - 1) * 32 * 4 * NT * 4 : 0;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    if (g_event_start) cudaEventRecord(g_event_start, stream);
    // launched as a programmatic dependent of the preceding kernel of the stream (the kernel orders
    // itself after that kernel with griddepcontrol.wait before it touches anything but the weights)
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((kStripSlots * WPS + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2]{};
    int na = 0;
    // measured: the overlap pays for short kernels (4096^2: 7.0 -> 6.2 us) and costs a long one 2 %
    if (P.weight_bytes <= (32ll << 20)) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    const cudaError_t launched = cudaLaunchKernelEx(&cfg, kernel, P);
    if (g_event_stop) cudaEventRecord(g_event_stop, stream);
    note_launch();
    return launched != cudaSuccess ? launched : cudaGetLastError();
}

}  // namespace

void set_gemv_events(cudaEvent_t start, cudaEvent_t stop) {
    g_event_start = start;
    g_event_stop = stop;
}

// The fused prologue holds rows*K <= 16384 inputs in registers and keeps their int8 codes resident
// in shared memory next to the ring; at most 8 rows.
int gemv_strip_fused_rows(int K) {
    if (!gemv_strip_supported(K)) return 0;
    const int rows = 16384 / K;
    return rows > 8 ? 8 : rows;
}

bool gemv_strip_supported(int K) { return K > 0 && K % 256 == 0 && K <= 65536; }

cudaError_t launch_relayout_strips(const uint32_t* words, int N, int K, void* strips, cudaStream_t stream) {
    const int64_t chunks = static_cast<int64_t>((N + 15) / 16) * 16 * (K / 64);
    const int blocks = static_cast<int>((chunks + 255) / 256);
    relayout_strips_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint4*>(words), N, K,
                                                       static_cast<uint4*>(strips), chunks);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_permute_q(const int8_t* q, int M, int K, int8_t* qp, int32_t* q_sums, cudaStream_t stream) {
    permute_q_kernel<<<M, 256, 0, stream>>>(q, M, K, qp, q_sums);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_gemv_strip(StripProblem* problems, int count, cudaStream_t stream) {
    if (count < 1 || count > TBL_MAX_GROUPS) return cudaErrorInvalidValue;
    StripParams P{};
    P.count = count;
    P.status = device_status_ptr();
    if (!P.status) return cudaErrorUnknown;
    int max_rows = 1, total = 0;
    for (int i = 0; i < count; ++i) {
        if (!gemv_strip_supported(problems[i].K)) return cudaErrorInvalidValue;
        max_rows = problems[i].rows > max_rows ? problems[i].rows : max_rows;
        P.prob[i] = problems[i];
        P.prob[i].strip_begin = total;
        total += (problems[i].N + 15) / 16;
        P.weight_bytes += static_cast<long long>((problems[i].N + 15) / 16) * 4 * problems[i].K;
    }
    P.total_strips = total;
    const int nt = max_rows <= 8 ? 1 : (max_rows <= 16 ? 2 : (max_rows <= 32 ? 4 : 8));
    // Stage depth in k.  Two slabs (2048) per stage halve the per-stage synchronisation of a consumer warp
    // (16384^2, M = 1: 20.8 -> 18.5 us); three are no better, with only two stages left in the ring.
    // Tall activation tiles leave room for one slab (long rows: 16384^2 M=64 70.9 -> 64.8 us) or half a slab.
    int max_k = 0;
    for (int i = 0; i < count; ++i) max_k = problems[i].K > max_k ? problems[i].K : max_k;
    P.ks = nt <= 2 ? (max_k >= 2048 ? 2048 : 1024) : (max_k >= 4096 ? 1024 : 512);
    P.stage_shift = P.ks == 2048 ? 3 : (P.ks == 1024 ? 2 : 1);
    int grid = (total + kStripSlots - 1) / kStripSlots;
    if (grid > kNumSm) grid = kNumSm;
    // spread small problems over more SMs (fewer strips per CTA)
    if (total < kNumSm * kStripSlots) grid = total < kNumSm ? total : kNumSm;
    // fused quantiser: one problem, or several that share the input rows (grouped projections)
    P.fused = problems[0].x != nullptr;
    for (int i = 0; i < count; ++i) {
        const bool same = problems[i].x == problems[0].x && problems[i].K == problems[0].K &&
                          problems[i].rows == problems[0].rows && problems[i].rms_fast == problems[0].rms_fast &&
                          problems[i].q_max == problems[0].q_max;
        if ((P.fused || problems[i].x != nullptr) && !same) return cudaErrorInvalidValue;
    }
    if (P.fused && (nt != 1 || problems[0].rows > gemv_strip_fused_rows(problems[0].K) || problems[0].rows_dev))
        return cudaErrorInvalidValue;
    const bool fast = nt == 1 && count == 1 && P.fused && problems[0].rows == 1 && P.ks == 2048 && problems[0].K % 2048 == 0;
    // up to 16 rows (no device-side row counts), every stage full
    const bool few_rows_fast = nt <= 2 && count == 1 && !problems[0].rows_dev && !problems[0].offset_dev &&
                               P.ks == 2048 && problems[0].K % 2048 == 0;
    // a CTA's passes take at most `slots` strips: size the stages for the largest share, not for 8
    P.share_base = total / grid;
    P.share_rem = total % grid;
    const int share = (total + grid - 1) / grid;
    const int passes = (share + kStripSlots - 1) / kStripSlots;
    P.slots = (share + passes - 1) / passes;
    P.act_rows = P.fused ? 0 : (max_rows < 8 * nt ? max_rows : 8 * nt);
    const size_t fused_bytes = P.fused ? 1024 + ((static_cast<size_t>(problems[0].rows) * problems[0].K + 127) & ~size_t(127)) : 0;
    const size_t stage_bytes = static_cast<size_t>(P.slots) * (P.ks / 256) * 1024 +
                               static_cast<size_t>(P.ks / 256) * P.act_rows * 256;
    // the ring takes what the 227 KB of a CTA leave after the fixed parts (barriers, fused quantiser state,
    // the slack below and the cross-warp reduction buffer the launcher adds for the two-warps-per-strip variant)
    const size_t fixed = 128 + fused_bytes + static_cast<size_t>(8 * nt) * 256 + (nt == 1 ? kStripSlots * 32 * 4 * 4 : 0);
    const size_t room = 227 * 1024 - fixed;
    P.stages = static_cast<int>(room / stage_bytes < static_cast<size_t>(kMaxStages) ? room / stage_bytes : kMaxStages);
    if (P.stages < 2) return cudaErrorInvalidValue;
    // slack after the last stage: lanes of activation rows >= act_rows read (and ignore) stale bytes
    const size_t smem = 128 + fused_bytes + P.stages * stage_bytes + static_cast<size_t>(8 * nt) * 256;
    switch (nt) {
        case 1:
            if (fast)
                return launch_variant<1, true, 2, 1>(P, grid, smem, stream);
            if (few_rows_fast)
                return launch_variant<1, true, 2, 2>(P, grid, smem, stream);
            return launch_variant<1, true, 2>(P, grid, smem, stream);
        case 2:
            if (few_rows_fast) return launch_variant<2, true, 1, 2>(P, grid, smem, stream);
            return launch_variant<2, true, 1>(P, grid, smem, stream);
        case 4: return launch_variant<4, true, 1>(P, grid, smem, stream);
        default: return launch_variant<8, false, 1>(P, grid, smem, stream);
    }
}

}  // namespace tbl
