// A stack of ternary linears in ONE persistent launch: y = L_{n-1}( ... L_1( L_0(x) ) ), few activation rows
// (decode).  Each layer is [RMSNorm] -> per-token absmax quantiser -> 2-bit ternary GEMV -> two-scale epilogue
// [-> squared ReLU], exactly as the single-layer strip GEMV computes it.
//
// Why one launch: a decode GEMV over 64 MiB of weights lasts about as long as the DRAM pipeline needs to ramp
// up and drain, so a chain of separate launches never reaches the streaming rate.  Here one CTA per SM stays
// resident for the whole stack.  Its producer warp depends on nothing but the weights, so it keeps the ring of
// shared-memory stages full across layer boundaries: while the consumer warps of the grid finish layer l, meet
// at a grid-wide barrier and quantise the new activation row, the first stages of layer l+1 are already
// landing.  The weight stream of the whole stack is one uninterrupted front-to-back sweep of HBM.
//
// Layer boundary (consumer warps only).  The epilogue warp of each strip stores its 16 outputs per row and counts
// its strip as arrived -- per warp, with no CTA-wide barrier and NO fence, so neither the round trips of the seven
// strips of a CTA nor a store's way to L2 are waited for.  The quantiser of the next layer polls the counter
// (bounded) until three quarters of the strips have arrived and then reads the row (L2-resident).  Nothing orders
// a strip's stores before its arrival, and the last strips have not even been counted at that point: every
// activation buffer starts the launch filled with all-ones words -- a bit pattern the writers never store (they
// replace that one NaN by the canonical one) -- so a load validates itself, and a 16-value group is fetched again
// (bounded) until none of its words is the filler.  The row maximum is then taken over the loaded values (max is
// exact in any order) and the row is quantised straight into shared memory.  The grid must be co-resident: the
// kernel is launched cooperatively.  Every wait is bounded; a wait that gives up sets TBL_DEV_WAIT_TIMEOUT and the
// CTA leaves.
//
// Weight layout, stage layout, widening and the MMA are those of gemv_strip.cu (strips of 16 rows, 1 KB
// blocks, slab-major order, mma.sync.m16n8k32.u8.s8 with the weights as the A operand); single-row layers with
// full 2048-deep stages take their dot products with dp4a on the same masked words instead (no tensor pipe).
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

constexpr int kMaxStages = 8;
constexpr int kSlots = 8;                  // strips a CTA works on concurrently
constexpr int kWps = 2;                    // warps per strip
constexpr int kConsumers = kSlots * kWps;  // 16 consumer warps + 1 producer warp
constexpr int kT = kConsumers * 32;
constexpr int kMaxRows = 8;
constexpr int kGroups = 16384 / 16 / kT;   // 16-element groups per thread in the quantiser
constexpr int kReduceBytes = kSlots * (kWps - 1) * 32 * 4 * 4;
constexpr int kStateBytes = 1024;
constexpr uint32_t kGridSpinLimit = 1u << 21;

struct ChainParams {
    ChainLayer layer[TBL_MAX_CHAIN];
    int count, rows;
    const float* x;        // [rows, K_0]
    float* y;              // [rows, N_last]
    float* act_base;       // activations between layers: buffer l holds layer l's output, [rows, width], all-ones bits at launch
    size_t act_stride;
    unsigned* sync;        // [count][16]: word 0 = strips of the layer that have arrived, counted up from 0xffffffff
                           // (the launch's memset fills counters and activation buffers with the same byte)
    int ks, stage_shift, stages, slots_max, acts_bytes;
    int* status;
    unsigned long long* trace;   // profiling aid: [cta][layer][8] nanosecond stamps, or null
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 10, %0;" ::"r"(kT) : "memory"); }

// Shared-memory state of the consumer warps.  The per-row scale and code sum are double-buffered by layer parity:
// the epilogue warps of layer l may still read theirs while the quantiser of layer l+1 fills the other copy.
struct ConsumerState {
    float scale[2][kMaxRows];
    int qsum[2][kMaxRows];
    float red[kConsumers * kMaxRows];
    uint32_t amax[kMaxRows];      // absmax reduction over the CTA's threads
    int ok;
};
static_assert(sizeof(ConsumerState) <= kStateBytes, "consumer state must fit its slot");

// Per-token absmax quantiser of rows*K <= 16384 inputs into the resident interleaved shared-memory copy; same
// arithmetic as the stand-alone quantiser.  `sync` != null: x is the previous layer's output; its strips have all
// been issued when that layer's arrival counter reaches `target`, and each loaded word tells whether it has landed.
// Returns false when a bounded wait gave up (status word set).
template <bool SINGLE>
__device__ __forceinline__ bool quantise_resident(const float* __restrict__ x, const int R, const int K,
                                                  const bool rms_fast, const float q_max, const unsigned* sync,
                                                  const unsigned target, const bool first_layer, const int par,
                                                  uint8_t* acts_resident, ConsumerState* cs, int* status,
                                                  unsigned long long* trace, const bool paired) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_groups = R * K / 16;
    constexpr int kRows = SINGLE ? 1 : kMaxRows;
    if (threadIdx.x < kMaxRows) {
        cs->qsum[par][threadIdx.x] = 0;
        cs->amax[threadIdx.x] = 0u;
    }
    if (sync) {
        if (threadIdx.x == 0) {
            bool ok = false;
            for (uint32_t spin = 0; spin < kGridSpinLimit; ++spin) {
                // the counter starts at 0xffffffff.  The loads start once three quarters of the strips have arrived:
                // they validate themselves, so the rest of the row can land while they are in flight and only the
                // groups that were too early are fetched again (measured: start at 0 / 1/4 / 1/2 / 3/4 / all arrived
                // = 13.86 / 13.60 / 13.46 / 13.45 / 13.72 us per layer)
                if (ld_acquire_gpu(sync) + 1u >= target - target / 4) { ok = true; break; }
            }
            if (!ok) { atomicOr(status, TBL_DEV_WAIT_TIMEOUT); cs->ok = 0; }
        }
        bar_consumers();     // every consumer warp has left the previous layer; zeroed sums and maxima visible
        if (*reinterpret_cast<volatile int*>(&cs->ok) == 0) return false;
    }
    if (trace && threadIdx.x == 0) trace[1] = global_ns();
    float4 xv[kGroups][4];
    int grow[kGroups];
#pragma unroll
    for (int i = 0; i < kGroups; ++i) {
        const int Gl = threadIdx.x + i * kT;
        grow[i] = -1;
        if (Gl < total_groups) {
            const int e = Gl * 16;
            int row = 0;
            if (!SINGLE) {
#pragma unroll
                for (int m = 1; m < kMaxRows; ++m) row += e >= m * K ? 1 : 0;
            }
            grow[i] = row;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) xv[i][q4] = __ldcg(reinterpret_cast<const float4*>(x + e + 4 * q4));
        } else {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) xv[i][q4] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (sync) {
        // the writers do not fence: a value may still be on its way when the counter is complete.  The buffers start as
        // all-ones words (never a result: the writers replace that one NaN pattern), so a load validates itself.
        uint32_t pending = 0u;
#pragma unroll
        for (int i = 0; i < kGroups; ++i) pending |= grow[i] >= 0 ? 1u << i : 0u;
        for (uint32_t spin = 0; spin < kGridSpinLimit && pending; ++spin) {
#pragma unroll
            for (int i = 0; i < kGroups; ++i) {
                if (pending >> i & 1u) {
                    uint32_t least = 1u;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        least = min(least, ~__float_as_uint(xv[i][q4].x)); least = min(least, ~__float_as_uint(xv[i][q4].y));
                        least = min(least, ~__float_as_uint(xv[i][q4].z)); least = min(least, ~__float_as_uint(xv[i][q4].w));
                    }
                    if (least != 0u) {
                        pending &= ~(1u << i);
                    } else {
                        const int Gl = threadIdx.x + i * kT;
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) xv[i][q4] = __ldcg(reinterpret_cast<const float4*>(x + Gl * 16 + 4 * q4));
                    }
                }
            }
        }
        if (pending) { atomicOr(status, TBL_DEV_WAIT_TIMEOUT); cs->ok = 0; }
    }
    // first layer only: the producer warp starts queueing weight copies once these loads are in flight
    if (first_layer) asm volatile("bar.arrive 11, %0;" ::"r"(kT + 32) : "memory");
    if (!sync) bar_consumers();     // zeroed sums visible (later layers passed a barrier above)
    if (trace && threadIdx.x == 0) {
        asm volatile("" ::"f"(xv[kGroups - 1][3].w), "f"(xv[0][0].x));
        trace[7] = global_ns();
    }
    float inv[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) inv[m] = 1.0f;
    if (rms_fast) {
        float ss[kRows];
#pragma unroll
        for (int m = 0; m < kRows; ++m) ss[m] = 0.0f;
#pragma unroll
        for (int i = 0; i < kGroups; ++i) {
            float q = 0.0f;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                q += xv[i][q4].x * xv[i][q4].x + xv[i][q4].y * xv[i][q4].y + xv[i][q4].z * xv[i][q4].z + xv[i][q4].w * xv[i][q4].w;
#pragma unroll
            for (int m = 0; m < kRows; ++m) if (grow[i] == m) ss[m] += q;
        }
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
            if (m < R) {
#pragma unroll
                for (int o = 16; o; o >>= 1) ss[m] += __shfl_xor_sync(0xffffffffu, ss[m], o);
                if (lane == 0) cs->red[warp * kMaxRows + m] = ss[m];
            }
        }
        bar_consumers();
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
            if (m < R) {
                float r = cs->red[m];
                for (int w = 1; w < kConsumers; ++w) r += cs->red[w * kMaxRows + m];
                inv[m] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(r, static_cast<float>(K)), 1e-6f)));
            }
        }
#pragma unroll
        for (int i = 0; i < kGroups; ++i) {
            float f = 1.0f;
#pragma unroll
            for (int m = 0; m < kRows; ++m) if (grow[i] == m) f = inv[m];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                xv[i][q4].x = __fmul_rn(xv[i][q4].x, f); xv[i][q4].y = __fmul_rn(xv[i][q4].y, f);
                xv[i][q4].z = __fmul_rn(xv[i][q4].z, f); xv[i][q4].w = __fmul_rn(xv[i][q4].w, f);
            }
        }
    }
    float amax[kRows];
    {
        float mx[kRows];
#pragma unroll
        for (int m = 0; m < kRows; ++m) mx[m] = 0.0f;
#pragma unroll
        for (int i = 0; i < kGroups; ++i) {
            float q = 0.0f;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
                q = fmaxf(q, fmaxf(fmaxf(fabsf(xv[i][q4].x), fabsf(xv[i][q4].y)), fmaxf(fabsf(xv[i][q4].z), fabsf(xv[i][q4].w))));
#pragma unroll
            for (int m = 0; m < kRows; ++m) if (grow[i] == m) mx[m] = fmaxf(mx[m], q);
        }
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
            if (m < R) {
                const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(mx[m]));
                if (lane == 0 && wmax != 0u) atomicMax(&cs->amax[m], wmax);
            }
        }
        bar_consumers();
#pragma unroll
        for (int m = 0; m < kRows; ++m) amax[m] = m < R ? __uint_as_float(cs->amax[m]) : 0.0f;
    }
    int qsum[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) qsum[m] = 0;
#pragma unroll
    for (int i = 0; i < kGroups; ++i) {
        if (grow[i] >= 0) {
            const int m = grow[i];
            float am = amax[0];
#pragma unroll
            for (int r = 1; r < kRows; ++r) if (m == r) am = amax[r];
            const float scale = __fdiv_rn(q_max, __fadd_rn(am, 1e-8f));
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
                for (int r = 0; r < kRows; ++r) if (m == r) qsum[r] += s4;
            }
            const int e = (threadIdx.x + i * kT) * 16;
            const uint4 codes = transpose4x4_bytes(make_uint4(wds[0], wds[1], wds[2], wds[3]));
            if (SINGLE && paired) {
                // single-row order of the full-stage path: word j (plane j) of quarter x goes to 128-bit slot
                // 2 * (x >> 1) + (j >> 1), word 2 * (j & 1) + (x & 1)
                const int kb = e >> 8, r = e & 255, tq = r >> 6, xq = (r >> 4) & 3;
                uint32_t* dst = reinterpret_cast<uint32_t*>(acts_resident + kb * 256 + (xq >> 1) * 128 + tq * 16) + (xq & 1);
                dst[0] = codes.x;
                dst[2] = codes.y;
                dst[16] = codes.z;
                dst[18] = codes.w;
            } else {
                *reinterpret_cast<uint4*>(acts_resident + qp_offset(m, R, K, e - m * K)) = codes;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
        if (m < R) {
            const int wsum = __reduce_add_sync(0xffffffffu, qsum[m]);
            if (lane == 0 && wsum != 0) atomicAdd(&cs->qsum[par][m], wsum);
        }
    }
    if (static_cast<int>(threadIdx.x) < R) {
        float am = amax[0];
#pragma unroll
        for (int r = 1; r < kRows; ++r) if (static_cast<int>(threadIdx.x) == r) am = amax[r];
        cs->scale[par][threadIdx.x] = __fdiv_rn(__fadd_rn(am, 1e-8f), q_max);
    }
    bar_consumers();
    return true;
}

__global__ void __launch_bounds__((kConsumers + 1) * 32, 1)
gemv_chain_kernel(const __grid_constant__ ChainParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk_stage = P.ks >> 8;
    const int stage_bytes = P.slots_max * nblk_stage * 1024;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    int* reduce_buf = reinterpret_cast<int*>(smem + 128);
    ConsumerState* cs = reinterpret_cast<ConsumerState*>(smem + 128 + kReduceBytes);
    uint8_t* acts_resident = smem + 128 + kReduceBytes + kStateBytes;
    uint8_t* stage_base = acts_resident + P.acts_bytes;
    const uint32_t stage_base_addr = smem_u32(stage_base);
    const uint32_t acts_resident_addr = smem_u32(acts_resident);
    const int nstages = P.stages;
    const int G = static_cast<int>(gridDim.x), bid = static_cast<int>(blockIdx.x);
    const int R = P.rows;
    auto stamp = [&](int l, int slot_id) {
        if (P.trace) P.trace[(static_cast<size_t>(bid) * P.count + l) * 8 + slot_id] = global_ns();
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumers);
        }
        fence_mbar_init();
        fence_proxy_async();
        cs->ok = 1;
    }
    __syncthreads();

    const bool producer = warp == kConsumers;
    const int slot = warp / kWps, part = warp % kWps;
    const int g = lane >> 2, t = lane & 3;
    int aoff[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) aoff[x] = g * 256 + ((((x ^ (g & 1)) << 2) + t) << 4);

    // the producer holds its first copies back until the consumers' loads of x are in flight
    if (producer) asm volatile("bar.sync 11, %0;" ::"r"(kT + 32) : "memory");

    int it = 0;
    bool alive = true;
    for (int l = 0; l < P.count && alive; ++l) {
        const ChainLayer& L = P.layer[l];
        const int K = L.K, N = L.N;
        const int nstrips = (N + 15) >> 4;
        const int share_base = nstrips / G, share_rem = nstrips % G;
        const int s_begin = bid * share_base + min(bid, share_rem);
        const int s_end = s_begin + share_base + (bid < share_rem ? 1 : 0);
        const int share = share_base + (share_rem ? 1 : 0);                 // largest share of any CTA
        const int passes = (share + kSlots - 1) / kSlots;
        const int slots = passes ? (share + passes - 1) / passes : 1;
        const int nblk = K >> 8;
        const int ksteps = (nblk + nblk_stage - 1) >> P.stage_shift;
        const bool fast = R == 1 && nblk_stage == 8 && (K & 2047) == 0;
        const int par = l & 1;

        if (producer) {
            const uint64_t stream_policy = l2_evict_first_policy();
            for (int s = s_begin; s < s_end && alive;) {
                const int cnt = min(slots, s_end - s);
                const int local = s;
                s += cnt;
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
                    if (lane == 0) mbar_arrive_expect_tx(&full[st], static_cast<uint32_t>(cnt) * nb * 1024);
                    __syncwarp();
                    // the stage is one or two slabs of cnt adjacent strips: one contiguous copy per slab,
                    // laid out [slab][strip][block in slab]
                    const int slab = b0 >> 2;
                    if (lane < ((nb + 3) >> 2)) {
                        const int sl = slab + lane;
                        const int sbs = min(4, nblk - 4 * sl);
                        bulk_g2s_hint(wst + lane * cnt * 4096,
                                      L.strips + ((static_cast<size_t>(4) * sl * nstrips + static_cast<size_t>(local) * sbs) << 10),
                                      cnt * sbs * 1024, &full[st], stream_policy);
                    }
                }
            }
            continue;
        }

        // ---------------- consumer warps ----------------
        const float* xin = l == 0 ? P.x : P.act_base + static_cast<size_t>(l - 1) * P.act_stride;
        float* yout = l == P.count - 1 ? P.y : P.act_base + static_cast<size_t>(l) * P.act_stride;
        const bool has_work = s_begin < s_end;
        if (threadIdx.x == 0) stamp(l, 0);
        if (has_work) {
            unsigned long long* tr = P.trace ? P.trace + (static_cast<size_t>(bid) * P.count + l) * 8 : nullptr;
            const unsigned* sync = l > 0 ? P.sync + (l - 1) * 16 : nullptr;
            const unsigned target = l > 0 ? static_cast<unsigned>((P.layer[l - 1].N + 15) >> 4) : 0u;
            const bool ok = R == 1
                ? quantise_resident<true>(xin, R, K, L.rms_fast != 0, L.q_max, sync, target, l == 0, par, acts_resident,
                                          cs, P.status, tr, fast)
                : quantise_resident<false>(xin, R, K, L.rms_fast != 0, L.q_max, sync, target, l == 0, par, acts_resident,
                                           cs, P.status, tr, false);
            if (!ok) { alive = false; break; }
        } else if (l == 0) {
            asm volatile("bar.arrive 11, %0;" ::"r"(kT + 32) : "memory");
        }
        if (threadIdx.x == 0) stamp(l, 2);
        bool first_stage = true;

        for (int s = s_begin; s < s_end && alive;) {
            const int cnt = min(slots, s_end - s);
            const int local = s;
            s += cnt;
            const bool active = slot < cnt;
            int acc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;

            for (int ksi = 0; ksi < ksteps; ++ksi, ++it) {
                const int st = it % nstages;
                alive = mbar_wait_bounded(&full[st], (it / nstages) & 1, P.status);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                if (first_stage && threadIdx.x == 0) stamp(l, 3);
                first_stage = false;
                if (active) {
                    const int nb = min(nblk_stage, nblk - ksi * nblk_stage);
                    const uint32_t stage_addr = stage_base_addr + st * stage_bytes;
                    if (fast) {
                        // single row, full 2048-deep stage: blocks part, part+2 of both slabs with constant
                        // offsets; the loads of a block are issued ahead of the arithmetic of the block before it
                        const uint32_t w0 = stage_addr + lane * 16 + (slot * 4 + part) * 1024;
                        const uint32_t w1 = w0 + cnt * 4096;
                        const uint32_t a0 = acts_resident_addr + t * 16 + (ksi * 8 + part) * 256;
                        struct Operands { uint4 lo, hi, b[4]; };
                        auto load_block = [&](const uint32_t wblk, const uint32_t ablk) {
                            Operands o;
                            o.lo = lds128(wblk);
                            o.hi = lds128(wblk + 512);
#pragma unroll
                            for (int x = 0; x < 4; ++x) o.b[x] = lds128(ablk + x * 64);
                            return o;
                        };
                        // One row: seven of an MMA's eight columns would be idle, and its 8 issues per block cost the
                        // tensor pipe as much as 32 dp4a cost the FMA pipe (measured: 14.3 against 14.8 us per layer).
                        // Each lane takes the dot products of its own 16-byte chunks (row g and row g + 8, 64 weights
                        // each) with the matching 64 codes, plane by plane; the four lanes of a row meet once per layer
                        // (shuffles below).  acc[p][0] / acc[p][2] are the plane-p sums of row g / g + 8, where the
                        // MMA form of the multi-row path keeps column 0 of the same rows.  The codes of plane p of
                        // quarter x sit in 128-bit slot 2 * (x >> 1) + (p >> 1), word 2 * (p & 1) + (x & 1) (the
                        // paired order the quantiser writes for these layers; with the plain order -- word p of slot
                        // x -- the same loop compiles to a schedule that is 3 % slower).
                        auto mma_block = [&](const Operands& o) {
                            const uint32_t lw[4] = {o.lo.x, o.lo.y, o.lo.z, o.lo.w};
                            const uint32_t hw[4] = {o.hi.x, o.hi.y, o.hi.z, o.hi.w};
#pragma unroll
                            for (int x = 0; x < 4; ++x) {
#pragma unroll
                                for (int pl = 0; pl < 4; ++pl) {
                                    const uint4& q = o.b[(x >> 1) * 2 + (pl >> 1)];
                                    const int idx = (pl & 1) * 2 + (x & 1);
                                    const uint32_t a = idx == 0 ? q.x : (idx == 1 ? q.y : (idx == 2 ? q.z : q.w));
                                    const uint32_t mk = 0x03030303u << (2 * pl);
                                    acc[pl][0] = dp4a_su(static_cast<int>(a), lw[x] & mk, acc[pl][0]);
                                    acc[pl][2] = dp4a_su(static_cast<int>(a), hw[x] & mk, acc[pl][2]);
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
                    } else {
                        // stage layout [slab][strip][block in slab]; this warp takes the blocks of its parity
                        const uint32_t ast = acts_resident_addr + ksi * nblk_stage * R * 256;
                        const uint32_t astep = kWps * R * 256;
                        for (int sl = 0; 4 * sl < nb; ++sl) {
                            const int sbs = min(4, nb - 4 * sl);
                            const uint32_t wslab = stage_addr + lane * 16 + sl * cnt * 4096 + (slot * sbs + part) * 1024;
                            uint32_t ablk = ast + (4 * sl + part) * R * 256;
#pragma unroll
                            for (int i = 0; i < 4 / kWps; ++i) {
                                if (part + i * kWps < sbs) {
                                    const uint32_t wblk = wslab + i * kWps * 1024;
                                    const uint4 lo = lds128(wblk);
                                    const uint4 hi = lds128(wblk + 512);
                                    const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w};
                                    const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                                    for (int xp = 0; xp < 2; ++xp) {
                                        const uint4 B0 = lds128(ablk + aoff[2 * xp]);
                                        const uint4 B1 = lds128(ablk + aoff[2 * xp + 1]);
                                        const uint32_t b0[4] = {B0.x, B0.y, B0.z, B0.w};
                                        const uint32_t b1[4] = {B1.x, B1.y, B1.z, B1.w};
#pragma unroll
                                        for (int j = 0; j < 4; ++j) {
                                            const uint32_t mk = 0x03030303u << (2 * j);
                                            mma_u8s8(acc[j], lw[2 * xp] & mk, hw[2 * xp] & mk, lw[2 * xp + 1] & mk,
                                                     hw[2 * xp + 1] & mk, b0[j], b1[j]);
                                        }
                                    }
                                }
                                ablk += astep;
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[st]);
            }
            if (!alive) break;
            if (threadIdx.x == 0) stamp(l, 4);

            if (active) {
                if (fast) {
                    // the four lanes of a row (t = 0..3) hold the sums of their quarters of every k-block
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            int v = acc[j][e];
                            v += __shfl_xor_sync(0xffffffffu, v, 1);
                            v += __shfl_xor_sync(0xffffffffu, v, 2);
                            acc[j][e] = v;
                        }
                    }
                }
                // exact recombination of the 4^j-scaled partial sums, then the two warps of a strip meet
                int tot[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) tot[e] = acc[0][e] + (acc[1][e] >> 2) + (acc[2][e] >> 4) + (acc[3][e] >> 6);
                int* mine = reduce_buf + (slot * 32 + lane) * 4;
                if (part > 0) *reinterpret_cast<int4*>(mine) = make_int4(tot[0], tot[1], tot[2], tot[3]);
                asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * kWps) : "memory");
                if (part == 0) {
                    const int4 v = *reinterpret_cast<const int4*>(mine);
                    tot[0] += v.x; tot[1] += v.y; tot[2] += v.z; tot[3] += v.w;
                }
                // the buffer is reused by the next pass: the reader must be done before the writer returns
                asm volatile("bar.sync %0, %1;" ::"r"(1 + slot), "r"(32 * kWps) : "memory");
                if (part == 0) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int n = (local + slot) * 16 + g + 8 * h;
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int m = 2 * t + c;
                            if (n < N && m < R) {
                                const int total = tot[2 * h + c] - cs->qsum[par][m];
                                float v = epilogue(total, __fmul_rn(cs->scale[par][m], L.weight_scale), L.magnitude, L.bias, n);
                                if (L.squared_relu) { v = fmaxf(v, 0.0f); v = __fmul_rn(v, v); }
                                if (__float_as_uint(v) == 0xffffffffu) v = __uint_as_float(0x7fffffffu);
                                yout[static_cast<size_t>(m) * N + n] = v;
                            }
                        }
                    }
                    if (l + 1 < P.count) {
                        // layer boundary, per strip: count the strip as arrived (no fence: the readers validate)
                        __syncwarp();
                        if (lane == 0) atomicAdd(P.sync + l * 16, 1u);
                    }
                }
            }
        }
        if (!alive) break;
        if (threadIdx.x == 0) stamp(l, 5);
    }
}

struct DeviceInfo {
    bool known;
    int sms;
    int cooperative;
};

DeviceInfo device_info() {
    static DeviceInfo info[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DeviceInfo{false, 0, 0};
    if (!info[dev].known) {
        int sms = 0, coop = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DeviceInfo{false, 0, 0};
        if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) return DeviceInfo{false, 0, 0};
        if (cudaFuncSetAttribute(gemv_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
            return DeviceInfo{false, 0, 0};
        info[dev] = DeviceInfo{true, sms, coop};
    }
    return info[dev];
}

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

unsigned long long* g_chain_trace = nullptr;
size_t g_chain_trace_bytes = 0;

}  // namespace

void set_chain_trace(void* buffer, size_t bytes) {
    g_chain_trace = static_cast<unsigned long long*>(buffer);
    g_chain_trace_bytes = buffer ? bytes : 0;
}

bool gemv_chain_supported(const ChainLayer* layers, int count, int rows) {
    if (!layers || count < 1 || count > TBL_MAX_CHAIN || rows < 1 || rows > kMaxRows) return false;
    for (int l = 0; l < count; ++l) {
        if (!layers[l].strips || !gemv_strip_supported(layers[l].K) || layers[l].N < 1) return false;
        if (static_cast<long long>(rows) * layers[l].K > 16384) return false;
        if (l > 0 && layers[l].K != layers[l - 1].N) return false;
    }
    return true;
}

namespace {
// [sync words | two activation buffers]
struct ChainScratch {
    size_t sync_bytes, act_bytes, total;
};
ChainScratch chain_scratch(const ChainLayer* layers, int count, int rows) {
    size_t width = 0;
    for (int l = 0; l + 1 < count; ++l) width = static_cast<size_t>(layers[l].N) > width ? layers[l].N : width;
    ChainScratch c{};
    c.sync_bytes = round_up(static_cast<size_t>(count) * 16 * sizeof(unsigned), 256);
    c.act_bytes = round_up(static_cast<size_t>(rows) * width * sizeof(float), 256);
    c.total = c.sync_bytes + static_cast<size_t>(count) * c.act_bytes;
    return c;
}
}  // namespace

size_t gemv_chain_workspace_bytes(const ChainLayer* layers, int count, int rows) {
    return chain_scratch(layers, count, rows).total;
}

cudaError_t launch_gemv_chain(const ChainLayer* layers, int count, int rows, const float* x, float* y,
                              void* workspace, cudaStream_t stream) {
    if (!gemv_chain_supported(layers, count, rows)) return cudaErrorInvalidValue;
    const DeviceInfo info = device_info();
    if (!info.known || !info.cooperative || info.sms < 1) return cudaErrorNotSupported;
    ChainParams P{};
    P.count = count;
    P.rows = rows;
    P.x = x;
    P.y = y;
    P.status = device_status_ptr();
    if (!P.status) return cudaErrorUnknown;
    int max_k = 0, max_strips = 0;
    for (int l = 0; l < count; ++l) {
        P.layer[l] = layers[l];
        max_k = layers[l].K > max_k ? layers[l].K : max_k;
        const int ns = (layers[l].N + 15) / 16;
        max_strips = ns > max_strips ? ns : max_strips;
    }
    const int grid = max_strips < info.sms ? max_strips : info.sms;
    P.trace = g_chain_trace_bytes >= static_cast<size_t>(grid) * count * 8 * sizeof(unsigned long long) ? g_chain_trace : nullptr;
    // one ring geometry for the whole stack: the deepest stage and the widest pass of any layer
    P.ks = max_k >= 2048 ? 2048 : 1024;
    P.stage_shift = P.ks == 2048 ? 3 : 2;
    P.slots_max = 1;
    for (int l = 0; l < count; ++l) {
        const int ns = (layers[l].N + 15) / 16;
        const int share = (ns + grid - 1) / grid;
        const int passes = (share + kSlots - 1) / kSlots;
        const int slots = (share + passes - 1) / passes;
        P.slots_max = slots > P.slots_max ? slots : P.slots_max;
    }
    P.acts_bytes = static_cast<int>(round_up(static_cast<size_t>(rows) * max_k, 128));
    const size_t stage_bytes = static_cast<size_t>(P.slots_max) * (P.ks / 256) * 1024;
    // slack after the last stage: lanes of activation rows >= rows read (and ignore) stale bytes
    const size_t fixed = 128 + kReduceBytes + kStateBytes + P.acts_bytes + 2048;
    const size_t room = 227 * 1024 - fixed;
    P.stages = static_cast<int>(room / stage_bytes < static_cast<size_t>(kMaxStages) ? room / stage_bytes : kMaxStages);
    if (P.stages < 2) return cudaErrorInvalidValue;
    const size_t smem = fixed + P.stages * stage_bytes;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const ChainScratch sc = chain_scratch(layers, count, rows);
    P.sync = reinterpret_cast<unsigned*>(ws);
    P.act_base = reinterpret_cast<float*>(ws + sc.sync_bytes);
    P.act_stride = sc.act_bytes / sizeof(float);
    // arrival counters and activation buffers start as all-ones words
    cudaError_t e = cudaMemsetAsync(ws, 0xff, sc.sync_bytes + static_cast<size_t>(count > 1 ? count - 1 : 0) * sc.act_bytes, stream);
    if (e != cudaSuccess) return e;

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((kConsumers + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1]{};
    attrs[0].id = cudaLaunchAttributeCooperative;     // CTAs wait on one another: they must be co-resident
    attrs[0].val.cooperative = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, gemv_chain_kernel, P);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace tbl
