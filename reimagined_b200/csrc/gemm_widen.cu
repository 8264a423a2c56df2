// Mid-size batches (up to 128 rows per pass) on the 2-bit weights: the words are widened to bytes INSIDE the
// kernel and multiplied on the 5th-generation tensor cores, so the weights cross HBM once at two bits each and
// the multiply-accumulate work leaves the SM's issue slots.  The weights are read in the strip-major layout of
// the decode GEMV (gemv_strip.cu): a tile's share of a 1024-deep slab is one contiguous run of memory, fetched
// with one bulk copy (a 2-D box over the row-major words costs one 128-byte DRAM access per row and k-block and
// ran at a third of the rate).
//
// y[m, n] = epilogue(sum_k t[n, k] * q[m, k]),  t = code - 1.  "Swap-AB": a tile is 128 weight rows (the MMA's
// M dimension, the accumulator's TMEM lanes) x all activation rows (the MMA's N dimension, padded to 16).
//
// Widening without shifts: a canonical word holds 16 codes, code i at bits 2i.  (word & (0x03030303 << 2p)) is
// the byte vector 4^p * code of weights {p, 4+p, 8+p, 12+p} of that word -- one AND per four weights.  Per
// k-block of 512 weights a weight row is 32 words; plane p of the block is the 128-byte row made of its 32
// masked words, i.e. one 128-byte-swizzle row of a tcgen05 A operand (unsigned 8-bit).  The activations are
// laid out to match (plane-major inside each 512-block: byte 4g + e of plane p is element 16g + 4e + p), and
// each plane accumulates into its own TMEM columns, so the 4^p scale is taken out exactly with shifts in the
// epilogue; the "-1" of the code is removed there too by subtracting sum_k q[m, k].
//
// One persistent CTA per SM, eleven warps:
//   warp 0     weight producer: per slab (two k-blocks) one bulk copy of the tile's 8 strips x 4 KB into a ring of
//              two raw stages (a stage is free again as soon as the widen warps hold its words in registers)
//   warp 1     MMA issuer (one lane): per half k-block (two planes) 8 x tcgen05.mma kind::i8 (u8 x s8 -> s32,
//              M = 128, N = n_pad, K = 32); owns the TMEM allocation
//   warp 2     activation producer: per half k-block two TMA boxes [n_pad rows x 128 B] (L2-resident) into a ring
//              of 2 (n_pad = 128) to 16 slots
//   warps 3-10 widen: warp w owns strip w of the tile; per k-block it reads the strip's two 1 KB blocks as four
//              512-byte half-blocks (lane = 4g + t holds the 16-byte chunk t of row g or g + 8) and writes the
//              planes of each chunk into a ring of three A buffers of two planes (conflict-free 128-bit shared
//              accesses both ways), fences them for the async proxy and arrives; after the last k-block of a tile the same
//              warps run the epilogue (tcgen05.ld, exact recombination, two-scale epilogue, coalesced stores
//              along n)
// Every wait is bounded: on a timeout the role records the status word and falls through to the common exit,
// where TMEM is released.  The kernel is launched as a programmatic dependent of the kernel before it (the row
// quantiser): weights are fetched and widened while that kernel still runs; only the activation producer and the
// epilogue wait for it.
//
// Measured (16384 x 16384, B200): 41 us per pass for any batch up to 64 rows (tensor pipe 42 % busy).  An MMA of this shape
// lasts 46 cycles for any N <= 64, so the 96 KB of widened planes that fit hold only ~1 100 cycles of tensor work,
// less than the round trip commit -> widen warps wake -> stores -> arrive -> issue that recycles a buffer: the
// kernel is bound by that loop, not by HBM (10 us), the widening (ALU 4 us) or the MMAs (12 us).  Neither the
// proxy fence nor the stores themselves matter (same time with both removed); a deeper activation ring does not
// help, a shallower A ring costs 6 us.  It beats the mma.sync strip kernel from 33 rows up (64 rows: 48 vs 65 us).
#include "common.cuh"
#include "kernels.cuh"
#include "tc05.cuh"

namespace tbl {
namespace {

using namespace tc05;

constexpr int kWidenWarps = 8;
constexpr int kWidenThreads = 32 * (3 + kWidenWarps);
constexpr int kBlockK = 512;                 // weights of K per k-block
constexpr int kRawBytes = 8 * 4096;          // one slab of a tile: 8 strips x 4 blocks of 1 KB
constexpr int kPlaneBytes = 128 * 128;       // one widened plane of a k-block
constexpr int kMaxNpad = 128;
constexpr int kRawStages = 2;
constexpr int kAStages = 3;                  // A buffers of two planes (half a k-block)
constexpr int kAHalfBytes = 2 * kPlaneBytes;
constexpr int kMaxBStages = 16;              // activation boxes of two planes: as many as fit kBRingBytes (2 at n_pad = 128)
constexpr int kBRingBytes = 64 * 1024;
constexpr int kNumSmW = 148;

struct WidenTiles {            // one weight matrix of the launch
    const uint8_t* strips;     // strip-major weights
    const float* magnitude;
    const float* bias;
    float* y;
    float weight_scale;
    int N, nstrips;
    int tile0;                 // its first tile in a row pass's tile list (128 weight rows per tile)
    int squared_relu;
    const int32_t* rows_dev;   // device row count of this matrix (null: the launch's M)
    const int32_t* offset_dev; // device index of its first row in the codes / scales / sums / y (null: 0)
};

struct WidenParams {
    const float* act_scales;
    const int32_t* q_sums;
    WidenTiles view[kWidenMaxViews];
    int views;
    int M, K, n_pad, kblocks;
    int tiles;                 // row_passes x tiles_per_pass
    int tiles_per_pass;        // weight-row tiles of all the views
    int* status;
};

// One unit of work: 128 weight rows of one view times one pass of up to 128 activation rows.  The tile list is
// pass-major (every view's first 128 rows come first), so the passes that device-side row counts leave empty are
// at its end.
struct WidenTile {
    int view;
    int wtile;                 // tile of 128 weight rows inside the view
    int row0;                  // first activation row (index into the codes / scales / sums / y)
    int rows;                  // activation rows of this pass; <= 0: nothing to do
};

__device__ __forceinline__ WidenTile decode_widen_tile(const WidenParams& p, int tile) {
    const int pass = tile / p.tiles_per_pass, t = tile - pass * p.tiles_per_pass;
    int v = 0;
    while (v + 1 < p.views && t >= p.view[v + 1].tile0) ++v;
    const WidenTiles& vw = p.view[v];
    const int total = vw.rows_dev ? __ldg(vw.rows_dev) : p.M;
    const int base = vw.offset_dev ? __ldg(vw.offset_dev) : 0;
    WidenTile w;
    w.view = v; w.wtile = t - vw.tile0; w.row0 = base + pass * kMaxNpad;
    w.rows = min(kMaxNpad, total - pass * kMaxNpad);
    return w;
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Row-major codes q[M, K] -> plane-major qw[M, K_pad] (K_pad a multiple of 512, zero past K): inside each block of
// 512 elements, byte 4g + e of plane p (128 bytes per plane) is element 16g + 4e + p -- a 4x4 byte transpose of
// every 16-element group, its four words going to the four planes.
__global__ void permute_planes_kernel(const int8_t* __restrict__ q, int M, int K, int K_pad, int8_t* __restrict__ qw) {
    const int groups_per_row = K_pad >> 4;
    const long long total = static_cast<long long>(M) * groups_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int m = static_cast<int>(i / groups_per_row), gg = static_cast<int>(i - static_cast<long long>(m) * groups_per_row);
        const int kb = gg >> 5, g = gg & 31;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (gg * 16 < K) v = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(m) * K + gg * 16);
        const uint4 t = transpose4x4_bytes(v);
        uint32_t* dst = reinterpret_cast<uint32_t*>(qw + static_cast<size_t>(m) * K_pad + kb * kBlockK) + g;
        dst[0] = t.x;
        dst[32] = t.y;
        dst[64] = t.z;
        dst[96] = t.w;
    }
}

__global__ void __launch_bounds__(kWidenThreads, 1)
gemm_widen_kernel(const __grid_constant__ CUtensorMap map_q, const WidenParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_buf = smem;                                           // kAStages x 32 KB
    uint8_t* raw_buf = a_buf + kAStages * kAHalfBytes;               // kRawStages x 32 KB
    uint8_t* b_buf = raw_buf + kRawStages * kRawBytes;               // b_stages x (2 planes x n_pad x 128 B)
    uint64_t* raw_full = reinterpret_cast<uint64_t*>(b_buf + kBRingBytes);
    uint64_t* raw_empty = raw_full + kRawStages;
    uint64_t* a_full = raw_empty + kRawStages;
    uint64_t* a_empty = a_full + kAStages;
    uint64_t* b_full = a_empty + kAStages;
    uint64_t* b_empty = b_full + kMaxBStages;
    uint64_t* tmem_full = b_empty + kMaxBStages;
    uint64_t* tmem_empty = tmem_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tmem_cols = p.n_pad > 64 ? 512u : 256u;      // 4 planes x n_pad columns, a power of two
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRawStages; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], kWidenWarps); }
        for (int s = 0; s < kAStages; ++s) { mbar_init(&a_full[s], kWidenWarps); mbar_init(&a_empty[s], 1); }
        for (int s = 0; s < kMaxBStages; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, kWidenWarps);
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n_pad = p.n_pad;
    const int b_stage_bytes = 2 * n_pad * 128;
    const int b_stages = min(kMaxBStages, kBRingBytes / b_stage_bytes);

    if (warp == 0) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            const uint64_t policy = l2_evict_first_policy();
            const int nblk = p.K >> 8;                       // 1 KB blocks of 256 weights per strip
            const int slabs = (nblk + 3) >> 2;
            int it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < p.tiles; tile += gridDim.x) {
                const WidenTile wt = decode_widen_tile(p, tile);
                if (wt.rows <= 0) continue;
                const WidenTiles& vw = p.view[wt.view];
                const int first = wt.wtile * 8, cnt = min(8, vw.nstrips - first);
                for (int sl = 0; sl < slabs; ++sl, ++it) {
                    const int s = it % kRawStages;
                    if (it >= kRawStages) {
                        alive = mbar_wait_bounded(&raw_empty[s], ((it / kRawStages) - 1) & 1, p.status);
                        if (!alive) break;
                    }
                    const int sbs = min(4, nblk - 4 * sl);
                    const uint32_t bytes = static_cast<uint32_t>(cnt) * sbs * 1024;
                    mbar_arrive_expect_tx(&raw_full[s], bytes);
                    bulk_g2s_hint(raw_buf + s * kRawBytes,
                                  vw.strips + ((static_cast<size_t>(4) * sl * vw.nstrips + static_cast<size_t>(first) * sbs) << 10), bytes,
                                  &raw_full[s], policy);
                }
            }
        }
    } else if (warp == 2) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            int hs = 0;
            bool alive = true;
            const uint32_t tx = 2u * n_pad * 128u;
            pdl_wait();                          // the codes come from the kernel before this one
            for (int tile = blockIdx.x; alive && tile < p.tiles; tile += gridDim.x) {
                const WidenTile wt = decode_widen_tile(p, tile);
                if (wt.rows <= 0) continue;
                for (int kh = 0; kh < 2 * p.kblocks; ++kh, ++hs) {
                    const int s = hs % b_stages;
                    if (hs >= b_stages) {
                        alive = mbar_wait_bounded(&b_empty[s], ((hs / b_stages) - 1) & 1, p.status);
                        if (!alive) break;
                    }
                    uint8_t* dst = b_buf + s * b_stage_bytes;
                    mbar_arrive_expect_tx(&b_full[s], tx);
                    const int x0 = (kh >> 1) * kBlockK + (kh & 1) * 256;
                    // rows past the pass's own (another view's, or past the end: zero-filled) are multiplied and ignored
                    tma_load_2d(dst, &map_q, x0, wt.row0, &b_full[s]);
                    tma_load_2d(dst + n_pad * 128, &map_q, x0 + 128, wt.row0, &b_full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // kind::i8: D = s32, A = unsigned 8-bit (scaled codes), B = signed 8-bit, both K-major, N = n_pad, M = 128
            const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(n_pad >> 3) << 17) | (8u << 24);
            // An MMA of this shape lasts 46 cycles, about as long as one thread needs to build two descriptors from
            // scratch: the descriptors of the ring slots are formed once, a k-step only adds its byte offset (>> 4;
            // the address field cannot carry out of its 14 bits inside the CTA's shared memory).
            const uint64_t a_desc0 = smem_desc_sw128(smem_u32(a_buf)), b_desc0 = smem_desc_sw128(smem_u32(b_buf));
            const uint32_t b_plane = static_cast<uint32_t>(n_pad) * 128u >> 4;
            int hs = 0, local = 0;
            bool alive = true;
            for (int tile = blockIdx.x; alive && tile < p.tiles; tile += gridDim.x) {
                if (decode_widen_tile(p, tile).rows <= 0) continue;
                if (local >= 1) {
                    alive = mbar_wait_bounded(tmem_empty, (local - 1) & 1, p.status);
                    if (!alive) break;
                }
                ++local;
                tc_fence_after();
                for (int kh = 0; kh < 2 * p.kblocks; ++kh, ++hs) {
                    const int sa = hs % kAStages, sb = hs % b_stages;
                    alive = mbar_wait_bounded(&b_full[sb], (hs / b_stages) & 1, p.status) &&
                            mbar_wait_bounded(&a_full[sa], (hs / kAStages) & 1, p.status);
                    if (!alive) break;
                    tc_fence_after();
                    const uint64_t ad = a_desc0 + static_cast<uint32_t>(sa * (kAHalfBytes >> 4));
                    const uint64_t bd = b_desc0 + static_cast<uint32_t>(sb * (b_stage_bytes >> 4));
                    const uint32_t d0 = tmem_base + (kh & 1) * 2 * n_pad;
                    const uint32_t first = (kh >> 1) != 0 ? 1u : 0u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            umma_i8(d0 + h * n_pad, ad + (h * (kPlaneBytes >> 4) + kk * 2), bd + (h * b_plane + kk * 2), idesc,
                                    kk != 0 ? 1u : first);
                        }
                    }
                    umma_commit(&a_empty[sa]);      // the widened planes may be overwritten once these MMAs have read them
                    umma_commit(&b_empty[sb]);      // ... and the activation boxes
                }
                if (alive) umma_commit(tmem_full);
            }
        }
    } else {
        // ---------------- widen warps, then epilogue ----------------
        const int ws = warp - 3;                    // strip of the tile this warp widens
        const int quarter = warp & 3;               // TMEM lanes 32*quarter .. +31 are this warp's
        const int ehalf = (warp - 3) >> 2;          // which of the two warps of the quarter
        const int g = lane >> 2, t = lane & 3;
        const int nblk = p.K >> 8;
        int it = 0, sit = 0, local = 0;             // k-blocks and slabs consumed so far
        bool alive = true;
        for (int tile = blockIdx.x; alive && tile < p.tiles; tile += gridDim.x) {
            const WidenTile wt = decode_widen_tile(p, tile);
            if (wt.rows <= 0) continue;
            for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                const int sl = kb >> 1, sbs = min(4, nblk - 4 * sl);
                const int s = sit % kRawStages;
                if ((kb & 1) == 0) alive = mbar_wait_bounded(&raw_full[s], (sit / kRawStages) & 1, p.status);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                // half-block (block bi of this k-block, rows g or g + 8): 32 lanes x 16 bytes, contiguous
                const uint32_t raw = smem_u32(raw_buf + s * kRawBytes) + ws * sbs * 1024 + (kb & 1) * 2048 + lane * 16;
                uint4 src[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) src[i] = lds128(raw + (i >> 1) * 1024 + (i & 1) * 512);
                const bool slab_done = (kb & 1) == 1 || 2 * (kb + 1) >= sbs + 4 * sl;
                if (slab_done) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&raw_empty[s]);      // the slab's words are in registers
                    ++sit;
                }
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    const int hs = 2 * it + h2, sa = hs % kAStages;
                    if (hs >= kAStages) alive = mbar_wait_bounded(&a_empty[sa], ((hs / kAStages) - 1) & 1, p.status);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    const uint32_t abase = smem_u32(a_buf + sa * kAHalfBytes);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        // src[i]: block i >> 1 of the k-block, rows g + 8 * (i & 1); chunk (i >> 1) * 4 + t of the 128-byte row
                        const int row = ws * 16 + (i & 1) * 8 + g, c = (i >> 1) * 4 + t;
                        const uint32_t dst = abase + row * 128 + ((c ^ (row & 7)) << 4);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t mk = 0x03030303u << (2 * (2 * h2 + h));
                            sts128(dst + h * kPlaneBytes, src[i].x & mk, src[i].y & mk, src[i].z & mk, src[i].w & mk);
                        }
                    }
                    fence_proxy_async();            // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[sa]);
                }
                if (!alive) break;
            }
            if (!alive) break;
            // epilogue of the tile: lane = weight row, columns = 4 planes x n_pad activation rows
            alive = mbar_wait_bounded(tmem_full, local & 1, p.status);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            tc_fence_after();
            pdl_wait();                          // scales and code sums come from the kernel before this one; y is written below
            ++local;
            const WidenTiles& vw = p.view[wt.view];
            const int n = wt.wtile * 128 + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            const float mag = (vw.magnitude && n < vw.N) ? __ldg(vw.magnitude + n) : 1.0f;
            const float bia = (vw.bias && n < vw.N) ? __ldg(vw.bias + n) : 0.0f;
            const float wscale = vw.weight_scale;
            const bool has_mag = vw.magnitude != nullptr, has_bias = vw.bias != nullptr, sq = vw.squared_relu != 0;
            float* yv = vw.y;
            const int N = vw.N;
            for (int m0 = ehalf * 16; m0 < n_pad; m0 += 32) {
                uint32_t d0[16], d1[16], d2[16], d3[16];
                tmem_ld16(t_row + m0, d0);
                tmem_ld16(t_row + n_pad + m0, d1);
                tmem_ld16(t_row + 2 * n_pad + m0, d2);
                tmem_ld16(t_row + 3 * n_pad + m0, d3);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = m0 + j;
                    if (m < wt.rows) {
                        const int row = wt.row0 + m;
                        // exact: plane p's sum is a multiple of 4^p
                        const int total = static_cast<int>(d0[j]) + (static_cast<int>(d1[j]) >> 2) + (static_cast<int>(d2[j]) >> 4) +
                                          (static_cast<int>(d3[j]) >> 6) - __ldg(p.q_sums + row);
                        float v = __fmul_rn(static_cast<float>(total), __fmul_rn(__ldg(p.act_scales + row), wscale));
                        if (has_mag) v = __fmul_rn(v, mag);
                        if (has_bias) v = __fadd_rn(v, bia);
                        if (sq) { v = fmaxf(v, 0.0f); v = __fmul_rn(v, v); }
                        if (n < N) yv[static_cast<size_t>(row) * N + n] = v;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_empty);
        }
    }

    // common exit: all roles meet, then the allocating warp releases TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

inline size_t round_up_w(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

bool gemm_widen_supported(int M, int K, int N) {
    return M >= 1 && M <= kMaxNpad && K >= 256 && (K & 255) == 0 && N >= 1;
}

int gemm_widen_plane_ld(int K) { return static_cast<int>(round_up_w(K, kBlockK)); }

size_t gemm_widen_scratch_bytes(int M, int K) {
    return round_up_w(static_cast<size_t>(M) * round_up_w(K, kBlockK), 256);
}

cudaError_t launch_gemm_widen(const WidenView* views, int count, const int8_t* q, int8_t* planes, const float* act_scales,
                              const int32_t* q_sums, int M, int K, cudaStream_t stream, const int32_t* rows_dev,
                              const int32_t* offsets_dev, int total_rows) {
    if (!views || count < 1 || count > kWidenMaxViews || !planes || M < 1) return cudaErrorInvalidValue;
    // device-side row counts (the experts of a MoE stage): view v multiplies rows offsets_dev[v] .. + rows_dev[v] of the
    // total_rows rows of codes, at most M of them, in passes of 128
    const bool counted = rows_dev != nullptr;
    if (counted ? (!offsets_dev || q || total_rows < 1) : M > kMaxNpad) return cudaErrorInvalidValue;
    const int pass_rows = M < kMaxNpad ? M : kMaxNpad;
    const int K_pad = gemm_widen_plane_ld(K);
    WidenParams p{};
    p.act_scales = act_scales; p.q_sums = q_sums; p.M = M; p.K = K; p.views = count;
    p.n_pad = (pass_rows + 15) & ~15;
    p.kblocks = K_pad / kBlockK;
    int tiles = 0;
    for (int v = 0; v < count; ++v) {
        if (!gemm_widen_supported(pass_rows, K, views[v].N) || !views[v].strips || !views[v].y) return cudaErrorInvalidValue;
        WidenTiles& t = p.view[v];
        t.strips = static_cast<const uint8_t*>(views[v].strips); t.magnitude = views[v].magnitude; t.bias = views[v].bias;
        t.y = views[v].y; t.weight_scale = views[v].weight_scale; t.N = views[v].N; t.nstrips = (views[v].N + 15) / 16;
        t.tile0 = tiles; t.squared_relu = views[v].squared_relu;
        t.rows_dev = counted ? rows_dev + v : nullptr;
        t.offset_dev = counted ? offsets_dev + v : nullptr;
        tiles += (views[v].N + 127) / 128;
    }
    p.tiles_per_pass = tiles;
    p.tiles = tiles * ((M + kMaxNpad - 1) / kMaxNpad);
    const int map_rows = counted ? total_rows : M;
    if (q) {
        const long long groups = static_cast<long long>(M) * (K_pad >> 4);
        const int grid = static_cast<int>((groups + 255) / 256 < 1184 ? (groups + 255) / 256 : 1184);
        permute_planes_kernel<<<grid, 256, 0, stream>>>(q, M, K, K_pad, planes);
        note_launch();
    }
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorUnknown;
    CUtensorMap mq;
    // the plane-major codes [rows, K_pad bytes], box 128 bytes x n_pad rows
    if (!make_map(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, planes, map_rows, K_pad, 128, p.n_pad)) return cudaErrorUnknown;
    const size_t smem = 1024 + kAStages * kAHalfBytes + kRawStages * kRawBytes + kBRingBytes + 512;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_widen_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int grid = p.tiles < kNumSmW ? p.tiles : kNumSmW;
    // Programmatic dependent launch: everything up to the first MMA -- TMEM allocation, the first weight slabs, the
    // first widened planes -- depends on nothing the kernel before this one writes, so it may run beside that
    // kernel's tail (the row quantiser releases its dependents at once); the activation producer and the epilogue
    // wait for its completion (pdl_wait).
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kWidenThreads); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_widen_kernel, mq, p);
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

}  // namespace tbl
