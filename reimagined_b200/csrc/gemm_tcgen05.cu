// Prefill GEMM: y[M,N] = epilogue(q[M,K] (int8) x w[N,K]^T (int8 ternary)) on the 5th-generation
// tensor cores.  tcgen05.mma kind::i8 (s8 x s8 -> s32), both operands K-major in shared memory in
// the 128-byte-swizzled canonical layout written by TMA, accumulators in tensor memory (TMEM).
//
// One persistent CTA per SM, ten warps:
//   warp 0    TMA producer: per k-block one box of q [128 rows x 128 B] and one of w [BN x 128 B]
//   warp 1    MMA issuer (one lane): 4 x tcgen05.mma (K = 32 each) per k-block, tcgen05.commit
//             releases the stage; also owns the TMEM allocation (512 columns = 2 accumulators)
//   warps 2-9 epilogue: tcgen05.ld the 128 x BN s32 tile (a TMEM lane quarter per warp pair), apply
//             float(acc) * (act_scale*weight_scale) [* magnitude] [+ bias], stage 32x32 fp32 blocks
//             in swizzled shared memory and write them with TMA stores (clipped at the edges)
// Grouped mode (GROUPED = true) runs a table of problems in one launch -- the expert stages of a
// mixture-of-experts block: problem g owns rows [offset[g], offset[g] + rows[g]) of the shared activation
// and output arrays and its own weight matrix (one tensor map each); the counts live on the device, so
// every role walks the same tile list derived from them, and the epilogue masks rows past a problem's
// end and stores rows with plain coalesced stores instead of box stores.
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1; the next
// block's tcgen05.ld is issued before the current block is converted and stored.
// Tall mode (MT = 2, large problems): a tile is 256 activation rows x 256 weight rows -- two M = 128 MMAs per
// k-step share one weight box, which cuts the operand bytes fetched through L2 per output by a third (the kernel
// is bound by that fetch at 8192-deep K, not by the tensor pipe).  The two accumulators then are the two halves
// of one tile: the epilogue of a tile overlaps the next tile's main loop only while its first half drains.
// Tiles are walked in groups of kGroupM row tiles x all column tiles, so that the tiles in flight at any time
// share a few activation and weight boxes in L2.
// Every wait is bounded: on a timeout the role records the status word and falls through to
// the common exit, where TMEM is released.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.cuh"
#include "tc05.cuh"

namespace tbl {
namespace {

constexpr int BM = 128;          // activation rows per tile (UMMA M)
constexpr int BK = 128;          // bytes of K per stage = one 128B swizzle atom
// ring depth: what fits beside the 32 KB of epilogue staging (narrow tiles get a deeper ring: with few
// rows the kernel streams weights and wants more bytes in flight per SM)
__host__ __device__ constexpr int stages_for(int bn, int mt = 1) { return mt == 2 ? 3 : (bn >= 256 ? 4 : (bn >= 128 ? 6 : 8)); }
constexpr int kGroupM = 16;      // row tiles per group of the tile walk
// Tall mode pays once every SM has a 256 x 256 tile and the k-loop is long enough to amortise the undoubled
// accumulator (measured: 1024 x 16384 x 16384 +13 %, 4096^3 +3 %, 8192 x 2048 x 2048 -1 %, 1024 x 4096 x 4096 -34 %).
__host__ inline bool tall_tiles_pay(long long tall_tiles, int K) {
    return tall_tiles >= 4 * 148 || (tall_tiles >= 148 && K >= 4096);
}
constexpr int kMaxStages = 8;
constexpr int kEpiWarps = 8;        // two warps per TMEM lane quarter, each taking every other 32-column block
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kNumSm = 148;

struct GemmParams {
    const float* act_scales;
    const float* magnitude;
    const float* bias;
    float* y;
    int32_t* acc_debug;
    float weight_scale;
    int M, K, N;
    int tiles_m, tiles_n;
    int use_tma_store;
    int* status;
    GemmScatter scatter;      // count > 0: tiles go to these arrays (plain 128-bit stores, peers included), not to y
};

// Grouped mode (mixture-of-experts stages): problem g multiplies rows [offset[g], offset[g] + rows[g]) of the
// shared activation / output arrays by its own weight matrix.  Row counts and offsets live on the device
// (they come from the routing kernel), so every role of the kernel derives the tile list from them itself.
struct GroupTable {
    CUtensorMap b[TBL_MAX_GROUPS];
    float weight_scale[TBL_MAX_GROUPS];
    const float* magnitude[TBL_MAX_GROUPS];
    const float* bias[TBL_MAX_GROUPS];
    const int* rows_dev;
    const int* offset_dev;
    int groups;
    int cap;              // host-side upper bound on the rows of any problem
    int squared_relu;
};
struct NoGroups {};

// Tile t of the launch -> (problem, first row in the shared arrays, rows left in the problem, n-tile).
template <bool GROUPED, int MT, typename Table>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, const Table& gt, int t, int& g, int& row0, int& rows,
                                            int& tn) {
    if constexpr (!GROUPED) {
        if (t >= p.tiles_m * p.tiles_n) return false;
        // groups of kGroupM row tiles; inside a group the row tile runs fastest, then the column tile
        const int per_group = kGroupM * p.tiles_n;
        const int grp = t / per_group, in_grp = t - grp * per_group;
        const int gm = min(kGroupM, p.tiles_m - grp * kGroupM);
        const int tm = grp * kGroupM + in_grp % gm;
        g = 0; tn = in_grp / gm; row0 = tm * (128 * MT); rows = p.M - row0;
        return true;
    } else {
        int base = 0;
        for (int e = 0; e < gt.groups; ++e) {
            const int r = min(__ldg(gt.rows_dev + e), gt.cap);
            const int tiles_m = (r + 127) >> 7;
            const int tiles = tiles_m * p.tiles_n;
            if (t < base + tiles) {
                const int local = t - base, tm = local % tiles_m;
                g = e; tn = local / tiles_m; row0 = __ldg(gt.offset_dev + e) + tm * 128; rows = r - tm * 128;
                return true;
            }
            base += tiles;
        }
        return false;
    }
}

using namespace tc05;


template <int BN, bool GROUPED, int MT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_y, const GemmParams p,
                    const __grid_constant__ std::conditional_t<GROUPED, GroupTable, NoGroups> gt) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment is required by the 128-byte swizzle pattern
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    static_assert(MT == 1 || (BN == 256 && !GROUPED), "tall tiles: 256 x 256, plain mode");
    constexpr int kStages = stages_for(BN, MT);
    constexpr int kABytes = MT * BM * BK;
    constexpr int kBBytes = BN * BK;
    constexpr int kStageBytes = kABytes + kBBytes;
    uint8_t* epi_stage = smem + kStages * kStageBytes;                 // 8 warps x 4 KB
    uint64_t* full = reinterpret_cast<uint64_t*>(epi_stage + kEpiWarps * 4096);
    uint64_t* empty = full + kMaxStages;
    uint64_t* tmem_full = empty + kMaxStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], kEpiWarps); }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int it = 0;
            bool alive = true;
            int g, row0, rows, tn;
            for (int tile = blockIdx.x; alive && decode_tile<GROUPED, MT>(p, gt, tile, g, row0, rows, tn); tile += gridDim.x) {
                const CUtensorMap* bmap = &map_b;
                if constexpr (GROUPED) bmap = &gt.b[g];
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (it >= kStages) {
                        alive = mbar_wait_bounded(&empty[s], ((it / kStages) - 1) & 1, p.status);
                        if (!alive) break;
                    }
                    uint8_t* a_dst = smem + s * kStageBytes;
                    uint8_t* b_dst = a_dst + kABytes;
                    mbar_arrive_expect_tx(&full[s], kStageBytes);
                    // (grouped: rows past the problem's last belong to the next problem or lie past the
                    // array, where the copy fills zeros; their accumulator rows are never stored)
                    tma_load_2d(a_dst, &map_a, kb * BK, row0, &full[s]);
                    if constexpr (MT == 2) tma_load_2d(a_dst + BM * BK, &map_a, kb * BK, row0 + BM, &full[s]);
                    tma_load_2d(b_dst, bmap, kb * BK, tn * BN, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // kind::i8 instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = BN, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                   (static_cast<uint32_t>(BM >> 4) << 24);
            int it = 0, local = 0;
            bool alive = true;
            int g, row0, rows, tn;
            for (int tile = blockIdx.x; alive && decode_tile<GROUPED, MT>(p, gt, tile, g, row0, rows, tn);
                 tile += gridDim.x, ++local) {
                // MT == 1: the tile's accumulator is buffer local & 1.  MT == 2: both buffers, one per half of the tile.
                const int buf = local & 1;
                if constexpr (MT == 1) {
                    if (local >= 2) {
                        alive = mbar_wait_bounded(&tmem_empty[buf], ((local >> 1) - 1) & 1, p.status);
                        if (!alive) break;
                    }
                }
                // (MT == 2: each half is waited for just before the first MMA that writes it, below: the epilogue
                // drains half 0 first, so this tile's first MMAs run while half 1 is still being stored)
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (MT == 1 ? buf * BN : 0);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % kStages;
                    alive = mbar_wait_bounded(&full[s], (it / kStages) & 1, p.status);
                    if (!alive) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                    const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                    for (int h = 0; h < MT; ++h) {
                        if constexpr (MT == 2) {
                            if (kb == 0 && local >= 1) {
                                alive = mbar_wait_bounded(&tmem_empty[h], (local - 1) & 1, p.status);
                                if (!alive) break;
                                tc_fence_after();
                            }
                        }
#pragma unroll
                        for (int kk = 0; kk < BK / 32; ++kk) {
                            umma_i8(d_tmem + h * BN, smem_desc_sw128(a_addr + h * (BM * BK) + kk * 32),
                                    smem_desc_sw128(b_addr + kk * 32), idesc, (kb | kk) != 0 ? 1u : 0u);
                        }
                    }
                    if (!alive) break;
                    umma_commit(&empty[s]);   // stage reusable once these MMAs have read it
                }
                if (alive) {
                    if constexpr (MT == 1) {
                        umma_commit(&tmem_full[buf]);
                    } else {
                        umma_commit(&tmem_full[0]);
                        umma_commit(&tmem_full[1]);
                    }
                }
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;          // TMEM lanes 32*quarter .. +31 are this warp's
        const int half = (warp - 2) >> 2;      // which of the two warps of the quarter: blocks half, half+2, ...
        uint8_t* stage = epi_stage + (warp - 2) * 4096;
        const uint64_t store_policy = l2_evict_first_policy();
        int local = 0;
        bool alive = true;
        int g, tile_row0, tile_rows, tn;
        for (int tile = blockIdx.x; alive && decode_tile<GROUPED, MT>(p, gt, tile, g, tile_row0, tile_rows, tn);
             tile += gridDim.x, ++local) {
          for (int h = 0; h < MT && alive; ++h) {
            // MT == 1: buffer local & 1 holds the tile.  MT == 2: buffer h holds rows h * 128 .. of the tile.
            const int buf = MT == 1 ? (local & 1) : h;
            alive = mbar_wait_bounded(&tmem_full[buf], (MT == 1 ? (local >> 1) : local) & 1, p.status);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            tc_fence_after();
            const int row0 = tile_row0 + h * BM, rows = tile_rows - h * BM;
            const int m = row0 + quarter * 32 + lane;            // row in the activation / output arrays
            const bool row_ok = quarter * 32 + lane < rows;
            float wscale = p.weight_scale;
            const float* magnitude = p.magnitude;
            const float* bias = p.bias;
            if constexpr (GROUPED) { wscale = gt.weight_scale[g]; magnitude = gt.magnitude[g]; bias = gt.bias[g]; }
            const float comb = row_ok ? __fmul_rn(__ldg(p.act_scales + m), wscale) : 0.0f;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * BN;
            // blocks of 32 columns this warp owns inside the tile, clipped at N
            const int nblocks = min(BN / 32, (p.N - tn * BN + 31) / 32);
            uint32_t r[32], rn[32];
            if (half < nblocks) tmem_ld32(t_row + half * 32, r);
#pragma unroll 1
            for (int c = half; c < nblocks; c += 2) {
                const int n0 = tn * BN + c * 32;
                tmem_ld_wait();
                if (c + 2 < nblocks) tmem_ld32(t_row + (c + 2) * 32, rn);   // in flight while this block is stored
                // float(acc) * (act_scale * weight_scale) [* magnitude[n]] [+ bias[n]], one rounding each.  The
                // per-column factors are loaded once per block (lane i holds column n0 + i) and handed round
                // with shuffles; columns past N are clipped by the store.  (An earlier form tested and
                // loaded per element: 825 instructions per 32 x 32 block, and the epilogue, not the tensor
                // pipe, set the pace of small-K shapes.)
                float v[32];
                if (!magnitude && !bias) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(static_cast<float>(static_cast<int>(r[i])), comb);
                } else {
                    const int nl = n0 + lane;
                    const float mag_l = magnitude && nl < p.N ? __ldg(magnitude + nl) : 1.0f;
                    const float bias_l = bias && nl < p.N ? __ldg(bias + nl) : 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float x = __fmul_rn(static_cast<float>(static_cast<int>(r[i])), comb);
                        if (magnitude) x = __fmul_rn(x, __shfl_sync(0xffffffffu, mag_l, i));
                        if (bias) x = __fadd_rn(x, __shfl_sync(0xffffffffu, bias_l, i));
                        v[i] = x;
                    }
                }
                if constexpr (GROUPED) {
                    if (gt.squared_relu) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) { const float x = fmaxf(v[i], 0.0f); v[i] = __fmul_rn(x, x); }
                    }
                }
                if (p.acc_debug && row_ok) {
                    for (int i = 0; i < 32; ++i)
                        if (n0 + i < p.N) p.acc_debug[static_cast<size_t>(m) * p.N + n0 + i] = static_cast<int>(r[i]);
                }
                if constexpr (GROUPED) {
                    // rows of other problems follow this one's in y: no clipped box store here.  Stage the
                    // block (row = lane, same swizzle as below), then one coalesced 128-byte store per row.
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 f = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = f;
                    }
                    __syncwarp();
                    const int valid = min(32, rows - quarter * 32);
                    const int col = n0 + lane;
                    for (int rr = 0; rr < valid; ++rr) {
                        const float x = *reinterpret_cast<const float*>(stage + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) +
                                                                        ((lane & 3) << 2));
                        if (col < p.N) p.y[static_cast<size_t>(row0 + quarter * 32 + rr) * p.N + col] = x;
                    }
                } else if (p.scatter.count > 0) {
                    // stage the block (row = lane, swizzled), then every destination gets it as 128-byte row
                    // segments: 4 rows x 8 chunks of 16 bytes per store instruction
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 f = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = f;
                    }
                    __syncwarp();
                    const int valid = min(32, rows - quarter * 32);
                    const int chunk = lane & 7, rsub = lane >> 3;
                    const int col = n0 + 4 * chunk;
#pragma unroll 1
                    for (int d = 0; d < p.scatter.count; ++d) {
                        float* base = p.scatter.dest[d] + p.scatter.col0 + col;
#pragma unroll
                        for (int i8 = 0; i8 < 8; ++i8) {
                            const int rr = 4 * i8 + rsub;
                            if (rr < valid && col < p.N) {      // N % 4 == 0 is checked on the host
                                const float4 f = *reinterpret_cast<const float4*>(stage + rr * 128 + ((chunk ^ (rr & 7)) << 4));
                                *reinterpret_cast<float4*>(base + static_cast<size_t>(row0 + quarter * 32 + rr) * p.scatter.ld) = f;
                            }
                        }
                    }
                } else if (p.use_tma_store) {
                    // the previous block's store must have finished reading the staging buffer
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
                    // row = lane; 16-byte chunk j of the 128-byte row goes to chunk j ^ (row & 7)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 f = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        *reinterpret_cast<float4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = f;
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d_hint(&map_y, n0, row0 + quarter * 32, stage, store_policy);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (row_ok) {
                    for (int i = 0; i < 32; ++i)
                        if (n0 + i < p.N) p.y[static_cast<size_t>(m) * p.N + n0 + i] = v[i];
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = rn[i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
          }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // common exit: all roles meet, then the allocating warp releases TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}


template <int BN, int MT = 1>
cudaError_t launch_bn(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& my, const GemmParams& p,
                      cudaStream_t stream) {
    auto kernel = gemm_tcgen05_kernel<BN, false, MT>;
    const size_t smem = 1024 + stages_for(BN, MT) * (MT * BM * BK + BN * BK) + kEpiWarps * 4096 + 256;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < kNumSm ? tiles : kNumSm;
    kernel<<<grid, kThreads, smem, stream>>>(ma, mb, my, p, NoGroups{});
    note_launch();
    return cudaGetLastError();
}

template <int BN>
cudaError_t launch_grouped_bn(const CUtensorMap& ma, const GemmParams& p, const GroupTable& gt, int grid,
                              cudaStream_t stream) {
    auto kernel = gemm_tcgen05_kernel<BN, true, 1>;
    const size_t smem = 1024 + stages_for(BN) * (BM * BK + BN * BK) + kEpiWarps * 4096 + 256;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kernel<<<grid, kThreads, smem, stream>>>(ma, ma, ma, p, gt);
    note_launch();
    return cudaGetLastError();
}

}  // namespace

// Grouped prefill GEMM: problem g = rows [offset_dev[g], offset_dev[g] + rows_dev[g]) of q / act_scales / y
// against w_i8[g]; `total_rows` is the extent of those arrays, `cap` an upper bound on any rows_dev[g].
cudaError_t launch_gemm_tcgen05_grouped(const int8_t* q, const float* act_scales, const int8_t* const* w_i8,
                                        const float* weight_scales, const float* const* magnitudes,
                                        const float* const* biases, const int* rows_dev, const int* offset_dev,
                                        int groups, int cap, int total_rows, int K, int N, float* y,
                                        int squared_relu, cudaStream_t stream) {
    if (groups < 1 || groups > TBL_MAX_GROUPS) return cudaErrorInvalidValue;
    GemmParams p{};
    p.act_scales = act_scales; p.y = y; p.K = K; p.N = N; p.M = total_rows;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorUnknown;
    // tile width: the one whose rounds over the 148 SMs cost least (rounds x width) among 256 and 128, and 64
    // too while even 256-wide tiles leave SMs without one (narrow tiles re-read the activations more often).  The row-tile count is an estimate: the real one depends
    // on the device-side row counts (about half a ragged tile per problem).
    const long long row_tiles = (total_rows + BM - 1) / BM + (groups + 1) / 2;
    int bn = 256;
    {
        const bool short_of_tiles = row_tiles * ((N + 255) / 256) < kNumSm;
        long long best = -1;
        for (int cand = 256; cand >= (short_of_tiles ? 64 : 128); cand >>= 1) {
            if (cand > 64 && N <= cand / 2) continue;
            const long long tiles = row_tiles * ((N + cand - 1) / cand);
            const long long cost = ((tiles + kNumSm - 1) / kNumSm) * cand;
            if (best < 0 || cost < best) { best = cost; bn = cand; }
        }
    }
    p.tiles_n = (N + bn - 1) / bn;
    GroupTable gt{};
    gt.groups = groups; gt.cap = cap; gt.squared_relu = squared_relu; gt.rows_dev = rows_dev; gt.offset_dev = offset_dev;
    CUtensorMap ma;
    if (!make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, total_rows, K, BK, BM)) return cudaErrorUnknown;
    for (int g = 0; g < groups; ++g) {
        if (!make_map(&gt.b[g], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_i8[g], N, K, BK, bn)) return cudaErrorUnknown;
        gt.weight_scale[g] = weight_scales[g];
        gt.magnitude[g] = magnitudes[g];
        gt.bias[g] = biases[g];
    }
    // tiles: at most ceil(total/128) + groups row tiles (one ragged tile per problem) times the n-tiles
    const long long tiles = (static_cast<long long>((total_rows + BM - 1) / BM) + groups) * p.tiles_n;
    const int grid = tiles < kNumSm ? static_cast<int>(tiles) : kNumSm;
    return bn == 256 ? launch_grouped_bn<256>(ma, p, gt, grid, stream)
                     : (bn == 128 ? launch_grouped_bn<128>(ma, p, gt, grid, stream) : launch_grouped_bn<64>(ma, p, gt, grid, stream));
}

cudaError_t launch_gemm_tcgen05(const int8_t* q, const float* act_scales, const int8_t* w_i8, float weight_scale,
                                const float* magnitude, const float* bias, int M, int K, int N, float* y,
                                int32_t* acc_debug, cudaStream_t stream, const GemmScatter* scatter) {
    GemmParams p{};
    if (scatter) {
        if (scatter->count < 1 || scatter->count > TBL_MAX_PEERS || (N & 3) || (scatter->ld & 3) || (scatter->col0 & 3))
            return cudaErrorInvalidValue;
        p.scatter = *scatter;
    }
    p.act_scales = act_scales; p.magnitude = magnitude; p.bias = bias; p.y = y; p.acc_debug = acc_debug;
    p.weight_scale = weight_scale; p.M = M; p.K = K; p.N = N;
    p.status = device_status_ptr();
    if (!p.status) return cudaErrorUnknown;
    // tall tiles (256 x 256) where there are enough of them: a third fewer operand bytes through L2 per output
    const long long tall_tiles = static_cast<long long>((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    const bool tall = N >= 256 && tall_tiles_pay(tall_tiles, K);
    // otherwise the tile width: 256 unless the narrower tile fills the 148 SMs clearly better (wave quantisation)
    int bn = N > 128 ? 256 : 128;
    if (bn == 256 && !tall) {
        const long long tm = (M + BM - 1) / BM;
        const long long t256 = tm * ((N + 255) / 256), t128 = tm * ((N + 127) / 128);
        const double e256 = static_cast<double>(t256) / (((t256 + kNumSm - 1) / kNumSm) * kNumSm);
        const double e128 = static_cast<double>(t128) / (((t128 + kNumSm - 1) / kNumSm) * kNumSm);
        if (e128 > 1.15 * e256) bn = 128;
        // few rows: the launch streams the weights once and wants every SM pulling -- narrower tiles
        if (bn == 128 && t128 < 100 && N > 64) bn = 64;
    }
    p.tiles_m = tall ? (M + 2 * BM - 1) / (2 * BM) : (M + BM - 1) / BM;
    p.tiles_n = (N + bn - 1) / bn;
    // TMA stores need a 16-byte row pitch and base
    p.use_tma_store = !scatter && (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    CUtensorMap ma, mb, my;
    if (!make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, M, K, BK, BM)) return cudaErrorUnknown;
    if (!make_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_i8, N, K, BK, bn)) return cudaErrorUnknown;
    if (p.use_tma_store) {
        if (!make_map(&my, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, y, M, N, 32, 32)) return cudaErrorUnknown;
    } else {
        my = ma;  // unused
    }
    if (tall) return launch_bn<256, 2>(ma, mb, my, p, stream);
    return bn == 256 ? launch_bn<256>(ma, mb, my, p, stream)
                     : (bn == 128 ? launch_bn<128>(ma, mb, my, p, stream) : launch_bn<64>(ma, mb, my, p, stream));
}

}  // namespace tbl
