// Ternary x int8 GEMV/GEMM for 5..64 activation rows per pass on the int8 mma.sync tensor path,
// with a problem table so one launch covers a group of independent linears (MoE experts,
// projections sharing an input).
//
// "Swap-AB": the MMA's 16-row A operand is a strip of 16 weight rows, its 8-column B operand is
// 8 activation rows.  A producer warp streams [16*W rows x KS] of canonical 2-bit words and
// [M x KS] of interleaved int8 activations into a shared-memory ring with 1-D bulk (TMA) copies,
// one per row segment; W consumer warps widen the codes in registers ((word >> 2j) & 0x03030303
// yields the unsigned bytes of weights {j,4+j,8+j,12+j}, which is exactly the order the
// activations were interleaved in) and issue m16n8k32 u8 x s8 MMAs.  The "-1" of the code is
// removed in the epilogue by subtracting sum_k q[m,k].
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

constexpr int kMaxProblems = TBL_MAX_GROUPS;
constexpr int kMaxStages = 4;
constexpr int kNumSm = 148;

struct MmaParams {
    MmaProblem prob[kMaxProblems];
    int count;
    int warps;   // consumer warps per CTA (row tile = 16 * warps)
    int ks;      // k elements per stage (multiple of 256)
    int stages;  // ring depth (2..kMaxStages)
    int* status; // device status word
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = activation tiles of 8 rows handled per pass (M_pad = 8*NT).
template <int NT>
__global__ void __launch_bounds__(9 * 32, 1) gemv_mma_kernel(const __grid_constant__ MmaParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = P.warps;
    const int RT = 16 * W;
    const int KS = P.ks;
    constexpr int MPAD = 8 * NT;

    // which problem / row tile is this CTA
    int pi = 0;
    while (pi + 1 < P.count && static_cast<int>(blockIdx.x) >= P.prob[pi + 1].cta_begin) ++pi;
    const MmaProblem& pr = P.prob[pi];
    const int n0 = (blockIdx.x - pr.cta_begin) * RT;
    const int K = pr.K, N = pr.N;
    int rows = pr.rows;
    if (pr.rows_dev) rows = min(rows, __ldg(pr.rows_dev));
    if (rows <= 0) return;
    const int row0 = pr.offset_dev ? __ldg(pr.offset_dev) : 0;
    const int8_t* qp_base = pr.qp + static_cast<size_t>(row0) * pr.K;

    const int wstride = KS / 4 + 64;    // bytes between weight rows of a stage (bank spread)
    const int astride = KS + 64;        // bytes between activation rows of a stage
    const int stage_bytes = RT * wstride + MPAD * astride;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    const int kStages = P.stages;
    uint8_t* stages = smem + 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], W);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    const int rows_valid = min(RT, N - n0);
    const int ksteps = (K + KS - 1) / KS;
    const int mtiles = (rows + MPAD - 1) / MPAD;
    const int row_bytes = K >> 2;
    const uint8_t* wbytes = reinterpret_cast<const uint8_t*>(pr.words) + static_cast<size_t>(n0) * row_bytes;

    if (warp == W) {
        // ---------------- producer warp ----------------
        int it = 0;
        bool alive = true;
        for (int mt = 0; mt < mtiles && alive; ++mt) {
            const int m0 = mt * MPAD;
            const int mcount = min(MPAD, rows - m0);
            for (int ksi = 0; ksi < ksteps && alive; ++ksi, ++it) {
                const int s = it % kStages;
                if (it >= kStages) {
                    alive = mbar_wait_bounded(&empty[s], ((it / kStages) - 1) & 1, P.status);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                }
                const int k0 = ksi * KS;
                const int kcur = min(KS, K - k0);
                uint8_t* wst = stages + static_cast<size_t>(s) * stage_bytes;
                uint8_t* ast = wst + RT * wstride;
                if (lane == 0)
                    mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(rows_valid) * (kcur >> 2) +
                                                        static_cast<uint32_t>(mcount) * kcur);
                __syncwarp();
                for (int r = lane; r < rows_valid; r += 32)
                    bulk_g2s(wst + r * wstride, wbytes + static_cast<size_t>(r) * row_bytes + (k0 >> 2),
                             kcur >> 2, &full[s]);
                for (int m = lane; m < mcount; m += 32)
                    bulk_g2s(ast + m * astride, qp_base + static_cast<size_t>(m0 + m) * K + k0, kcur, &full[s]);
            }
        }
        return;
    }
    if (warp > W) return;

    // ---------------- consumer warps ----------------
    const int g = lane >> 2, t = lane & 3;
    const int wr = 16 * warp;  // first row of this warp inside the CTA tile
    int it = 0;
    bool alive = true;
    for (int mt = 0; mt < mtiles && alive; ++mt) {
        const int m0 = mt * MPAD;
        int acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0;

        for (int ksi = 0; ksi < ksteps; ++ksi, ++it) {
            const int s = it % kStages;
            alive = mbar_wait_bounded(&full[s], (it / kStages) & 1, P.status);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            const int kcur = min(KS, K - ksi * KS);
            const uint8_t* wst = stages + static_cast<size_t>(s) * stage_bytes;
            const uint8_t* ast = wst + RT * wstride;
            const uint8_t* wlo = wst + (wr + g) * wstride + t * 16;
            const uint8_t* whi = wlo + 8 * wstride;
            const uint8_t* ab = ast + g * astride + t * 16;
            for (int step = 0; step < (kcur >> 8); ++step) {
                const uint4 lo = *reinterpret_cast<const uint4*>(wlo + step * 64);
                const uint4 hi = *reinterpret_cast<const uint4*>(whi + step * 64);
                const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w};
                const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
                uint32_t alo[4][4], ahi[4][4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        alo[x][j] = (lw[x] >> (2 * j)) & 0x03030303u;
                        ahi[x][j] = (hw[x] >> (2 * j)) & 0x03030303u;
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint8_t* ap = ab + nt * 8 * astride + step * 256;
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const uint4 b = *reinterpret_cast<const uint4*>(ap + x * 64);
                        mma_u8s8(acc[nt], alo[x][0], ahi[x][0], alo[x][1], ahi[x][1], b.x, b.y);
                        mma_u8s8(acc[nt], alo[x][2], ahi[x][2], alo[x][3], ahi[x][3], b.z, b.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!alive) break;

        // epilogue of this activation tile
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int n = n0 + wr + g + 8 * h;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int m = m0 + nt * 8 + 2 * t + c;
                    if (n < N && m < rows) {
                        const int gm = row0 + m;
                        const int total = acc[nt][2 * h + c] - __ldg(pr.q_sums + gm);
                        if (pr.acc_debug) pr.acc_debug[static_cast<size_t>(gm) * pr.ldy + n] = total;
                        float v = epilogue(total, __fmul_rn(__ldg(pr.act_scales + gm), pr.weight_scale),
                                           pr.magnitude, pr.bias, n);
                        if (pr.squared_relu) { v = fmaxf(v, 0.0f); v = __fmul_rn(v, v); }
                        pr.y[static_cast<size_t>(gm) * pr.ldy + n] = v;
                    }
                }
            }
        }
    }
}

// q row-major -> interleaved order + per-row sums; one CTA per row, 16 elements per thread-step.
__global__ void __launch_bounds__(256) permute_q_kernel(const int8_t* __restrict__ q, int K,
                                                        int8_t* __restrict__ qp, int32_t* __restrict__ q_sums) {
    __shared__ int partial[8];
    const int row = blockIdx.x;
    const int8_t* src = q + static_cast<size_t>(row) * K;
    int8_t* dst = qp + static_cast<size_t>(row) * K;
    int sum = 0;
    for (int j = threadIdx.x * 16; j < K; j += 256 * 16) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + j));
        sum = dp4a_ss(static_cast<int>(v.x), 0x01010101, sum);
        sum = dp4a_ss(static_cast<int>(v.y), 0x01010101, sum);
        sum = dp4a_ss(static_cast<int>(v.z), 0x01010101, sum);
        sum = dp4a_ss(static_cast<int>(v.w), 0x01010101, sum);
        *reinterpret_cast<uint4*>(dst + qp_offset16(j)) = transpose4x4_bytes(v);
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

template <int NT>
cudaError_t launch_nt(const MmaParams& P, int grid, size_t smem, cudaStream_t stream) {
    auto kernel = gemv_mma_kernel<NT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    kernel<<<grid, (P.warps + 1) * 32, smem, stream>>>(P);
    note_launch();
    return cudaGetLastError();
}

}  // namespace

bool gemv_mma_supported(int K) { return K > 0 && K % 256 == 0; }

cudaError_t launch_permute_q(const int8_t* q, int M, int K, int8_t* qp, int32_t* q_sums, cudaStream_t stream) {
    permute_q_kernel<<<M, 256, 0, stream>>>(q, K, qp, q_sums);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_gemv_mma(MmaProblem* problems, int count, cudaStream_t stream) {
    if (count < 1 || count > kMaxProblems) return cudaErrorInvalidValue;
    MmaParams P{};
    P.count = count;
    P.status = device_status_ptr();
    if (!P.status) return cudaErrorUnknown;
    int max_rows = 1, max_n = 1;
    for (int i = 0; i < count; ++i) {
        if (!gemv_mma_supported(problems[i].K)) return cudaErrorInvalidValue;
        max_rows = problems[i].rows > max_rows ? problems[i].rows : max_rows;
        max_n = problems[i].N > max_n ? problems[i].N : max_n;
    }
    const int nt = max_rows <= 8 ? 1 : (max_rows <= 16 ? 2 : (max_rows <= 32 ? 4 : 8));
    // consumer warps: the largest row tile that still gives every SM a CTA
    int warps = 8;
    while (warps > 1) {
        int ctas = 0;
        for (int i = 0; i < count; ++i) ctas += (problems[i].N + 16 * warps - 1) / (16 * warps);
        if (ctas >= kNumSm - 28) break;
        warps >>= 1;
    }
    P.warps = warps;
    P.ks = nt <= 2 ? 1024 : 512;
    int grid = 0;
    for (int i = 0; i < count; ++i) {
        P.prob[i] = problems[i];
        P.prob[i].cta_begin = grid;
        grid += (problems[i].N + 16 * warps - 1) / (16 * warps);
    }
    const size_t stage_bytes = static_cast<size_t>(16 * warps) * (P.ks / 4 + 64) + static_cast<size_t>(8 * nt) * (P.ks + 64);
    P.stages = kMaxStages;
    while (P.stages > 2 && 128 + P.stages * stage_bytes > 220 * 1024) --P.stages;
    const size_t smem = 128 + P.stages * stage_bytes;
    switch (nt) {
        case 1: return launch_nt<1>(P, grid, smem, stream);
        case 2: return launch_nt<2>(P, grid, smem, stream);
        case 4: return launch_nt<4>(P, grid, smem, stream);
        default: return launch_nt<8>(P, grid, smem, stream);
    }
}

}  // namespace tbl
