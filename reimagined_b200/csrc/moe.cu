// MoE helpers around the grouped ternary kernels: device-side routing lists (which rows go to
// which expert, without a host round trip) and the final weighted merge in expert order.
#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

constexpr int kRouteThreads = 256;

// One CTA walks the experts in index order and, inside an expert, the rows in row order, handing
// out consecutive slots: slots of expert e are [offsets[e], offsets[e] + counts[e]).  The routing weights are
// read once, up front (a bit per expert and row, kept in registers for up to kRouteChunks x 256 rows): the walk
// itself then touches only shared memory, instead of one dependent global round trip per expert.
constexpr int kRouteChunks = 8;
__global__ void __launch_bounds__(kRouteThreads)
moe_route_kernel(const float* __restrict__ routing, int rows, int experts, int capacity, MoeLists L,
                 int* status) {
    __shared__ int warp_totals[kRouteThreads / 32];
    __shared__ int base;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    const bool cached = rows <= kRouteChunks * kRouteThreads && experts <= 32;
    uint32_t mask[kRouteChunks];
#pragma unroll
    for (int c = 0; c < kRouteChunks; ++c) {
        mask[c] = 0u;
        const int r = c * kRouteThreads + threadIdx.x;
        if (cached && r < rows) {
            for (int e = 0; e < experts; ++e)
                mask[c] |= routing[static_cast<size_t>(r) * experts + e] != 0.0f ? 1u << e : 0u;
        }
    }
    __syncthreads();
    for (int e = 0; e < experts; ++e) {
        const int start = base;
#pragma unroll 1
        for (int r0 = 0, c = 0; r0 < rows; r0 += kRouteThreads, ++c) {
            const int r = r0 + threadIdx.x;
            bool hit;
            if (cached) {
                uint32_t mk = mask[0];
#pragma unroll
                for (int i = 1; i < kRouteChunks; ++i) if (c == i) mk = mask[i];
                hit = (mk >> e & 1u) != 0u;
            } else {
                hit = r < rows && routing[static_cast<size_t>(r) * experts + e] != 0.0f;
            }
            const unsigned ballot = __ballot_sync(0xffffffffu, hit);
            const int before = __popc(ballot & ((1u << lane) - 1));
            if (lane == 0) warp_totals[warp] = __popc(ballot);
            __syncthreads();
            int prefix = 0, total = 0;
            for (int w = 0; w < kRouteThreads / 32; ++w) {
                if (w < warp) prefix += warp_totals[w];
                total += warp_totals[w];
            }
            const int chunk_base = base;
            if (r < rows) {
                int slot = -1;
                if (hit) {
                    slot = chunk_base + prefix + before;
                    if (slot < capacity) {
                        L.slot_row[slot] = r;
                    } else {
                        slot = -1;
                        atomicOr(status, TBL_DEV_ROUTE_OVERFLOW);
                    }
                }
                L.slot_of[static_cast<size_t>(r) * experts + e] = slot;
            }
            __syncthreads();
            if (threadIdx.x == 0) base = chunk_base + total;
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            const int end = min(base, capacity);
            const int begin = min(start, capacity);
            L.offsets[e] = begin;
            L.counts[e] = end - begin;
        }
    }
    if (threadIdx.x == 0) *L.total = min(base, capacity);
}

// out[r,n] = sum over experts in index order of contrib[slot(r,e), n] * routing[r,e], each term and
// each addition separately rounded (the CPU composition accumulates expert by expert).
__global__ void __launch_bounds__(256)
moe_merge_kernel(const float* __restrict__ routing, const float* __restrict__ contrib,
                 const int32_t* __restrict__ slot_of, int experts, int dim, float* __restrict__ out) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (n >= dim) return;
    float sum = 0.0f;
    for (int e = 0; e < experts; ++e) {
        const float w = routing[static_cast<size_t>(r) * experts + e];
        if (w != 0.0f) {
            const int slot = slot_of[static_cast<size_t>(r) * experts + e];
            if (slot >= 0) sum = __fadd_rn(sum, __fmul_rn(contrib[static_cast<size_t>(slot) * dim + n], w));
        }
    }
    out[static_cast<size_t>(r) * dim + n] = sum;
}


// Router post-processing, one thread per token: softmax over the experts' logits (max-subtracted,
// 1/max(sum, 1e-8)), keep the top_k largest (ties -> lower index), renormalise by 1/max(sum_selected, 1e-9),
// zero the rest.  Sums run in the reference's order (expert index, then rank).
__global__ void router_topk_kernel(const float* __restrict__ logits, int rows, int experts, int top_k,
                                   float* __restrict__ weights) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const float* l = logits + static_cast<size_t>(r) * experts;
    float* w = weights + static_cast<size_t>(r) * experts;
    float p[TBL_MAX_GROUPS];
    float mx = l[0];
    for (int e = 1; e < experts; ++e) mx = l[e] > mx ? l[e] : mx;
    float sum = 0.0f;
    for (int e = 0; e < experts; ++e) { p[e] = expf(__fsub_rn(l[e], mx)); sum = __fadd_rn(sum, p[e]); }
    const float inv = __fdiv_rn(1.0f, sum > 1e-8f ? sum : 1e-8f);
    for (int e = 0; e < experts; ++e) p[e] = __fmul_rn(p[e], inv);
    if (top_k > 0 && top_k < experts) {
        unsigned keep = 0u;
        float selected = 0.0f;
        for (int rank = 0; rank < top_k; ++rank) {
            int best = -1;
            for (int e = 0; e < experts; ++e)
                if (!((keep >> e) & 1u) && (best < 0 || p[e] > p[best])) best = e;
            keep |= 1u << best;
            selected = __fadd_rn(selected, p[best]);
        }
        const float inv_sel = __fdiv_rn(1.0f, selected > 1e-9f ? selected : 1e-9f);
        for (int e = 0; e < experts; ++e) p[e] = ((keep >> e) & 1u) ? __fmul_rn(p[e], inv_sel) : 0.0f;
    }
    for (int e = 0; e < experts; ++e) w[e] = p[e];
}

}  // namespace

cudaError_t launch_moe_route(const float* routing, int rows, int experts, int capacity, MoeLists lists,
                             int* status, cudaStream_t stream) {
    moe_route_kernel<<<1, kRouteThreads, 0, stream>>>(routing, rows, experts, capacity, lists, status);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_moe_merge(const float* routing, const float* contrib, const int32_t* slot_of, int rows,
                             int experts, int dim, float* out, cudaStream_t stream) {
    const dim3 grid((dim + 255) / 256, rows);
    moe_merge_kernel<<<grid, 256, 0, stream>>>(routing, contrib, slot_of, experts, dim, out);
    note_launch();
    return cudaGetLastError();
}

cudaError_t launch_router_topk(const float* logits, int rows, int experts, int top_k, float* weights,
                               cudaStream_t stream) {
    if (experts < 1 || experts > TBL_MAX_GROUPS) return cudaErrorInvalidValue;
    router_topk_kernel<<<(rows + 127) / 128, 128, 0, stream>>>(logits, rows, experts, top_k, weights);
    note_launch();
    return cudaGetLastError();
}

}  // namespace tbl
