// Internal launcher declarations shared by the translation units of libternary_b200.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ternary_b200.h"

namespace tbl {

// ---- interleaved activation order read by the strip GEMV ------------------------------------
// Rows are grouped in tiles of kQpTile; a tile with R rows is stored block-major over K:
// [k/256][R][256 bytes], so the activations of one k-slab of a tile are contiguous (one bulk copy).
// Inside a 256-byte row-block the sixteen 16-element groups (chunk t = 0..3 of 64 elements,
// quarter i = 0..3) sit at group position ((i ^ (m & 1)) * 4 + t) -- the XOR spreads odd and even
// rows over different shared-memory banks -- and each group is 4x4 byte-transposed so that byte e
// of word j is element 4e + j (the order the 2-bit extraction pairs weights in).
// Byte offset of the group starting at element j (j % 16 == 0) of row `row` out of `rows`:
constexpr int kQpTile = 64;
__host__ __device__ __forceinline__ size_t qp_offset(int row, int rows, int K, int j) {
    const int mt = row / kQpTile, m = row % kQpTile;
    const int remaining = rows - mt * kQpTile;
    const int R = remaining < kQpTile ? remaining : kQpTile;
    const int kb = j >> 8, r = j & 255;
    const int t = r >> 6, i = (r >> 4) & 3;
    return static_cast<size_t>(mt) * kQpTile * K + static_cast<size_t>(kb) * R * 256 + m * 256 +
           ((((i ^ (m & 1)) << 2) + t) << 4);
}

// quantize.cu
// active_rows (device, may be null): rows >= *active_rows are skipped.
// qp (may be null) receives the interleaved copy; its tiling follows the row's problem: either the
// whole call is one problem of M rows, or seg_offsets/seg_counts (device, `segs` entries) give the
// first row and row count of each problem.
struct QuantSegments {
    const int32_t* offsets;
    const int32_t* counts;
    int segs;
};
cudaError_t launch_quantize_rows(const float* x, const int32_t* row_index, int M, int K, int bits,
                                 int rms_mode, int tie_mode, int8_t* q, int8_t* qp, float* act_scales,
                                 int32_t* q_sums, float* inv_norm_scratch, const int32_t* active_rows,
                                 QuantSegments segments, cudaStream_t stream, int plane_ld = 0);
cudaError_t launch_expand_i8(const uint32_t* words, int N, int K, int8_t* out, cudaStream_t stream);

// gemv_stream.cu — M <= 4, CUDA-core dp4a, weights streamed by per-warp TMA rings.
struct GemvSmallArgs {
    const float* x;          // fp32 [M,K] when fused, else null
    const int8_t* q;         // int8 [M,K] row-major when not fused, else null
    const float* act_scales; // fp32 [M] when not fused
    const uint32_t* words;   // canonical packed [N, K/16]
    const float* magnitude;  // [N] or null
    const float* bias;       // [N] or null
    float* y;                // fp32 [M,N]
    int32_t* acc_debug;      // int32 [M,N] or null
    int8_t* q_out;           // fused only: int8 [M,K] codes written by CTA 0, or null
    float* scales_out;       // fused only: fp32 [M] written by CTA 0, or null
    float weight_scale;
    float q_max;
    int M, K, N;
    int rms_mode;            // fused only: TBL_RMS_NONE or TBL_RMS_FAST
};
bool gemv_small_supported(int M, int K, int N);
cudaError_t launch_gemv_small(const GemvSmallArgs& a, cudaStream_t stream);

// gemv_generic.cu — any K % 16 == 0, any M: one warp per output row (correctness fallback).
// rows_dev / offset_dev (device, may be null): the row count and first row come from device memory
// (rows of q, act_scales and y are then taken relative to *offset_dev; M is the upper bound).
cudaError_t launch_gemv_generic(const int8_t* q, const float* act_scales, const uint32_t* words,
                                float weight_scale, const float* magnitude, const float* bias,
                                int M, int K, int N, float* y, int32_t* acc_debug, int squared_relu,
                                const int32_t* rows_dev, const int32_t* offset_dev, cudaStream_t stream);

// gemv_strip.cu -- 1 <= M <= 64 rows per pass, int8 mma.sync tensor cores, strip-major weights,
// problem table for grouped launches.
// Optional work in front of the fused quantiser of a strip GEMV (single problem, or several sharing the input rows):
// the residual add that closes a block of the hybrid and the RMSNorm x weight that opens the next stage, so that
// neither needs a launch of its own:  x <- x + a * ga [+ b * gb]  (ga null: x + a), stored to hidden_out / trace_out
// by CTA 0, then  x <- (x * rsqrt(mean(x^2) + norm_eps)) * norm_w.  All arrays are [rows, K] or [K], 16-byte aligned.
struct StripPrologue {
    const float* a;
    const float* ga;
    const float* b;
    const float* gb;
    const float* norm_w;      // null: no norm
    float norm_eps;
    float* hidden_out;        // may be null
    float* trace_out;         // may be null
};

struct StripProblem {
    const uint8_t* strips;    // strip-major packed weights (launch_relayout_strips)
    const int8_t* qp;         // interleaved int8 activations
    const float* act_scales;  // [rows]
    const int32_t* q_sums;    // [rows]
    const float* magnitude;
    const float* bias;
    float* y;                 // fp32 [rows, ldy]
    int32_t* acc_debug;       // int32 [rows, ldy] or null
    const int32_t* rows_dev;  // device row count (overrides rows when non-null)
    const int32_t* offset_dev;// device index of this problem's first row in qp/act_scales/q_sums/y
    float weight_scale;
    int rows;                 // host-known row count (upper bound when rows_dev is set)
    int N, K, ldy;
    int squared_relu;
    int strip_begin;          // global index of this problem's first strip (filled by the launcher)
    // fused quantiser (single-problem launches with few rows): when x != null the kernel quantises
    // x fp32 [rows, K] itself in its prologue and ignores qp / act_scales / q_sums
    const float* x;
    float q_max;
    int rms_fast;             // apply the (parallel-sum) input RMSNorm before quantising
    StripPrologue pre;        // fused launches only (problem 0's is used); all null = none
};
// rows the strip kernel can quantise in its own prologue for this K (0 = none)
int gemv_strip_fused_rows(int K);
bool gemv_strip_supported(int K);
void set_gemv_events(cudaEvent_t start, cudaEvent_t stop);
cudaError_t launch_relayout_strips(const uint32_t* words, int N, int K, void* strips, cudaStream_t stream);
cudaError_t launch_gemv_strip(StripProblem* problems, int count, cudaStream_t stream);
cudaError_t launch_permute_q(const int8_t* q, int M, int K, int8_t* qp, int32_t* q_sums, cudaStream_t stream);

// gemv_chain.cu -- a stack of ternary linears (each layer's output is the next one's input) for <= 8 rows in one
// persistent cooperative launch; layers need strip-major weights, K % 256 == 0 and rows*K <= 16384.
struct ChainLayer {
    const uint8_t* strips;
    const float* magnitude;
    const float* bias;
    float weight_scale;
    float q_max;
    int N, K;
    int rms_fast;        // input RMSNorm (parallel sum) before the quantiser
    int squared_relu;    // max(y,0)^2 after the epilogue
};
bool gemv_chain_supported(const ChainLayer* layers, int count, int rows);
size_t gemv_chain_workspace_bytes(const ChainLayer* layers, int count, int rows);
void set_chain_trace(void* buffer, size_t bytes);
cudaError_t launch_gemv_chain(const ChainLayer* layers, int count, int rows, const float* x, float* y,
                              void* workspace, cudaStream_t stream);

// api.cu -- the same two calls with a residual add / RMSNorm x weight in the GEMV's own prologue (StripPrologue).
// They serve only shapes the fused-prologue strip kernel takes (strip copies present, rows <= gemv_strip_fused_rows(K),
// 16-byte aligned arrays) and return TBL_ERR_UNSUPPORTED otherwise: the caller then runs the pieces separately.
int grouped_forward_rows_pre(const tbl_linear_view* views, int groups, const float* x, int rows, float* out,
                             long long out_stride, const StripPrologue& pre, cudaStream_t st);
int linear_view_forward_pre(const tbl_linear_view& v, const float* x, int rows, bool squared_relu, const StripPrologue& pre,
                            float* y, cudaStream_t st);

// api.cu -- one view's forward with an optional squared ReLU (fused into the GEMV epilogue where possible)
int linear_view_forward(const tbl_linear_view& v, const float* x, int rows, int rms_mode, bool squared_relu, float* y,
                        void* workspace, size_t workspace_bytes, cudaStream_t st);

// gemm_widen.cu -- up to 128 rows per pass on the strip-major 2-bit weights: widened to bytes inside the kernel,
// tcgen05 int8 MMAs with the weights as the A operand.  Up to kWidenMaxViews weight matrices that share the input
// rows (and K) run in one launch.  `planes` holds gemm_widen_scratch_bytes(M, K) bytes: the plane-major codes,
// written by the row quantiser itself (plane_ld = gemm_widen_plane_ld(K)) or, when `q` (row-major codes) is given,
// by a permutation pass inside the launcher.
constexpr int kWidenMaxViews = 16;
struct WidenView {
    const void* strips;
    const float* magnitude;
    const float* bias;
    float* y;               // [M, N] row-major
    float weight_scale;
    int N;
    int squared_relu;       // y = max(y, 0)^2 after the affine epilogue
};
bool gemm_widen_supported(int M, int K, int N);
int gemm_widen_plane_ld(int K);
size_t gemm_widen_scratch_bytes(int M, int K);
// rows_dev / offsets_dev (device, one entry per view; optional): view v multiplies only rows offsets_dev[v] ..
// + rows_dev[v] of the total_rows rows of codes (the experts of a MoE stage); M is then the upper bound of a view's
// row count and may exceed 128 (passes of 128 rows inside the launch; q must be null).
cudaError_t launch_gemm_widen(const WidenView* views, int count, const int8_t* q, int8_t* planes, const float* act_scales,
                              const int32_t* q_sums, int M, int K, cudaStream_t stream, const int32_t* rows_dev = nullptr,
                              const int32_t* offsets_dev = nullptr, int total_rows = 0);

// gemm_tcgen05.cu — M > 64, tcgen05 int8 MMA, TMEM accumulators, TMA operands.
// `scatter` (optional): instead of y, the epilogue writes every output tile into `count` arrays -- this GPU's and
// its peers' mappings of one [M, ld] output -- at column col0 + n: the column-split exchange done by the GEMM's own
// stores over NVLink.
struct GemmScatter {
    float* dest[TBL_MAX_PEERS];
    int count;
    long long ld, col0;
};
cudaError_t launch_gemm_tcgen05(const int8_t* q, const float* act_scales, const int8_t* w_i8,
                                float weight_scale, const float* magnitude, const float* bias,
                                int M, int K, int N, float* y, int32_t* acc_debug, cudaStream_t stream,
                                const GemmScatter* scatter = nullptr);
cudaError_t launch_gemm_tcgen05_grouped(const int8_t* q, const float* act_scales, const int8_t* const* w_i8,
                                        const float* weight_scales, const float* const* magnitudes,
                                        const float* const* biases, const int* rows_dev, const int* offset_dev,
                                        int groups, int cap, int total_rows, int K, int N, float* y,
                                        int squared_relu, cudaStream_t stream);

// moe.cu — routing lists and the final merge.
struct MoeLists {
    int32_t* counts;    // [E] rows routed to each expert
    int32_t* offsets;   // [E] first slot of each expert
    int32_t* total;     // [1] slots in use
    int32_t* slot_row;  // [capacity] source row of each slot
    int32_t* slot_of;   // [rows,E] slot of (row, expert) or -1
};
cudaError_t launch_moe_route(const float* routing, int rows, int experts, int capacity, MoeLists lists,
                             int* status, cudaStream_t stream);
cudaError_t launch_router_topk(const float* logits, int rows, int experts, int top_k, float* weights,
                               cudaStream_t stream);
// glue.cu -- row norms around a linear (block RMSNorm x weight; SiLU gate -> RMSNorm x weight), optionally
// fused with the per-token quantiser.  gate / weight / out / q may be null (q and out not both); q needs
// dim % 16 == 0.  The row is cached in shared memory, which bounds dim.
constexpr int kRowNormMaxDim = 49152;
cudaError_t launch_row_norm(const float* value, const float* gate, const float* weight, int rows, int dim, float eps,
                            int bits, float* out, int8_t* q, float* act_scales, int32_t* q_sums,
                            cudaStream_t stream);
// column-split outputs after an all-gather, [parts][rows][cols] -> [rows][parts*cols]
cudaError_t launch_retile_columns(const float* gathered, int parts, int rows, int cols, float* out, cudaStream_t stream);
// max(x,0)^2 in place over n floats (OXN/nsos/src/tensor.cpp:3209-3226).
cudaError_t launch_squared_relu(float* x, int64_t n, cudaStream_t stream);
cudaError_t launch_moe_merge(const float* routing, const float* contrib, const int32_t* slot_of, int rows,
                             int experts, int dim, float* out, cudaStream_t stream);

}  // namespace tbl
