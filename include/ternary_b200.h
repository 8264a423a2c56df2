/*
 * ternary_b200 — C ABI of the B200 (sm_100a) BitNet b1.58 ternary linear path.
 *
 * Drop-in boundary for the NSOS runtime's packed BitLinear path.  Every entry point
 *   - is extern "C", takes plain pointers and sizes, and returns an int status
 *     (0 = ok, negative = rejected by validation, nothing was launched);
 *   - never throws, never allocates device memory, never synchronises unless its comment
 *     says so; all work is enqueued on the caller's stream (a cudaStream_t passed as
 *     void*; NULL = the legacy default stream);
 *   - borrows every pointer: the owner keeps buffers alive until the stream has drained.
 * Device-side waits are bounded; a kernel that gives up records a code readable with
 * tbl_device_status().
 *
 * Numeric contract (identical to the reference's CPU packed path):
 *   weight_scale = float(sum_i double|w_i| / n) + 1e-8f, sequential sum;
 *   t = w/(weight_scale+1e-8f) > 0.5 ? +1 : (< -0.5 ? -1 : 0);
 *   2-bit code t+1 at bits 2*(i%16) of word i/16, i = n*K + k;
 *   per row: m = max|x|, q = round_half_even(x * (qmax/(m+1e-8f))), act_scale = (m+1e-8f)/qmax;
 *   acc = sum_k q*t (int32);  y = float(acc) * (act_scale*weight_scale) [* magnitude[n]] [+ bias[n]].
 */
#ifndef TERNARY_B200_H
#define TERNARY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------ */
#define TBL_OK 0
#define TBL_ERR_INVALID_ARG (-1)   /* null pointer, non-positive size, bad flag          */
#define TBL_ERR_SHAPE (-2)         /* K % 16 != 0, M*N > INT_MAX, M out of a kernel's range */
#define TBL_ERR_OVERFLOW (-3)      /* K > INT_MAX/254: int32 accumulation could overflow  */
#define TBL_ERR_SCALE (-4)         /* weight_scale not finite or not > 0                  */
#define TBL_ERR_BITS (-5)          /* activation bits outside [2,8]                       */
#define TBL_ERR_ALIGNMENT (-6)     /* a device pointer is not 16-byte aligned             */
#define TBL_ERR_WORKSPACE (-7)     /* workspace too small                                 */
#define TBL_ERR_CODE (-8)          /* packed words contain the illegal code 0b11          */
#define TBL_ERR_CUDA (-9)          /* a CUDA runtime call or launch failed                */
#define TBL_ERR_UNSUPPORTED (-10)  /* descriptor mode this library does not implement     */
#define TBL_ERR_FORMAT (-11)       /* edge pack: bad magic/version, truncated, bad flag, non-finite value */
#define TBL_ERR_INTEGRITY (-12)    /* edge pack: trailer missing or SHA-256 mismatch      */

const char* tbl_status_string(int status);

/* Library/ABI version (bumped when a signature changes). */
int tbl_abi_version(void);

/* ---- flags ------------------------------------------------------------------------- */
/* rms_mode: input RMSNorm applied before quantisation (eps 1e-6).
 *   0 none; 1 parallel reduction (fast, sum order differs from the CPU reference by
 *   rounding); 2 reference order (sequential fp32 sum, bit-identical to Tensor::rmsnorm). */
#define TBL_RMS_NONE 0
#define TBL_RMS_FAST 1
#define TBL_RMS_REFERENCE_ORDER 2
/* tie rule for the quantiser: 0 = round-half-to-even (the default x86-64 reference build),
 * 1 = round-half-away-from-zero (the reference's scalar build and MoE decode kernel). */
#define TBL_TIE_EVEN 0
#define TBL_TIE_AWAY 1

/* ---- offline packer (host) ---------------------------------------------------------- */

/* Number of uint32 words of the canonical packing of an [N,K] matrix.
 * Replaces: size computation in BitLinear::pack_weights, OXN/nsos/src/bitlinear.cpp:162-166. */
int64_t tbl_packed_words(int N, int K);

/* Absmean-ternarises w_host (fp32 [N,K], row-major) and writes the canonical 2-bit words
 * and the per-matrix scale.  Host-only, sequential double sum (bit-exact with the reference).
 * Replaces: BitLinear::pack_weights (OXN/nsos/src/bitlinear.cpp:152-193), tensor_abs_mean
 * (OXN/nsos/src/tensor.cpp:2097-2102), BitLinear::quantize_weights
 * (OXN/nsos/src/bitlinear.cpp:1359-1379), BitNetAdapter::pack_weights_microsoft_style
 * (OXN/nsos/src/bitnet_adapter.cpp:570-588). */
int tbl_pack_weights(const float* w_host, int N, int K, uint32_t* words_host, float* weight_scale);

/* Decodes canonical words to int8 {-1,0,+1} [N,K] on the host (code 3 decodes to 0).
 * Replaces: BitNetAdapter::unpack_weights_microsoft_style_to_i8,
 * OXN/nsos/src/bitnet_adapter.cpp:590-606. */
int tbl_unpack_weights_i8(const uint32_t* words_host, int N, int K, int8_t* t_host);

/* Validates an imported packed state: sizes, finite positive scale, no code 0b11, finite
 * magnitude/bias (either may be NULL).
 * Replaces: the checks of BitLinear::prepare_packed_state, OXN/nsos/src/bitlinear.cpp:834-900. */
int tbl_validate_packed(const uint32_t* words_host, int64_t n_words, int N, int K,
                        float weight_scale, const float* magnitude_host, const float* bias_host);

/* ---- device: weight layouts derived from the canonical words ------------------------------ */

/* The device entry points below take words that passed tbl_validate_packed (or came out of tbl_pack_weights /
 * tbl_edge_pack_open): they do not look for the reserved code 0b11.  The host decoder maps that code to 0
 * (like the reference's CPU decoders); the device kernels compute code - 1 and would read it as +2 (like the
 * reference's GPU kernels, OXN/nsos/src/cuda/kernels.cu:991,1043).  Validate before uploading. */

/* Bytes of the strip-major copy of an [N,K] matrix (K % 256 == 0; rows padded to a multiple of 16). */
size_t tbl_strip_bytes(int N, int K);

/* Re-orders canonical words (device) into the strip-major layout the decode GEMV streams:
 * strips of 16 rows, each a contiguous run of K/256 blocks of 1 KB whose 16-byte chunks are in
 * warp-lane order (rows g and g+8 of lane 4g+t).  A permutation of the canonical 16-byte chunks
 * plus zero-weight padding rows; done once per matrix at load time.  Needs K % 256 == 0.
 * Replaces: the H2D upload of the packed words in BitLinear::forward
 * (OXN/nsos/src/bitlinear.cpp:632-643), which is where the reference fixes its device layout. */
int tbl_relayout_strips(const uint32_t* words_dev, int N, int K, void* strips_dev, void* stream);


/* Expands canonical words (device) into int8 {-1,0,+1} [N,K] row-major (device), the K-major
 * operand the tcgen05 GEMM reads through TMA.  Mirrors the unpacked copy the reference keeps
 * beside its packed words (BitLinear::unpacked_weights_i8, OXN/nsos/src/bitlinear.cpp:186-188). */
int tbl_expand_weights_i8(const uint32_t* words_dev, int N, int K, int8_t* w_i8_dev, void* stream);

/* ---- device: activation quantiser --------------------------------------------------- */

/* Per-row absmax quantiser: x fp32 [M,K] -> q int8 [M,K] + act_scales fp32 [M]
 * (+ optional q_sums int32 [M] = sum_k q, NULL to skip).  row_index (device int32 [M], may be
 * NULL) gathers input rows: output row i is computed from x row row_index[i].
 * Replaces: BitLinear::quantize_activations_bitnet (OXN/nsos/src/bitlinear.cpp:240-291),
 * launch_quantize_activations_bitnet_kernel (OXN/nsos/src/cuda/bitnet_kernels.cu:70-130,296-304)
 * and, with rms_mode != 0, the Tensor::rmsnorm(1e-6) in BitLinear::forward
 * (OXN/nsos/src/bitlinear.cpp:460-463). */
int tbl_quantize_rows(const float* x_dev, const int32_t* row_index_dev, int M, int K, int bits,
                      int rms_mode, int tie_mode, int8_t* q_dev, float* act_scales_dev,
                      int32_t* q_sums_dev, void* stream);

/* ---- device: GEMV / GEMM on already-quantised activations ----------------------------- */

/* Bytes of scratch tbl_gemv needs for (M,K). */
size_t tbl_gemv_workspace_bytes(int M, int K);

/* Decode GEMV, 1 <= M <= 64: y[M,N] = epilogue(q[M,K] x ternary[N,K]^T).
 * Weights: strips_dev (tbl_relayout_strips, the fast tensor-core stream) and/or words_dev
 * (canonical; used when strips_dev is NULL or K % 256 != 0).  At least one must be given.
 * acc_debug (device int32 [M,N], may be NULL) receives the raw accumulators.
 * Replaces: launch_bitnet_gemv_scaled (OXN/nsos/src/cuda/kernels.cu:1027-1066,1110-1130) and,
 * for 1 < M <= 64, launch_bitnet_gemm + launch_bitnet_apply_act_scales_kernel
 * (OXN/nsos/src/cuda/kernels.cu:966-1022, OXN/nsos/src/cuda/bitnet_kernels.cu:140-149). */
int tbl_gemv(const int8_t* q_dev, const float* act_scales_dev, const uint32_t* words_dev,
             const void* strips_dev, float weight_scale, const float* magnitude_dev,
             const float* bias_dev, int M, int K, int N, float* y_dev, int32_t* acc_debug_dev,
             void* workspace_dev, size_t workspace_bytes, void* stream);

/* Prefill GEMM on tcgen05 int8 tensor cores (any M >= 1, intended for M >= 128):
 * y[M,N] = epilogue(q[M,K] x w_i8[N,K]^T), accumulators in tensor memory.
 * w_i8_dev is the output of tbl_expand_weights_i8.  Needs K % 16 == 0.
 * Replaces: launch_bitnet_gemm + launch_bitnet_apply_act_scales_kernel + the magnitude/bias
 * tensor ops of bitnet_gemm_158bit_gpu (OXN/nsos/src/bitnet_gpu_dispatch.cpp:157-171). */
int tbl_gemm(const int8_t* q_dev, const float* act_scales_dev, const int8_t* w_i8_dev,
             float weight_scale, const float* magnitude_dev, const float* bias_dev,
             int M, int K, int N, float* y_dev, int32_t* acc_debug_dev, void* stream);

/* ---- device: the fused layer forward -------------------------------------------------- */

/* Bytes of scratch tbl_linear_forward needs for (M,K,N). */
size_t tbl_linear_workspace_bytes(int M, int K, int N);

/* x fp32 [M,K] (device) -> y fp32 [M,N] (device): [RMSNorm] -> quantise -> ternary GEMV
 * (M <= 32 on the strip copy; 33 <= M <= 256 with K % 256 == 0 on the strip copy too, widened to
 * bytes inside a tcgen05 kernel, so batches up to 256 rows need no int8 copy) or tcgen05 GEMM
 * (M > 64 when w_i8_dev != NULL) -> two-scale epilogue [* magnitude] [+ bias].  strips_dev /
 * w_i8_dev may be NULL: then the call runs on what it is given (canonical words alone serve
 * every M, at lower speed).
 * Replaces: bitnet_gemm_158bit_gpu (OXN/nsos/include/bitnet_gpu_dispatch.h:46-51,
 * OXN/nsos/src/bitnet_gpu_dispatch.cpp:65-174) and the packed branch of BitLinear::forward
 * (OXN/nsos/src/bitlinear.cpp:606-659,690-741). */
int tbl_linear_forward(const float* x_dev, const uint32_t* words_dev, const void* strips_dev,
                       const int8_t* w_i8_dev, float weight_scale, int M, int K, int N, int bits, int rms_mode,
                       const float* magnitude_dev, const float* bias_dev, float* y_dev,
                       void* workspace_dev, size_t workspace_bytes, void* stream);

/* The same forward for a column-split layer whose output every GPU of the node needs whole: this GPU holds
 * the weight rows [col0, col0 + N) of an [N_total, K] layer and writes its [M, N] block of y straight into
 * `n_dest` arrays -- its own and its peers' mappings of the full output, row pitch `ldy` elements -- from the
 * GEMM epilogue (plain 128-bit stores over NVLink for the peers), so that no all-gather and no re-tile pass
 * follow.  The caller orders the GPUs before the output is read (a barrier across the ranks on the stream).
 * Needs M > 64 and the int8 expansion (the tcgen05 path); N, ldy and col0 multiples of 4; y_dest_host holds
 * device pointers that are valid on this GPU (peer access enabled or a symmetric-memory mapping).  Shapes the
 * tensor-core path does not serve return TBL_ERR_UNSUPPORTED: write into a local slot and all-gather instead.
 * The reference has no multi-GPU inference (OXN/nsos/src/fabric_v2.cpp stages gradients through the host);
 * this is the B200 counterpart of one model spread over the NVLink domain. */
#define TBL_MAX_PEERS 8
int tbl_linear_forward_scatter(const float* x_dev, const int8_t* w_i8_dev, float weight_scale, int M, int K, int N,
                               int bits, int rms_mode, const float* magnitude_dev, const float* bias_dev,
                               float* const* y_dest_host, int n_dest, long long ldy, long long col0,
                               void* workspace_dev, size_t workspace_bytes, void* stream);

/* Largest scratch tbl_linear_forward_noalloc can serve: tbl_linear_workspace_bytes(M,K,N) must not
 * exceed this (e.g. M*K <= 1 MiB of int8 codes: 64 rows of K = 16384, or 1365 rows of K = 768). */
#define TBL_NOALLOC_SCRATCH_BYTES (2u * 1024u * 1024u + 64u * 1024u)

/* tbl_linear_forward for callers that have no way to obtain device scratch memory: code running
 * inside a latency-critical decode loop where cudaMalloc is forbidden, plugins handed only their
 * input and output buffers by a host runtime that owns the allocator, and bindings (cgo/JNI/ctypes)
 * whose side of the boundary cannot manage device lifetimes.  Same arithmetic and same results as
 * tbl_linear_forward; the quantiser's scratch (int8 codes, scales, row sums) lives in a fixed array
 * inside the library image instead of a caller workspace.
 *   - The array is TBL_NOALLOC_SCRATCH_BYTES large and is part of every device's copy of the library
 *     from load until exit; shapes whose scratch would not fit are refused with TBL_ERR_WORKSPACE
 *     and nothing is launched.
 *   - The first call on each device looks the array's device address up (with that device current);
 *     make that first call before any stream capture begins.
 *   - No cudaMalloc/cudaFree or other allocating call is made, on any call.
 *   - Every call uses the same array and leaves its last contents there.  Nothing in it has to start
 *     at zero (each call overwrites all it later reads), but two calls that overlap on the GPU --
 *     different streams, or one stream fed from several threads without ordering -- race on it: keep
 *     calls on one stream or order them yourself.
 * This entry point has no counterpart in the reference (whose dispatch always borrows scratch from
 * its ExecutionContext). */
int tbl_linear_forward_noalloc(const float* x_dev, const uint32_t* words_dev, const void* strips_dev,
                               const int8_t* w_i8_dev, float weight_scale, int M, int K, int N, int bits,
                               int rms_mode, const float* magnitude_dev, const float* bias_dev,
                               float* y_dev, void* stream);

/* ---- grouped variant ------------------------------------------------------------------- */

/* Borrowed descriptor of one linear; the first nine fields are field-for-field the reference's
 * GpuLinearView (OXN/nsos/include/gpu_linear_view.h:8-26); `strips` and `w_i8` are this library's
 * additions (strip-major copy of `packed` from tbl_relayout_strips, int8 expansion from
 * tbl_expand_weights_i8; either may be NULL).  Only the packed mode (packed != NULL, weight == NULL,
 * activation_bits in [2,8]) is implemented; others -> TBL_ERR_UNSUPPORTED. */
typedef struct tbl_linear_view {
    const float* weight;
    const uint32_t* packed;
    const float* magnitude;
    const float* bias;
    int inputs;
    int outputs;
    int activation_bits;
    int rms_input;
    float weight_scale;
    const void* strips;
    const int8_t* w_i8;
} tbl_linear_view;

#define TBL_MAX_GROUPS 32

/* Bytes of scratch for tbl_grouped_forward with `groups` views of at most max_inputs inputs. */
size_t tbl_grouped_workspace_bytes(int groups, int max_inputs);

/* `groups` independent linears sharing ONE input row (QKV, Mamba x/z/B/C/dt): views is a
 * HOST array; view g reads input_dev[0..inputs) and writes output_dev[g*output_stride ..].
 * All views must share inputs, activation_bits and rms_input so the row is quantised once.
 * Replaces: launch_grouped_decode_projections (OXN/nsos/src/cuda/moe_kernels.cu:779-784) and
 * GpuProjectionGroup::forward (OXN/nsos/src/gpu_projection_group.cpp:12-52). */
int tbl_grouped_forward(const tbl_linear_view* views_host, int groups, const float* input_dev,
                        float* output_dev, int output_stride, int rms_mode,
                        void* workspace_dev, size_t workspace_bytes, void* stream);

/* tbl_grouped_forward for `rows` <= 64 input rows (batched decode: B sequences go through the same
 * projections).  input_dev is fp32 [rows, inputs]; view g writes a contiguous [rows, outputs_g] block at
 * output_dev + g*output_stride (output_stride in floats, >= rows*outputs_g).  One launch when
 * rows*inputs <= 16384 (the rows are quantised in the prologue of the grouped GEMV), else two.
 * No counterpart in the reference: its grouped launch takes a single row
 * (OXN/nsos/src/gpu_projection_group.cpp:12-47) and batches fall back to one BitLinear call per projection. */
size_t tbl_grouped_rows_workspace_bytes(int groups, int rows, int max_inputs);
int tbl_grouped_forward_rows(const tbl_linear_view* views_host, int groups, const float* input_dev, int rows,
                             float* output_dev, long long output_stride, int rms_mode, void* workspace_dev,
                             size_t workspace_bytes, void* stream);

/* ---- a stack of linears in one launch --------------------------------------------------------- */

#define TBL_MAX_CHAIN 16

/* Bytes of scratch for tbl_chain_forward (activations between the layers, the barrier words of the persistent
 * kernel and, for shapes that take the layer-by-layer route, one layer's quantiser scratch). */
size_t tbl_chain_workspace_bytes(const tbl_linear_view* views_host, int count, int rows);

/* y = L[count-1]( ... L[1]( L[0](x) ) ): `count` <= TBL_MAX_CHAIN ternary linears applied one after the other to
 * x fp32 [rows, views[0].inputs]; views[i].inputs must equal views[i-1].outputs.  Layer i is exactly one
 * tbl_linear_forward (input RMSNorm when views[i].rms_input, quantiser, ternary GEMV, magnitude, bias) followed,
 * when squared_relu_host != NULL and squared_relu_host[i] != 0, by max(y,0)^2.  y_dev is fp32 [rows, last outputs].
 * With rows <= 8, every view carrying `strips`, inputs % 256 == 0 and rows*inputs <= 16384, the whole stack runs
 * as ONE persistent cooperative kernel: a CTA per SM streams the weights of all layers back to back while the
 * grid meets at a bounded barrier between layers (the weight stream never stops at a layer boundary).  Other
 * shapes run layer by layer through tbl_linear_forward.  rms_mode as in tbl_linear_forward (used by the layers
 * whose view has rms_input set; TBL_RMS_NONE there selects TBL_RMS_FAST).
 * Replaces: a run of BitLinear::forward calls whose only glue is an optional squared ReLU -- the block FFN
 * ffn_gate_up -> squared_relu -> ffn_down (OXN/nsos/src/jamba.cpp:3286-3367), an expert's
 * expert_gate_up -> squared_relu -> expert_down (OXN/nsos/src/jamba.cpp:3938-3941), and the fixed launch
 * sequence the reference replays from a captured graph (JambaModel::forward_ids_decode_graph,
 * OXN/nsos/src/jamba.cpp:2074-2376). */
int tbl_chain_forward(const tbl_linear_view* views_host, int count, const int* squared_relu_host,
                      const float* x_dev, int rows, int rms_mode, float* y_dev, void* workspace_dev,
                      size_t workspace_bytes, void* stream);

/* Column-split layers (one rank per block of output columns, see tbl_linear_forward: each rank writes its
 * [rows, cols] block straight into its slot of the all-gather buffer): gathered_dev fp32 [parts, rows, cols] as the
 * all-gather leaves it -> out_dev fp32 [rows, parts*cols].  Local memory only.  No counterpart in the reference,
 * which has no multi-GPU inference (its optional host-staged MPI layer is OXN/nsos/src/fabric_v2.cpp:192-258). */
int tbl_retile_columns(const float* gathered_dev, int parts, int rows, int cols, float* out_dev, void* stream);

/* Router post-processing on the device: logits fp32 [rows, experts] (the gate's output) -> routing weights
 * [rows, experts] as tbl_moe_forward takes them: softmax, keep the top_k largest per row (ties -> lower
 * index), renormalise, zero the rest; top_k == 0 or >= experts leaves the softmax.  May run in place.
 * Sums follow the reference's order; exp is the device's expf, so weights agree with the CPU path to a few
 * ulp, not bit for bit.  Replaces: Tensor::softmax + moe_topk_mask_kernel / the CPU partial_sort in
 * MoERouter::forward (OXN/nsos/src/tensor.cpp:3402-3450, src/cuda/moe_kernels.cu:32-91,
 * src/jamba.cpp:8268-8296). */
int tbl_router_topk(const float* logits_dev, int rows, int experts, int top_k, float* weights_dev, void* stream);

/* ---- device: the norms either side of a linear ---------------------------------------- */

/* Row-wise RMSNorm x weight, with the SiLU gate that precedes it in the Mamba-2 epilogue and, optionally, the
 * per-token quantiser that follows it, in one launch (one CTA per row, the row kept in shared memory):
 *   gate_dev == NULL:  n = value.rmsnorm(eps) * weight           block norm, OXN/nsos/src/jamba.cpp:3175-3179
 *                                                                (Tensor::rmsnorm, OXN/nsos/src/tensor.cpp:3455-3490)
 *   gate_dev != NULL:  n = (value * silu(gate)).rmsnorm(eps) * weight
 *                      Replaces: launch_mamba_gated_rmsnorm (OXN/nsos/src/cuda/mamba_kernels.cu:3421-3446) and the
 *                      unfused y.mul(z.silu()).rmsnorm(eps).mul(weight) (OXN/nsos/src/mamba2.cpp:4011).
 * value / gate / out are fp32 [rows, dim], weight_dev fp32 [dim] or NULL (no learnable weight).
 * out_dev (may be NULL) receives n.  q_dev (may be NULL; needs dim % 16 == 0) receives the int8 codes of n with
 * act_scales_dev [rows] and, if not NULL, q_sums_dev [rows]: bit for bit what tbl_quantize_rows(n, bits,
 * TBL_RMS_NONE, TBL_TIE_EVEN) gives, ready for tbl_gemm (prefill: no quantiser launch, no fp32 round trip) or
 * tbl_gemv.  At decode sizes prefer out_dev + tbl_linear_forward: its GEMV quantises in its own prologue.
 * At least one of out_dev / q_dev.  dim <= 49152.  fp32 results agree with the reference's CPU ops to 1e-5
 * relative (the sum of squares is a tree, exp is the device's expf), not bit for bit. */
int tbl_row_norm(const float* value_dev, const float* gate_dev, const float* weight_dev, int rows, int dim,
                 float eps, float* out_dev, int bits, int8_t* q_dev, float* act_scales_dev,
                 int32_t* q_sums_dev, void* stream);

/* ---- one decode step of the Mamba-2 / attention hybrid ----------------------------------------- */

/* The streaming single-token step of the reference's model (JambaModel::forward_ids_last on one token per
 * sequence in streaming mode, OXN/nsos/src/jamba.cpp:851-992, 1963-1980; its graph form
 * JambaModel::forward_ids_decode_graph, :2074-2376) for a batch of independent sequences:
 *   embedding gather (OXN/nsos/src/embedding.cpp:618) -> per block { RMSNorm x weight; Mamba-2 branch: x / z / B / C / dt
 *   projections, causal-conv step + SiLU, SSD recurrence step, SiLU-gated RMSNorm, out projection
 *   (Mamba2SSD::forward_faithful_step, OXN/nsos/src/mamba2.cpp:3947-4125; device forms
 *   OXN/nsos/src/cuda/mamba_kernels.cu:3332-3405); hybrid blocks add, in parallel on their own norm of the same
 *   residual stream, attention over the KV cache with RoPE (OXN/nsos/src/jamba.cpp:6291-6295, 6500-6640;
 *   OXN/nsos/src/cuda/kernels.cu:2853-2990), the per-channel gates (OXN/nsos/src/jamba.cpp:3195-3230) and the FFN
 *   up -> squared ReLU -> down (OXN/nsos/src/jamba.cpp:3286-3367) } -> final RMSNorm x weight -> LM head.
 * Every projection is a ternary linear described by a tbl_linear_view (packed mode; `strips` where inputs % 256 == 0
 * gives the fast path).  All pointers are device pointers except `blocks`, which is a host array. */
#define TBL_MAX_DECODE_BLOCKS 128

typedef struct tbl_mamba_block {
    tbl_linear_view x, z;          /* d_model -> d_inner                                   */
    tbl_linear_view B, C;          /* d_model -> n_groups * d_state                        */
    tbl_linear_view dt;            /* d_model -> n_heads (its bias is the dt bias)         */
    tbl_linear_view out;           /* d_inner -> d_model                                   */
    const float* A_log;            /* [n_heads]                                            */
    const float* D;                /* [n_heads]                                            */
    const float* conv_w;           /* [d_inner + 2*n_groups*d_state, conv_kernel]          */
    const float* conv_b;           /* [d_inner + 2*n_groups*d_state]                       */
    const float* norm_w;           /* [d_inner], weight of the gated norm                  */
    int d_inner, n_heads, d_head, n_groups, d_state, conv_kernel;
    float norm_eps;
} tbl_mamba_block;

typedef struct tbl_attention_block {
    tbl_linear_view q;             /* d_model -> n_heads * head_dim                        */
    tbl_linear_view kv;            /* d_model -> 2 * n_kv_heads * head_dim (k then v)      */
    tbl_linear_view out;           /* d_model -> d_model                                   */
    const float* rope_cos;         /* [rope_positions, head_dim / 2]                       */
    const float* rope_sin;
    int n_heads, n_kv_heads, head_dim, sliding_window, rope_positions;
} tbl_attention_block;

typedef struct tbl_decode_block {
    int hybrid;                    /* 0: x + mamba(norm(x)); 1: gated mamba + attention, then the gated FFN */
    const float* core_norm_w;      /* [d_model] or NULL                                    */
    float core_norm_eps;
    tbl_mamba_block mamba;
    /* hybrid blocks only */
    const float* attn_norm_w;      /* [d_model] or NULL                                    */
    const float* ff_norm_w;        /* [d_model] or NULL                                    */
    const float* mamba_gate;       /* [d_model]                                            */
    const float* attn_gate;        /* [d_model]                                            */
    const float* ffn_gate;         /* [d_model]                                            */
    tbl_attention_block attn;
    tbl_linear_view ffn_up, ffn_down;
} tbl_decode_block;

typedef struct tbl_decode_model {
    int d_model, vocab, n_blocks;
    const float* embedding;        /* [vocab, d_model]                                     */
    const tbl_decode_block* blocks;/* HOST array of n_blocks entries                       */
    const float* final_norm_w;     /* [d_model] or NULL                                    */
    float final_norm_eps;
    tbl_linear_view head;          /* d_model -> vocab                                     */
} tbl_decode_model;

/* The glue kernels of the step, one entry point each (all enqueue on `stream`, fp32, row-major).
 *
 * tbl_embedding_gather: out[i,:] = table[ids[i],:], a zero row for an id outside [0, vocab).
 *   Replaces: launch_embedding_gather_kernel (OXN/nsos/src/cuda/kernels.cu:639), Embedding::forward
 *   (OXN/nsos/src/embedding.cpp:618).
 * tbl_mamba_conv_step: causal depthwise conv over the concatenated channels [x | B | C] with the window kept in
 *   ring_dev [rows, conv_kernel-1, d_inner + 2*group_state] (oldest tap first; shifted here), bias, SiLU.
 *   Replaces: launch_mamba2_faithful_conv_step (OXN/nsos/src/cuda/mamba_kernels.cu:3332-3359),
 *   host form OXN/nsos/src/mamba2.cpp:4062-4094.
 * tbl_mamba_ssd_step: h = decay*h + delta*B*x, y = D*x + sum_n h*C with delta = softplus(dt),
 *   decay = exp(-delta*exp(A_log)) (in double); state_dev [rows, n_heads*d_head, d_state] is updated.
 *   Replaces: launch_mamba2_faithful_step (OXN/nsos/src/cuda/mamba_kernels.cu:3376-3405), host form
 *   OXN/nsos/src/mamba2.cpp:443-473, 4096-4118.
 * tbl_attention_decode: one new token per row: RoPE (halves i / i + head_dim/2) on q and k at positions_dev[row],
 *   k | v appended to the caches [rows, capacity, n_kv_heads*head_dim], softmax(q.k / sqrt(head_dim)) over the last
 *   sliding_window tokens, weighted sum of v -> out [rows, n_heads*head_dim].  positions_dev is NOT advanced.
 *   Replaces: launch_gqa_append_kv_cache_kernel + launch_gqa_cached_attention_decode_kernel
 *   (OXN/nsos/src/cuda/kernels.cu:2853-2990), host form OXN/nsos/src/jamba.cpp:5140-5190, 6520-6640.
 * tbl_gated_residual: out = x + (a*gate_a [+ b*gate_b]) with per-channel gates [dim]; gate_a NULL: out = x + a.
 *   Replaces: the Tensor mul/add chains of JambaBlock::forward (OXN/nsos/src/jamba.cpp:3224-3251, 3367-3371). */
int tbl_embedding_gather(const int32_t* ids_dev, int count, const float* table_dev, int vocab, int dim, float* out_dev,
                         void* stream);
int tbl_mamba_conv_step(const float* x_dev, const float* B_dev, const float* C_dev, const float* conv_w_dev,
                        const float* conv_b_dev, float* ring_dev, float* xbc_dev, int d_inner, int group_state,
                        int conv_kernel, int rows, void* stream);
int tbl_mamba_ssd_step(const float* xbc_dev, const float* dt_dev, const float* A_log_dev, const float* D_dev,
                       float* state_dev, float* y_dev, int n_heads, int d_head, int d_state, int n_groups, int rows,
                       void* stream);
int tbl_attention_decode(const float* q_dev, const float* kv_dev, float* k_cache_dev, float* v_cache_dev, int capacity,
                         const int32_t* positions_dev, const float* rope_cos_dev, const float* rope_sin_dev,
                         int rope_positions, int n_heads, int n_kv_heads, int head_dim, int sliding_window, int rows,
                         float* out_dev, void* stream);
int tbl_gated_residual(const float* x_dev, const float* a_dev, const float* gate_a_dev, const float* b_dev,
                       const float* gate_b_dev, int rows, int dim, float* out_dev, void* stream);

/* Device state of `batch` sequences with room for `capacity` cached tokens each (positions, conv windows, SSM
 * states, KV caches): size, and reset to the empty session (JambaModel::reset_session + reserve_kv_cache). */
size_t tbl_decode_state_bytes(const tbl_decode_model* model, int batch, int capacity);
int tbl_decode_state_reset(const tbl_decode_model* model, int batch, int capacity, void* state_dev, size_t state_bytes,
                           void* stream);
size_t tbl_decode_workspace_bytes(const tbl_decode_model* model, int batch);

/* Enqueues one step: token_ids_dev int32 [batch] -> logits_dev fp32 [batch, vocab]; the state advances by one
 * token per sequence (positions live on the device, so a captured step can be replayed).  hidden_trace_dev
 * (may be NULL) receives the residual stream fp32 [n_blocks + 1, batch, d_model]: the embedding rows, then the
 * stream after every block.  state_dev and workspace_dev must be 256-byte aligned.  A sequence whose cache is
 * full is reported through the device status (TBL_DEV_CACHE_FULL).  fp32 results agree with the reference's CPU
 * path to ~1e-5 relative per operation (device expf / exp / log, tree-shaped norm and softmax sums), not bit for
 * bit; the ternary linears themselves are bit-exact on identical inputs. */
int tbl_decode_step(const tbl_decode_model* model, int batch, int capacity, void* state_dev,
                    const int32_t* token_ids_dev, float* logits_dev, float* hidden_trace_dev, void* workspace_dev,
                    size_t workspace_bytes, void* stream);

/* Bytes of scratch for tbl_moe_forward. */
size_t tbl_moe_workspace_bytes(int rows, int dim, int hidden_dim, int experts, int max_routes_per_row);

/* MoE expert FFN: out[r,:] = sum_e routing[r,e] * down_e(relu(up_e(x_r))^2), experts summed in
 * index order, experts with routing weight 0 skipped (their weights are never read).
 * views_host holds 2*experts views: [0,E) the up linears (dim -> hidden_dim), [E,2E) the down
 * linears (hidden_dim -> dim).  routing_dev fp32 [rows,experts].  At most max_routes_per_row
 * non-zero routing weights per row (else the device status reports TBL_DEV_ROUTE_OVERFLOW).
 * With >= 16 routed rows per expert on average and `w_i8` set in every view, both expert stages run as
 * one grouped tensor-core GEMM each (row counts stay on the device); otherwise on the strip / canonical
 * GEMV path.
 * Replaces: launch_moe_sparse_decode (OXN/nsos/src/cuda/moe_kernels.cu:786-795) and the CPU
 * composition in JambaBlock::forward_moe (OXN/nsos/src/jamba.cpp:3865-3972). */
int tbl_moe_forward(const tbl_linear_view* views_host, const float* routing_dev, const float* x_dev,
                    int rows, int dim, int hidden_dim, int experts, int max_routes_per_row,
                    int rms_mode, int tie_mode, float* out_dev,
                    void* workspace_dev, size_t workspace_bytes, void* stream);

/* ---- edge-linear pack ("DGE1") ---------------------------------------------------------- */

/* The file in which the reference ships a model's packed linears (JambaModel::save_edge_linear_pack /
 * load_edge_linear_pack, OXN/nsos/src/jamba.cpp:1325-1663; helpers :505-606; format in csrc/edge_pack.cpp).
 * Host only, over a memory image of the file.  Payload offsets are in bytes from the start of the image and
 * are NOT aligned (copy out with memcpy). */
typedef struct tbl_edge_layer {
    int sensitive, in_features, out_features, use_bias;
    float weight_scale;
    uint64_t packed_offset, packed_words;        /* canonical 2-bit words, ceil(in*out/16)          */
    uint64_t magnitude_offset;                   /* fp32 [out]                                       */
    uint64_t bias_offset;                        /* fp32 [out] when use_bias                         */
    uint64_t flat_alpha_offset, flat_beta_offset;/* fp32 [in] each                                   */
    uint64_t weight_offset, weight_count;        /* fp32 [out*in] of a sensitive layer, else 0       */
} tbl_edge_layer;

typedef struct tbl_edge_layer_src {
    int sensitive, in_features, out_features, use_bias;
    float weight_scale;
    const uint32_t* packed;
    const float* magnitude;
    const float* bias;
    const float* flat_alpha;
    const float* flat_beta;
    const float* weight;                         /* sensitive layers only */
} tbl_edge_layer_src;

/* Validates the whole image (header, every layer's lengths / finite values / scale / codes, nothing after the
 * last layer, version-3 trailer length and SHA-256) and reports version (2 or 3) and layer count.
 * Replaces: the parsing and validation half of load_edge_linear_pack (jamba.cpp:1451-1616). */
int tbl_edge_pack_open(const void* data, size_t bytes, int* version_out, int* layers_out);
/* Layer `index` of a pack that tbl_edge_pack_open accepted: walks the record headers up to it and scans only that
 * layer's payload; the digest is not recomputed. */
int tbl_edge_pack_layer(const void* data, size_t bytes, int index, tbl_edge_layer* out);
/* Everything in one pass: digest, full validation and every layer record (`capacity` entries; TBL_ERR_WORKSPACE
 * with *layers_out set when there are more).  Loading a pack costs one hash and one scan of the file. */
int tbl_edge_pack_layers(const void* data, size_t bytes, tbl_edge_layer* out, int capacity, int* version_out,
                         int* layers_out);
/* Size of, and writer for, a version-3 pack.  Replaces: save_edge_linear_pack's serialisation
 * (jamba.cpp:1345-1439); the caller does the atomic temp-file replace. */
size_t tbl_edge_pack_bytes(const tbl_edge_layer_src* layers, int count);
int tbl_edge_pack_write(const tbl_edge_layer_src* layers, int count, void* out, size_t capacity, size_t* written);
/* Lower-case hex SHA-256 of a buffer (the trailer's digest; integrity::sha256_hex,
 * OXN/nsos/include/nsos/sha256.h:12). */
void tbl_sha256_hex(const void* data, size_t bytes, char out[65]);

/* ---- device status ---------------------------------------------------------------------- */
#define TBL_DEV_OK 0
#define TBL_DEV_WAIT_TIMEOUT 1     /* a bounded mbarrier / TMA wait gave up                */
#define TBL_DEV_ROUTE_OVERFLOW 2   /* a row had more routes than max_routes_per_row        */
#define TBL_DEV_CACHE_FULL 4       /* decode step: a sequence's KV cache or rotary table is full */

/* Synchronises `stream`, returns the sticky device status word of the current device and
 * clears it.  Negative on a CUDA error. */
int tbl_device_status(void* stream);

/* Self-test of the give-up path of the device-side waits: launches one CTA that waits, with a limit of 4096 polls,
 * on a barrier nobody arrives on.  The kernel must return on its own (within milliseconds), write 1 to *gave_up_dev
 * and leave TBL_DEV_WAIT_TIMEOUT in the device status word; the context stays usable.  No counterpart in the
 * reference, whose kernels have no inter-thread waits. */
int tbl_selftest_bounded_wait(int* gave_up_dev, void* stream);

/* Profiling aid: while set (non-NULL cudaEvent_t handles), every launch of the decode GEMV kernel
 * records `start_event` just before and `stop_event` just after it on its stream, so a harness can
 * time that kernel alone with cudaEventElapsedTime.  Pass NULLs to switch it off.  Process-wide.
 * Replaces: the per-kernel timing the reference's benchmarks take around launch_bitnet_gemv_scaled
 * (OXN/nsos/benchmarks/bench_decode_gemv.cpp:75-90). */
void tbl_set_kernel_events(void* start_event, void* stop_event);

/* Profiling aid for tbl_chain_forward's persistent kernel: while a device buffer of at least
 * CTAs * count * 8 * sizeof(uint64_t) bytes is set (CTAs = SM count of the device), each CTA records, per layer,
 * globaltimer nanosecond stamps: [0] layer entered, [1] grid barrier passed, [2] input quantised, [3] first
 * weight stage landed, [4] last stage consumed, [5] outputs stored, [6] arrived on the layer's counter,
 * [7] producer warp finished issuing the layer's copies.  Pass NULL to switch it off.  Process-wide.
 * Replaces: the per-layer timing the reference prints with NSOS_LAYER_TIMING=1 (OXN/nsos/src/jamba.cpp:902-963). */
void tbl_set_chain_trace(void* buffer_dev, size_t bytes);

/* Number of kernels this library has launched in this process (all streams). */
uint64_t tbl_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TERNARY_B200_H */
