// extern "C" entry points: validation, workspace carving and kernel selection.  No allocation,
// no synchronisation (except tbl_device_status), no exceptions across the boundary.
#include <atomic>
#include <climits>
#include <cmath>

#include "common.cuh"
#include "kernels.cuh"

namespace tbl {

static std::atomic<uint64_t> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? TBL_OK : TBL_ERR_CUDA; }

// Shape rules shared by every device entry point; they are the reference's own
// (bitnet_gemm_158bit_gpu: positive sizes, K % 16 == 0, K <= INT_MAX/254, M*N <= INT_MAX,
// finite positive scale, bits in [2,8]).
int check_problem(int M, int K, int N, float weight_scale, int bits) {
    if (M <= 0 || K <= 0 || N <= 0) return TBL_ERR_INVALID_ARG;
    if (bits < 2 || bits > 8) return TBL_ERR_BITS;
    if (K > INT_MAX / 254) return TBL_ERR_OVERFLOW;
    if (!std::isfinite(weight_scale) || weight_scale <= 0.0f) return TBL_ERR_SCALE;
    if (K % 16 != 0) return TBL_ERR_SHAPE;
    if (static_cast<int64_t>(M) * N > INT_MAX) return TBL_ERR_SHAPE;
    return TBL_OK;
}

struct Workspace {
    int8_t* q;
    int8_t* qp;
    float* act_scales;
    int32_t* q_sums;
    float* inv_norm;
    size_t bytes;
};

constexpr int kWidenMinRows = 32;     // more rows than this (and <= 256, K % 256 == 0): the widening tensor-core kernel

Workspace carve(void* base, int M, int K) {
    Workspace w;
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    const size_t mk = round_up(static_cast<size_t>(M) * K, 256);
    w.q = reinterpret_cast<int8_t*>(p + off); off += mk;
    // the second copy is the interleaved one (M * K bytes) or the plane-major one (rows padded to 512 codes)
    w.qp = reinterpret_cast<int8_t*>(p + off); off += round_up(static_cast<size_t>(M) * round_up(static_cast<size_t>(K), 512), 256);
    const size_t vec = round_up(static_cast<size_t>(M) * 4, 256);
    w.act_scales = reinterpret_cast<float*>(p + off); off += vec;
    w.q_sums = reinterpret_cast<int32_t*>(p + off); off += vec;
    w.inv_norm = reinterpret_cast<float*>(p + off); off += vec;
    w.bytes = off;
    return w;
}

// Mid-size batches (kWidenMinRows < M <= 256) of up to kWidenMaxViews weight matrices that share the input rows: the
// rows are quantised once, straight into the plane-major layout where the register quantiser serves the width, and
// every pass of up to 128 rows is one launch of the widening tensor-core kernel over all the matrices.
bool widen_rows_ok(int M, int K) { return M > kWidenMinRows && M <= 2 * 128 && K >= 256 && (K & 255) == 0; }

int widen_forward(const WidenView* views, int count, const float* x, int M, int K, int bits, int rms_mode,
                  const Workspace& w, cudaStream_t st) {
    const int ld = gemm_widen_plane_ld(K);
    const bool direct = K <= 32768;            // the register quantiser writes the planes itself
    cudaError_t e = launch_quantize_rows(x, nullptr, M, K, bits, rms_mode, TBL_TIE_EVEN, direct ? nullptr : w.q,
                                         direct ? w.qp : nullptr, w.act_scales, w.q_sums, w.inv_norm, nullptr,
                                         QuantSegments{}, st, direct ? ld : 0);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    for (int m0 = 0; m0 < M; m0 += 128) {
        const int rows = M - m0 < 128 ? M - m0 : 128;
        WidenView pass[kWidenMaxViews];
        for (int v = 0; v < count; ++v) {
            pass[v] = views[v];
            pass[v].y = views[v].y + static_cast<size_t>(m0) * views[v].N;
        }
        e = launch_gemm_widen(pass, count, direct ? nullptr : w.q + static_cast<size_t>(m0) * K,
                              w.qp + static_cast<size_t>(m0) * ld, w.act_scales + m0, w.q_sums + m0, rows, K, st);
        if (e != cudaSuccess) return TBL_ERR_CUDA;
    }
    return TBL_OK;
}

// GEMV on already-quantised activations for any M (the tensor-core kernel walks M in tiles of 64).
int run_gemv(const int8_t* q, const int8_t* qp, const float* act_scales, const int32_t* q_sums,
             const uint32_t* words, const void* strips, float weight_scale, const float* magnitude,
             const float* bias, int M, int K, int N, float* y, int32_t* acc_debug, cudaStream_t stream) {
    if (qp && strips && gemv_strip_supported(K)) {
        StripProblem pr{};
        pr.strips = static_cast<const uint8_t*>(strips); pr.qp = qp; pr.act_scales = act_scales;
        pr.q_sums = q_sums; pr.magnitude = magnitude; pr.bias = bias; pr.y = y; pr.acc_debug = acc_debug;
        pr.weight_scale = weight_scale; pr.rows = M; pr.N = N; pr.K = K; pr.ldy = N;
        return cuda_status(launch_gemv_strip(&pr, 1, stream));
    }
    if (!words || !q) return TBL_ERR_INVALID_ARG;
    if (M <= 4 && gemv_small_supported(M, K, N) && aligned16(words) && aligned16(q)) {
        GemvSmallArgs a{};
        a.q = q; a.act_scales = act_scales; a.words = words; a.magnitude = magnitude; a.bias = bias;
        a.y = y; a.acc_debug = acc_debug; a.weight_scale = weight_scale; a.q_max = 127.0f;
        a.M = M; a.K = K; a.N = N; a.rms_mode = TBL_RMS_NONE;
        return cuda_status(launch_gemv_small(a, stream));
    }
    return cuda_status(launch_gemv_generic(q, act_scales, words, weight_scale, magnitude, bias, M, K, N, y,
                                           acc_debug, 0, nullptr, nullptr, stream));
}

}  // namespace
}  // namespace tbl

namespace tbl {
namespace {
// One CTA waits, with a limit of a few thousand polls, on an mbarrier nobody arrives on: the wait runs out, the
// kernel records it and returns.  Exercises the give-up path every pipelined kernel of the library shares.
__global__ void bounded_wait_selftest_kernel(int* status, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    const bool ok = mbar_wait_bounded(&bar, 0, status, 4096);
    if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}
}  // namespace
}  // namespace tbl


using namespace tbl;

extern "C" {

const char* tbl_status_string(int status) {
    switch (status) {
        case TBL_OK: return "ok";
        case TBL_ERR_INVALID_ARG: return "invalid argument (null pointer, non-positive size or bad flag)";
        case TBL_ERR_SHAPE: return "unsupported shape (K must be a multiple of 16, M*N <= INT_MAX, M within the kernel's range)";
        case TBL_ERR_OVERFLOW: return "K too large: int32 accumulation could overflow";
        case TBL_ERR_SCALE: return "weight_scale must be finite and positive";
        case TBL_ERR_BITS: return "activation bits must be in [2,8]";
        case TBL_ERR_ALIGNMENT: return "device pointer must be 16-byte aligned";
        case TBL_ERR_WORKSPACE: return "workspace too small";
        case TBL_ERR_FORMAT: return "edge pack malformed";
        case TBL_ERR_INTEGRITY: return "edge pack integrity trailer missing or digest mismatch";
        case TBL_ERR_CODE: return "packed words contain the reserved code 0b11";
        case TBL_ERR_CUDA: return "CUDA runtime error";
        case TBL_ERR_UNSUPPORTED: return "descriptor mode not implemented";
        default: return "unknown status";
    }
}

int tbl_abi_version(void) { return 3; }

uint64_t tbl_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void tbl_set_kernel_events(void* start_event, void* stop_event) {
    set_gemv_events(static_cast<cudaEvent_t>(start_event), static_cast<cudaEvent_t>(stop_event));
}

void tbl_set_chain_trace(void* buffer_dev, size_t bytes) { set_chain_trace(buffer_dev, bytes); }

int tbl_selftest_bounded_wait(int* gave_up_dev, void* stream) {
    if (!gave_up_dev) return TBL_ERR_INVALID_ARG;
    int* status = device_status_ptr();
    if (!status) return TBL_ERR_CUDA;
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, gave_up_dev);
    note_launch();
    return cuda_status(cudaGetLastError());
}

int tbl_device_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    int status = 0;
    if (read_and_clear_device_status(&status) != 0) return TBL_ERR_CUDA;
    return status;
}

size_t tbl_strip_bytes(int N, int K) {
    if (N <= 0 || K <= 0 || K % 256 != 0) return 0;
    return static_cast<size_t>((N + 15) / 16) * 16 * (K / 4);
}

int tbl_relayout_strips(const uint32_t* words_dev, int N, int K, void* strips_dev, void* stream) {
    if (!words_dev || !strips_dev || N <= 0 || K <= 0) return TBL_ERR_INVALID_ARG;
    if (!gemv_strip_supported(K)) return TBL_ERR_SHAPE;
    if (!aligned16(words_dev) || !aligned16(strips_dev)) return TBL_ERR_ALIGNMENT;
    return cuda_status(launch_relayout_strips(words_dev, N, K, strips_dev, static_cast<cudaStream_t>(stream)));
}

int tbl_expand_weights_i8(const uint32_t* words_dev, int N, int K, int8_t* w_i8_dev, void* stream) {
    if (!words_dev || !w_i8_dev || N <= 0 || K <= 0) return TBL_ERR_INVALID_ARG;
    if (!aligned16(words_dev) || !aligned16(w_i8_dev)) return TBL_ERR_ALIGNMENT;
    return cuda_status(launch_expand_i8(words_dev, N, K, w_i8_dev, static_cast<cudaStream_t>(stream)));
}

int tbl_quantize_rows(const float* x_dev, const int32_t* row_index_dev, int M, int K, int bits, int rms_mode,
                      int tie_mode, int8_t* q_dev, float* act_scales_dev, int32_t* q_sums_dev, void* stream) {
    if (!x_dev || !q_dev || !act_scales_dev || M <= 0 || K <= 0) return TBL_ERR_INVALID_ARG;
    if (bits < 2 || bits > 8) return TBL_ERR_BITS;
    if (rms_mode != TBL_RMS_NONE && rms_mode != TBL_RMS_FAST) {
        // the reference-order factor needs one float of scratch per row; this entry point has no
        // workspace argument, so only the layer-level calls offer that mode
        return TBL_ERR_INVALID_ARG;
    }
    if (tie_mode != TBL_TIE_EVEN && tie_mode != TBL_TIE_AWAY) return TBL_ERR_INVALID_ARG;
    return cuda_status(launch_quantize_rows(x_dev, row_index_dev, M, K, bits, rms_mode, tie_mode, q_dev,
                                            nullptr, act_scales_dev, q_sums_dev, nullptr, nullptr,
                                            QuantSegments{}, static_cast<cudaStream_t>(stream)));
}

size_t tbl_gemv_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return round_up(static_cast<size_t>(M) * K, 256) + round_up(static_cast<size_t>(M) * 4, 256);
}

int tbl_gemv(const int8_t* q_dev, const float* act_scales_dev, const uint32_t* words_dev, const void* strips_dev,
             float weight_scale, const float* magnitude_dev, const float* bias_dev, int M, int K, int N,
             float* y_dev, int32_t* acc_debug_dev, void* workspace_dev, size_t workspace_bytes, void* stream) {
    if (!q_dev || !act_scales_dev || (!words_dev && !strips_dev) || !y_dev) return TBL_ERR_INVALID_ARG;
    const int rc = check_problem(M, K, N, weight_scale, 8);
    if (rc != TBL_OK) return rc;
    if (M > 64) return TBL_ERR_SHAPE;
    if (!aligned16(q_dev) || (words_dev && !aligned16(words_dev)) || (strips_dev && !aligned16(strips_dev)))
        return TBL_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int8_t* qp = nullptr;
    int32_t* q_sums = nullptr;
    const bool strip = strips_dev != nullptr && gemv_strip_supported(K);
    if (!strip && !words_dev) return TBL_ERR_SHAPE;
    if (strip) {
        if (!workspace_dev || workspace_bytes < tbl_gemv_workspace_bytes(M, K)) return TBL_ERR_WORKSPACE;
        if (!aligned16(workspace_dev)) return TBL_ERR_ALIGNMENT;
        qp = static_cast<int8_t*>(workspace_dev);
        q_sums = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace_dev) +
                                            round_up(static_cast<size_t>(M) * K, 256));
        const cudaError_t e = launch_permute_q(q_dev, M, K, qp, q_sums, st);
        if (e != cudaSuccess) return TBL_ERR_CUDA;
    }
    return run_gemv(q_dev, qp, act_scales_dev, q_sums, words_dev, strip ? strips_dev : nullptr, weight_scale,
                    magnitude_dev, bias_dev, M, K, N, y_dev, acc_debug_dev, st);
}

int tbl_gemm(const int8_t* q_dev, const float* act_scales_dev, const int8_t* w_i8_dev, float weight_scale,
             const float* magnitude_dev, const float* bias_dev, int M, int K, int N, float* y_dev,
             int32_t* acc_debug_dev, void* stream) {
    if (!q_dev || !act_scales_dev || !w_i8_dev || !y_dev) return TBL_ERR_INVALID_ARG;
    const int rc = check_problem(M, K, N, weight_scale, 8);
    if (rc != TBL_OK) return rc;
    if (!aligned16(q_dev) || !aligned16(w_i8_dev)) return TBL_ERR_ALIGNMENT;
    return cuda_status(launch_gemm_tcgen05(q_dev, act_scales_dev, w_i8_dev, weight_scale, magnitude_dev,
                                           bias_dev, M, K, N, y_dev, acc_debug_dev,
                                           static_cast<cudaStream_t>(stream)));
}

size_t tbl_linear_workspace_bytes(int M, int K, int N) {
    (void)N;
    if (M <= 0 || K <= 0) return 0;
    return carve(nullptr, M, K).bytes;
}

int tbl_linear_forward(const float* x_dev, const uint32_t* words_dev, const void* strips_dev,
                       const int8_t* w_i8_dev, float weight_scale, int M, int K, int N, int bits, int rms_mode,
                       const float* magnitude_dev, const float* bias_dev, float* y_dev, void* workspace_dev,
                       size_t workspace_bytes, void* stream) {
    if (!x_dev || !y_dev) return TBL_ERR_INVALID_ARG;
    const int rc = check_problem(M, K, N, weight_scale, bits);
    if (rc != TBL_OK) return rc;
    if (rms_mode < TBL_RMS_NONE || rms_mode > TBL_RMS_REFERENCE_ORDER) return TBL_ERR_INVALID_ARG;
    if (!aligned16(x_dev) || (words_dev && !aligned16(words_dev)) || (strips_dev && !aligned16(strips_dev)) ||
        (w_i8_dev && !aligned16(w_i8_dev)))
        return TBL_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool use_gemm = w_i8_dev != nullptr && M > 64;
    const bool strip = !use_gemm && strips_dev != nullptr && gemv_strip_supported(K);
    if (!use_gemm && !strip && !words_dev) return TBL_ERR_INVALID_ARG;

    // canonical words only, M <= 4: one kernel, the quantiser runs in the GEMV's prologue
    if (!use_gemm && !strip && M <= 4 && rms_mode != TBL_RMS_REFERENCE_ORDER && gemv_small_supported(M, K, N)) {
        GemvSmallArgs a{};
        a.x = x_dev; a.words = words_dev; a.magnitude = magnitude_dev; a.bias = bias_dev; a.y = y_dev;
        a.weight_scale = weight_scale; a.q_max = qmax_for_bits(bits);
        a.M = M; a.K = K; a.N = N; a.rms_mode = rms_mode;
        return cuda_status(launch_gemv_small(a, st));
    }

    // few rows on the strip layout: one kernel, the quantiser runs in the GEMV's prologue while the
    // first weight stages are already in flight
    if (strip && rms_mode != TBL_RMS_REFERENCE_ORDER && M <= gemv_strip_fused_rows(K)) {
        StripProblem pr{};
        pr.strips = static_cast<const uint8_t*>(strips_dev); pr.x = x_dev; pr.q_max = qmax_for_bits(bits);
        pr.rms_fast = rms_mode == TBL_RMS_FAST; pr.magnitude = magnitude_dev; pr.bias = bias_dev; pr.y = y_dev;
        pr.weight_scale = weight_scale; pr.rows = M; pr.N = N; pr.K = K; pr.ldy = N;
        return cuda_status(launch_gemv_strip(&pr, 1, st));
    }

    if (!workspace_dev || workspace_bytes < tbl_linear_workspace_bytes(M, K, N)) return TBL_ERR_WORKSPACE;
    if (!aligned16(workspace_dev)) return TBL_ERR_ALIGNMENT;
    const Workspace w = carve(workspace_dev, M, K);
    // mid-size batches on the strip-major 2-bit weights: widened in shared memory, multiplied on the tcgen05 tensor cores, up to
    // 128 rows per pass (the plane-major copy of the codes takes the place of the interleaved one in the workspace)
    if (strip && widen_rows_ok(M, K)) {
        WidenView v{};
        v.strips = strips_dev; v.magnitude = magnitude_dev; v.bias = bias_dev; v.y = y_dev; v.weight_scale = weight_scale; v.N = N;
        return widen_forward(&v, 1, x_dev, M, K, bits, rms_mode, w, st);
    }
    // the strip GEMV reads only the interleaved copy; the other paths read the row-major codes
    cudaError_t e = launch_quantize_rows(x_dev, nullptr, M, K, bits, rms_mode, TBL_TIE_EVEN, strip ? nullptr : w.q,
                                         strip ? w.qp : nullptr, w.act_scales, w.q_sums, w.inv_norm, nullptr,
                                         QuantSegments{}, st);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    if (use_gemm)
        return cuda_status(launch_gemm_tcgen05(w.q, w.act_scales, w_i8_dev, weight_scale, magnitude_dev,
                                               bias_dev, M, K, N, y_dev, nullptr, st));
    return run_gemv(strip ? nullptr : w.q, strip ? w.qp : nullptr, w.act_scales, w.q_sums, words_dev,
                    strip ? strips_dev : nullptr, weight_scale, magnitude_dev, bias_dev, M, K, N, y_dev, nullptr, st);
}

int tbl_linear_forward_scatter(const float* x_dev, const int8_t* w_i8_dev, float weight_scale, int M, int K, int N,
                               int bits, int rms_mode, const float* magnitude_dev, const float* bias_dev,
                               float* const* y_dest_host, int n_dest, long long ldy, long long col0,
                               void* workspace_dev, size_t workspace_bytes, void* stream) {
    if (!x_dev || !w_i8_dev || !y_dest_host) return TBL_ERR_INVALID_ARG;
    const int rc = check_problem(M, K, N, weight_scale, bits);
    if (rc != TBL_OK) return rc;
    if (rms_mode < TBL_RMS_NONE || rms_mode > TBL_RMS_REFERENCE_ORDER) return TBL_ERR_INVALID_ARG;
    if (n_dest < 1 || n_dest > TBL_MAX_PEERS || ldy < col0 + N || col0 < 0) return TBL_ERR_INVALID_ARG;
    if (M <= 64) return TBL_ERR_UNSUPPORTED;
    if ((N & 3) || (ldy & 3) || (col0 & 3)) return TBL_ERR_ALIGNMENT;
    if (!aligned16(x_dev) || !aligned16(w_i8_dev)) return TBL_ERR_ALIGNMENT;
    GemmScatter sc{};
    sc.count = n_dest; sc.ld = ldy; sc.col0 = col0;
    for (int d = 0; d < n_dest; ++d) {
        if (!y_dest_host[d]) return TBL_ERR_INVALID_ARG;
        if (!aligned16(y_dest_host[d])) return TBL_ERR_ALIGNMENT;
        sc.dest[d] = y_dest_host[d];
    }
    if (!workspace_dev || workspace_bytes < tbl_linear_workspace_bytes(M, K, N)) return TBL_ERR_WORKSPACE;
    if (!aligned16(workspace_dev)) return TBL_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const Workspace w = carve(workspace_dev, M, K);
    cudaError_t e = launch_quantize_rows(x_dev, nullptr, M, K, bits, rms_mode, TBL_TIE_EVEN, w.q, nullptr, w.act_scales,
                                         w.q_sums, w.inv_norm, nullptr, QuantSegments{}, st);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    return cuda_status(launch_gemm_tcgen05(w.q, w.act_scales, w_i8_dev, weight_scale, magnitude_dev, bias_dev, M, K, N,
                                           nullptr, nullptr, st, &sc));
}

}  // extern "C"

namespace tbl {

// tbl_linear_forward on a view, optionally followed by max(y,0)^2: fused into the strip GEMV's epilogue where that
// kernel serves the shape (one launch), a separate elementwise pass otherwise.
int linear_view_forward(const tbl_linear_view& v, const float* x, int rows, int rms_mode, bool squared_relu, float* y,
                        void* workspace, size_t workspace_bytes, cudaStream_t st) {
    const int mode = v.rms_input ? (rms_mode == TBL_RMS_NONE ? TBL_RMS_FAST : rms_mode) : TBL_RMS_NONE;
    if (squared_relu && v.strips && aligned16(v.strips) && gemv_strip_supported(v.inputs) && mode != TBL_RMS_REFERENCE_ORDER &&
        rows <= gemv_strip_fused_rows(v.inputs)) {
        StripProblem pr{};
        pr.strips = static_cast<const uint8_t*>(v.strips); pr.x = x; pr.q_max = qmax_for_bits(v.activation_bits);
        pr.rms_fast = mode == TBL_RMS_FAST; pr.magnitude = v.magnitude; pr.bias = v.bias; pr.y = y;
        pr.weight_scale = v.weight_scale; pr.rows = rows; pr.N = v.outputs; pr.K = v.inputs; pr.ldy = v.outputs;
        pr.squared_relu = 1;
        return cuda_status(launch_gemv_strip(&pr, 1, st));
    }
    if (squared_relu && v.strips && aligned16(v.strips) && aligned16(x) && gemv_strip_supported(v.inputs) &&
        !(v.w_i8 && rows > 64) && widen_rows_ok(rows, v.inputs) &&
        check_problem(rows, v.inputs, v.outputs, v.weight_scale, v.activation_bits) == TBL_OK) {
        // mid-size batches: the widening tensor-core kernel squares in its epilogue too
        if (!workspace || workspace_bytes < tbl_linear_workspace_bytes(rows, v.inputs, v.outputs)) return TBL_ERR_WORKSPACE;
        if (!aligned16(workspace)) return TBL_ERR_ALIGNMENT;
        WidenView wv{};
        wv.strips = v.strips; wv.magnitude = v.magnitude; wv.bias = v.bias; wv.y = y; wv.weight_scale = v.weight_scale;
        wv.N = v.outputs; wv.squared_relu = 1;
        return widen_forward(&wv, 1, x, rows, v.inputs, v.activation_bits, mode, carve(workspace, rows, v.inputs), st);
    }
    const int rc = tbl_linear_forward(x, v.packed, v.strips, rows > 64 ? v.w_i8 : nullptr, v.weight_scale, rows, v.inputs,
                                      v.outputs, v.activation_bits, mode, v.magnitude, v.bias, y, workspace, workspace_bytes, st);
    if (rc != TBL_OK || !squared_relu) return rc;
    return cuda_status(launch_squared_relu(y, static_cast<int64_t>(rows) * v.outputs, st));
}

}  // namespace tbl

namespace tbl {

namespace {
bool prologue_ok(const StripPrologue& pre) {
    const void* ptrs[] = {pre.a, pre.ga, pre.b, pre.gb, pre.norm_w, pre.hidden_out, pre.trace_out};
    for (const void* q : ptrs)
        if (q && (reinterpret_cast<uintptr_t>(q) & 15)) return false;
    return (pre.b == nullptr) == (pre.gb == nullptr) && (pre.a != nullptr || (pre.ga == nullptr && pre.b == nullptr));
}
}  // namespace

int grouped_forward_rows_pre(const tbl_linear_view* views, int groups, const float* x, int rows, float* out,
                             long long out_stride, const StripPrologue& pre, cudaStream_t st) {
    if (!views || !x || !out || groups <= 0 || groups > TBL_MAX_GROUPS || rows <= 0) return TBL_ERR_INVALID_ARG;
    const int K = views[0].inputs;
    if (!gemv_strip_supported(K) || rows > gemv_strip_fused_rows(K) || !prologue_ok(pre) ||
        (reinterpret_cast<uintptr_t>(x) & 15))
        return TBL_ERR_UNSUPPORTED;
    StripProblem pr[TBL_MAX_GROUPS];
    for (int g = 0; g < groups; ++g) {
        const tbl_linear_view& v = views[g];
        if (!v.strips || (reinterpret_cast<uintptr_t>(v.strips) & 15) || v.inputs != K || v.weight != nullptr ||
            v.activation_bits != views[0].activation_bits || (v.rms_input != 0) != (views[0].rms_input != 0))
            return TBL_ERR_UNSUPPORTED;
        if (static_cast<long long>(v.outputs) * rows > out_stride) return TBL_ERR_SHAPE;
        pr[g] = StripProblem{};
        pr[g].strips = static_cast<const uint8_t*>(v.strips);
        pr[g].magnitude = v.magnitude; pr[g].bias = v.bias;
        pr[g].y = out + static_cast<size_t>(g) * out_stride;
        pr[g].weight_scale = v.weight_scale; pr[g].rows = rows;
        pr[g].N = v.outputs; pr[g].K = K; pr[g].ldy = v.outputs;
        pr[g].x = x; pr[g].q_max = 127.0f;
        if (v.activation_bits != 8) return TBL_ERR_UNSUPPORTED;
        pr[g].rms_fast = v.rms_input != 0;
        pr[g].pre = pre;
    }
    const cudaError_t e = launch_gemv_strip(pr, groups, st);
    return e == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

int linear_view_forward_pre(const tbl_linear_view& v, const float* x, int rows, bool squared_relu, const StripPrologue& pre,
                            float* y, cudaStream_t st) {
    if (!x || !y || rows <= 0) return TBL_ERR_INVALID_ARG;
    if (!v.strips || (reinterpret_cast<uintptr_t>(v.strips) & 15) || v.weight != nullptr || v.activation_bits != 8 ||
        !gemv_strip_supported(v.inputs) || rows > gemv_strip_fused_rows(v.inputs) || !prologue_ok(pre) ||
        (reinterpret_cast<uintptr_t>(x) & 15))
        return TBL_ERR_UNSUPPORTED;
    StripProblem pr{};
    pr.strips = static_cast<const uint8_t*>(v.strips); pr.x = x; pr.q_max = 127.0f;
    pr.rms_fast = v.rms_input != 0; pr.magnitude = v.magnitude; pr.bias = v.bias; pr.y = y;
    pr.weight_scale = v.weight_scale; pr.rows = rows; pr.N = v.outputs; pr.K = v.inputs; pr.ldy = v.outputs;
    pr.squared_relu = squared_relu ? 1 : 0;
    pr.pre = pre;
    const cudaError_t e = launch_gemv_strip(&pr, 1, st);
    return e == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

}  // namespace tbl

// ---- grouped variant ---------------------------------------------------------------------------

namespace {

int check_view(const tbl_linear_view& v) {
    if (v.weight != nullptr || v.packed == nullptr) return TBL_ERR_UNSUPPORTED;
    if (v.activation_bits == 0) return TBL_ERR_UNSUPPORTED;
    const int rc = check_problem(1, v.inputs, v.outputs, v.weight_scale, v.activation_bits);
    if (rc != TBL_OK) return rc;
    if (!aligned16(v.packed)) return TBL_ERR_ALIGNMENT;
    return TBL_OK;
}

struct MoeWorkspace {
    MoeLists lists;
    int8_t* q1;          // [capacity, dim]   quantised expert inputs (interleaved or row-major)
    int8_t* q2;          // [capacity, hidden]
    float* scales1; int32_t* sums1; float* inv1;
    float* scales2; int32_t* sums2; float* inv2;
    float* hidden;       // [capacity, hidden] fp32
    float* contrib;      // [capacity, dim] fp32
    size_t bytes;
};

MoeWorkspace carve_moe(void* base, int rows, int dim, int hidden_dim, int experts, int capacity) {
    MoeWorkspace w;
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { uint8_t* r = p + off; off += round_up(bytes, 256); return r; };
    w.lists.counts = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * experts));
    w.lists.offsets = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * experts));
    w.lists.total = reinterpret_cast<int32_t*>(take(sizeof(int32_t)));
    w.lists.slot_row = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * capacity));
    w.lists.slot_of = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * static_cast<size_t>(rows) * experts));
    // (rows padded to 512 codes: the plane-major layout of the widening GEMM)
    w.q1 = reinterpret_cast<int8_t*>(take(static_cast<size_t>(capacity) * round_up(static_cast<size_t>(dim), 512)));
    w.q2 = reinterpret_cast<int8_t*>(take(static_cast<size_t>(capacity) * round_up(static_cast<size_t>(hidden_dim), 512)));
    w.scales1 = reinterpret_cast<float*>(take(sizeof(float) * capacity));
    w.sums1 = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * capacity));
    w.inv1 = reinterpret_cast<float*>(take(sizeof(float) * capacity));
    w.scales2 = reinterpret_cast<float*>(take(sizeof(float) * capacity));
    w.sums2 = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * capacity));
    w.inv2 = reinterpret_cast<float*>(take(sizeof(float) * capacity));
    w.hidden = reinterpret_cast<float*>(take(sizeof(float) * static_cast<size_t>(capacity) * hidden_dim));
    w.contrib = reinterpret_cast<float*>(take(sizeof(float) * static_cast<size_t>(capacity) * dim));
    w.bytes = off;
    return w;
}

// One grouped linear stage of the MoE: problem e multiplies the rows of expert e's slot range.
int run_expert_stage(const tbl_linear_view* views, int experts, const int8_t* q, bool strip, const float* scales,
                     const int32_t* sums, const MoeLists& lists, int capacity, float* y, int squared_relu,
                     cudaStream_t st) {
    const int K = views[0].inputs, N = views[0].outputs;
    if (strip) {
        StripProblem pr[TBL_MAX_GROUPS];
        for (int e = 0; e < experts; ++e) {
            pr[e] = StripProblem{};
            pr[e].strips = static_cast<const uint8_t*>(views[e].strips); pr[e].qp = q;
            pr[e].act_scales = scales; pr[e].q_sums = sums;
            pr[e].magnitude = views[e].magnitude; pr[e].bias = views[e].bias; pr[e].y = y;
            pr[e].rows_dev = lists.counts + e; pr[e].offset_dev = lists.offsets + e;
            pr[e].weight_scale = views[e].weight_scale; pr[e].rows = capacity;
            pr[e].N = N; pr[e].K = K; pr[e].ldy = N; pr[e].squared_relu = squared_relu;
        }
        return cuda_status(launch_gemv_strip(pr, experts, st));
    }
    for (int e = 0; e < experts; ++e) {
        const cudaError_t err = launch_gemv_generic(q, scales, views[e].packed, views[e].weight_scale,
                                                    views[e].magnitude, views[e].bias, capacity, K, N, y,
                                                    nullptr, squared_relu, lists.counts + e,
                                                    lists.offsets + e, st);
        if (err != cudaSuccess) return TBL_ERR_CUDA;
    }
    return TBL_OK;
}

bool all_have_i8(const tbl_linear_view* views, int count) {
    for (int i = 0; i < count; ++i)
        if (!views[i].w_i8 || !aligned16(views[i].w_i8)) return false;
    return views[0].inputs % 16 == 0;
}

// One expert stage as a grouped tensor-core GEMM on the int8 expansions.
int run_expert_stage_gemm(const tbl_linear_view* views, int experts, const int8_t* q, const float* scales,
                          const MoeLists& lists, int capacity, int rows_cap, float* y, int squared_relu,
                          cudaStream_t st) {
    const int8_t* w[TBL_MAX_GROUPS];
    float ws[TBL_MAX_GROUPS];
    const float* mag[TBL_MAX_GROUPS];
    const float* bias[TBL_MAX_GROUPS];
    for (int e = 0; e < experts; ++e) {
        w[e] = views[e].w_i8; ws[e] = views[e].weight_scale; mag[e] = views[e].magnitude; bias[e] = views[e].bias;
    }
    return cuda_status(launch_gemm_tcgen05_grouped(q, scales, w, ws, mag, bias, lists.counts, lists.offsets, experts,
                                                   rows_cap, capacity, views[0].inputs, views[0].outputs, y,
                                                   squared_relu, st));
}

bool all_have_strips(const tbl_linear_view* views, int count) {
    for (int i = 0; i < count; ++i)
        if (!views[i].strips || !aligned16(views[i].strips)) return false;
    return gemv_strip_supported(views[0].inputs);
}

// The persistent route serves a stack when every layer has strips and the kernel's shape rules hold.
bool chain_layers(const tbl_linear_view* views, int count, const int* squared_relu, int rows, int rms_mode,
                  ChainLayer* out) {
    if (rms_mode == TBL_RMS_REFERENCE_ORDER) {
        for (int i = 0; i < count; ++i) if (views[i].rms_input) return false;
    }
    for (int i = 0; i < count; ++i) {
        if (!views[i].strips || !aligned16(views[i].strips)) return false;
        out[i] = ChainLayer{static_cast<const uint8_t*>(views[i].strips), views[i].magnitude, views[i].bias,
                            views[i].weight_scale, qmax_for_bits(views[i].activation_bits), views[i].outputs,
                            views[i].inputs, views[i].rms_input ? 1 : 0, squared_relu && squared_relu[i] ? 1 : 0};
    }
    return gemv_chain_supported(out, count, rows);
}
size_t chain_act_bytes(const tbl_linear_view* views, int count, int rows) {
    size_t width = 0;
    for (int i = 0; i + 1 < count; ++i) width = static_cast<size_t>(views[i].outputs) > width ? views[i].outputs : width;
    return round_up(static_cast<size_t>(rows) * width * sizeof(float), 256);
}
}  // namespace

extern "C" {

size_t tbl_grouped_workspace_bytes(int groups, int max_inputs) {
    if (groups <= 0 || max_inputs <= 0) return 0;
    return carve(nullptr, 1, max_inputs).bytes;
}

size_t tbl_grouped_rows_workspace_bytes(int groups, int rows, int max_inputs) {
    if (groups <= 0 || rows <= 0 || max_inputs <= 0) return 0;
    return carve(nullptr, rows, max_inputs).bytes;
}

int tbl_grouped_forward_rows(const tbl_linear_view* views_host, int groups, const float* input_dev, int rows,
                             float* output_dev, long long output_stride, int rms_mode, void* workspace_dev,
                             size_t workspace_bytes, void* stream) {
    if (!views_host || !input_dev || !output_dev || groups <= 0 || groups > TBL_MAX_GROUPS || rows <= 0 ||
        output_stride <= 0)
        return TBL_ERR_INVALID_ARG;
    if (rows > 64) return TBL_ERR_SHAPE;      // one activation tile; larger batches go through tbl_linear_forward
    if (rms_mode < TBL_RMS_NONE || rms_mode > TBL_RMS_REFERENCE_ORDER) return TBL_ERR_INVALID_ARG;
    const int K = views_host[0].inputs;
    for (int g = 0; g < groups; ++g) {
        const int rc = check_view(views_host[g]);
        if (rc != TBL_OK) return rc;
        // the shared input rows are quantised once, so the views must agree on how
        if (views_host[g].inputs != K || views_host[g].activation_bits != views_host[0].activation_bits ||
            (views_host[g].rms_input != 0) != (views_host[0].rms_input != 0))
            return TBL_ERR_UNSUPPORTED;
        if (static_cast<long long>(views_host[g].outputs) * rows > output_stride) return TBL_ERR_SHAPE;
    }
    if (!workspace_dev || workspace_bytes < tbl_grouped_rows_workspace_bytes(groups, rows, K)) return TBL_ERR_WORKSPACE;
    if (!aligned16(workspace_dev) || !aligned16(input_dev)) return TBL_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const Workspace w = carve(workspace_dev, rows, K);
    const int mode = views_host[0].rms_input ? (rms_mode == TBL_RMS_NONE ? TBL_RMS_FAST : rms_mode) : TBL_RMS_NONE;
    const bool mma = all_have_strips(views_host, groups);
    auto fill = [&](StripProblem& pr, int g) {
        pr = StripProblem{};
        pr.strips = static_cast<const uint8_t*>(views_host[g].strips);
        pr.magnitude = views_host[g].magnitude; pr.bias = views_host[g].bias;
        pr.y = output_dev + static_cast<size_t>(g) * output_stride;
        pr.weight_scale = views_host[g].weight_scale; pr.rows = rows;
        pr.N = views_host[g].outputs; pr.K = K; pr.ldy = views_host[g].outputs;
    };
    if (mma && mode != TBL_RMS_REFERENCE_ORDER && rows <= gemv_strip_fused_rows(K)) {
        // one launch: the shared input rows are quantised in the prologue of the grouped GEMV
        StripProblem pr[TBL_MAX_GROUPS];
        for (int g = 0; g < groups; ++g) {
            fill(pr[g], g);
            pr[g].x = input_dev; pr[g].q_max = qmax_for_bits(views_host[0].activation_bits);
            pr[g].rms_fast = mode == TBL_RMS_FAST;
        }
        return cuda_status(launch_gemv_strip(pr, groups, st));
    }
    if (mma && groups <= kWidenMaxViews && widen_rows_ok(rows, K)) {
        // more rows than the GEMV's tiles serve well: one launch of the widening tensor-core kernel over all the views
        WidenView wv[kWidenMaxViews];
        for (int g = 0; g < groups; ++g) {
            wv[g] = WidenView{};
            wv[g].strips = views_host[g].strips; wv[g].magnitude = views_host[g].magnitude; wv[g].bias = views_host[g].bias;
            wv[g].y = output_dev + static_cast<size_t>(g) * output_stride;
            wv[g].weight_scale = views_host[g].weight_scale; wv[g].N = views_host[g].outputs;
        }
        return widen_forward(wv, groups, input_dev, rows, K, views_host[0].activation_bits, mode, w, st);
    }
    cudaError_t e = launch_quantize_rows(input_dev, nullptr, rows, K, views_host[0].activation_bits, mode,
                                         TBL_TIE_EVEN, mma ? nullptr : w.q, mma ? w.qp : nullptr, w.act_scales,
                                         w.q_sums, w.inv_norm, nullptr, QuantSegments{}, st);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    if (mma) {
        StripProblem pr[TBL_MAX_GROUPS];
        for (int g = 0; g < groups; ++g) {
            fill(pr[g], g);
            pr[g].qp = w.qp; pr[g].act_scales = w.act_scales; pr[g].q_sums = w.q_sums;
        }
        return cuda_status(launch_gemv_strip(pr, groups, st));
    }
    for (int g = 0; g < groups; ++g) {
        e = launch_gemv_generic(w.q, w.act_scales, views_host[g].packed, views_host[g].weight_scale,
                                views_host[g].magnitude, views_host[g].bias, rows, K, views_host[g].outputs,
                                output_dev + static_cast<size_t>(g) * output_stride, nullptr, 0, nullptr,
                                nullptr, st);
        if (e != cudaSuccess) return TBL_ERR_CUDA;
    }
    return TBL_OK;
}

int tbl_grouped_forward(const tbl_linear_view* views_host, int groups, const float* input_dev,
                        float* output_dev, int output_stride, int rms_mode, void* workspace_dev,
                        size_t workspace_bytes, void* stream) {
    return tbl_grouped_forward_rows(views_host, groups, input_dev, 1, output_dev, output_stride, rms_mode,
                                    workspace_dev, workspace_bytes, stream);
}

size_t tbl_chain_workspace_bytes(const tbl_linear_view* views_host, int count, int rows) {
    if (!views_host || count <= 0 || count > TBL_MAX_CHAIN || rows <= 0) return 0;
    size_t lin = 0;
    for (int i = 0; i < count; ++i) {
        const size_t b = tbl_linear_workspace_bytes(rows, views_host[i].inputs, views_host[i].outputs);
        lin = b > lin ? b : lin;
    }
    // the persistent kernel's scratch (barrier words, strip flags, activations) or the layer-by-layer route's
    // (activations + one layer's quantiser scratch), whichever is larger
    ChainLayer layers[TBL_MAX_CHAIN];
    for (int i = 0; i < count; ++i) { layers[i] = ChainLayer{}; layers[i].N = views_host[i].outputs; layers[i].K = views_host[i].inputs; }
    const size_t persistent = gemv_chain_workspace_bytes(layers, count, rows);
    const size_t stepwise = 1024 + 2 * chain_act_bytes(views_host, count, rows) + lin;
    return persistent > stepwise ? persistent : stepwise;
}

int tbl_chain_forward(const tbl_linear_view* views_host, int count, const int* squared_relu_host,
                      const float* x_dev, int rows, int rms_mode, float* y_dev, void* workspace_dev,
                      size_t workspace_bytes, void* stream) {
    if (!views_host || !x_dev || !y_dev || count <= 0 || count > TBL_MAX_CHAIN || rows <= 0) return TBL_ERR_INVALID_ARG;
    if (rms_mode < TBL_RMS_NONE || rms_mode > TBL_RMS_REFERENCE_ORDER) return TBL_ERR_INVALID_ARG;
    for (int i = 0; i < count; ++i) {
        const int rc = check_view(views_host[i]);
        if (rc != TBL_OK) return rc;
        if (static_cast<int64_t>(rows) * views_host[i].outputs > INT_MAX) return TBL_ERR_SHAPE;
        if (i > 0 && views_host[i].inputs != views_host[i - 1].outputs) return TBL_ERR_SHAPE;
    }
    if (!workspace_dev || workspace_bytes < tbl_chain_workspace_bytes(views_host, count, rows)) return TBL_ERR_WORKSPACE;
    if (!aligned16(workspace_dev) || !aligned16(x_dev) || !aligned16(y_dev)) return TBL_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ChainLayer layers[TBL_MAX_CHAIN];
    if (chain_layers(views_host, count, squared_relu_host, rows, rms_mode, layers))
        return cuda_status(launch_gemv_chain(layers, count, rows, x_dev, y_dev, workspace_dev, st));
    // layer by layer: same arithmetic, one tbl_linear_forward per layer, activations ping-pong in the workspace
    uint8_t* ws = static_cast<uint8_t*>(workspace_dev);
    const size_t act = chain_act_bytes(views_host, count, rows);
    float* bufs[2] = {reinterpret_cast<float*>(ws + 1024), reinterpret_cast<float*>(ws + 1024 + act)};
    void* lin_ws = ws + 1024 + 2 * act;
    const size_t lin_bytes = workspace_bytes - (1024 + 2 * act);
    const float* in = x_dev;
    for (int i = 0; i < count; ++i) {
        const tbl_linear_view& v = views_host[i];
        float* out = i == count - 1 ? y_dev : bufs[i & 1];
        const int rc = linear_view_forward(v, in, rows, rms_mode, squared_relu_host && squared_relu_host[i], out, lin_ws,
                                           lin_bytes, st);
        if (rc != TBL_OK) return rc;
        in = out;
    }
    return TBL_OK;
}

int tbl_router_topk(const float* logits_dev, int rows, int experts, int top_k, float* weights_dev, void* stream) {
    if (!logits_dev || !weights_dev || rows <= 0 || experts <= 0 || experts > TBL_MAX_GROUPS || top_k < 0)
        return TBL_ERR_INVALID_ARG;
    return cuda_status(launch_router_topk(logits_dev, rows, experts, top_k, weights_dev,
                                          static_cast<cudaStream_t>(stream)));
}

int tbl_row_norm(const float* value_dev, const float* gate_dev, const float* weight_dev, int rows, int dim,
                 float eps, float* out_dev, int bits, int8_t* q_dev, float* act_scales_dev, int32_t* q_sums_dev,
                 void* stream) {
    if (!value_dev || (!out_dev && !q_dev) || rows <= 0 || dim <= 0) return TBL_ERR_INVALID_ARG;
    if (!(eps > 0.0f) || !std::isfinite(eps)) return TBL_ERR_INVALID_ARG;     // Tensor::rmsnorm refuses the same
    if (dim > kRowNormMaxDim) return TBL_ERR_SHAPE;
    if (q_dev) {
        if (!act_scales_dev) return TBL_ERR_INVALID_ARG;
        if (bits < 2 || bits > 8) return TBL_ERR_BITS;
        if (dim % 16 || (reinterpret_cast<uintptr_t>(q_dev) & 3)) return TBL_ERR_SHAPE;
    }
    return cuda_status(launch_row_norm(value_dev, gate_dev, weight_dev, rows, dim, eps, bits, out_dev, q_dev,
                                       act_scales_dev, q_sums_dev, static_cast<cudaStream_t>(stream)));
}

int tbl_retile_columns(const float* gathered_dev, int parts, int rows, int cols, float* out_dev, void* stream) {
    if (!gathered_dev || !out_dev || parts <= 0 || rows <= 0 || cols <= 0 || gathered_dev == out_dev) return TBL_ERR_INVALID_ARG;
    return cuda_status(launch_retile_columns(gathered_dev, parts, rows, cols, out_dev, static_cast<cudaStream_t>(stream)));
}

size_t tbl_moe_workspace_bytes(int rows, int dim, int hidden_dim, int experts, int max_routes_per_row) {
    if (rows <= 0 || dim <= 0 || hidden_dim <= 0 || experts <= 0 || max_routes_per_row <= 0) return 0;
    if (max_routes_per_row > experts) max_routes_per_row = experts;
    return carve_moe(nullptr, rows, dim, hidden_dim, experts, rows * max_routes_per_row).bytes;
}

int tbl_moe_forward(const tbl_linear_view* views_host, const float* routing_dev, const float* x_dev, int rows,
                    int dim, int hidden_dim, int experts, int max_routes_per_row, int rms_mode, int tie_mode,
                    float* out_dev, void* workspace_dev, size_t workspace_bytes, void* stream) {
    if (!views_host || !routing_dev || !x_dev || !out_dev || rows <= 0 || dim <= 0 || hidden_dim <= 0 ||
        experts <= 0 || experts > TBL_MAX_GROUPS || max_routes_per_row <= 0)
        return TBL_ERR_INVALID_ARG;
    if (rms_mode < TBL_RMS_NONE || rms_mode > TBL_RMS_REFERENCE_ORDER) return TBL_ERR_INVALID_ARG;
    if (tie_mode != TBL_TIE_EVEN && tie_mode != TBL_TIE_AWAY) return TBL_ERR_INVALID_ARG;
    if (max_routes_per_row > experts) max_routes_per_row = experts;
    if (static_cast<int64_t>(rows) * max_routes_per_row > INT_MAX / 2) return TBL_ERR_SHAPE;
    for (int e = 0; e < 2 * experts; ++e) {
        const int rc = check_view(views_host[e]);
        if (rc != TBL_OK) return rc;
        const tbl_linear_view& v = views_host[e];
        const int want_in = e < experts ? dim : hidden_dim, want_out = e < experts ? hidden_dim : dim;
        if (v.inputs != want_in || v.outputs != want_out) return TBL_ERR_SHAPE;
        if (v.activation_bits != views_host[0].activation_bits ||
            (v.rms_input != 0) != (views_host[0].rms_input != 0))
            return TBL_ERR_UNSUPPORTED;
    }
    if (!workspace_dev ||
        workspace_bytes < tbl_moe_workspace_bytes(rows, dim, hidden_dim, experts, max_routes_per_row))
        return TBL_ERR_WORKSPACE;
    if (!aligned16(workspace_dev) || !aligned16(x_dev)) return TBL_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int capacity = rows * max_routes_per_row;
    const MoeWorkspace w = carve_moe(workspace_dev, rows, dim, hidden_dim, experts, capacity);
    const int bits = views_host[0].activation_bits;
    const int mode = views_host[0].rms_input ? (rms_mode == TBL_RMS_NONE ? TBL_RMS_FAST : rms_mode) : TBL_RMS_NONE;
    int* status = device_status_ptr();
    if (!status) return TBL_ERR_CUDA;

    cudaError_t e = launch_moe_route(routing_dev, rows, experts, capacity, w.lists, status, st);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    // expert inputs: gather routed rows, [RMSNorm], quantise once per slot
    const QuantSegments seg{w.lists.offsets, w.lists.counts, experts};
    // enough rows per expert for 128-row tensor-core tiles, and the int8 expansions at hand: grouped GEMMs
    if (capacity >= 16 * experts && all_have_i8(views_host, 2 * experts)) {
        e = launch_quantize_rows(x_dev, w.lists.slot_row, capacity, dim, bits, mode, tie_mode, w.q1, nullptr, w.scales1,
                                 nullptr, w.inv1, w.lists.total, QuantSegments{}, st);
        if (e != cudaSuccess) return TBL_ERR_CUDA;
        int rcg = run_expert_stage_gemm(views_host, experts, w.q1, w.scales1, w.lists, capacity, rows, w.hidden, 1, st);
        if (rcg != TBL_OK) return rcg;
        e = launch_quantize_rows(w.hidden, nullptr, capacity, hidden_dim, bits, mode, tie_mode, w.q2, nullptr,
                                 w.scales2, nullptr, w.inv2, w.lists.total, QuantSegments{}, st);
        if (e != cudaSuccess) return TBL_ERR_CUDA;
        rcg = run_expert_stage_gemm(views_host + experts, experts, w.q2, w.scales2, w.lists, capacity, rows, w.contrib,
                                    0, st);
        if (rcg != TBL_OK) return rcg;
        return cuda_status(launch_moe_merge(routing_dev, w.contrib, w.lists.slot_of, rows, experts, dim, out_dev, st));
    }
    const bool mma1 = all_have_strips(views_host, experts);
    const bool mma2 = all_have_strips(views_host + experts, experts);
    // enough rows per expert for the widening tensor-core kernel on the 2-bit weights: one grouped launch per stage,
    // every expert's rows in passes of 128 by its device-side count
    if (mma1 && mma2 && capacity >= 16 * experts && experts <= kWidenMaxViews && dim % 256 == 0 && hidden_dim % 256 == 0 &&
        dim <= 32768 && hidden_dim <= 32768) {
        const int rows_cap = rows;                      // a row reaches an expert at most once
        auto stage = [&](const tbl_linear_view* v, const int8_t* planes, const float* scales, const int32_t* sums, int K,
                         float* y, int squared) {
            WidenView wv[kWidenMaxViews];
            for (int x = 0; x < experts; ++x) {
                wv[x] = WidenView{};
                wv[x].strips = v[x].strips; wv[x].magnitude = v[x].magnitude; wv[x].bias = v[x].bias; wv[x].y = y;
                wv[x].weight_scale = v[x].weight_scale; wv[x].N = v[x].outputs; wv[x].squared_relu = squared;
            }
            return launch_gemm_widen(wv, experts, nullptr, const_cast<int8_t*>(planes), scales, sums, rows_cap, K, st,
                                     w.lists.counts, w.lists.offsets, capacity);
        };
        e = launch_quantize_rows(x_dev, w.lists.slot_row, capacity, dim, bits, mode, tie_mode, nullptr, w.q1, w.scales1,
                                 w.sums1, w.inv1, w.lists.total, QuantSegments{}, st, gemm_widen_plane_ld(dim));
        if (e != cudaSuccess) return TBL_ERR_CUDA;
        if (stage(views_host, w.q1, w.scales1, w.sums1, dim, w.hidden, 1) != cudaSuccess) return TBL_ERR_CUDA;
        e = launch_quantize_rows(w.hidden, nullptr, capacity, hidden_dim, bits, mode, tie_mode, nullptr, w.q2, w.scales2,
                                 w.sums2, w.inv2, w.lists.total, QuantSegments{}, st, gemm_widen_plane_ld(hidden_dim));
        if (e != cudaSuccess) return TBL_ERR_CUDA;
        if (stage(views_host + experts, w.q2, w.scales2, w.sums2, hidden_dim, w.contrib, 0) != cudaSuccess) return TBL_ERR_CUDA;
        return cuda_status(launch_moe_merge(routing_dev, w.contrib, w.lists.slot_of, rows, experts, dim, out_dev, st));
    }
    e = launch_quantize_rows(x_dev, w.lists.slot_row, capacity, dim, bits, mode, tie_mode, mma1 ? nullptr : w.q1,
                             mma1 ? w.q1 : nullptr, w.scales1, w.sums1, w.inv1, w.lists.total, seg, st);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    int rc = run_expert_stage(views_host, experts, w.q1, mma1, w.scales1, w.sums1, w.lists, capacity, w.hidden,
                              1, st);
    if (rc != TBL_OK) return rc;
    e = launch_quantize_rows(w.hidden, nullptr, capacity, hidden_dim, bits, mode, tie_mode, mma2 ? nullptr : w.q2,
                             mma2 ? w.q2 : nullptr, w.scales2, w.sums2, w.inv2, w.lists.total, seg, st);
    if (e != cudaSuccess) return TBL_ERR_CUDA;
    rc = run_expert_stage(views_host + experts, experts, w.q2, mma2, w.scales2, w.sums2, w.lists, capacity,
                          w.contrib, 0, st);
    if (rc != TBL_OK) return rc;
    return cuda_status(launch_moe_merge(routing_dev, w.contrib, w.lists.slot_of, rows, experts, dim, out_dev, st));
}

}  // extern "C"

// ---- allocation-free variant of the layer forward --------------------------------------------

// Scratch for tbl_linear_forward_noalloc.  In host code this name is only a stand-in for the
// symbol: the device address has to be asked for, per device, with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[TBL_NOALLOC_SCRATCH_BYTES];

namespace {

// Device address of g_noalloc_scratch on the current device; looked up once per device.
void* noalloc_scratch_address() {
    static void* cached[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cached[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess) return nullptr;
        cached[dev] = ptr;
    }
    return cached[dev];
}

}  // namespace

extern "C" int tbl_linear_forward_noalloc(const float* x_dev, const uint32_t* words_dev, const void* strips_dev,
                                          const int8_t* w_i8_dev, float weight_scale, int M, int K, int N, int bits,
                                          int rms_mode, const float* magnitude_dev, const float* bias_dev,
                                          float* y_dev, void* stream) {
    if (M <= 0 || K <= 0 || N <= 0) return TBL_ERR_INVALID_ARG;
    // refuse, before anything is enqueued, what the fixed array cannot hold
    if (tbl_linear_workspace_bytes(M, K, N) > TBL_NOALLOC_SCRATCH_BYTES) return TBL_ERR_WORKSPACE;
    void* scratch = noalloc_scratch_address();
    if (!scratch) return TBL_ERR_CUDA;
    return tbl_linear_forward(x_dev, words_dev, strips_dev, w_i8_dev, weight_scale, M, K, N, bits, rms_mode,
                              magnitude_dev, bias_dev, y_dev, scratch, TBL_NOALLOC_SCRATCH_BYTES, stream);
}
