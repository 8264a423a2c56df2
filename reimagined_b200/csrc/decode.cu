// One streaming decode step of the Mamba-2 / attention hybrid whose every projection is a ternary linear:
// the glue kernels between the linears (embedding gather, causal-conv step, SSD recurrence step, single-token
// attention over the KV cache with RoPE, gated residual adds) and the host routine that enqueues the whole
// step on one stream -- no allocation, no synchronisation, positions kept on the device -- so a caller can
// capture it once in a CUDA graph and replay it per token.
//
// The arithmetic follows the reference's host branches operation by operation (separately rounded products
// and sums, the same summation orders) so that results differ from them only through the device's expf / exp /
// log and the tree-shaped sums of the norms and the softmax denominator.
#include <cmath>

#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.cuh"

namespace tbl {
namespace {

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- embedding gather: out[b,:] = table[ids[b],:]; an id outside [0, vocab) gives a zero row ----------------
__global__ void __launch_bounds__(256) embedding_gather_kernel(const int32_t* __restrict__ ids,
                                                               const float* __restrict__ table, int vocab, int D,
                                                               float* __restrict__ out, float* __restrict__ trace) {
    const int b = blockIdx.x;
    const int id = __ldg(ids + b);
    const bool ok = id >= 0 && id < vocab;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = ok ? __ldg(table + static_cast<size_t>(id) * D + d) : 0.0f;
        out[static_cast<size_t>(b) * D + d] = v;
        if (trace) trace[static_cast<size_t>(b) * D + d] = v;
    }
}

__device__ __forceinline__ float silu_stable(float x) {
    float sig;
    if (x >= 0.0f) {
        const float z = expf(-x);
        sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, z));
    } else {
        const float z = expf(x);
        sig = __fdiv_rn(z, __fadd_rn(1.0f, z));
    }
    return __fmul_rn(x, sig);
}

// ---- Mamba-2 causal depthwise conv step + SiLU over [x | B | C], then the ring shift ------------------------
// One thread per (row, channel).  ring [R][K-1][conv_dim], oldest tap first.
__global__ void __launch_bounds__(256) mamba_conv_step_kernel(const float* __restrict__ xv, const float* __restrict__ Bv,
                                                              const float* __restrict__ Cv,
                                                              const float* __restrict__ conv_w,
                                                              const float* __restrict__ conv_b, float* __restrict__ ring,
                                                              int d_inner, int GS, int K, float* __restrict__ xBC) {
    const int conv_dim = d_inner + 2 * GS;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (c >= conv_dim) return;
    const int taps = K - 1;
    float* rr = ring + static_cast<size_t>(r) * taps * conv_dim;
    const float current = c < d_inner ? xv[static_cast<size_t>(r) * d_inner + c]
                                      : (c < d_inner + GS ? Bv[static_cast<size_t>(r) * GS + c - d_inner]
                                                          : Cv[static_cast<size_t>(r) * GS + c - d_inner - GS]);
    float value = __ldg(conv_b + c);
    for (int j = 0; j < K; ++j) {
        const float tap = j < taps ? rr[static_cast<size_t>(j) * conv_dim + c] : current;
        value = __fadd_rn(value, __fmul_rn(__ldg(conv_w + static_cast<size_t>(c) * K + j), tap));
    }
    xBC[static_cast<size_t>(r) * conv_dim + c] = silu_stable(value);
    for (int s = 0; s + 1 < taps; ++s) rr[static_cast<size_t>(s) * conv_dim + c] = rr[static_cast<size_t>(s + 1) * conv_dim + c];
    if (taps > 0) rr[static_cast<size_t>(taps - 1) * conv_dim + c] = current;
}


// One channel of the SSD recurrence: h[n] = decay*h[n] + (delta*B[n])*x ; y = D*x + sum_n h[n]*C[n], n ascending.
// The state row is staged through registers in chunks of 16 so that its loads are issued together (a load placed
// after the previous element's store would wait for it: the compiler cannot prove they do not alias).
__device__ __forceinline__ float ssd_channel(float* __restrict__ st, const float* __restrict__ Bg, const float* __restrict__ Cg,
                                             int N, float decay, float delta, float input, float y) {
    int n0 = 0;
    for (; n0 + 16 <= N; n0 += 16) {
        float hv[16];
        if ((reinterpret_cast<uintptr_t>(st + n0) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 v = *reinterpret_cast<const float4*>(st + n0 + 4 * q);
                hv[4 * q] = v.x; hv[4 * q + 1] = v.y; hv[4 * q + 2] = v.z; hv[4 * q + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int n = 0; n < 16; ++n) hv[n] = st[n0 + n];
        }
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            hv[n] = __fadd_rn(__fmul_rn(decay, hv[n]), __fmul_rn(__fmul_rn(delta, Bg[n0 + n]), input));
            y = __fadd_rn(y, __fmul_rn(hv[n], Cg[n0 + n]));
        }
#pragma unroll
        for (int n = 0; n < 16; ++n) st[n0 + n] = hv[n];
    }
    for (int n = n0; n < N; ++n) {
        const float hv = __fadd_rn(__fmul_rn(decay, st[n]), __fmul_rn(__fmul_rn(delta, Bg[n]), input));
        st[n] = hv;
        y = __fadd_rn(y, __fmul_rn(hv, Cg[n]));
    }
    return y;
}

// ---- SSD recurrence step: h = decay*h + delta*B*x ; y = D*x + sum_n h*C -------------------------------------
// One thread per (row, channel); delta = softplus(dt), decay = exp(-delta*exp(A_log)) in double.
__global__ void __launch_bounds__(128) mamba_ssd_step_kernel(const float* __restrict__ xBC, const float* __restrict__ dt,
                                                             const float* __restrict__ A_log, const float* __restrict__ Dp,
                                                             float* __restrict__ state, int n_heads, int d_head, int N,
                                                             int n_groups, float* __restrict__ y) {
    const int d_inner = n_heads * d_head, GS = n_groups * N, conv_dim = d_inner + 2 * GS;
    const int chan = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (chan >= d_inner) return;
    const int h = chan / d_head;
    const int group = (h * n_groups) / n_heads;
    const float dt_raw = dt[static_cast<size_t>(r) * n_heads + h];
    const float a_log = __ldg(A_log + h);
    const float delta = dt_raw > 20.0f ? dt_raw : (dt_raw < -20.0f ? expf(dt_raw) : log1pf(expf(dt_raw)));
    float decay;
    if (!isfinite(dt_raw) || !isfinite(a_log)) {
        decay = nanf("");
    } else {
        const double log_delta = dt_raw < -20.0f ? static_cast<double>(dt_raw) : log(static_cast<double>(delta));
        const double log_q = log_delta + static_cast<double>(a_log);
        decay = log_q > 50.0 ? 0.0f : static_cast<float>(exp(-exp(log_q)));
    }
    const float* row = xBC + static_cast<size_t>(r) * conv_dim;
    const float input = row[chan];
    float* st = state + (static_cast<size_t>(r) * d_inner + chan) * N;
    y[static_cast<size_t>(r) * d_inner + chan] = ssd_channel(st, row + d_inner + group * N, row + d_inner + GS + group * N, N, decay,
                                                           delta, input, __fmul_rn(__ldg(Dp + h), input));
}

// ---- single-token attention over the KV cache ----------------------------------------------------------------
// One CTA per (query head, row).  RoPE on q and on the new key at the row's position; the first head of a
// KV group appends the rotated key and the value to the cache; every CTA keeps the new key / value of its group
// in shared memory, so no CTA reads what another one writes in this launch.
//   scores   one cached token per thread, the dot product in dimension order (a thread streams a whole key row)
//   softmax  warp shuffles, then one value per warp through shared memory
//   values   head_dim / 4 threads cover one value row with 128-bit loads; the CTA's thread groups take the cached
//            tokens round-robin, several rows in flight per thread, and their partial sums are added in group
//            order.  (With one dimension per thread and the tokens in sequence the launch's time was the cache's
//            load latency times the context length.)
constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnPartial = 4 * kAttnThreads;     // floats: one float4 of partial sums per thread
constexpr int kAttnMaxHeadDim = 4 * kAttnThreads;  // a value row is covered by at most one CTA's worth of float4s

static size_t attention_smem_bytes(int head_dim, int capacity) {
    return sizeof(float) * (static_cast<size_t>(3) * head_dim + kAttnWarps + kAttnPartial + capacity);
}

__global__ void __launch_bounds__(kAttnThreads)
attention_decode_kernel(const float* __restrict__ q, const float* __restrict__ kv, float* __restrict__ k_cache,
                        float* __restrict__ v_cache, int capacity, const int32_t* __restrict__ positions,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rope_positions,
                        int n_heads, int n_kv_heads, int head_dim, int sliding_window, float* __restrict__ out,
                        int* status) {
    extern __shared__ __align__(16) float sm[];
    float* qr = sm;                       // [head_dim]
    float* knew = qr + head_dim;          // [head_dim]
    float* vnew = knew + head_dim;        // [head_dim]
    float* red = vnew + head_dim;         // [kAttnWarps]
    float* partial = red + kAttnWarps;    // [kAttnPartial]
    float* scores = partial + kAttnPartial;   // [capacity]
    const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kv_dim = n_kv_heads * head_dim, half = head_dim / 2, d_model = n_heads * head_dim;
    const int group = n_heads / n_kv_heads > 0 ? n_heads / n_kv_heads : 1;
    const int kvh = min(h / group, n_kv_heads - 1);
    const int pos = __ldg(positions + r);
    if (pos < 0 || pos >= capacity || pos >= rope_positions) {
        // the cache (or the rotary table) is full: report it and leave this row's output at zero
        if (tid == 0) atomicOr(status, TBL_DEV_CACHE_FULL);
        for (int d = tid; d < head_dim; d += kAttnThreads) out[static_cast<size_t>(r) * d_model + h * head_dim + d] = 0.0f;
        return;
    }
    const float* c = cos_t + static_cast<size_t>(pos) * half;
    const float* s = sin_t + static_cast<size_t>(pos) * half;
    const float* qh = q + static_cast<size_t>(r) * d_model + h * head_dim;
    const float* kh = kv + static_cast<size_t>(r) * 2 * kv_dim + kvh * head_dim;
    for (int i = tid; i < half; i += kAttnThreads) {
        const float cv = __ldg(c + i), sv = __ldg(s + i);
        const float q0 = qh[i], q1 = qh[i + half];
        qr[i] = __fsub_rn(__fmul_rn(q0, cv), __fmul_rn(q1, sv));
        qr[i + half] = __fadd_rn(__fmul_rn(q0, sv), __fmul_rn(q1, cv));
        const float k0 = kh[i], k1 = kh[i + half];
        knew[i] = __fsub_rn(__fmul_rn(k0, cv), __fmul_rn(k1, sv));
        knew[i + half] = __fadd_rn(__fmul_rn(k0, sv), __fmul_rn(k1, cv));
        vnew[i] = kh[kv_dim + i];
        vnew[i + half] = kh[kv_dim + i + half];
    }
    __syncthreads();
    const size_t head_base = static_cast<size_t>(r) * capacity * kv_dim + static_cast<size_t>(kvh) * head_dim;
    if (h == kvh * group) {
        float* kc = k_cache + head_base + static_cast<size_t>(pos) * kv_dim;
        float* vc = v_cache + head_base + static_cast<size_t>(pos) * kv_dim;
        for (int d = tid; d < head_dim; d += kAttnThreads) { kc[d] = knew[d]; vc[d] = vnew[d]; }
    }
    const int cached = pos + 1;
    const int first = max(0, cached - sliding_window);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(static_cast<float>(head_dim)));
    // scores: one token per thread, the dot product in dimension order; the new token's key is the one in shared memory
    float local_max = -1e30f;
    for (int t = first + tid; t < cached; t += kAttnThreads) {
        float dot = 0.0f;
        if (t == pos) {
            for (int d = 0; d < head_dim; ++d) dot = __fadd_rn(dot, __fmul_rn(qr[d], knew[d]));
        } else {
            const float4* key = reinterpret_cast<const float4*>(k_cache + head_base + static_cast<size_t>(t) * kv_dim);
            for (int d4 = 0; d4 < head_dim / 4; ++d4) {
                const float4 k4 = key[d4];
                dot = __fadd_rn(dot, __fmul_rn(qr[4 * d4], k4.x));
                dot = __fadd_rn(dot, __fmul_rn(qr[4 * d4 + 1], k4.y));
                dot = __fadd_rn(dot, __fmul_rn(qr[4 * d4 + 2], k4.z));
                dot = __fadd_rn(dot, __fmul_rn(qr[4 * d4 + 3], k4.w));
            }
        }
        const float sc = __fmul_rn(dot, scale);
        scores[t - first] = sc;
        local_max = fmaxf(local_max, sc);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, o));
    if (lane == 0) red[warp] = local_max;
    __syncthreads();
    float max_s = red[0];
#pragma unroll
    for (int w = 1; w < kAttnWarps; ++w) max_s = fmaxf(max_s, red[w]);
    __syncthreads();
    float local_sum = 0.0f;
    for (int t = first + tid; t < cached; t += kAttnThreads) {
        const float e = expf(__fsub_rn(scores[t - first], max_s));
        scores[t - first] = e;
        local_sum += e;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) local_sum += __shfl_xor_sync(0xffffffffu, local_sum, o);
    if (lane == 0) red[warp] = local_sum;
    __syncthreads();                      // also: every thread's exp() is in scores[] now
    float total = red[0];
#pragma unroll
    for (int w = 1; w < kAttnWarps; ++w) total += red[w];
    const float inv_sum = __fdiv_rn(1.0f, fmaxf(total, 1e-9f));
    // weighted sum of the values
    const int row_threads = head_dim / 4;                     // threads that cover one value row
    const int groups = kAttnThreads / row_threads;            // token groups of this CTA (>= 1: head_dim <= 4 * threads)
    const int g = tid / row_threads, d4 = tid - g * row_threads;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (g < groups) {
        const float4* vrow = reinterpret_cast<const float4*>(v_cache + head_base) + d4;
        const size_t step = static_cast<size_t>(kv_dim / 4);   // float4s between two tokens' rows
        constexpr int kInFlight = 8;
        int t = first + g;
        for (; t + (kInFlight - 1) * groups < pos; t += kInFlight * groups) {
            float4 v[kInFlight];
#pragma unroll
            for (int j = 0; j < kInFlight; ++j) v[j] = vrow[static_cast<size_t>(t + j * groups) * step];
#pragma unroll
            for (int j = 0; j < kInFlight; ++j) {
                const float p = __fmul_rn(scores[t + j * groups - first], inv_sum);
                acc.x = __fadd_rn(acc.x, __fmul_rn(p, v[j].x));
                acc.y = __fadd_rn(acc.y, __fmul_rn(p, v[j].y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(p, v[j].z));
                acc.w = __fadd_rn(acc.w, __fmul_rn(p, v[j].w));
            }
        }
        for (; t < cached; t += groups) {
            const float4 v = t == pos ? reinterpret_cast<const float4*>(vnew)[d4] : vrow[static_cast<size_t>(t) * step];
            const float p = __fmul_rn(scores[t - first], inv_sum);
            acc.x = __fadd_rn(acc.x, __fmul_rn(p, v.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(p, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(p, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(p, v.w));
        }
        reinterpret_cast<float4*>(partial)[tid] = acc;        // partial[g][4 * d4 ..]: tid = g * row_threads + d4
    }
    __syncthreads();
    for (int d = tid; d < head_dim; d += kAttnThreads) {
        float sum = partial[d];
        for (int j = 1; j < groups; ++j) sum = __fadd_rn(sum, partial[j * head_dim + d]);
        out[static_cast<size_t>(r) * d_model + h * head_dim + d] = sum;
    }
}


// ---- fused glue of the step (one CTA per sequence) -------------------------------------------------------------
constexpr int kFusedThreads = 512;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; ++w) t += scratch[w];     // fixed order: the same result in every thread
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = scratch[0];
    for (int w = 1; w < nw; ++w) t = fmaxf(t, scratch[w]);
    return t;
}

// Where a glue kernel leaves the rows it produces as 8-bit codes for the GEMM behind it (the widening tensor-core
// kernel, gemm_widen.cu, or the tiled strip GEMV, gemv_strip.cu) instead of fp32 values, which saves the stand-alone row quantiser between the two: per row the
// absmax, scale = 127 / (absmax + 1e-8), code = round-half-even(v * scale) -- the arithmetic of
// quantize_rows_reg_kernel (quantize.cu) for 8 bits without an input norm, so the codes are the same bit for bit.
// Two layouts, after the kernel that reads them:
//   tile_rows == 0  plane-major (widening GEMM): inside each block of 512 codes of a row (leading dimension ld, a
//                   multiple of 512, zero past the row's width), byte 4g + e of plane p (128 bytes per plane) is
//                   element 16g + 4e + p;
//   tile_rows > 0   the interleaved activation tiles of the strip GEMV (qp_offset) for a batch of tile_rows rows:
//                   every 16-element group is stored as its 4x4 byte transpose (ld = the row's width).
struct RowCodes {
    int8_t* codes;         // null: the kernel writes fp32 as usual
    float* act_scales;     // [rows] (absmax + 1e-8) / 127
    int32_t* q_sums;       // [rows] sum of the row's codes
    int ld;
    int tile_rows;
};

__device__ __forceinline__ size_t code_offset(const RowCodes& c, int row, int k) {
    if (c.tile_rows > 0) return qp_offset(row, c.tile_rows, c.ld, k & ~15) + (k & 3) * 4 + ((k >> 2) & 3);
    return static_cast<size_t>(row) * c.ld + (k >> 9) * 512 + (k & 3) * 128 + ((k >> 4) & 31) * 4 + ((k >> 2) & 3);
}

// hidden_out = x + (a*ga [+ b*gb]) (or x itself when a == null; x = table[ids[row]] when ids != null), and up to two
// RMSNorm x weight views of it (eps shared): out1 = rmsnorm(h)*w1, out2 = rmsnorm(h)*w2.  Replaces the residual
// add that closes one block and the norm(s) that open the next (OXN/nsos/src/jamba.cpp:3175-3179, 3195-3251).
__global__ void __launch_bounds__(kFusedThreads)
residual_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ ids, const float* __restrict__ table,
                     int vocab, const float* __restrict__ a, const float* __restrict__ ga, const float* __restrict__ b,
                     const float* __restrict__ gb, int D, float eps, const float* __restrict__ w1,
                     const float* __restrict__ w2, float* __restrict__ hidden_out, float* __restrict__ trace,
                     float* __restrict__ out1, float* __restrict__ out2, RowCodes codes1) {
    extern __shared__ float sm[];
    float* row = sm;                 // [D]
    float* scratch = sm + D;         // [32]
    __shared__ int code_sum;
    // a dependent launch (the widening GEMM behind out1's codes) may fetch and widen its first weights meanwhile
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const float* src = x ? x + static_cast<size_t>(r) * D : nullptr;
    bool id_ok = true;
    if (ids) {
        const int id = __ldg(ids + r);
        id_ok = id >= 0 && id < vocab;
        src = table + static_cast<size_t>(id_ok ? id : 0) * D;
    }
    float ss = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = id_ok ? src[d] : 0.0f;
        if (a) {
            const size_t i = static_cast<size_t>(r) * D + d;
            float contrib = ga ? __fmul_rn(a[i], __ldg(ga + d)) : a[i];
            if (b) contrib = __fadd_rn(contrib, __fmul_rn(b[i], __ldg(gb + d)));
            v = __fadd_rn(v, contrib);
        }
        row[d] = v;
        if (hidden_out) hidden_out[static_cast<size_t>(r) * D + d] = v;
        if (trace) trace[static_cast<size_t>(r) * D + d] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(D)), eps)));
    float mx = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float n = __fmul_rn(row[d], inv);
        const float v1 = w1 ? __fmul_rn(n, __ldg(w1 + d)) : n;
        if (out1) out1[static_cast<size_t>(r) * D + d] = v1;
        if (out2) out2[static_cast<size_t>(r) * D + d] = w2 ? __fmul_rn(n, __ldg(w2 + d)) : n;
        if (codes1.codes) { row[d] = v1; mx = fmaxf(mx, fabsf(v1)); }     // the thread's own elements: no barrier needed
    }
    if (!codes1.codes) return;
    if (threadIdx.x == 0) code_sum = 0;
    mx = block_max(mx, scratch);
    const float denom = __fadd_rn(mx, 1e-8f);
    const float scale = __fdiv_rn(127.0f, denom);
    int local = 0;
    for (int d = threadIdx.x; d < codes1.ld; d += blockDim.x) {
        int c = 0;
        if (d < D) c = round_code(__fmul_rn(row[d], scale), false);
        local += static_cast<int8_t>(c);
        codes1.codes[code_offset(codes1, r, d)] = static_cast<int8_t>(c);
    }
    local = __reduce_add_sync(0xffffffffu, local);
    if ((threadIdx.x & 31) == 0 && local != 0) atomicAdd(&code_sum, local);
    __syncthreads();
    if (threadIdx.x == 0) {
        codes1.act_scales[r] = __fdiv_rn(denom, 127.0f);
        codes1.q_sums[r] = code_sum;
    }
}

__device__ __forceinline__ float silu_two_sided(float g) {     // Tensor::silu (OXN/nsos/src/tensor.cpp:3273-3280)
    const float e = expf(-fabsf(g));
    const float sig = __fdiv_rn(g >= 0.0f ? 1.0f : e, __fadd_rn(1.0f, e));
    return __fmul_rn(g, sig);
}

// conv step -> SSD step -> (y * silu(z)).rmsnorm(eps) * weight for one sequence per CTA: the three stages of
// Mamba2SSD::forward_faithful_step between the projections and the out projection
// (OXN/nsos/src/mamba2.cpp:4062-4123), with the conv output and the per-head decay terms kept in shared memory.
__global__ void __launch_bounds__(kFusedThreads)
mamba_mix_kernel(const float* __restrict__ xv, const float* __restrict__ zv, const float* __restrict__ Bv,
                 const float* __restrict__ Cv, const float* __restrict__ dt, const float* __restrict__ conv_w,
                 const float* __restrict__ conv_b, const float* __restrict__ A_log, const float* __restrict__ Dp,
                 const float* __restrict__ norm_w, float* __restrict__ ring, float* __restrict__ state, int n_heads,
                 int d_head, int N, int n_groups, int K, float eps, float* __restrict__ out) {
    extern __shared__ float sm[];
    const int d_inner = n_heads * d_head, GS = n_groups * N, conv_dim = d_inner + 2 * GS;
    float* xbc = sm;                          // [conv_dim]
    float* gated = xbc + conv_dim;            // [d_inner]
    float* delta_s = gated + d_inner;         // [n_heads]
    float* decay_s = delta_s + n_heads;       // [n_heads]
    float* scratch = decay_s + n_heads;       // [32]
    const int r = blockIdx.x;
    const int taps = K - 1;
    float* rr = ring + static_cast<size_t>(r) * (taps > 0 ? taps : 1) * conv_dim;
    // The kernel runs as one CTA per sequence, so its duration is a sum of memory round trips: every phase issues
    // all of a thread's loads before it uses any of them (kBatch channels at a time).
    constexpr int kBatch = 4, kMaxK = 4;
    // per-head step sizes and decays, by the last warp while the others start on the convolution
    if (static_cast<int>(threadIdx.x) >= static_cast<int>(blockDim.x) - 32) {
        for (int h = threadIdx.x - (blockDim.x - 32); h < n_heads; h += 32) {
            const float dt_raw = dt[static_cast<size_t>(r) * n_heads + h];
            const float a_log = __ldg(A_log + h);
            const float delta = dt_raw > 20.0f ? dt_raw : (dt_raw < -20.0f ? expf(dt_raw) : log1pf(expf(dt_raw)));
            float decay;
            if (!isfinite(dt_raw) || !isfinite(a_log)) {
                decay = nanf("");
            } else {
                const double log_delta = dt_raw < -20.0f ? static_cast<double>(dt_raw) : log(static_cast<double>(delta));
                const double log_q = log_delta + static_cast<double>(a_log);
                decay = log_q > 50.0 ? 0.0f : static_cast<float>(exp(-exp(log_q)));
            }
            delta_s[h] = delta;
            decay_s[h] = decay;
        }
    }
    for (int c0 = threadIdx.x; c0 < conv_dim; c0 += blockDim.x * kBatch) {
        float tapv[kBatch][kMaxK], wv[kBatch][kMaxK], bias[kBatch];
        if (K <= kMaxK) {
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const int c = c0 + i * blockDim.x;
                if (c < conv_dim) {
                    const float current = c < d_inner ? xv[static_cast<size_t>(r) * d_inner + c]
                                                      : (c < d_inner + GS ? Bv[static_cast<size_t>(r) * GS + c - d_inner]
                                                                          : Cv[static_cast<size_t>(r) * GS + c - d_inner - GS]);
#pragma unroll
                    for (int j = 0; j < kMaxK; ++j) {
                        if (j < K) {
                            tapv[i][j] = j < taps ? rr[static_cast<size_t>(j) * conv_dim + c] : current;
                            wv[i][j] = __ldg(conv_w + static_cast<size_t>(c) * K + j);
                        }
                    }
                    bias[i] = __ldg(conv_b + c);
                }
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const int c = c0 + i * blockDim.x;
                if (c < conv_dim) {
                    float value = bias[i];
#pragma unroll
                    for (int j = 0; j < kMaxK; ++j)
                        if (j < K) value = __fadd_rn(value, __fmul_rn(wv[i][j], tapv[i][j]));
                    xbc[c] = silu_stable(value);
                    // the window moves on: taps 1.. become 0.., the newest input goes last
#pragma unroll
                    for (int j = 0; j + 1 < kMaxK; ++j)
                        if (j < taps) rr[static_cast<size_t>(j) * conv_dim + c] = tapv[i][j + 1];
                }
            }
        } else {
            for (int i = 0; i < kBatch; ++i) {
                const int c = c0 + i * blockDim.x;
                if (c >= conv_dim) break;
                const float current = c < d_inner ? xv[static_cast<size_t>(r) * d_inner + c]
                                                  : (c < d_inner + GS ? Bv[static_cast<size_t>(r) * GS + c - d_inner]
                                                                      : Cv[static_cast<size_t>(r) * GS + c - d_inner - GS]);
                float value = __ldg(conv_b + c);
                for (int j = 0; j < K; ++j) {
                    const float tap = j < taps ? rr[static_cast<size_t>(j) * conv_dim + c] : current;
                    value = __fadd_rn(value, __fmul_rn(__ldg(conv_w + static_cast<size_t>(c) * K + j), tap));
                }
                xbc[c] = silu_stable(value);
                for (int s2 = 0; s2 + 1 < taps; ++s2) rr[static_cast<size_t>(s2) * conv_dim + c] = rr[static_cast<size_t>(s2 + 1) * conv_dim + c];
                if (taps > 0) rr[static_cast<size_t>(taps - 1) * conv_dim + c] = current;
            }
        }
    }
    __syncthreads();
    float ss = 0.0f;
    for (int ch0 = threadIdx.x; ch0 < d_inner; ch0 += blockDim.x * kBatch) {
        float zval[kBatch], dval[kBatch];
        float hv[kBatch][16];
        const bool fast = N == 16;
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const int chan = ch0 + i * blockDim.x;
            if (chan < d_inner) {
                zval[i] = zv[static_cast<size_t>(r) * d_inner + chan];
                dval[i] = __ldg(Dp + chan / d_head);
                if (fast) {
                    const float4* st4 = reinterpret_cast<const float4*>(state + (static_cast<size_t>(r) * d_inner + chan) * 16);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 v = st4[q];
                        hv[i][4 * q] = v.x; hv[i][4 * q + 1] = v.y; hv[i][4 * q + 2] = v.z; hv[i][4 * q + 3] = v.w;
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const int chan = ch0 + i * blockDim.x;
            if (chan < d_inner) {
                const int h = chan / d_head;
                const int group = (h * n_groups) / n_heads;
                const float delta = delta_s[h], decay = decay_s[h];
                const float input = xbc[chan];
                const float* Bg = xbc + d_inner + group * N;
                const float* Cg = xbc + d_inner + GS + group * N;
                float* st = state + (static_cast<size_t>(r) * d_inner + chan) * N;
                float y = __fmul_rn(dval[i], input);
                if (fast) {
#pragma unroll
                    for (int n = 0; n < 16; ++n) {
                        hv[i][n] = __fadd_rn(__fmul_rn(decay, hv[i][n]), __fmul_rn(__fmul_rn(delta, Bg[n]), input));
                        y = __fadd_rn(y, __fmul_rn(hv[i][n], Cg[n]));
                    }
                    float4* st4 = reinterpret_cast<float4*>(st);
#pragma unroll
                    for (int q = 0; q < 4; ++q) st4[q] = make_float4(hv[i][4 * q], hv[i][4 * q + 1], hv[i][4 * q + 2], hv[i][4 * q + 3]);
                } else {
                    y = ssd_channel(st, Bg, Cg, N, decay, delta, input, y);
                }
                const float gv = __fmul_rn(y, silu_two_sided(zval[i]));
                gated[chan] = gv;
                ss += gv * gv;
            }
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(d_inner)), eps)));
    for (int chan = threadIdx.x; chan < d_inner; chan += blockDim.x) {
        const float n = __fmul_rn(gated[chan], inv);
        out[static_cast<size_t>(r) * d_inner + chan] = norm_w ? __fmul_rn(n, __ldg(norm_w + chan)) : n;
    }
}

// The same three stages with a sequence's channels spread over a thread-block cluster of kMixCluster CTAs (one SM
// cannot hide the latency of a sequence's 100 KB of state on its own: 20 us per launch as one CTA).  CTA `rank` owns
// a contiguous slice of the d_inner channels: their conv taps, ring rows, SSD state rows and outputs.  The B and C
// channels of the convolution (2 * n_groups * d_state values every CTA needs) are recomputed by every CTA from the
// same ring taps; only rank 0 moves their window on, after a cluster barrier behind which every CTA holds the taps
// in registers.  The gated norm's sum of squares is the fixed-order sum of the CTAs' partial sums, exchanged through
// rank 0's shared memory (distributed shared memory).  One channel per thread; kernel width K <= 4, d_state = 16.
constexpr int kMixCluster = 8;
constexpr int kMixThreads = 256;
__global__ void __launch_bounds__(kMixThreads)
mamba_mix_cluster_kernel(const float* __restrict__ xv, const float* __restrict__ zv, const float* __restrict__ Bv,
                         const float* __restrict__ Cv, const float* __restrict__ dt, const float* __restrict__ conv_w,
                         const float* __restrict__ conv_b, const float* __restrict__ A_log, const float* __restrict__ Dp,
                         const float* __restrict__ norm_w, float* __restrict__ ring, float* __restrict__ state,
                         int n_heads, int d_head, int n_groups, int K, float eps, float* __restrict__ out, RowCodes codes) {
    namespace cg = cooperative_groups;
    // a dependent launch (the widening GEMM of the out projection) may fetch and widen its first weights meanwhile
    pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int N = 16, kMaxK = 4;
    extern __shared__ float sm[];
    const int d_inner = n_heads * d_head, GS = n_groups * N, conv_dim = d_inner + 2 * GS;
    const int rank = static_cast<int>(cluster.block_rank());
    const int r = blockIdx.x / kMixCluster;
    const int per = (d_inner + kMixCluster - 1) / kMixCluster;
    const int c_lo = min(d_inner, rank * per), n_own = min(d_inner, c_lo + per) - c_lo;
    float* xs = sm;                           // [per]     conv outputs of the CTA's own channels
    float* bc = xs + per;                     // [2 * GS]  conv outputs of the B and C channels
    float* delta_s = bc + 2 * GS;             // [n_heads]
    float* decay_s = delta_s + n_heads;       // [n_heads]
    float* scratch = decay_s + n_heads;       // [32]
    float* parts = scratch + 32;              // [kMixCluster], rank 0's copy is the one used
    float* maxes = parts + kMixCluster;       // [kMixCluster], likewise: the CTAs' absmax of the outputs
    int* code_sums = reinterpret_cast<int*>(maxes + kMixCluster);   // [kMixCluster], likewise: the CTAs' sums of codes
    const int taps = K - 1;
    float* rr = ring + static_cast<size_t>(r) * (taps > 0 ? taps : 1) * conv_dim;
    // per-head step sizes and decays, by the last warp while the others start on the convolution
    if (static_cast<int>(threadIdx.x) >= kMixThreads - 32) {
        for (int h = threadIdx.x - (kMixThreads - 32); h < n_heads; h += 32) {
            const float dt_raw = dt[static_cast<size_t>(r) * n_heads + h];
            const float a_log = __ldg(A_log + h);
            const float delta = dt_raw > 20.0f ? dt_raw : (dt_raw < -20.0f ? expf(dt_raw) : log1pf(expf(dt_raw)));
            float decay;
            if (!isfinite(dt_raw) || !isfinite(a_log)) {
                decay = nanf("");
            } else {
                const double log_delta = dt_raw < -20.0f ? static_cast<double>(dt_raw) : log(static_cast<double>(delta));
                const double log_q = log_delta + static_cast<double>(a_log);
                decay = log_q > 50.0 ? 0.0f : static_cast<float>(exp(-exp(log_q)));
            }
            delta_s[h] = delta;
            decay_s[h] = decay;
        }
    }
    // convolution: thread i < n_own takes channel c_lo + i, the next 2 * GS threads the B and C channels
    const int idx = threadIdx.x;
    const int c = idx < n_own ? c_lo + idx : (idx < n_own + 2 * GS ? d_inner + (idx - n_own) : -1);
    float tapv[kMaxK];
    if (c >= 0) {
        const float current = c < d_inner ? xv[static_cast<size_t>(r) * d_inner + c]
                                          : (c < d_inner + GS ? Bv[static_cast<size_t>(r) * GS + c - d_inner]
                                                              : Cv[static_cast<size_t>(r) * GS + c - d_inner - GS]);
        float wv[kMaxK];
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            if (j < K) {
                tapv[j] = j < taps ? rr[static_cast<size_t>(j) * conv_dim + c] : current;
                wv[j] = __ldg(conv_w + static_cast<size_t>(c) * K + j);
            }
        }
        float value = __ldg(conv_b + c);
#pragma unroll
        for (int j = 0; j < kMaxK; ++j)
            if (j < K) value = __fadd_rn(value, __fmul_rn(wv[j], tapv[j]));
        const float act = silu_stable(value);
        if (c < d_inner) xs[idx] = act; else bc[c - d_inner] = act;
    }
    // SSD state row, gate and skip weight of the thread's channel: in flight across the barrier
    float hv[N], zval = 0.0f, dval = 0.0f;
    const int chan = c_lo + idx;
    if (idx < n_own) {
        zval = zv[static_cast<size_t>(r) * d_inner + chan];
        dval = __ldg(Dp + chan / d_head);
        const float4* st4 = reinterpret_cast<const float4*>(state + (static_cast<size_t>(r) * d_inner + chan) * N);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 v = st4[q];
            hv[4 * q] = v.x; hv[4 * q + 1] = v.y; hv[4 * q + 2] = v.z; hv[4 * q + 3] = v.w;
        }
    }
    cluster.sync();          // every CTA holds the taps it needs: the windows may move on; conv outputs visible
    if (c >= 0 && (c < d_inner || rank == 0)) {
#pragma unroll
        for (int j = 0; j + 1 < kMaxK; ++j)
            if (j < taps) rr[static_cast<size_t>(j) * conv_dim + c] = tapv[j + 1];
    }
    float ss = 0.0f, gv = 0.0f;
    if (idx < n_own) {
        const int h = chan / d_head;
        const int group = (h * n_groups) / n_heads;
        const float delta = delta_s[h], decay = decay_s[h];
        const float input = xs[idx];
        const float* Bg = bc + group * N;
        const float* Cg = bc + GS + group * N;
        float y = __fmul_rn(dval, input);
#pragma unroll
        for (int n = 0; n < N; ++n) {
            hv[n] = __fadd_rn(__fmul_rn(decay, hv[n]), __fmul_rn(__fmul_rn(delta, Bg[n]), input));
            y = __fadd_rn(y, __fmul_rn(hv[n], Cg[n]));
        }
        float4* st4 = reinterpret_cast<float4*>(state + (static_cast<size_t>(r) * d_inner + chan) * N);
#pragma unroll
        for (int q = 0; q < 4; ++q) st4[q] = make_float4(hv[4 * q], hv[4 * q + 1], hv[4 * q + 2], hv[4 * q + 3]);
        gv = __fmul_rn(y, silu_two_sided(zval));
        ss = gv * gv;
    }
    const float partial = block_sum(ss, scratch);
    if (threadIdx.x == 0) cluster.map_shared_rank(parts, 0)[rank] = partial;
    cluster.sync();
    const float* all = cluster.map_shared_rank(parts, 0);
    float total = 0.0f;
    for (int k = 0; k < kMixCluster; ++k) total += all[k];        // fixed order: the same sum in every CTA
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(d_inner)), eps)));
    float o = 0.0f;
    if (idx < n_own) {
        const float n = __fmul_rn(gv, inv);
        o = norm_w ? __fmul_rn(n, __ldg(norm_w + chan)) : n;
        if (!codes.codes) out[static_cast<size_t>(r) * d_inner + chan] = o;
    }
    if (codes.codes) {
        // the row as 8-bit codes for the out projection: absmax over the cluster, then every thread rounds its channel
        const float cta_max = block_max(fabsf(o), scratch);
        if (threadIdx.x == 0) cluster.map_shared_rank(maxes, 0)[rank] = cta_max;
        cluster.sync();
        const float* all_max = cluster.map_shared_rank(maxes, 0);
        float mx = 0.0f;
        for (int k = 0; k < kMixCluster; ++k) mx = fmaxf(mx, all_max[k]);
        const float denom = __fadd_rn(mx, 1e-8f);
        const float scale = __fdiv_rn(127.0f, denom);
        int c = 0;
        if (idx < n_own) {
            c = static_cast<int8_t>(round_code(__fmul_rn(o, scale), false));
            codes.codes[code_offset(codes, r, chan)] = static_cast<int8_t>(c);
        }
        if (rank == kMixCluster - 1)            // the padding up to the leading dimension
            for (int k = d_inner + idx; k < codes.ld; k += kMixThreads) codes.codes[code_offset(codes, r, k)] = 0;
        c = __reduce_add_sync(0xffffffffu, c);
        __syncthreads();                        // block_max's readers are done with scratch
        int* iscratch = reinterpret_cast<int*>(scratch);
        if ((threadIdx.x & 31) == 0) iscratch[threadIdx.x >> 5] = c;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < kMixThreads / 32; ++w) t += iscratch[w];
            cluster.map_shared_rank(code_sums, 0)[rank] = t;
            if (rank == 0) codes.act_scales[r] = __fdiv_rn(denom, 127.0f);
        }
    }
    cluster.sync();          // rank 0's shared memory stays alive until every CTA has read (and written) what it exchanges there
    if (codes.codes && rank == 0 && threadIdx.x == 0) {
        int t = 0;
        for (int k = 0; k < kMixCluster; ++k) t += code_sums[k];
        codes.q_sums[r] = t;
    }
}

// ---- out = x + (a * ga [+ b * gb]); ga == null: out = x + a ----------------------------------------------------
__global__ void __launch_bounds__(256) gated_residual_kernel(const float* __restrict__ x, const float* __restrict__ a,
                                                             const float* __restrict__ ga, const float* __restrict__ b,
                                                             const float* __restrict__ gb, int rows, int D,
                                                             float* __restrict__ out, float* __restrict__ trace) {
    const int64_t n = static_cast<int64_t>(rows) * D;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int d = static_cast<int>(i % D);
        float contrib = ga ? __fmul_rn(a[i], __ldg(ga + d)) : a[i];
        if (b) contrib = __fadd_rn(contrib, __fmul_rn(b[i], __ldg(gb + d)));
        const float v = __fadd_rn(x[i], contrib);
        out[i] = v;
        if (trace) trace[i] = v;
    }
}

__global__ void advance_positions_kernel(int32_t* positions, int rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) positions[r] += 1;
}

// ---- state layout ----------------------------------------------------------------------------------------------
struct BlockState {
    float* ring;
    float* ssm;
    float* k_cache;
    float* v_cache;
};

struct StateLayout {
    int32_t* positions;
    BlockState block[TBL_MAX_DECODE_BLOCKS];
    size_t bytes;
};

StateLayout carve_state(const tbl_decode_model& m, int batch, int capacity, void* base) {
    StateLayout L{};
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { uint8_t* r = p + off; off += round_up(bytes, 256); return r; };
    L.positions = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * batch));
    for (int i = 0; i < m.n_blocks; ++i) {
        const tbl_decode_block& b = m.blocks[i];
        const int conv_dim = b.mamba.d_inner + 2 * b.mamba.n_groups * b.mamba.d_state;
        const int taps = b.mamba.conv_kernel > 1 ? b.mamba.conv_kernel - 1 : 0;
        L.block[i].ring = reinterpret_cast<float*>(take(sizeof(float) * batch * (taps ? taps : 1) * conv_dim));
        L.block[i].ssm = reinterpret_cast<float*>(take(sizeof(float) * batch * static_cast<size_t>(b.mamba.d_inner) * b.mamba.d_state));
        if (b.hybrid) {
            const size_t kv = sizeof(float) * batch * static_cast<size_t>(capacity) * b.attn.n_kv_heads * b.attn.head_dim;
            L.block[i].k_cache = reinterpret_cast<float*>(take(kv));
            L.block[i].v_cache = reinterpret_cast<float*>(take(kv));
        }
    }
    L.bytes = off;
    return L;
}

int check_model(const tbl_decode_model* m, int batch, int capacity) {
    if (!m || !m->blocks || !m->embedding || batch <= 0 || capacity <= 0) return TBL_ERR_INVALID_ARG;
    if (m->n_blocks <= 0 || m->n_blocks > TBL_MAX_DECODE_BLOCKS || m->d_model <= 0 || m->vocab <= 0) return TBL_ERR_INVALID_ARG;
    for (int i = 0; i < m->n_blocks; ++i) {
        const tbl_decode_block& b = m->blocks[i];
        const tbl_mamba_block& mm = b.mamba;
        if (mm.d_inner <= 0 || mm.n_heads <= 0 || mm.d_head <= 0 || mm.n_groups <= 0 || mm.d_state <= 0 ||
            mm.conv_kernel < 1 || mm.n_heads * mm.d_head != mm.d_inner || mm.n_heads % mm.n_groups)
            return TBL_ERR_SHAPE;
        if (!mm.A_log || !mm.D || !mm.conv_w || !mm.conv_b) return TBL_ERR_INVALID_ARG;
        const int GS = mm.n_groups * mm.d_state;
        if (mm.x.inputs != m->d_model || mm.x.outputs != mm.d_inner || mm.z.outputs != mm.d_inner || mm.B.outputs != GS ||
            mm.C.outputs != GS || mm.dt.outputs != mm.n_heads || mm.out.inputs != mm.d_inner || mm.out.outputs != m->d_model)
            return TBL_ERR_SHAPE;
        if (b.hybrid) {
            const tbl_attention_block& a = b.attn;
            if (a.n_heads <= 0 || a.n_kv_heads <= 0 || a.head_dim <= 0 || a.head_dim % 4 || a.n_heads * a.head_dim != m->d_model ||
                a.sliding_window <= 0 || !a.rope_cos || !a.rope_sin || a.rope_positions <= 0)
                return TBL_ERR_SHAPE;
            if (a.q.outputs != m->d_model || a.kv.outputs != 2 * a.n_kv_heads * a.head_dim || a.out.inputs != m->d_model)
                return TBL_ERR_SHAPE;
            if (!b.mamba_gate || !b.attn_gate || !b.ffn_gate) return TBL_ERR_INVALID_ARG;
            if (b.ffn_up.inputs != m->d_model || b.ffn_down.inputs != b.ffn_up.outputs || b.ffn_down.outputs != m->d_model)
                return TBL_ERR_SHAPE;
        }
    }
    if (m->head.inputs != m->d_model || m->head.outputs != m->vocab) return TBL_ERR_SHAPE;
    return TBL_OK;
}

struct Scratch {
    float *hidden[2], *core, *attn_in, *proj, *xbc, *y, *gated, *mamba_out, *qkv, *heads, *attn_out, *res, *ffn_in, *ffn_mid, *ffn_out;
    void* lin;
    // rows that a glue kernel hands to the widening GEMM as 8-bit codes (RowCodes), with their scales and code sums
    int8_t* codes;
    float* code_scales;
    int32_t* code_sums;
    size_t lin_bytes, proj_stride, qkv_stride, bytes;
};

Scratch carve_scratch(const tbl_decode_model& m, int batch, void* base) {
    Scratch S{};
    uint8_t* p = static_cast<uint8_t*>(base);
    size_t off = 0;
    auto take = [&](size_t floats) { float* r = reinterpret_cast<float*>(p + off); off += round_up(floats * sizeof(float), 256); return r; };
    int max_inner = 1, max_conv = 1, max_kvout = 1, max_ffn = 1;
    size_t lin = 0;
    auto want = [&](size_t b) { lin = b > lin ? b : lin; };
    const int D = m.d_model;
    for (int i = 0; i < m.n_blocks; ++i) {
        const tbl_decode_block& b = m.blocks[i];
        max_inner = b.mamba.d_inner > max_inner ? b.mamba.d_inner : max_inner;
        const int conv_dim = b.mamba.d_inner + 2 * b.mamba.n_groups * b.mamba.d_state;
        max_conv = conv_dim > max_conv ? conv_dim : max_conv;
        want(tbl_grouped_rows_workspace_bytes(5, batch < 64 ? batch : 64, D));
        want(tbl_linear_workspace_bytes(batch, D, b.mamba.d_inner));
        want(tbl_linear_workspace_bytes(batch, b.mamba.d_inner, D));
        if (b.hybrid) {
            max_kvout = b.attn.kv.outputs > max_kvout ? b.attn.kv.outputs : max_kvout;
            max_kvout = D > max_kvout ? D : max_kvout;
            max_ffn = b.ffn_up.outputs > max_ffn ? b.ffn_up.outputs : max_ffn;
            want(tbl_linear_workspace_bytes(batch, D, b.ffn_up.outputs));
            want(tbl_linear_workspace_bytes(batch, b.ffn_up.outputs, D));
            want(tbl_linear_workspace_bytes(batch, D, D));
        }
    }
    want(tbl_linear_workspace_bytes(batch, D, m.vocab));
    const size_t BD = static_cast<size_t>(batch) * D;
    S.hidden[0] = take(BD); S.hidden[1] = take(BD);
    S.core = take(BD); S.attn_in = take(BD);
    S.proj_stride = static_cast<size_t>(batch) * max_inner;
    S.proj = take(5 * S.proj_stride);
    S.xbc = take(static_cast<size_t>(batch) * max_conv);
    S.y = take(static_cast<size_t>(batch) * max_inner);
    S.gated = take(static_cast<size_t>(batch) * max_inner);
    S.mamba_out = take(BD);
    S.qkv_stride = static_cast<size_t>(batch) * max_kvout;
    S.qkv = take(2 * S.qkv_stride);
    S.heads = take(BD); S.attn_out = take(BD); S.res = take(BD); S.ffn_in = take(BD); S.ffn_out = take(BD);
    S.ffn_mid = take(static_cast<size_t>(batch) * max_ffn);
    S.lin = p + off;
    S.lin_bytes = round_up(lin, 256);
    off += S.lin_bytes;
    const int widest = max_inner > D ? max_inner : D;
    S.codes = reinterpret_cast<int8_t*>(p + off);
    off += round_up(static_cast<size_t>(batch) * gemm_widen_plane_ld(widest), 256);
    S.code_scales = take(batch);
    S.code_sums = reinterpret_cast<int32_t*>(take(batch));
    S.bytes = off;
    return S;
}

}  // namespace
}  // namespace tbl

using namespace tbl;

extern "C" {

int tbl_embedding_gather(const int32_t* ids_dev, int count, const float* table_dev, int vocab, int dim, float* out_dev,
                         void* stream) {
    if (!ids_dev || !table_dev || !out_dev || count <= 0 || vocab <= 0 || dim <= 0) return TBL_ERR_INVALID_ARG;
    embedding_gather_kernel<<<count, 256, 0, static_cast<cudaStream_t>(stream)>>>(ids_dev, table_dev, vocab, dim, out_dev, nullptr);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

int tbl_mamba_conv_step(const float* x_dev, const float* B_dev, const float* C_dev, const float* conv_w_dev,
                        const float* conv_b_dev, float* ring_dev, float* xbc_dev, int d_inner, int group_state,
                        int conv_kernel, int rows, void* stream) {
    if (!x_dev || !B_dev || !C_dev || !conv_w_dev || !conv_b_dev || !ring_dev || !xbc_dev) return TBL_ERR_INVALID_ARG;
    if (d_inner <= 0 || group_state <= 0 || conv_kernel < 1 || rows <= 0) return TBL_ERR_INVALID_ARG;
    const int conv_dim = d_inner + 2 * group_state;
    mamba_conv_step_kernel<<<dim3((conv_dim + 255) / 256, rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        x_dev, B_dev, C_dev, conv_w_dev, conv_b_dev, ring_dev, d_inner, group_state, conv_kernel, xbc_dev);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

int tbl_mamba_ssd_step(const float* xbc_dev, const float* dt_dev, const float* A_log_dev, const float* D_dev,
                       float* state_dev, float* y_dev, int n_heads, int d_head, int d_state, int n_groups, int rows,
                       void* stream) {
    if (!xbc_dev || !dt_dev || !A_log_dev || !D_dev || !state_dev || !y_dev) return TBL_ERR_INVALID_ARG;
    if (n_heads <= 0 || d_head <= 0 || d_state <= 0 || n_groups <= 0 || n_heads % n_groups || rows <= 0) return TBL_ERR_INVALID_ARG;
    mamba_ssd_step_kernel<<<dim3((n_heads * d_head + 127) / 128, rows), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        xbc_dev, dt_dev, A_log_dev, D_dev, state_dev, n_heads, d_head, d_state, n_groups, y_dev);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

int tbl_attention_decode(const float* q_dev, const float* kv_dev, float* k_cache_dev, float* v_cache_dev, int capacity,
                         const int32_t* positions_dev, const float* rope_cos_dev, const float* rope_sin_dev,
                         int rope_positions, int n_heads, int n_kv_heads, int head_dim, int sliding_window, int rows,
                         float* out_dev, void* stream) {
    if (!q_dev || !kv_dev || !k_cache_dev || !v_cache_dev || !positions_dev || !rope_cos_dev || !rope_sin_dev || !out_dev)
        return TBL_ERR_INVALID_ARG;
    if (capacity <= 0 || rope_positions <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || head_dim % 4 ||
        sliding_window <= 0 || rows <= 0)
        return TBL_ERR_INVALID_ARG;
    if (head_dim > kAttnMaxHeadDim || (n_kv_heads * head_dim) % 4) return TBL_ERR_SHAPE;
    const size_t smem = attention_smem_bytes(head_dim, capacity);
    if (smem > 200 * 1024) return TBL_ERR_SHAPE;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return TBL_ERR_CUDA;
    int* status = device_status_ptr();
    if (!status) return TBL_ERR_CUDA;
    attention_decode_kernel<<<dim3(n_heads, rows), kAttnThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        q_dev, kv_dev, k_cache_dev, v_cache_dev, capacity, positions_dev, rope_cos_dev, rope_sin_dev, rope_positions, n_heads,
        n_kv_heads, head_dim, sliding_window, out_dev, status);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

int tbl_gated_residual(const float* x_dev, const float* a_dev, const float* gate_a_dev, const float* b_dev,
                       const float* gate_b_dev, int rows, int dim, float* out_dev, void* stream) {
    if (!x_dev || !a_dev || !out_dev || rows <= 0 || dim <= 0 || (b_dev && !gate_b_dev)) return TBL_ERR_INVALID_ARG;
    const int64_t n = static_cast<int64_t>(rows) * dim;
    const int grid = static_cast<int>((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    gated_residual_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(x_dev, a_dev, gate_a_dev, b_dev, gate_b_dev, rows,
                                                                               dim, out_dev, nullptr);
    note_launch();
    return cudaGetLastError() == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
}

size_t tbl_decode_state_bytes(const tbl_decode_model* model, int batch, int capacity) {
    if (check_model(model, batch, capacity) != TBL_OK) return 0;
    return carve_state(*model, batch, capacity, nullptr).bytes;
}

int tbl_decode_state_reset(const tbl_decode_model* model, int batch, int capacity, void* state_dev, size_t state_bytes,
                           void* stream) {
    const int rc = check_model(model, batch, capacity);
    if (rc != TBL_OK) return rc;
    if (!state_dev || state_bytes < tbl_decode_state_bytes(model, batch, capacity)) return TBL_ERR_WORKSPACE;
    const StateLayout L = carve_state(*model, batch, capacity, state_dev);
    // positions, conv rings and SSM states start at zero; the KV caches are only read below the positions
    const size_t head = reinterpret_cast<uint8_t*>(L.block[0].ring) - static_cast<uint8_t*>(state_dev);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(state_dev, 0, head, st) != cudaSuccess) return TBL_ERR_CUDA;
    for (int i = 0; i < model->n_blocks; ++i) {
        const tbl_mamba_block& mm = model->blocks[i].mamba;
        const int conv_dim = mm.d_inner + 2 * mm.n_groups * mm.d_state;
        const int taps = mm.conv_kernel > 1 ? mm.conv_kernel - 1 : 1;
        if (cudaMemsetAsync(L.block[i].ring, 0, sizeof(float) * batch * taps * conv_dim, st) != cudaSuccess) return TBL_ERR_CUDA;
        if (cudaMemsetAsync(L.block[i].ssm, 0, sizeof(float) * batch * static_cast<size_t>(mm.d_inner) * mm.d_state, st) != cudaSuccess)
            return TBL_ERR_CUDA;
    }
    return TBL_OK;
}

size_t tbl_decode_workspace_bytes(const tbl_decode_model* model, int batch) {
    if (check_model(model, batch, 1) != TBL_OK) return 0;
    return carve_scratch(*model, batch, nullptr).bytes;
}

int tbl_decode_step(const tbl_decode_model* model, int batch, int capacity, void* state_dev, const int32_t* token_ids_dev,
                    float* logits_dev, float* hidden_trace_dev, void* workspace_dev, size_t workspace_bytes, void* stream) {
    int rc = check_model(model, batch, capacity);
    if (rc != TBL_OK) return rc;
    if (!state_dev || !token_ids_dev || !logits_dev) return TBL_ERR_INVALID_ARG;
    if (!workspace_dev || workspace_bytes < tbl_decode_workspace_bytes(model, batch)) return TBL_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace_dev) & 255) || (reinterpret_cast<uintptr_t>(state_dev) & 255)) return TBL_ERR_ALIGNMENT;
    const tbl_decode_model& m = *model;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const StateLayout state = carve_state(m, batch, capacity, state_dev);
    const Scratch S = carve_scratch(m, batch, workspace_dev);
    int* status = device_status_ptr();
    if (!status) return TBL_ERR_CUDA;
    const int D = m.d_model, B = batch;
    const size_t BD = static_cast<size_t>(B) * D;
    if (sizeof(float) * (D + 32) > 48 * 1024) return TBL_ERR_SHAPE;   // the fused glue keeps a row of the residual stream in shared memory
    auto launched = [&]() { note_launch(); return cudaGetLastError() == cudaSuccess ? TBL_OK : TBL_ERR_CUDA; };
    auto linear = [&](const tbl_linear_view& v, const float* x, float* y) {
        return tbl_linear_forward(x, v.packed, v.strips, B > 64 ? v.w_i8 : nullptr, v.weight_scale, B, v.inputs, v.outputs,
                                  v.activation_bits, v.rms_input ? TBL_RMS_FAST : TBL_RMS_NONE, v.magnitude, v.bias, y,
                                  S.lin, S.lin_bytes, stream);
    };
    auto group = [&](const tbl_linear_view* views, int count, const float* x, float* out, size_t stride) {
        if (B <= 64) return tbl_grouped_forward_rows(views, count, x, B, out, static_cast<long long>(stride), TBL_RMS_NONE,
                                                      S.lin, S.lin_bytes, stream);
        for (int g = 0; g < count; ++g) {
            const int r = linear(views[g], x, out + g * stride);
            if (r != TBL_OK) return r;
        }
        return TBL_OK;
    };
    // closes the pending residual add (x + a*ga [+ b*gb]) into `hidden_out` and opens the next stage with up to
    // two norms of the sum; with ids: x is the embedding row
    auto residual_norm = [&](const float* x, const int32_t* ids, const float* a, const float* ga, const float* b2,
                             const float* gb, float eps, const float* w1, const float* w2, float* hidden_out, float* trace,
                             float* out1, float* out2, RowCodes codes1 = RowCodes{}) {
        residual_norm_kernel<<<B, kFusedThreads, sizeof(float) * (D + 32), st>>>(x, ids, m.embedding, m.vocab, a, ga, b2, gb, D, eps,
                                                                                 w1, w2, hidden_out, trace, out1, out2, codes1);
        return launched();
    };
    // Batches past the fused-prologue GEMV's range: the kernel that produces a projection's input rows also quantises
    // them (RowCodes), and the projections run straight on the codes -- no stand-alone quantiser launch.  Up to 16
    // rows the codes go to the tiled strip GEMV, from 17 to 64 rows to the widening tensor-core GEMM.
    const bool fold = B <= gemv_strip_fused_rows(D);
    // (the widening kernel's fixed cost per launch beats the strip GEMV's 8-row passes from 17 rows on at the widths of
    // a decode step; on their own, large matrices switch at 33 rows)
    constexpr int kCodeWidenMinRows = 16;
    const bool code_widen = B > kCodeWidenMinRows && B <= 64;
    const bool code_strip = !fold && B <= kCodeWidenMinRows;
    auto takes_codes = [&](const tbl_linear_view* v, int count) {
        if (!(code_widen || code_strip) || count > (code_widen ? kWidenMaxViews : TBL_MAX_GROUPS)) return false;
        for (int g = 0; g < count; ++g) {
            if (!v[g].strips || (reinterpret_cast<uintptr_t>(v[g].strips) & 15) || v[g].rms_input || v[g].activation_bits != 8 ||
                v[g].inputs != v[0].inputs)
                return false;
            if (code_widen ? !gemm_widen_supported(B, v[g].inputs, v[g].outputs) : !gemv_strip_supported(v[g].inputs)) return false;
        }
        return true;
    };
    auto row_codes = [&](int K) {
        return RowCodes{S.codes, S.code_scales, S.code_sums, code_widen ? gemm_widen_plane_ld(K) : K, code_widen ? 0 : B};
    };
    auto gemm_on_codes = [&](const tbl_linear_view* v, int count, float* out, size_t stride) {
        cudaError_t e;
        if (code_widen) {
            WidenView wv[kWidenMaxViews];
            for (int g = 0; g < count; ++g) {
                wv[g] = WidenView{};
                wv[g].strips = v[g].strips; wv[g].magnitude = v[g].magnitude; wv[g].bias = v[g].bias;
                wv[g].y = out + g * stride; wv[g].weight_scale = v[g].weight_scale; wv[g].N = v[g].outputs;
            }
            e = launch_gemm_widen(wv, count, nullptr, S.codes, S.code_scales, S.code_sums, B, v[0].inputs, st);
        } else {
            StripProblem pr[TBL_MAX_GROUPS];
            for (int g = 0; g < count; ++g) {
                pr[g] = StripProblem{};
                pr[g].strips = static_cast<const uint8_t*>(v[g].strips); pr[g].qp = S.codes;
                pr[g].act_scales = S.code_scales; pr[g].q_sums = S.code_sums;
                pr[g].magnitude = v[g].magnitude; pr[g].bias = v[g].bias; pr[g].y = out + g * stride;
                pr[g].weight_scale = v[g].weight_scale; pr[g].rows = B; pr[g].N = v[g].outputs; pr[g].K = v[g].inputs;
                pr[g].ldy = v[g].outputs;
            }
            e = launch_gemv_strip(pr, count, st);
        }
        return e == cudaSuccess ? TBL_OK : TBL_ERR_CUDA;
    };

    // The residual add that ends a block is carried as "pending" and applied by the kernel that opens the next
    // stage: h = x_pending + (a*ga + b*gb).  For few rows (B * D <= 16384) that kernel is the GEMV itself: the
    // add, the store of the residual stream and the RMSNorm x weight run in its prologue (StripPrologue), so a block
    // costs no launch for them; the first block (embedding rows) and larger batches use residual_norm_kernel.
    struct Pending { const float* x; const int32_t* ids; const float* a; const float* ga; const float* b; const float* gb; };
    Pending pend{nullptr, token_ids_dev, nullptr, nullptr, nullptr, nullptr};
    auto pre_of = [](const Pending& pd, const float* norm_w, float eps, float* hidden_out, float* trace) {
        StripPrologue pre{};
        pre.a = pd.a; pre.ga = pd.ga; pre.b = pd.b; pre.gb = pd.gb;
        pre.norm_w = norm_w; pre.norm_eps = eps; pre.hidden_out = hidden_out; pre.trace_out = trace;
        return pre;
    };
    int cur = 0;
    for (int i = 0; i < m.n_blocks; ++i) {
        const tbl_decode_block& b = m.blocks[i];
        const tbl_mamba_block& mm = b.mamba;
        if (mm.d_inner > 16 * 1024) return TBL_ERR_SHAPE;
        float* h = S.hidden[cur];
        float* trace = hidden_trace_dev ? hidden_trace_dev + static_cast<size_t>(i) * BD : nullptr;
        const tbl_linear_view proj[5] = {mm.x, mm.z, mm.B, mm.C, mm.dt};
        // hidden state entering this block (+ trace of the previous block's output), core norm, then the five
        // projections of the normalised row
        bool folded = false;
        if (fold && !pend.ids) {
            rc = grouped_forward_rows_pre(proj, 5, pend.x, B, S.proj, static_cast<long long>(S.proj_stride),
                                          pre_of(pend, b.core_norm_w, b.core_norm_eps, h, trace), st);
            if (rc == TBL_OK) folded = true;
            else if (rc != TBL_ERR_UNSUPPORTED) return rc;
        }
        if (!folded) {
            const bool coded = takes_codes(proj, 5) && proj[0].inputs == D;
            if ((rc = residual_norm(pend.x, pend.ids, pend.a, pend.ga, pend.b, pend.gb, b.core_norm_eps, b.core_norm_w,
                                    b.hybrid ? b.attn_norm_w : nullptr, h, trace, coded ? nullptr : S.core,
                                    b.hybrid ? S.attn_in : nullptr, coded ? row_codes(D) : RowCodes{})) != TBL_OK)
                return rc;
            if ((rc = coded ? gemm_on_codes(proj, 5, S.proj, S.proj_stride) : group(proj, 5, S.core, S.proj, S.proj_stride)) != TBL_OK)
                return rc;
        }
        // conv step + SSD step + gated norm in one kernel, then the out projection
        const int GS = mm.n_groups * mm.d_state, conv_dim = mm.d_inner + 2 * GS;
        const size_t mix_smem = sizeof(float) * (conv_dim + mm.d_inner + 2 * mm.n_heads + 32);
        if (mix_smem > 48 * 1024) {
            static bool configured[64] = {};
            int dev = 0;
            cudaGetDevice(&dev);
            if (dev < 0 || dev >= 64 || !configured[dev]) {
                if (cudaFuncSetAttribute(mamba_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
                    return TBL_ERR_CUDA;
                if (dev >= 0 && dev < 64) configured[dev] = true;
            }
        }
        const int per_cta = (mm.d_inner + kMixCluster - 1) / kMixCluster;
        const bool clustered = mm.d_state == 16 && mm.conv_kernel >= 1 && mm.conv_kernel <= 4 && per_cta + 2 * GS <= kMixThreads;
        const bool out_coded = clustered && takes_codes(&mm.out, 1) && mm.out.inputs == mm.d_inner;
        if (clustered) {
            // a sequence's channels over a cluster of 8 CTAs
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(static_cast<unsigned>(kMixCluster) * B);
            cfg.blockDim = dim3(kMixThreads);
            cfg.dynamicSmemBytes = sizeof(float) * (per_cta + 2 * GS + 2 * mm.n_heads + 32 + 3 * kMixCluster);
            cfg.stream = st;
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = kMixCluster; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            if (cudaLaunchKernelEx(&cfg, mamba_mix_cluster_kernel, static_cast<const float*>(S.proj),
                                   static_cast<const float*>(S.proj + S.proj_stride),
                                   static_cast<const float*>(S.proj + 2 * S.proj_stride),
                                   static_cast<const float*>(S.proj + 3 * S.proj_stride),
                                   static_cast<const float*>(S.proj + 4 * S.proj_stride), mm.conv_w, mm.conv_b, mm.A_log, mm.D,
                                   mm.norm_w, state.block[i].ring, state.block[i].ssm, mm.n_heads, mm.d_head, mm.n_groups,
                                   mm.conv_kernel, mm.norm_eps, S.gated, out_coded ? row_codes(mm.d_inner) : RowCodes{}) != cudaSuccess)
                return TBL_ERR_CUDA;
        } else {
            mamba_mix_kernel<<<B, kFusedThreads, mix_smem, st>>>(
                S.proj, S.proj + S.proj_stride, S.proj + 2 * S.proj_stride, S.proj + 3 * S.proj_stride, S.proj + 4 * S.proj_stride,
                mm.conv_w, mm.conv_b, mm.A_log, mm.D, mm.norm_w, state.block[i].ring, state.block[i].ssm, mm.n_heads, mm.d_head,
                mm.d_state, mm.n_groups, mm.conv_kernel, mm.norm_eps, S.gated);
        }
        if ((rc = launched()) != TBL_OK) return rc;
        if ((rc = out_coded ? gemm_on_codes(&mm.out, 1, S.mamba_out, 0) : linear(mm.out, S.gated, S.mamba_out)) != TBL_OK) return rc;
        if (!b.hybrid) {
            pend = Pending{h, nullptr, S.mamba_out, nullptr, nullptr, nullptr};
            cur ^= 1;
            continue;
        }
        // attention branch on its own norm of the same residual stream
        const tbl_attention_block& a = b.attn;
        const tbl_linear_view qkv[2] = {a.q, a.kv};
        bool qkv_folded = false;
        if (folded) {
            rc = grouped_forward_rows_pre(qkv, 2, h, B, S.qkv, static_cast<long long>(S.qkv_stride),
                                          pre_of(Pending{}, b.attn_norm_w, b.core_norm_eps, nullptr, nullptr), st);
            if (rc == TBL_OK) qkv_folded = true;
            else if (rc != TBL_ERR_UNSUPPORTED) return rc;
            if (!qkv_folded) {
                // the attention norm alone (x = h, nothing pending), then the projections
                if ((rc = residual_norm(h, nullptr, nullptr, nullptr, nullptr, nullptr, b.core_norm_eps, b.attn_norm_w, nullptr,
                                        nullptr, nullptr, S.attn_in, nullptr)) != TBL_OK)
                    return rc;
            }
        }
        if (!qkv_folded && (rc = group(qkv, 2, S.attn_in, S.qkv, S.qkv_stride)) != TBL_OK) return rc;
        if (a.head_dim > kAttnMaxHeadDim || a.head_dim % 4) return TBL_ERR_SHAPE;
        const size_t attn_smem = attention_smem_bytes(a.head_dim, capacity);
        if (attn_smem > 200 * 1024) return TBL_ERR_SHAPE;
        if (attn_smem > 48 * 1024) {
            static bool configured[64] = {};
            int dev = 0;
            cudaGetDevice(&dev);
            if (dev < 0 || dev >= 64 || !configured[dev]) {
                if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
                    return TBL_ERR_CUDA;
                if (dev >= 0 && dev < 64) configured[dev] = true;
            }
        }
        attention_decode_kernel<<<dim3(a.n_heads, B), kAttnThreads, attn_smem, st>>>(
            S.qkv, S.qkv + S.qkv_stride, state.block[i].k_cache, state.block[i].v_cache, capacity, state.positions,
            a.rope_cos, a.rope_sin, a.rope_positions, a.n_heads, a.n_kv_heads, a.head_dim, a.sliding_window, S.heads, status);
        if ((rc = launched()) != TBL_OK) return rc;
        if ((rc = linear(a.out, S.heads, S.attn_out)) != TBL_OK) return rc;
        // res = h + (mamba*gate + attn*gate), and its norm for the FFN: up -> squared ReLU -> down (two launches with
        // the squared ReLU in the first one's epilogue: at this width a launch boundary is cheaper than the persistent
        // stack's grid-wide layer boundary)
        bool up_folded = false;
        if (fold) {
            rc = linear_view_forward_pre(b.ffn_up, h, B, true,
                                         pre_of(Pending{nullptr, nullptr, S.mamba_out, b.mamba_gate, S.attn_out, b.attn_gate},
                                                b.ff_norm_w, 1e-5f, S.res, nullptr),
                                         S.ffn_mid, st);
            if (rc == TBL_OK) up_folded = true;
            else if (rc != TBL_ERR_UNSUPPORTED) return rc;
        }
        if (!up_folded) {
            if ((rc = residual_norm(h, nullptr, S.mamba_out, b.mamba_gate, S.attn_out, b.attn_gate, 1e-5f, b.ff_norm_w, nullptr, S.res,
                                    nullptr, S.ffn_in, nullptr)) != TBL_OK)
                return rc;
            if ((rc = linear_view_forward(b.ffn_up, S.ffn_in, B, TBL_RMS_FAST, true, S.ffn_mid, S.lin, S.lin_bytes, st)) != TBL_OK) return rc;
        }
        if ((rc = linear_view_forward(b.ffn_down, S.ffn_mid, B, TBL_RMS_FAST, false, S.ffn_out, S.lin, S.lin_bytes, st)) != TBL_OK) return rc;
        pend = Pending{S.res, nullptr, S.ffn_out, b.ffn_gate, nullptr, nullptr};
        cur ^= 1;
    }
    // the last block's residual add, the final norm and the LM head
    float* last_trace = hidden_trace_dev ? hidden_trace_dev + static_cast<size_t>(m.n_blocks) * BD : nullptr;
    bool head_folded = false;
    if (fold && !pend.ids) {
        rc = linear_view_forward_pre(m.head, pend.x, B, false, pre_of(pend, m.final_norm_w, m.final_norm_eps, S.hidden[cur], last_trace),
                                     logits_dev, st);
        if (rc == TBL_OK) head_folded = true;
        else if (rc != TBL_ERR_UNSUPPORTED) return rc;
    }
    if (!head_folded) {
        if ((rc = residual_norm(pend.x, pend.ids, pend.a, pend.ga, pend.b, pend.gb, m.final_norm_eps, m.final_norm_w, nullptr,
                                S.hidden[cur], last_trace, S.core, nullptr)) != TBL_OK)
            return rc;
        if ((rc = linear(m.head, S.core, logits_dev)) != TBL_OK) return rc;
    }
    advance_positions_kernel<<<(B + 127) / 128, 128, 0, st>>>(state.positions, B);
    return launched();
}

}  // extern "C"
