/*
 * CPU oracle for the BitNet b1.58 ternary linear path (TEST INFRASTRUCTURE ONLY).
 *
 * This file restates, in plain scalar C, the arithmetic of the NSOS runtime's packed
 * ternary linear (OXN/nsos).  It exists so the CUDA kernels can be checked against an
 * independent implementation; it is never linked into, imported by, or called from the
 * shipped library.  Only the tests, the smoke check and the bench's CPU-baseline legs
 * may use it.
 *
 * Parity status: PINNED.  Every function here is compared bit-for-bit against the
 * reference's own C++ (compiled from its sources by oracle/Makefile into oracle/_ref)
 * and against golden vectors generated from that build (tests/golden).
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared (no -mfma, no -ffast-math): the
 * reference's default x86-64 build has no FMA contraction on this path, so every
 * multiply and add below must stay a separately rounded fp32 operation.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- A1: absmean ---------------------------------------------------------------
 * OXN/nsos/src/tensor.cpp:2097-2102 (tensor_abs_mean, CPU branch): a strictly
 * left-to-right sum of |w| in double, divided by n in double, narrowed to float. */
float tor_abs_mean(const float* w, int64_t n) {
    if (n <= 0) return 0.0f;
    double total = 0.0;
    for (int64_t i = 0; i < n; ++i) total += fabs((double)w[i]);
    return (float)(total / (double)n);
}

/* ---- A2: ternary codes ---------------------------------------------------------
 * OXN/nsos/src/bitlinear.cpp:1359-1379 (BitLinear::quantize_weights):
 * scale = absmean + 1e-8f; v = w / (scale + 1e-8f); strict 0.5 thresholds. */
void tor_quantize_weights(const float* w, int64_t n, int8_t* t) {
    const float scale = tor_abs_mean(w, n) + 1e-8f;
    const float denom = scale + 1e-8f;
    for (int64_t i = 0; i < n; ++i) {
        const float v = w[i] / denom;
        t[i] = v > 0.5f ? 1 : (v < -0.5f ? -1 : 0);
    }
}

/* ---- A3: packer ------------------------------------------------------------------
 * OXN/nsos/src/bitlinear.cpp:152-193 (BitLinear::pack_weights) and
 * OXN/nsos/src/bitnet_adapter.cpp:570-606 (pack/unpack "microsoft style"):
 * weight_scale = absmean + 1e-8f; code (t+1) at bits 2*(i%4) of byte i/4, i = n*K+k,
 * bytes little-endian inside uint32 words; word count ceil(ceil(N*K/4)/4).
 * words must hold tor_packed_words(N,K) entries.  t_out / row_sums may be NULL.
 * Returns weight_scale. */
int64_t tor_packed_words(int N, int K) {
    const int64_t bytes = ((int64_t)N * K + 3) / 4;
    return (bytes + 3) / 4;
}

float tor_pack_weights(const float* w, int N, int K, uint32_t* words,
                       int8_t* t_out, int32_t* row_sums) {
    const int64_t total = (int64_t)N * K;
    const float weight_scale = tor_abs_mean(w, total) + 1e-8f;
    int8_t* t = t_out ? t_out : (int8_t*)malloc((size_t)total);
    tor_quantize_weights(w, total, t);
    const int64_t nwords = tor_packed_words(N, K);
    memset(words, 0, (size_t)nwords * sizeof(uint32_t));
    uint8_t* bytes = (uint8_t*)words;
    for (int64_t i = 0; i < total; ++i) {
        const uint8_t code = (uint8_t)(t[i] + 1);
        bytes[i >> 2] |= (uint8_t)(code << ((i & 3) << 1));
    }
    if (row_sums) {
        /* OXN/nsos/src/bitlinear.cpp:36-73 (compute_weight_row_sums) */
        for (int n = 0; n < N; ++n) {
            int32_t s = 0;
            for (int k = 0; k < K; ++k) s += t[(int64_t)n * K + k];
            row_sums[n] = s;
        }
    }
    if (!t_out) free(t);
    return weight_scale;
}

/* OXN/nsos/src/bitnet_adapter.cpp:590-606: decode {0,1,2,3} -> {-1,0,+1,0}. */
void tor_unpack_i8(const uint32_t* words, int N, int K, int8_t* t) {
    static const int8_t decode[4] = {-1, 0, 1, 0};
    const uint8_t* bytes = (const uint8_t*)words;
    const int64_t total = (int64_t)N * K;
    for (int64_t i = 0; i < total; ++i)
        t[i] = decode[(bytes[i >> 2] >> ((i & 3) << 1)) & 3];
}

/* ---- A7: optional input RMSNorm -----------------------------------------------
 * OXN/nsos/src/tensor.cpp:3476-3486 (Tensor::rmsnorm, CPU branch): sequential fp32
 * sum of squares, inv = 1/sqrt(sum/K + eps), x*inv. */
void tor_rmsnorm_rows(const float* x, int M, int K, float eps, float* out) {
    for (int i = 0; i < M; ++i) {
        const float* src = x + (int64_t)i * K;
        float* dst = out + (int64_t)i * K;
        float sum_sq = 0.0f;
        for (int j = 0; j < K; ++j) {
            const float v = src[j];
            sum_sq += v * v;
        }
        const float inv = 1.0f / sqrtf(sum_sq / (float)(K > 1 ? K : 1) + eps);
        for (int j = 0; j < K; ++j) dst[j] = src[j] * inv;
    }
}

/* q_max for an activation bit width.
 * OXN/nsos/src/bitlinear.cpp:250-254: 127 default, 1 for bits<=2, 2^(b-1)-1 else. */
float tor_qmax(int bits) {
    if (bits <= 2) return 1.0f;
    return powf(2.0f, (float)(bits - 1)) - 1.0f;
}

/* ---- A5: per-row absmax activation quantiser -------------------------------------
 * OXN/nsos/src/bitlinear.cpp:240-291 + OXN/nsos/src/bitlinear_quantize_avx2.cpp:65-103.
 * tie_mode 0 = the default x86-64 build: round-half-to-even for the 8-wide body
 * (_mm256_round_ps) and std::round (half away from zero) for the K%8 tail;
 * tie_mode 1 = the scalar build: std::round everywhere.
 * q is float-valued integers like the reference's x_q tensor; q_i8 (nullable) receives
 * the int8 the GEMM derives from it (re-round + clamp to [-127,127],
 * OXN/nsos/src/bitnet_adapter_avx2.cpp:94-126). */
void tor_quantize_rows(const float* x, int M, int K, int bits, int tie_mode,
                       float* q, int8_t* q_i8, float* act_scales) {
    const float q_max = tor_qmax(bits);
    const int body = tie_mode == 0 ? (K / 8) * 8 : 0;
    for (int i = 0; i < M; ++i) {
        const float* row = x + (int64_t)i * K;
        float max_val = 0.0f;
        for (int j = 0; j < K; ++j) {
            const float a = fabsf(row[j]);
            if (a > max_val) max_val = a;
        }
        const float denom = max_val + 1e-8f;
        const float scale = q_max / denom;
        act_scales[i] = denom / q_max;
        for (int j = 0; j < K; ++j) {
            const float v = row[j] * scale;
            const float r = j < body ? nearbyintf(v) : roundf(v);
            if (q) q[(int64_t)i * K + j] = r;
            if (q_i8) {
                float c = r;
                if (c < -127.0f) c = -127.0f;
                if (c > 127.0f) c = 127.0f;
                q_i8[(int64_t)i * K + j] = (int8_t)c;
            }
        }
    }
}

/* ---- A6: int8 x ternary GEMM with the two-scale epilogue -------------------------
 * OXN/nsos/src/bitnet_adapter_avx2.cpp:52-158 (default build) and
 * OXN/nsos/src/bitnet_adapter.cpp:109-151 (scalar): acc = sum_k q*t (int32, exact);
 * y = float(acc) * (act_scale * weight_scale); then *magnitude[n]; then +bias[n].
 * acc_out (nullable) receives the raw int32 accumulators. */
void tor_gemm_i8(const int8_t* q_i8, const int8_t* t, const float* act_scales,
                 float weight_scale, int M, int K, int N, const float* magnitude,
                 const float* bias, float* y, int32_t* acc_out) {
    for (int m = 0; m < M; ++m) {
        const float combined = act_scales[m] * weight_scale;
        const int8_t* qr = q_i8 + (int64_t)m * K;
        for (int n = 0; n < N; ++n) {
            const int8_t* tr = t + (int64_t)n * K;
            int32_t acc = 0;
            for (int k = 0; k < K; ++k) acc += (int32_t)qr[k] * (int32_t)tr[k];
            if (acc_out) acc_out[(int64_t)m * N + n] = acc;
            float v = (float)acc * combined;
            if (magnitude) v *= magnitude[n];
            if (bias) v += bias[n];
            y[(int64_t)m * N + n] = v;
        }
    }
}

/* ---- A7 wrapper: one packed BitLinear forward --------------------------------------
 * OXN/nsos/src/bitlinear.cpp:439-466,690-741 (BitLinear::forward, packed branch):
 * optional rmsnorm(1e-6) -> quantise -> int GEMM -> (magnitude, bias) -> fp32 [M,N].
 * In exact-linear mode the caller passes rms_input = 0 and magnitude = NULL
 * (OXN/nsos/include/bitlinear.h:99-108).  Debug outputs (nullable): q_out int8 [M,K],
 * scales_out fp32 [M], acc_out int32 [M,N]. */
void tor_linear_forward(const float* x, int M, int K, int N, const uint32_t* words,
                        float weight_scale, int rms_input, int bits, int tie_mode,
                        const float* magnitude, const float* bias, float* y,
                        int8_t* q_out, float* scales_out, int32_t* acc_out) {
    float* xn = NULL;
    const float* src = x;
    if (rms_input) {
        xn = (float*)malloc((size_t)M * K * sizeof(float));
        tor_rmsnorm_rows(x, M, K, 1e-6f, xn);
        src = xn;
    }
    int8_t* t = (int8_t*)malloc((size_t)N * K);
    tor_unpack_i8(words, N, K, t);
    int8_t* q = q_out ? q_out : (int8_t*)malloc((size_t)M * K);
    float* sc = scales_out ? scales_out : (float*)malloc((size_t)M * sizeof(float));
    tor_quantize_rows(src, M, K, bits, tie_mode, NULL, q, sc);
    tor_gemm_i8(q, t, sc, weight_scale, M, K, N, magnitude, bias, y, acc_out);
    if (!q_out) free(q);
    if (!scales_out) free(sc);
    free(t);
    free(xn);
}

/* Same as tor_linear_forward but with already-unpacked int8 ternary weights, so a timing
 * loop does not pay for the unpack on every call (the reference keeps the unpacked copy
 * resident too, OXN/nsos/src/bitlinear.cpp:186-188). */
void tor_linear_forward_i8(const float* x, int M, int K, int N, const int8_t* t,
                           float weight_scale, int rms_input, int bits, int tie_mode,
                           const float* magnitude, const float* bias, float* y) {
    float* xn = NULL;
    const float* src = x;
    if (rms_input) {
        xn = (float*)malloc((size_t)M * K * sizeof(float));
        tor_rmsnorm_rows(x, M, K, 1e-6f, xn);
        src = xn;
    }
    int8_t* q = (int8_t*)malloc((size_t)M * K);
    float* sc = (float*)malloc((size_t)M * sizeof(float));
    tor_quantize_rows(src, M, K, bits, tie_mode, NULL, q, sc);
    tor_gemm_i8(q, t, sc, weight_scale, M, K, N, magnitude, bias, y, NULL);
    free(q);
    free(sc);
    free(xn);
}

/* OXN/nsos/src/tensor.cpp:3209-3226 (Tensor::squared_relu): max(x,0)^2. */
void tor_squared_relu(const float* x, int64_t n, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i] > 0.0f ? x[i] : 0.0f;
        out[i] = v * v;
    }
}

/* ---- A9: router post-processing --------------------------------------------------
 * OXN/nsos/src/tensor.cpp:3402-3450 (softmax, max-subtracted, 1/max(sum,1e-8)) and
 * OXN/nsos/src/jamba.cpp:8268-8296 (keep the top_k largest, ties -> lower index,
 * renormalise by 1/max(sum_selected,1e-9), others 0).  logits [rows,E] -> weights. */
void tor_router_topk(const float* logits, int rows, int E, int top_k, float* weights) {
    for (int r = 0; r < rows; ++r) {
        const float* l = logits + (int64_t)r * E;
        float* w = weights + (int64_t)r * E;
        float mx = l[0];
        for (int e = 1; e < E; ++e) if (l[e] > mx) mx = l[e];
        float sum = 0.0f;
        for (int e = 0; e < E; ++e) { w[e] = expf(l[e] - mx); sum += w[e]; }
        const float inv = 1.0f / (sum > 1e-8f ? sum : 1e-8f);
        for (int e = 0; e < E; ++e) w[e] *= inv;
        if (top_k > 0 && top_k < E) {
            char keep[64] = {0};
            float selected = 0.0f;
            for (int rank = 0; rank < top_k; ++rank) {
                int best = -1;
                for (int e = 0; e < E; ++e)
                    if (!keep[e] && (best < 0 || w[e] > w[best])) best = e;
                keep[best] = 1;
                selected += w[best];
            }
            const float inv_sel = 1.0f / (selected > 1e-9f ? selected : 1e-9f);
            for (int e = 0; e < E; ++e) w[e] = keep[e] ? w[e] * inv_sel : 0.0f;
        }
    }
}

/* ---- A9: MoE expert FFN, CPU composition -------------------------------------------
 * OXN/nsos/src/jamba.cpp:3865-3972 (JambaBlock::forward_moe, CPU branch): for each
 * expert in index order, gather the rows routed to it (row order), up -> squared ReLU
 * -> down (both default-mode BitLinears: rmsnorm 1e-6 input, magnitude, bias), scale by
 * the routing weight, add into the output.  Rows are "routed" when their routing weight
 * is non-zero (the router leaves exactly top_k non-zeros per row).
 * up_words[e]: [H,D] packed; down_words[e]: [D,H] packed; magnitude / bias arrays may be
 * NULL (then no affine), else up_mag[e] has H entries, down_mag[e] D entries, ... */
void tor_moe_forward(const float* x, int rows, int D, int H, int E, const float* routing,
                     const uint32_t* const* up_words, const float* up_scale,
                     const float* const* up_mag, const float* const* up_bias,
                     const uint32_t* const* down_words, const float* down_scale,
                     const float* const* down_mag, const float* const* down_bias,
                     int rms_input, int bits, int tie_mode, float* out) {
    memset(out, 0, (size_t)rows * D * sizeof(float));
    int* sel = (int*)malloc((size_t)rows * sizeof(int));
    for (int e = 0; e < E; ++e) {
        int cnt = 0;
        for (int r = 0; r < rows; ++r)
            if (routing[(int64_t)r * E + e] != 0.0f) sel[cnt++] = r;
        if (!cnt) continue;
        float* xin = (float*)malloc((size_t)cnt * D * sizeof(float));
        float* hid = (float*)malloc((size_t)cnt * H * sizeof(float));
        float* yo = (float*)malloc((size_t)cnt * D * sizeof(float));
        for (int i = 0; i < cnt; ++i)
            memcpy(xin + (int64_t)i * D, x + (int64_t)sel[i] * D, (size_t)D * sizeof(float));
        tor_linear_forward(xin, cnt, D, H, up_words[e], up_scale[e], rms_input, bits, tie_mode,
                           up_mag ? up_mag[e] : NULL, up_bias ? up_bias[e] : NULL, hid,
                           NULL, NULL, NULL);
        tor_squared_relu(hid, (int64_t)cnt * H, hid);
        tor_linear_forward(hid, cnt, H, D, down_words[e], down_scale[e], rms_input, bits,
                           tie_mode, down_mag ? down_mag[e] : NULL,
                           down_bias ? down_bias[e] : NULL, yo, NULL, NULL, NULL);
        for (int i = 0; i < cnt; ++i) {
            const float wgt = routing[(int64_t)sel[i] * E + e];
            float* dst = out + (int64_t)sel[i] * D;
            for (int d = 0; d < D; ++d) dst[d] = dst[d] + yo[(int64_t)i * D + d] * wgt;
        }
        free(xin); free(hid); free(yo);
    }
    free(sel);
}

/* ---- F1: the norms either side of a linear in the decode step ---------------------
 * gate == NULL: block norm x.rmsnorm(eps).mul(weight) (OXN/nsos/src/jamba.cpp:3175-3179).
 * gate != NULL: Mamba-2 epilogue y.mul(z.silu()).rmsnorm(eps).mul(weight)
 * (OXN/nsos/src/mamba2.cpp:4011; the fused device form is
 * OXN/nsos/src/cuda/mamba_kernels.cu:3421-3441).  silu follows Tensor::silu's CPU branch
 * (OXN/nsos/src/tensor.cpp:3273-3280: the two-sided sigmoid), the norm follows tor_rmsnorm_rows;
 * every product is rounded on its own.  weight may be NULL (non-learnable norm). */
void tor_row_norm(const float* value, const float* gate, const float* weight, int rows, int dim,
                  float eps, float* out) {
    for (int r = 0; r < rows; ++r) {
        const float* v = value + (int64_t)r * dim;
        const float* z = gate ? gate + (int64_t)r * dim : 0;
        float* dst = out + (int64_t)r * dim;
        float sum_sq = 0.0f;
        for (int j = 0; j < dim; ++j) {
            float a = v[j];
            if (z) {
                const float g = z[j];
                const float sig = g >= 0.0f ? 1.0f / (1.0f + expf(-g)) : expf(g) / (1.0f + expf(g));
                a = a * (g * sig);
            }
            dst[j] = a;
            sum_sq += a * a;
        }
        const float inv = 1.0f / sqrtf(sum_sq / (float)(dim > 1 ? dim : 1) + eps);
        for (int j = 0; j < dim; ++j) {
            const float n = dst[j] * inv;
            dst[j] = weight ? n * weight[j] : n;
        }
    }
}

/* ---- F1: decode-step glue of the hybrid -----------------------------------------------
 * Streaming single-token forms, restated from the reference's host branches.  Every product and
 * sum is rounded on its own, in the reference's order (the file is compiled with contraction off,
 * like the reference objects it is pinned against). */

/* OXN/nsos/src/mamba2.cpp:727-739 (sigmoid_stable / silu_stable). */
static float tor_silu_stable(float x) {
    float sig;
    if (x >= 0.0f) {
        const float z = expf(-x);
        sig = 1.0f / (1.0f + z);
    } else {
        const float z = expf(x);
        sig = z / (1.0f + z);
    }
    return x * sig;
}

/* Causal depthwise conv step + SiLU over the concatenated [x | B | C] channels, then the ring shift.
 * OXN/nsos/src/mamba2.cpp:4062-4094 (Mamba2SSD::forward_faithful_step, host branch); the device form is
 * mamba2_faithful_conv_step_kernel, OXN/nsos/src/cuda/mamba_kernels.cu:3332-3359.
 * ring [R][K-1][conv_dim] (oldest tap first), conv_w [conv_dim][K], xBC [R][conv_dim]. */
void tor_mamba_conv_step(const float* xv, const float* Bv, const float* Cv, const float* conv_w,
                         const float* conv_b, float* ring, int R, int d_inner, int GS, int K, float* xBC) {
    const int conv_dim = d_inner + 2 * GS;
    const int taps = K - 1 > 0 ? K - 1 : 0;
    for (int r = 0; r < R; ++r) {
        float* rr = ring + (int64_t)r * taps * conv_dim;
        for (int c = 0; c < conv_dim; ++c) {
            const float current = c < d_inner ? xv[(int64_t)r * d_inner + c]
                                              : (c < d_inner + GS ? Bv[(int64_t)r * GS + c - d_inner]
                                                                  : Cv[(int64_t)r * GS + c - d_inner - GS]);
            float value = conv_b[c];
            for (int j = 0; j < K; ++j)
                value += conv_w[(int64_t)c * K + j] * (j < taps ? rr[(int64_t)j * conv_dim + c] : current);
            xBC[(int64_t)r * conv_dim + c] = tor_silu_stable(value);
            if (taps > 0) {
                for (int s = 0; s + 1 < taps; ++s) rr[(int64_t)s * conv_dim + c] = rr[(int64_t)(s + 1) * conv_dim + c];
                rr[(int64_t)(taps - 1) * conv_dim + c] = current;
            }
        }
    }
}

/* delta = softplus(dt), decay = exp(-delta * exp(A_log)) evaluated in double.
 * OXN/nsos/src/mamba2.cpp:443-473 (mamba_decay_terms; the gradient terms are not needed here). */
static void tor_decay_terms(float dt_raw, float a_log, float* delta_out, float* decay_out) {
    const float delta = dt_raw > 20.0f ? dt_raw : (dt_raw < -20.0f ? expf(dt_raw) : log1pf(expf(dt_raw)));
    *delta_out = delta;
    if (!isfinite(dt_raw) || !isfinite(a_log)) { *decay_out = NAN; return; }
    const double log_delta = dt_raw < -20.0f ? (double)dt_raw : log((double)delta);
    const double log_q = log_delta + (double)a_log;
    if (log_q > 50.0) { *decay_out = 0.0f; return; }
    *decay_out = (float)exp(-exp(log_q));
}

/* One SSD recurrence step: h = decay*h + delta*B*x ; y = D*x + sum_n h*C.
 * OXN/nsos/src/mamba2.cpp:4096-4118; device form mamba2_faithful_step_kernel,
 * OXN/nsos/src/cuda/mamba_kernels.cu:3376-3405.  xBC [R][d_inner + 2*G*N], dt [R][H],
 * state [R][d_inner][N], y [R][d_inner]. */
void tor_mamba_ssd_step(const float* xBC, const float* dt, const float* A_log, const float* D, float* state,
                        int R, int n_heads, int d_head, int N, int n_groups, float* y) {
    const int d_inner = n_heads * d_head, GS = n_groups * N, conv_dim = d_inner + 2 * GS;
    for (int r = 0; r < R; ++r) {
        const float* row = xBC + (int64_t)r * conv_dim;
        float* st = state + (int64_t)r * d_inner * N;
        for (int h = 0; h < n_heads; ++h) {
            const int group = (h * n_groups) / n_heads;
            float delta, decay;
            tor_decay_terms(dt[(int64_t)r * n_heads + h], A_log[h], &delta, &decay);
            for (int p = 0; p < d_head; ++p) {
                const int chan = h * d_head + p;
                const float input = row[chan];
                float out = D[h] * input;
                for (int n = 0; n < N; ++n) {
                    const int64_t si = (int64_t)chan * N + n;
                    const float Bvalue = row[d_inner + group * N + n];
                    const float Cvalue = row[d_inner + GS + group * N + n];
                    st[si] = decay * st[si] + delta * Bvalue * input;
                    out += st[si] * Cvalue;
                }
                y[(int64_t)r * d_inner + chan] = out;
            }
        }
    }
}

/* Single-token attention over the KV cache: RoPE on q and k at the row's position, append k/v, per-head
 * softmax(q.k * scale) over the window, weighted sum of v.
 * OXN/nsos/src/jamba.cpp:5140-5190 (apply_rope: halves i / i + head_dim/2), :6520-6542 (k | v split, append),
 * :6604-6638 (scores, softmax with 1/max(sum,1e-9), accumulation in token order); device form
 * gqa_cached_attention_decode, OXN/nsos/src/cuda/kernels.cu:2853-2990.
 * q [R][H*hd], kv [R][2*KV*hd] (k then v), caches [R][capacity][KV*hd], tokens[r] = entries already cached
 * (advanced here), cos/sin [positions][hd/2], out [R][H*hd]. */
void tor_attention_decode(const float* q, const float* kv, float* k_cache, float* v_cache, int capacity,
                          int* tokens, const float* cos_t, const float* sin_t, int R, int n_heads,
                          int n_kv_heads, int head_dim, int sliding_window, float* out) {
    const int kv_dim = n_kv_heads * head_dim, half = head_dim / 2, d_model = n_heads * head_dim;
    const int group = n_heads / n_kv_heads > 0 ? n_heads / n_kv_heads : 1;
    const float scale = 1.0f / sqrtf((float)head_dim);
    float* qr = (float*)malloc(sizeof(float) * d_model);
    float* scores = (float*)malloc(sizeof(float) * (capacity + 1));
    for (int r = 0; r < R; ++r) {
        const int pos = tokens[r];
        const float* c = cos_t + (int64_t)pos * half;
        const float* s = sin_t + (int64_t)pos * half;
        for (int h = 0; h < n_heads; ++h)
            for (int i = 0; i < half; ++i) {
                const float q0 = q[(int64_t)r * d_model + h * head_dim + i];
                const float q1 = q[(int64_t)r * d_model + h * head_dim + i + half];
                qr[h * head_dim + i] = q0 * c[i] - q1 * s[i];
                qr[h * head_dim + i + half] = q0 * s[i] + q1 * c[i];
            }
        float* kc = k_cache + ((int64_t)r * capacity + pos) * kv_dim;
        float* vc = v_cache + ((int64_t)r * capacity + pos) * kv_dim;
        for (int h = 0; h < n_kv_heads; ++h)
            for (int i = 0; i < half; ++i) {
                const float k0 = kv[(int64_t)r * 2 * kv_dim + h * head_dim + i];
                const float k1 = kv[(int64_t)r * 2 * kv_dim + h * head_dim + i + half];
                kc[h * head_dim + i] = k0 * c[i] - k1 * s[i];
                kc[h * head_dim + i + half] = k0 * s[i] + k1 * c[i];
            }
        memcpy(vc, kv + (int64_t)r * 2 * kv_dim + kv_dim, sizeof(float) * kv_dim);
        const int cached = pos + 1;
        tokens[r] = cached;
        const int first = cached - sliding_window > 0 ? cached - sliding_window : 0;
        for (int h = 0; h < n_heads; ++h) {
            int kvh = h / group;
            if (kvh > n_kv_heads - 1) kvh = n_kv_heads - 1;
            float max_s = -1e30f;
            for (int t = first; t < cached; ++t) {
                const float* key = k_cache + ((int64_t)r * capacity + t) * kv_dim + kvh * head_dim;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; ++d) dot += qr[h * head_dim + d] * key[d];
                scores[t] = dot * scale;
                if (scores[t] > max_s) max_s = scores[t];
            }
            float sum_exp = 0.0f;
            for (int t = first; t < cached; ++t) { scores[t] = expf(scores[t] - max_s); sum_exp += scores[t]; }
            const float inv_sum = 1.0f / (sum_exp > 1e-9f ? sum_exp : 1e-9f);
            for (int t = first; t < cached; ++t) scores[t] *= inv_sum;
            float* oh = out + (int64_t)r * d_model + h * head_dim;
            for (int d = 0; d < head_dim; ++d) oh[d] = 0.0f;
            for (int t = first; t < cached; ++t) {
                const float* val = v_cache + ((int64_t)r * capacity + t) * kv_dim + kvh * head_dim;
                for (int d = 0; d < head_dim; ++d) oh[d] += scores[t] * val[d];
            }
        }
    }
    free(qr);
    free(scores);
}

/* Multi-threaded wrapper for the CPU-baseline timing legs: rows are sharded over
 * `threads` OpenMP workers (the reference's GEMM itself is single-threaded,
 * OXN/nsos/src/bitnet_adapter_avx2.cpp has no OpenMP; sharding rows is the fair
 * multi-core figure).  Compiled only when OpenMP is on. */
#ifdef _OPENMP
#include <omp.h>
void tor_linear_forward_i8_mt(const float* x, int M, int K, int N, const int8_t* t,
                              float weight_scale, int rms_input, int bits, int tie_mode,
                              const float* magnitude, const float* bias, float* y,
                              int threads) {
    if (threads < 1) threads = 1;
    if (threads > M) threads = M;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int p = 0; p < threads; ++p) {
        const int lo = (int)((int64_t)M * p / threads);
        const int hi = (int)((int64_t)M * (p + 1) / threads);
        if (hi > lo)
            tor_linear_forward_i8(x + (int64_t)lo * K, hi - lo, K, N, t, weight_scale,
                                  rms_input, bits, tie_mode, magnitude, bias,
                                  y + (int64_t)lo * N);
    }
}
#endif
