// C-callable shim around the UNMODIFIED reference implementation (TEST INFRASTRUCTURE ONLY).
//
// oracle/Makefile compiles this file together with the reference's own sources, read in
// place from the reference checkout, into oracle/_ref/libnsos_ref.so.  Nothing here
// restates any arithmetic: every function drives nsos::BitLinear through its public
// interface (OXN/nsos/include/bitlinear.h:77-212) so that the C restatement in
// ternary_oracle.c and the CUDA kernels can be compared with what the reference itself
// computes, and so the bench can time the reference's CPU path.
#include "bitlinear.h"
#include "bitnet_adapter.h"
#include "nsos/sha256.h"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

using nsos::BitLinear;
using nsos::Device;
using nsos::Tensor;

namespace {

// Builds a layer in inference mode on the packed path with caller-supplied weights.
// exact_linear != 0 -> no input RMSNorm, no magnitude (bitlinear.h:99-108); otherwise the
// default mode (RMS_PERI input norm + magnitude [+ bias]).
std::unique_ptr<BitLinear> make_layer(const float* W, int N, int K, int exact_linear,
                                      const float* magnitude, const float* bias, int bits) {
    auto L = std::make_unique<BitLinear>(K, N, bias != nullptr, /*seed=*/1);
    std::memcpy(L->weight.data.data(), W, sizeof(float) * static_cast<size_t>(N) * K);
    L->weight.mark_updated();
    if (magnitude) std::memcpy(L->magnitude.data.data(), magnitude, sizeof(float) * N);
    if (bias) std::memcpy(L->bias.data.data(), bias, sizeof(float) * N);
    L->set_exact_linear_mode(exact_linear != 0);
    L->set_training_mode(false);
    L->precision_bits = bits;
    L->repack_weights();
    L->set_reference_path(false);
    return L;
}

void run_forward(BitLinear& L, const float* x, int M, float* y) {
    const int K = L.input_features();
    const int N = L.output_features();
    Tensor in({M, K}, Device::CPU);
    std::memcpy(in.data(), x, sizeof(float) * static_cast<size_t>(M) * K);
    Tensor out = L.forward(in);
    std::memcpy(y, out.data(), sizeof(float) * static_cast<size_t>(M) * N);
}

}  // namespace

extern "C" {

// Packs W [N,K] with BitLinear::repack_weights and returns the canonical words and scale
// through export_packed_state().  words must hold ceil(N*K/16) entries.  Returns the
// number of words written, or -1 on error.
long long ref_pack(const float* W, int N, int K, uint32_t* words, float* weight_scale) {
    try {
        auto L = make_layer(W, N, K, 1, nullptr, nullptr, 8);
        const nsos::BitLinearPackedState st = L->export_packed_state();
        std::memcpy(words, st.packed_weights.data(), st.packed_weights.size() * sizeof(uint32_t));
        *weight_scale = st.weight_scale;
        return static_cast<long long>(st.packed_weights.size());
    } catch (...) {
        return -1;
    }
}

// One BitLinear::forward on the packed CPU path.  Returns 0, or -1 on an exception.
int ref_linear_forward(const float* W, int N, int K, const float* x, int M, int exact_linear,
                       const float* magnitude, const float* bias, int bits, float* y) {
    try {
        auto L = make_layer(W, N, K, exact_linear, magnitude, bias, bits);
        run_forward(*L, x, M, y);
        return 0;
    } catch (...) {
        return -1;
    }
}

// Handle API so a timing loop pays for packing once.
void* ref_layer_create(const float* W, int N, int K, int exact_linear, const float* magnitude,
                       const float* bias, int bits) {
    try {
        return make_layer(W, N, K, exact_linear, magnitude, bias, bits).release();
    } catch (...) {
        return nullptr;
    }
}

int ref_layer_forward(void* handle, const float* x, int M, float* y) {
    try {
        run_forward(*static_cast<BitLinear*>(handle), x, M, y);
        return 0;
    } catch (...) {
        return -1;
    }
}

// Rows sharded over `threads` OpenMP workers, each calling BitLinear::forward on its own
// copy of the layer handle list (one handle per worker: forward() mutates saved state).
int ref_layer_forward_mt(void* const* handles, int threads, const float* x, int M, float* y) {
    if (threads < 1) return -1;
    auto* first = static_cast<BitLinear*>(handles[0]);
    const int K = first->input_features();
    const int N = first->output_features();
    if (threads > M) threads = M;
    int failed = 0;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (int p = 0; p < threads; ++p) {
        const int lo = static_cast<int>(static_cast<long long>(M) * p / threads);
        const int hi = static_cast<int>(static_cast<long long>(M) * (p + 1) / threads);
        if (hi <= lo) continue;
        try {
            run_forward(*static_cast<BitLinear*>(handles[p]), x + static_cast<size_t>(lo) * K,
                        hi - lo, y + static_cast<size_t>(lo) * N);
        } catch (...) {
#pragma omp atomic write
            failed = 1;
        }
    }
    return failed ? -1 : 0;
}

// `count` independent layers (e.g. column shards of one wide layer, one per host thread) each run
// BitLinear::forward on the same x [M,K]; y_out[p] receives layer p's [M, N_p] result.
int ref_layers_forward_parallel(void* const* handles, int count, const float* x, int M, float* const* y_out) {
    int failed = 0;
#pragma omp parallel for num_threads(count) schedule(static)
    for (int p = 0; p < count; ++p) {
        try {
            run_forward(*static_cast<BitLinear*>(handles[p]), x, M, y_out[p]);
        } catch (...) {
#pragma omp atomic write
            failed = 1;
        }
    }
    return failed ? -1 : 0;
}

void ref_layer_destroy(void* handle) { delete static_cast<BitLinear*>(handle); }

// MoE expert FFN built from public pieces exactly as the CPU branch of
// JambaBlock::forward_moe composes them (OXN/nsos/src/jamba.cpp:3865-3972): per expert in
// index order, gather routed rows, up -> Tensor::squared_relu -> down, scale by the routing
// weight, accumulate.  up_w: E x [H,D] fp32 concatenated; down_w: E x [D,H] fp32
// concatenated.  Experts are default-mode layers (RMS input norm, magnitude 1, no bias).
int ref_moe_forward(const float* x, int rows, int D, int H, int E, const float* routing,
                    const float* up_w, const float* down_w, int bits, float* out) {
    try {
        std::fill_n(out, static_cast<size_t>(rows) * D, 0.0f);
        for (int e = 0; e < E; ++e) {
            std::vector<int> sel;
            for (int r = 0; r < rows; ++r)
                if (routing[static_cast<size_t>(r) * E + e] != 0.0f) sel.push_back(r);
            if (sel.empty()) continue;
            auto up = make_layer(up_w + static_cast<size_t>(e) * H * D, H, D, 0, nullptr, nullptr, bits);
            auto down = make_layer(down_w + static_cast<size_t>(e) * D * H, D, H, 0, nullptr, nullptr, bits);
            const int cnt = static_cast<int>(sel.size());
            Tensor xin({cnt, D}, Device::CPU);
            for (int i = 0; i < cnt; ++i)
                std::memcpy(xin.data() + static_cast<size_t>(i) * D,
                            x + static_cast<size_t>(sel[i]) * D, sizeof(float) * D);
            Tensor hidden = up->forward(xin).squared_relu();
            Tensor yo = down->forward(hidden);
            Tensor scale({cnt, 1}, Device::CPU);
            for (int i = 0; i < cnt; ++i)
                scale.data()[i] = routing[static_cast<size_t>(sel[i]) * E + e];
            Tensor scaled = yo.mul(scale);
            Tensor scatter = Tensor::zeros({rows, D}, Device::CPU);
            for (int i = 0; i < cnt; ++i)
                std::memcpy(scatter.data() + static_cast<size_t>(sel[i]) * D,
                            scaled.data() + static_cast<size_t>(i) * D, sizeof(float) * D);
            Tensor acc({rows, D}, Device::CPU);
            std::memcpy(acc.data(), out, sizeof(float) * static_cast<size_t>(rows) * D);
            Tensor sum = acc.add(scatter);
            std::memcpy(out, sum.data(), sizeof(float) * static_cast<size_t>(rows) * D);
        }
        return 0;
    } catch (...) {
        return -1;
    }
}

// The reference's own SHA-256 (integrity::sha256_hex, include/nsos/sha256.h:12): pins the digest of the
// edge-pack trailer.  out must hold 65 bytes.
void ref_sha256_hex(const void* data, size_t size, char* out) {
    const std::string hex = nsos::integrity::sha256_hex(data, size);
    std::memcpy(out, hex.c_str(), hex.size() + 1);
}

// The decode glue either side of a linear, composed from the reference's own Tensor ops exactly as its host
// branches compose them.  gate == NULL: block norm, x.rmsnorm(eps).mul(weight) (OXN/nsos/src/jamba.cpp:3175-3179;
// weight may be NULL for the non-learnable norm).  gate != NULL: the Mamba-2 epilogue
// y.mul(z.silu()).rmsnorm(eps).mul(weight) (OXN/nsos/src/mamba2.cpp:4011).  Returns 0, or -1 on error.
int ref_row_norm(const float* value, const float* gate, const float* weight, int rows, int dim, float eps,
                 float* out) {
    try {
        const size_t n = static_cast<size_t>(rows) * dim;
        Tensor v({rows, dim}, Device::CPU);
        std::memcpy(v.data(), value, sizeof(float) * n);
        if (gate) {
            Tensor z({rows, dim}, Device::CPU);
            std::memcpy(z.data(), gate, sizeof(float) * n);
            v = v.mul(z.silu());
        }
        Tensor normed = v.rmsnorm(eps);
        if (weight) {
            Tensor w({dim}, Device::CPU);
            std::memcpy(w.data(), weight, sizeof(float) * dim);
            normed = normed.mul(w);
        }
        std::memcpy(out, normed.data(), sizeof(float) * n);
        return 0;
    } catch (...) {
        return -1;
    }
}

}  // extern "C"
