// C-callable shim around the UNMODIFIED reference MODEL code (TEST INFRASTRUCTURE ONLY).
//
// oracle/Makefile compiles this file with every translation unit of the reference's core library, read in
// place from the reference checkout, into oracle/_ref/libnsos_model_ref.so.  Nothing here restates any
// arithmetic.  The shim builds an nsos::JambaModel from a ModelConfig, re-draws every BitLinear weight from
// N(0, 0.02) with a seeded std::mt19937, puts every projection on the packed ternary CPU path, and then
//   - runs streaming single-token steps through the model's public API (forward_ids_last),
//   - runs the same step block by block (embedding -> blocks -> final norm -> head) to hand out the hidden
//     state after every block,
//   - hands out every parameter the decode step needs (packed words, scales, norm weights, conv taps, ...)
//     through a callback, and writes the model's own edge-linear pack,
//   - runs MoERouter::forward.
// Private members are read (never written, except the weights the public API also exposes) by compiling this
// one file with the access keywords neutralised; the reference's own objects are compiled normally.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <random>
#include <string>
#include <vector>
#include <map>
#include <set>
#include <unordered_map>
#include <unordered_set>
#include <mutex>
#include <atomic>
#include <thread>
#include <functional>
#include <fstream>
#include <sstream>
#include <iostream>
#include <array>
#include <tuple>
#include <optional>
#include <variant>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <queue>
#include <list>
#include <numeric>
#include <limits>
#include <stdexcept>
#include <filesystem>
#include <future>
#include <shared_mutex>
#include <typeindex>
#include <any>
#include <bitset>
#include <complex>
#include <iomanip>
#include <regex>
#include <cassert>
#include <cstdio>
#include <cstdlib>
#include <immintrin.h>

#define private public
#define protected public
#include "jamba.h"
#include "mamba2.h"
#include "embedding.h"
#include "bitlinear.h"
#undef private
#undef protected

using namespace nsos;

namespace {

struct Model {
    std::unique_ptr<JambaModel> m;
};

typedef void (*emit_fn)(const char* name, int dtype, const void* data, long long count, void* user);
enum { F32 = 0, U32 = 1, I32 = 2 };

void emit_f32(emit_fn cb, void* user, const std::string& name, const Tensor& t) {
    Tensor h = t;
    cb(name.c_str(), F32, h.data(), static_cast<long long>(h.size), user);
}

void emit_ints(emit_fn cb, void* user, const std::string& name, std::vector<int32_t> v) {
    cb(name.c_str(), I32, v.data(), static_cast<long long>(v.size()), user);
}

// One BitLinear: the canonical packed state (the reference's own export) plus its mode flags.
void emit_linear(emit_fn cb, void* user, const std::string& name, BitLinear& L) {
    const BitLinearPackedState st = L.export_packed_state();
    cb((name + ".words").c_str(), U32, st.packed_weights.data(), static_cast<long long>(st.packed_weights.size()), user);
    float scale = st.weight_scale;
    cb((name + ".scale").c_str(), F32, &scale, 1, user);
    cb((name + ".magnitude").c_str(), F32, st.magnitude.data(), static_cast<long long>(st.magnitude.size()), user);
    if (st.use_bias) cb((name + ".bias").c_str(), F32, st.bias.data(), static_cast<long long>(st.bias.size()), user);
    // [in, out, use_bias, rms_input (norm strategy != NONE), magnitude applied, activation bits]
    const bool exact = L.exact_linear_mode();
    emit_ints(cb, user, name + ".meta",
              {st.in_features, st.out_features, st.use_bias ? 1 : 0, exact ? 0 : 1, exact ? 0 : 1, L.precision_bits});
}

void redraw(BitLinear& L, std::mt19937& rng) {
    std::normal_distribution<float> dist(0.0f, 0.02f);
    float* w = L.weight.data.data();
    for (int64_t i = 0; i < L.weight.data.size; ++i) w[i] = dist(rng);
    L.weight.mark_updated();
}

}  // namespace

extern "C" {

// cfg: [num_layers, d_model, vocab, n_heads, n_kv_heads, d_state, expand, conv_kernel, head_dim, n_groups,
//       attention_period, attention_slot].  Returns a handle or NULL.
void* refm_create(const int* cfg, unsigned seed) {
    try {
        ModelConfig c;
        c.num_layers = cfg[0]; c.d_model = cfg[1]; c.vocab_size = cfg[2]; c.n_heads = cfg[3]; c.n_kv_heads = cfg[4];
        c.mamba_d_state = cfg[5]; c.mamba_expand = cfg[6]; c.mamba_conv_kernel = cfg[7]; c.mamba_head_dim = cfg[8];
        c.mamba_n_groups = cfg[9]; c.attention_period = cfg[10]; c.attention_slot = cfg[11];
        c.hybrid_composition = HybridComposition::ParallelGated;
        c.use_moe = false; c.use_ttt = false; c.mamba2_faithful = true;
        auto model = std::make_unique<JambaModel>(c, Device::CPU);
        std::mt19937 rng(seed);
        // every projection ternary: weights N(0, 0.02), no layer kept in fp32, packed CPU path
        for (BitLinear* L : model->collect_bitlinear_layers()) {
            redraw(*L, rng);
            L->set_quantization_sensitive(false);
        }
        // the norms and gates start as ones / small constants: perturb them so a wrong pairing would show
        std::uniform_real_distribution<float> jitter(0.5f, 1.5f);
        for (auto& blk : model->layers) {
            for (Parameter* p : {&blk->core_norm_weight_, &blk->attention_norm_weight_, &blk->ff_norm_weight_,
                                 &blk->mamba_gate_, &blk->attention_gate_, &blk->ffn_gate_}) {
                float* d = p->data.size > 0 ? p->data.data() : nullptr;
                for (int64_t i = 0; d && i < p->data.size; ++i) d[i] *= jitter(rng);
            }
            if (blk->mamba_layer) {
                // the constructor draws these from a process-wide generator: draw them again from the seeded
                // one, over the constructor's own ranges (OXN/nsos/src/mamba2.cpp:560-563,616-626,676-686)
                Mamba2SSD& mm = *blk->mamba_layer;
                const float bound = 1.0f / std::sqrt(static_cast<float>(std::max(mm.conv_kernel_, 1)));
                std::uniform_real_distribution<float> conv(-bound, bound), a(1.0f, 16.0f),
                    logdt(std::log(1e-3f), std::log(1e-1f));
                for (int64_t i = 0; i < mm.conv_weight_.data.size; ++i) mm.conv_weight_.data.data()[i] = conv(rng);
                for (int64_t i = 0; i < mm.conv_bias_.data.size; ++i) mm.conv_bias_.data.data()[i] = conv(rng);
                for (int64_t i = 0; i < mm.A.data.size; ++i) mm.A.data.data()[i] = std::log(a(rng));
                for (int64_t i = 0; i < mm.dt_proj_->bias.data.size; ++i) {
                    const float dt_value = std::max(std::exp(logdt(rng)), 1e-4f);
                    mm.dt_proj_->bias.data.data()[i] = dt_value + std::log(-std::expm1(-dt_value));
                }
                float* d = blk->mamba_layer->norm_weight_.data.data();
                for (int64_t i = 0; i < blk->mamba_layer->norm_weight_.data.size; ++i) d[i] *= jitter(rng);
                float* dd = blk->mamba_layer->D.data.data();
                for (int64_t i = 0; i < blk->mamba_layer->D.data.size; ++i) dd[i] *= jitter(rng);
            }
        }
        {
            float* d = model->final_norm_weight_.data.data();
            for (int64_t i = 0; i < model->final_norm_weight_.data.size; ++i) d[i] *= jitter(rng);
        }
        model->set_training_mode(false);
        model->set_reference_path(false);
        for (BitLinear* L : model->collect_bitlinear_layers()) {
            L->set_training_mode(false);
            L->repack_weights();
            L->set_reference_path(false);
        }
        model->set_streaming_inference(true);
        model->reset_session();
        auto* h = new Model{std::move(model)};
        return h;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refm_create: %s\n", e.what());
        return nullptr;
    } catch (...) {
        return nullptr;
    }
}

void refm_destroy(void* handle) { delete static_cast<Model*>(handle); }

int refm_reset(void* handle) {
    try {
        static_cast<Model*>(handle)->m->reset_session();
        static_cast<Model*>(handle)->m->set_streaming_inference(true);
        return 0;
    } catch (...) { return -1; }
}

// One streaming decode step through the public API; logits must hold vocab floats.
int refm_step(void* handle, int token, float* logits) {
    try {
        JambaModel& m = *static_cast<Model*>(handle)->m;
        Tensor out = m.forward_ids_last({token});
        std::memcpy(logits, out.data(), sizeof(float) * static_cast<size_t>(out.size));
        return static_cast<int>(out.size);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refm_step: %s\n", e.what());
        return -1;
    }
}

// The same step taken block by block with the model's own objects: hidden [layers + 1, d_model] receives the
// embedding row and the residual stream after every block; logits as above.
int refm_step_trace(void* handle, int token, float* hidden, float* logits) {
    try {
        JambaModel& m = *static_cast<Model*>(handle)->m;
        const int D = m.model_config().d_model;
        Tensor h = m.embedding->forward(std::vector<int>{token});
        std::memcpy(hidden, h.data(), sizeof(float) * D);
        int i = 1;
        for (auto& layer : m.layers) {
            h = layer->forward(h, nullptr);
            std::memcpy(hidden + static_cast<size_t>(i++) * D, h.data(), sizeof(float) * D);
        }
        Tensor normed = h.rmsnorm(1e-5f).mul(m.final_norm_weight_.data);
        Tensor out = m.value_head->forward(normed);
        std::memcpy(logits, out.data(), sizeof(float) * static_cast<size_t>(out.size));
        return static_cast<int>(out.size);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refm_step_trace: %s\n", e.what());
        return -1;
    }
}

// Hands every parameter of the decode step to `cb` (name, dtype 0 f32 / 1 u32 / 2 i32, data, count).
int refm_export(void* handle, emit_fn cb, void* user) {
    try {
        JambaModel& m = *static_cast<Model*>(handle)->m;
        const ModelConfig& c = m.model_config();
        emit_ints(cb, user, "config", {c.num_layers, c.d_model, c.vocab_size, c.n_heads, c.n_kv_heads, c.mamba_d_state,
                                       c.mamba_expand, c.mamba_conv_kernel, c.mamba_head_dim, c.mamba_n_groups,
                                       c.attention_period, c.attention_slot});
        emit_f32(cb, user, "embedding", m.embedding->weight.data);
        emit_f32(cb, user, "final_norm", m.final_norm_weight_.data);
        emit_linear(cb, user, "head", *m.value_head);
        int li = 0;
        for (auto& blk : m.layers) {
            const std::string p = "L" + std::to_string(li++) + ".";
            emit_ints(cb, user, p + "kind", {blk->hybrid_parallel_ ? 1 : 0, blk->faithful_mamba_core_only_ ? 1 : 0,
                                             blk->learnable_core_norm_ ? 1 : 0});
            float eps = blk->core_norm_eps_;
            cb((p + "core_norm_eps").c_str(), F32, &eps, 1, user);
            if (blk->learnable_core_norm_) emit_f32(cb, user, p + "core_norm", blk->core_norm_weight_.data);
            Mamba2SSD& mm = *blk->mamba_layer;
            emit_ints(cb, user, p + "mamba.dims", {mm.d_inner, mm.n_heads, mm.d_head, mm.n_groups, mm.d_state,
                                                   mm.conv_dim, mm.conv_kernel_});
            float meps = mm.config_.rms_norm_eps;
            cb((p + "mamba.norm_eps").c_str(), F32, &meps, 1, user);
            emit_linear(cb, user, p + "mamba.x", *mm.x_proj_);
            emit_linear(cb, user, p + "mamba.z", *mm.z_proj_);
            emit_linear(cb, user, p + "mamba.B", *mm.B_proj_);
            emit_linear(cb, user, p + "mamba.C", *mm.C_proj_);
            emit_linear(cb, user, p + "mamba.dt", *mm.dt_proj_);
            emit_linear(cb, user, p + "mamba.out", mm.out_proj);
            emit_f32(cb, user, p + "mamba.A_log", mm.A.data);
            emit_f32(cb, user, p + "mamba.D", mm.D.data);
            emit_f32(cb, user, p + "mamba.conv_w", mm.conv_weight_.data);
            emit_f32(cb, user, p + "mamba.conv_b", mm.conv_bias_.data);
            emit_f32(cb, user, p + "mamba.norm_w", mm.norm_weight_.data);
            if (blk->hybrid_parallel_) {
                Attention& a = *blk->attn_layer;
                emit_f32(cb, user, p + "attn_norm", blk->attention_norm_weight_.data);
                emit_f32(cb, user, p + "ff_norm", blk->ff_norm_weight_.data);
                emit_f32(cb, user, p + "mamba_gate", blk->mamba_gate_.data);
                emit_f32(cb, user, p + "attn_gate", blk->attention_gate_.data);
                emit_f32(cb, user, p + "ffn_gate", blk->ffn_gate_.data);
                emit_ints(cb, user, p + "attn.dims", {a.n_heads, a.n_kv_heads, a.head_dim, a.kv_group_size,
                                                      a.sliding_window_, a.max_seq_len});
                a.ensure_freqs_capacity(1024);
                cb((p + "attn.cos").c_str(), F32, a.cos_cached.data(), static_cast<long long>(a.cos_cached.size()), user);
                cb((p + "attn.sin").c_str(), F32, a.sin_cached.data(), static_cast<long long>(a.sin_cached.size()), user);
                emit_linear(cb, user, p + "attn.q", *a.q_down_proj);
                emit_linear(cb, user, p + "attn.kv", *a.kv_down_proj);
                emit_linear(cb, user, p + "attn.out", *a.out_proj);
                emit_linear(cb, user, p + "ffn.up", *blk->ffn_gate_up);
                emit_linear(cb, user, p + "ffn.down", *blk->ffn_down);
            }
        }
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refm_export: %s\n", e.what());
        return -1;
    }
}

// The model's own edge-linear pack (JambaModel::save_edge_linear_pack).
int refm_save_edge_pack(void* handle, const char* path) {
    try {
        static_cast<Model*>(handle)->m->save_edge_linear_pack(path);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refm_save_edge_pack: %s\n", e.what());
        return -1;
    }
}

// MoERouter::forward on x [rows, D] with the gate's fp32 weight [E, D] (the router keeps its gate on the
// float path): logits and routing weights, both [rows, E].
int refm_router(const float* x, int rows, int D, int E, int top_k, const float* gate_w, float* logits, float* weights) {
    try {
        MoERouter router(D, E, top_k);
        std::memcpy(router.gate->weight.data.data(), gate_w, sizeof(float) * static_cast<size_t>(E) * D);
        router.gate->weight.mark_updated();
        Tensor in({rows, D}, Device::CPU);
        std::memcpy(in.data(), x, sizeof(float) * static_cast<size_t>(rows) * D);
        auto [lg, w] = router.forward(in);
        std::memcpy(logits, lg.data(), sizeof(float) * static_cast<size_t>(rows) * E);
        std::memcpy(weights, w.data(), sizeof(float) * static_cast<size_t>(rows) * E);
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refm_router: %s\n", e.what());
        return -1;
    }
}

}  // extern "C"
