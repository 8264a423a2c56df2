// Offline packer (host): fp32 weights -> absmean ternary {-1,0,+1} -> canonical 2-bit words plus
// one fp32 scale per matrix; the inverse decode; and the import-time validation of a packed state.
// The canonical words are also the device layout of the GEMV kernels: rows are contiguous and,
// for K % 64 == 0, start on 16-byte boundaries, so a run of rows is one 128-bit-coalesced stream.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <initializer_list>

#include "../../include/ternary_b200.h"

extern "C" {

int64_t tbl_packed_words(int N, int K) {
    if (N <= 0 || K <= 0) return 0;
    const int64_t bytes = (static_cast<int64_t>(N) * K + 3) / 4;
    return (bytes + 3) / 4;
}

int tbl_pack_weights(const float* w_host, int N, int K, uint32_t* words_host, float* weight_scale) {
    if (!w_host || !words_host || !weight_scale || N <= 0 || K <= 0) return TBL_ERR_INVALID_ARG;
    const int64_t total = static_cast<int64_t>(N) * K;
    // sequential double-precision sum: the order is part of the numeric contract
    double sum = 0.0;
    for (int64_t i = 0; i < total; ++i) sum += std::fabs(static_cast<double>(w_host[i]));
    const float absmean = static_cast<float>(sum / static_cast<double>(total));
    const float scale = absmean + 1e-8f;
    *weight_scale = scale;
    // the ternary rule divides by (scale + 1e-8f): the epsilon really is applied twice
    volatile float denom_v = scale + 1e-8f;
    const float denom = denom_v;
    const int64_t n_words = tbl_packed_words(N, K);
    std::memset(words_host, 0, static_cast<size_t>(n_words) * sizeof(uint32_t));
    for (int64_t i = 0; i < total; ++i) {
        const float v = w_host[i] / denom;
        const uint32_t code = v > 0.5f ? 2u : (v < -0.5f ? 0u : 1u);
        words_host[i >> 4] |= code << ((i & 15) << 1);
    }
    return TBL_OK;
}

int tbl_unpack_weights_i8(const uint32_t* words_host, int N, int K, int8_t* t_host) {
    if (!words_host || !t_host || N <= 0 || K <= 0) return TBL_ERR_INVALID_ARG;
    static const int8_t decode[4] = {-1, 0, 1, 0};
    const int64_t total = static_cast<int64_t>(N) * K;
    for (int64_t i = 0; i < total; ++i)
        t_host[i] = decode[(words_host[i >> 4] >> ((i & 15) << 1)) & 3u];
    return TBL_OK;
}

int tbl_validate_packed(const uint32_t* words_host, int64_t n_words, int N, int K, float weight_scale,
                        const float* magnitude_host, const float* bias_host) {
    if (!words_host || N <= 0 || K <= 0) return TBL_ERR_INVALID_ARG;
    const int64_t total = static_cast<int64_t>(N) * K;
    if (n_words != (total + 15) / 16) return TBL_ERR_SHAPE;
    if (!std::isfinite(weight_scale) || weight_scale <= 0.0f) return TBL_ERR_SCALE;
    for (int64_t i = 0; i < total; ++i)
        if (((words_host[i >> 4] >> ((i & 15) << 1)) & 3u) == 3u) return TBL_ERR_CODE;
    for (const float* v : {magnitude_host, bias_host}) {
        if (!v) continue;
        for (int n = 0; n < N; ++n)
            if (!std::isfinite(v[n])) return TBL_ERR_INVALID_ARG;
    }
    return TBL_OK;
}

}  // extern "C"
