// Compiled as C++17 against include/ternary_b200.hpp: the shim's status -> exception mapping and the
// host packer, without touching a GPU (the device entry point is only reached with arguments that its
// validation rejects before any CUDA call).
#include <cmath>
#include <cstdio>
#include <vector>

#include "ternary_b200.hpp"

int main() {
    namespace tb = ternary_b200;
    const int N = 7, K = 48;
    std::vector<float> w(N * K);
    for (int i = 0; i < N * K; ++i) w[i] = 0.03f * std::cos(0.61f * static_cast<float>(i + 3));
    std::vector<std::uint32_t> words(static_cast<std::size_t>(tbl_packed_words(N, K)));
    const float scale = tb::pack_weights(w.data(), N, K, words.data());
    if (!(scale > 0.0f)) return 1;
    tb::validate_packed(words.data(), static_cast<long long>(words.size()), N, K, scale);

    int caught = 0;
    try { tb::validate_packed(words.data(), static_cast<long long>(words.size()), N, K, -1.0f); }
    catch (const std::invalid_argument&) { ++caught; }                       // scale must be positive
    words[0] |= 3u;
    try { tb::validate_packed(words.data(), static_cast<long long>(words.size()), N, K, scale); }
    catch (const std::runtime_error&) { ++caught; }                          // reserved 2-bit code
    tb::DeviceWeights dw;                                                     // no device pointers at all
    dw.weight_scale = scale; dw.out_features = N; dw.in_features = K;
    try { tb::bitnet_gemm_158bit_gpu(nullptr, dw, 1, 8, nullptr, nullptr, nullptr, nullptr, 0, nullptr); }
    catch (const std::invalid_argument&) { ++caught; }
    dw.in_features = 8454672;                                                 // K > INT_MAX / 254, K % 16 == 0
    float dummy = 0.0f;
    try {
        tb::bitnet_gemm_158bit_gpu(&dummy, dw, 1, 8, nullptr, nullptr, &dummy, &dummy, 1u << 30, nullptr);
    } catch (const std::overflow_error&) { ++caught; }
    catch (const std::exception&) { caught += 100; }
    try { tb::mamba_gated_rmsnorm(&dummy, &dummy, &dummy, &dummy, 0, 64, 1e-5f, nullptr); }   // rows < 1
    catch (const std::invalid_argument&) { ++caught; }
    try { tb::rmsnorm_weight(&dummy, nullptr, &dummy, 4, 64, 0.0f, nullptr); }               // eps must be > 0
    catch (const std::invalid_argument&) { ++caught; }
    if (caught != 6) { std::printf("caught %d\n", caught); return 2; }
    if (tb::workspace_bytes(4, 1024, 8) < 2u * 4u * 1024u) return 3;
    std::printf("shim ok\n");
    return 0;
}
