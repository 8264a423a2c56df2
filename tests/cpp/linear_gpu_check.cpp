// A C++17 host, as the NSOS runtime is, drives a layer through ternary_b200::TernaryLinear on a GPU and compares
// with reference outputs handed in as raw files (written by the pytest that builds this program):
//   argv[1]/meta.txt  "N K M exact"      w.bin fp32 [N,K]   x.bin fp32 [M,K]   y.bin fp32 [M,N] (expected)
//   magnitude.bin / bias.bin fp32 [N] when not exact
// Checks: import -> forward is bit-identical to the expected output (reference-order input norm in default mode);
// export returns what was imported; a rejected import (reserved code) throws and leaves the layer serving the old
// weights; the grouped view describes the same buffers.
#include <cuda_runtime_api.h>

#include <cstdio>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "ternary_b200.hpp"

namespace tb = ternary_b200;

template <typename T>
static std::vector<T> read_all(const std::string& path, size_t count) {
    std::vector<T> v(count);
    std::ifstream f(path, std::ios::binary);
    if (!f.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(count * sizeof(T)))) {
        std::cerr << "cannot read " << path << "\n";
        std::exit(2);
    }
    return v;
}

#define CHECK(cond) do { if (!(cond)) { std::cerr << "FAILED: " #cond " (line " << __LINE__ << ")\n"; return 1; } } while (0)

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const std::string dir = argv[1];
    int N = 0, K = 0, M = 0, exact = 0;
    { std::ifstream meta(dir + "/meta.txt"); meta >> N >> K >> M >> exact; }
    CHECK(N > 0 && K > 0 && M > 0);
    const auto w = read_all<float>(dir + "/w.bin", static_cast<size_t>(N) * K);
    const auto x = read_all<float>(dir + "/x.bin", static_cast<size_t>(M) * K);
    const auto want = read_all<float>(dir + "/y.bin", static_cast<size_t>(M) * N);

    int live_allocations = 0;
    tb::DeviceMemory mem;
    mem.allocate = [&](std::size_t bytes) { void* p = nullptr; if (cudaMalloc(&p, bytes) != cudaSuccess) return static_cast<void*>(nullptr); ++live_allocations; return p; };
    mem.release = [&](void* p) { cudaFree(p); --live_allocations; };
    mem.upload = [](void* dst, const void* src, std::size_t bytes, void* stream) {
        cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
    };
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream) == cudaSuccess);

    tb::PackedState st;
    st.in_features = K; st.out_features = N; st.use_bias = !exact;
    st.packed_weights.resize((static_cast<size_t>(N) * K + 15) / 16);
    st.weight_scale = tb::pack_weights(w.data(), N, K, st.packed_weights.data());
    st.magnitude = exact ? std::vector<float>(N, 1.0f) : read_all<float>(dir + "/magnitude.bin", N);
    if (!exact) st.bias = read_all<float>(dir + "/bias.bin", N);
    st.flat_alpha.assign(K, 1.0f);
    st.flat_beta.assign(K, 0.0f);
    {
        tb::TernaryLinear layer(K, N, !exact, mem);
        layer.set_exact_linear_mode(exact != 0);
        // the retained-weights cross-check accepts the weights the state was packed from ...
        layer.commit_prepared_packed_state(layer.prepare_packed_state(st, stream, true, w.data()));
        // ... and refuses others
        std::vector<float> other = w;
        other[0] = -other[0] + 1.0f;
        bool threw = false;
        try { layer.prepare_packed_state(st, stream, true, other.data()); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw);

        float *dx = nullptr, *dy = nullptr;
        void* scratch = nullptr;
        const size_t ws = layer.workspace_bytes(M);
        CHECK(cudaMalloc(reinterpret_cast<void**>(&dx), x.size() * 4) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&dy), want.size() * 4) == cudaSuccess &&
              cudaMalloc(&scratch, ws ? ws : 16) == cudaSuccess);
        cudaMemcpyAsync(dx, x.data(), x.size() * 4, cudaMemcpyHostToDevice, stream);
        std::vector<float> got(want.size());
        auto run = [&]() {
            layer.forward(dx, M, dy, scratch, ws, stream, TBL_RMS_REFERENCE_ORDER);
            cudaMemcpyAsync(got.data(), dy, got.size() * 4, cudaMemcpyDeviceToHost, stream);
            tb::check_device(stream);
        };
        run();
        CHECK(std::memcmp(got.data(), want.data(), got.size() * 4) == 0);

        const tb::PackedState back = layer.export_packed_state();
        CHECK(back.packed_weights == st.packed_weights && back.weight_scale == st.weight_scale && back.magnitude == st.magnitude &&
              back.bias == st.bias);

        // a state with a reserved code is refused and nothing changes
        tb::PackedState bad = st;
        bad.packed_weights[bad.packed_weights.size() / 2] |= 0x3u;
        const int before = live_allocations;
        threw = false;
        try { layer.import_packed_state(bad, stream); } catch (const std::runtime_error& e) { threw = std::string(e.what()).find("reserved code") != std::string::npos; }
        CHECK(threw);
        CHECK(live_allocations == before);
        std::fill(got.begin(), got.end(), 0.0f);
        run();
        CHECK(std::memcmp(got.data(), want.data(), got.size() * 4) == 0);

        // re-importing swaps in fresh buffers and frees the old ones
        layer.import_packed_state(st, stream);
        cudaStreamSynchronize(stream);
        CHECK(live_allocations == before);
        run();
        CHECK(std::memcmp(got.data(), want.data(), got.size() * 4) == 0);

        tbl_linear_view view;
        CHECK(layer.prepare_gpu_decode_view(view));
        CHECK(view.inputs == K && view.outputs == N && view.packed != nullptr && view.rms_input == (exact ? 0 : 1));
        // the grouped seam with the reference's argument list: two descriptors of this layer on the first input row
        {
            const tbl_linear_view views[2] = {view, view};
            const size_t prepared_floats = 2 * static_cast<size_t>(K) + 1024;
            float *prepared = nullptr, *scales = nullptr, *grouped = nullptr;
            CHECK(cudaMalloc(reinterpret_cast<void**>(&prepared), prepared_floats * 4) == cudaSuccess &&
                  cudaMalloc(reinterpret_cast<void**>(&scales), 2 * 4) == cudaSuccess &&
                  cudaMalloc(reinterpret_cast<void**>(&grouped), 2 * static_cast<size_t>(N) * 4) == cudaSuccess);
            tb::launch_grouped_decode_projections(views, dx, prepared, prepared_floats, scales, grouped, 2, N, stream,
                                                  TBL_RMS_REFERENCE_ORDER);
            std::vector<float> rows(2 * static_cast<size_t>(N));
            cudaMemcpyAsync(rows.data(), grouped, rows.size() * 4, cudaMemcpyDeviceToHost, stream);
            tb::check_device(stream);
            CHECK(std::memcmp(rows.data(), want.data(), static_cast<size_t>(N) * 4) == 0);
            CHECK(std::memcmp(rows.data() + N, want.data(), static_cast<size_t>(N) * 4) == 0);
            bool small = false;
            try { tb::launch_grouped_decode_projections(views, dx, prepared, 8, scales, grouped, 2, N, stream); }
            catch (const std::invalid_argument&) { small = true; }
            CHECK(small);
            cudaFree(prepared); cudaFree(scales); cudaFree(grouped);
        }
        cudaFree(dx); cudaFree(dy); cudaFree(scratch);
    }
    CHECK(live_allocations == 0);     // the layer released everything it was given
    std::printf("linear gpu ok: %d x %d, %d rows, %llu launches\n", N, K, M, static_cast<unsigned long long>(tbl_launch_count()));
    return 0;
}
