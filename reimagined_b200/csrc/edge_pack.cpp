// Edge-linear pack ("DGE1"): the file in which the NSOS runtime ships the packed ternary linears of a model.
// Host-only reader, validator and writer over memory buffers (the caller maps or reads the file).
//
// Format (OXN/nsos/src/jamba.cpp:104-108, 505-560, 1345-1439; little-endian, no padding):
//   u32 magic 'DGE1' (0x31454744), u32 version (3; legacy 2 has no trailer), u32 layer count
//   per layer: u8 sensitive, i32 in_features, i32 out_features, u8 use_bias, f32 weight_scale,
//              vec<u32> packed words, vec<f32> magnitude[out], vec<f32> bias[out or 0],
//              vec<f32> flat_alpha[in], vec<f32> flat_beta[in], and for a sensitive layer vec<f32> weight[out*in]
//              (vec = u64 count + payload)
//   version 3 trailer: u32 'EGI3' (0x33494745), u64 payload bytes, 64 hex characters of SHA-256(payload)
// Validation follows validate_edge_packed_state (jamba.cpp:546-606) and the loader (jamba.cpp:1451-1616):
// exact vector lengths, finite values, weight_scale > 0, no reserved 2-bit code, flags in {0,1},
// nothing after the last layer, trailer length and digest.
#include <cmath>
#include <cstdint>
#include <cstring>

#include "../../include/ternary_b200.h"

namespace {

// ---- SHA-256 (FIPS 180-4) ----
struct Sha256 {
    uint32_t h[8];
    uint8_t block[64];
    uint64_t bytes;
    size_t fill;
};

const uint32_t kRound[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

inline uint32_t rotr(uint32_t v, int s) { return (v >> s) | (v << (32 - s)); }

void sha_compress(Sha256& c, const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
        w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
        const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
        const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
        w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = c.h[0], b = c.h[1], cc = c.h[2], d = c.h[3], e = c.h[4], f = c.h[5], g = c.h[6], h = c.h[7];
    for (int i = 0; i < 64; ++i) {
        const uint32_t t1 = h + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + kRound[i] + w[i];
        const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & cc) ^ (b & cc));
        h = g; g = f; f = e; e = d + t1; d = cc; cc = b; b = a; a = t1 + t2;
    }
    c.h[0] += a; c.h[1] += b; c.h[2] += cc; c.h[3] += d; c.h[4] += e; c.h[5] += f; c.h[6] += g; c.h[7] += h;
}

void sha_init(Sha256& c) {
    const uint32_t iv[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    std::memcpy(c.h, iv, sizeof iv);
    c.bytes = 0;
    c.fill = 0;
}

void sha_update(Sha256& c, const uint8_t* p, size_t n) {
    c.bytes += n;
    if (c.fill) {
        const size_t take = n < 64 - c.fill ? n : 64 - c.fill;
        std::memcpy(c.block + c.fill, p, take);
        c.fill += take; p += take; n -= take;
        if (c.fill == 64) { sha_compress(c, c.block); c.fill = 0; }
    }
    for (; n >= 64; p += 64, n -= 64) sha_compress(c, p);
    if (n) { std::memcpy(c.block, p, n); c.fill = n; }
}

void sha_hex(Sha256& c, char out[65]) {
    const uint64_t bits = c.bytes * 8;
    uint8_t pad[72] = {0x80};
    const size_t padlen = (c.fill < 56 ? 56 : 120) - c.fill;
    for (int i = 0; i < 8; ++i) pad[padlen + i] = static_cast<uint8_t>(bits >> (56 - 8 * i));
    sha_update(c, pad, padlen + 8);
    static const char* digits = "0123456789abcdef";
    for (int i = 0; i < 8; ++i)
        for (int b = 0; b < 4; ++b) {
            const uint8_t v = static_cast<uint8_t>(c.h[i] >> (24 - 8 * b));
            out[8 * i + 2 * b] = digits[v >> 4];
            out[8 * i + 2 * b + 1] = digits[v & 15];
        }
    out[64] = '\0';
}

}  // namespace

namespace {

constexpr uint32_t kMagic = 0x31454744u;          // "DGE1"
constexpr uint32_t kLegacyVersion = 2, kVersion = 3;
constexpr uint32_t kTrailerMagic = 0x33494745u;   // "EGI3"
constexpr uint64_t kTrailerBytes = 4 + 8 + 64;

// Bounds-checked little-endian cursor over the payload.
struct Cursor {
    const uint8_t* base;
    uint64_t end;      // payload bytes (the trailer is not readable through the cursor)
    uint64_t pos;
    bool ok;

    template <typename T>
    T pod() {
        T v{};
        if (!ok || end - pos < sizeof(T)) { ok = false; return v; }
        std::memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    // vec<T>: u64 count + payload; returns the payload's offset, fails unless count == want
    uint64_t vec(uint64_t want, size_t elem, bool* length_ok) {
        const uint64_t count = pod<uint64_t>();
        if (!ok) return 0;
        if (count != want) { *length_ok = false; ok = false; return 0; }
        if (count > (end - pos) / elem) { ok = false; return 0; }
        const uint64_t at = pos;
        pos += count * elem;
        return at;
    }
};

bool all_finite(const uint8_t* base, uint64_t offset, uint64_t count) {
    for (uint64_t i = 0; i < count; ++i) {
        float v;
        std::memcpy(&v, base + offset + 4 * i, 4);
        if (!std::isfinite(v)) return false;
    }
    return true;
}

// Parses layer records up to and including `stop_at` (or all when stop_at < 0).  Structure (flags, sizes, vector
// lengths, truncation) is always checked; the payload scans -- finite values, reserved codes -- run for every layer
// when validating the whole pack and only for the requested layer otherwise.  `all_out` (may be null, `capacity`
// entries) receives every record.
int walk(const uint8_t* data, uint64_t payload, int stop_at, uint32_t* layers_out, tbl_edge_layer* out,
         tbl_edge_layer* all_out = nullptr, int capacity = 0) {
    Cursor c{data, payload, 8, true};
    const uint32_t layers = c.pod<uint32_t>();
    if (!c.ok) return TBL_ERR_FORMAT;
    if (layers_out) *layers_out = layers;
    for (uint32_t index = 0; index < layers; ++index) {
        tbl_edge_layer L{};
        const uint8_t sensitive = c.pod<uint8_t>();
        L.in_features = c.pod<int32_t>();
        L.out_features = c.pod<int32_t>();
        const uint8_t use_bias = c.pod<uint8_t>();
        L.weight_scale = c.pod<float>();
        if (!c.ok || sensitive > 1 || use_bias > 1 || L.in_features <= 0 || L.out_features <= 0) return TBL_ERR_FORMAT;
        L.sensitive = sensitive;
        L.use_bias = use_bias;
        const uint64_t in = static_cast<uint64_t>(L.in_features), outf = static_cast<uint64_t>(L.out_features);
        const uint64_t total = in * outf;
        bool length_ok = true;
        L.packed_words = (total + 15) / 16;
        L.packed_offset = c.vec(L.packed_words, 4, &length_ok);
        L.magnitude_offset = c.vec(outf, 4, &length_ok);
        L.bias_offset = c.vec(use_bias ? outf : 0, 4, &length_ok);
        L.flat_alpha_offset = c.vec(in, 4, &length_ok);
        L.flat_beta_offset = c.vec(in, 4, &length_ok);
        if (sensitive) { L.weight_offset = c.vec(total, 4, &length_ok); L.weight_count = total; }
        if (!c.ok) return length_ok ? TBL_ERR_FORMAT : TBL_ERR_SHAPE;
        if (!std::isfinite(L.weight_scale) || L.weight_scale <= 0.0f) return TBL_ERR_SCALE;
        if (all_out && static_cast<int>(index) < capacity) all_out[index] = L;
        const bool scan = stop_at < 0 || static_cast<int>(index) == stop_at;
        if (scan && (!all_finite(data, L.magnitude_offset, outf) || !all_finite(data, L.bias_offset, use_bias ? outf : 0) ||
            !all_finite(data, L.flat_alpha_offset, in) || !all_finite(data, L.flat_beta_offset, in) ||
            !all_finite(data, L.weight_offset, L.weight_count)))
            return TBL_ERR_FORMAT;
        for (uint64_t w = 0; scan && w < L.packed_words; ++w) {
            uint32_t word;
            std::memcpy(&word, data + L.packed_offset + 4 * w, 4);
            // a field is reserved when both of its bits are set; fields past the last weight are not checked
            uint32_t both = word & (word >> 1) & 0x55555555u;
            if (w + 1 == L.packed_words && (total & 15)) both &= (1u << (2 * (total & 15))) - 1u;
            if (both) return TBL_ERR_CODE;
        }
        if (static_cast<int>(index) == stop_at) { if (out) *out = L; return TBL_OK; }
    }
    if (stop_at >= 0) return TBL_ERR_INVALID_ARG;          // index past the last layer
    return c.pos == payload ? TBL_OK : TBL_ERR_FORMAT;     // nothing may follow the last layer
}

// Header and (version 3) trailer checks; returns the payload length.
int open_pack(const uint8_t* data, size_t bytes, uint32_t* version_out, uint64_t* payload_out, bool verify_digest = true) {
    if (!data || bytes < 12) return TBL_ERR_FORMAT;
    uint32_t magic, version;
    std::memcpy(&magic, data, 4);
    std::memcpy(&version, data + 4, 4);
    if (magic != kMagic || (version != kLegacyVersion && version != kVersion)) return TBL_ERR_FORMAT;
    uint64_t payload = bytes;
    if (version >= kVersion) {
        if (bytes < 12 + kTrailerBytes) return TBL_ERR_FORMAT;
        payload = bytes - kTrailerBytes;
        uint32_t tmagic;
        uint64_t tbytes;
        std::memcpy(&tmagic, data + payload, 4);
        std::memcpy(&tbytes, data + payload + 4, 8);
        if (tmagic != kTrailerMagic || tbytes != payload) return TBL_ERR_INTEGRITY;
        if (verify_digest) {
            Sha256 c;
            sha_init(c);
            sha_update(c, data, payload);
            char hex[65];
            sha_hex(c, hex);
            if (std::memcmp(hex, data + payload + 12, 64) != 0) return TBL_ERR_INTEGRITY;
        }
    }
    *version_out = version;
    *payload_out = payload;
    return TBL_OK;
}

}  // namespace

extern "C" {

void tbl_sha256_hex(const void* data, size_t bytes, char out[65]) {
    Sha256 c;
    sha_init(c);
    if (bytes) sha_update(c, static_cast<const uint8_t*>(data), bytes);
    sha_hex(c, out);
}

int tbl_edge_pack_open(const void* data, size_t bytes, int* version_out, int* layers_out) {
    uint32_t version = 0, layers = 0;
    uint64_t payload = 0;
    int rc = open_pack(static_cast<const uint8_t*>(data), bytes, &version, &payload);
    if (rc != TBL_OK) return rc;
    rc = walk(static_cast<const uint8_t*>(data), payload, -1, &layers, nullptr);
    if (rc != TBL_OK) return rc;
    if (version_out) *version_out = static_cast<int>(version);
    if (layers_out) *layers_out = static_cast<int>(layers);
    return TBL_OK;
}

int tbl_edge_pack_layer(const void* data, size_t bytes, int index, tbl_edge_layer* out) {
    if (!out || index < 0) return TBL_ERR_INVALID_ARG;
    uint32_t version = 0;
    uint64_t payload = 0;
    // header and trailer framing only: the digest was checked by tbl_edge_pack_open
    const int rc = open_pack(static_cast<const uint8_t*>(data), bytes, &version, &payload, /*verify_digest=*/false);
    if (rc != TBL_OK) return rc;
    return walk(static_cast<const uint8_t*>(data), payload, index, nullptr, out);
}

int tbl_edge_pack_layers(const void* data, size_t bytes, tbl_edge_layer* out, int capacity, int* version_out,
                         int* layers_out) {
    if (!out || capacity < 0) return TBL_ERR_INVALID_ARG;
    uint32_t version = 0, layers = 0;
    uint64_t payload = 0;
    int rc = open_pack(static_cast<const uint8_t*>(data), bytes, &version, &payload, true);
    if (rc != TBL_OK) return rc;
    rc = walk(static_cast<const uint8_t*>(data), payload, -1, &layers, nullptr, out, capacity);
    if (rc != TBL_OK) return rc;
    if (version_out) *version_out = static_cast<int>(version);
    if (layers_out) *layers_out = static_cast<int>(layers);
    return static_cast<int>(layers) <= capacity ? TBL_OK : TBL_ERR_WORKSPACE;
}

}  // extern "C"

// ---- writer ----
namespace {

struct Sink {
    uint8_t* out;       // null: only count
    size_t cap, pos;
    bool ok;
    void put(const void* p, size_t n) {
        if (out) {
            if (cap - pos < n) { ok = false; return; }
            std::memcpy(out + pos, p, n);
        }
        pos += n;
    }
    template <typename T> void pod(T v) { put(&v, sizeof(T)); }
    void vec(const void* p, uint64_t count, size_t elem) {
        pod<uint64_t>(count);
        if (count) put(p, count * elem);
    }
};

int emit(const tbl_edge_layer_src* layers, int count, Sink& s) {
    s.pod<uint32_t>(kMagic);
    s.pod<uint32_t>(kVersion);
    s.pod<uint32_t>(static_cast<uint32_t>(count));
    for (int i = 0; i < count; ++i) {
        const tbl_edge_layer_src& L = layers[i];
        if (L.in_features <= 0 || L.out_features <= 0 || !L.packed || !L.magnitude || !L.flat_alpha || !L.flat_beta ||
            (L.use_bias && !L.bias) || (L.sensitive && !L.weight))
            return TBL_ERR_INVALID_ARG;
        const uint64_t in = static_cast<uint64_t>(L.in_features), outf = static_cast<uint64_t>(L.out_features);
        s.pod<uint8_t>(L.sensitive ? 1 : 0);
        s.pod<int32_t>(L.in_features);
        s.pod<int32_t>(L.out_features);
        s.pod<uint8_t>(L.use_bias ? 1 : 0);
        s.pod<float>(L.weight_scale);
        s.vec(L.packed, (in * outf + 15) / 16, 4);
        s.vec(L.magnitude, outf, 4);
        s.vec(L.bias, L.use_bias ? outf : 0, 4);
        s.vec(L.flat_alpha, in, 4);
        s.vec(L.flat_beta, in, 4);
        if (L.sensitive) s.vec(L.weight, in * outf, 4);
    }
    return s.ok ? TBL_OK : TBL_ERR_WORKSPACE;
}

}  // namespace

extern "C" {

size_t tbl_edge_pack_bytes(const tbl_edge_layer_src* layers, int count) {
    if (!layers || count < 0) return 0;
    Sink s{nullptr, 0, 0, true};
    if (emit(layers, count, s) != TBL_OK) return 0;
    return s.pos + kTrailerBytes;
}

int tbl_edge_pack_write(const tbl_edge_layer_src* layers, int count, void* out, size_t capacity, size_t* written) {
    if (!layers || count < 0 || !out) return TBL_ERR_INVALID_ARG;
    Sink s{static_cast<uint8_t*>(out), capacity, 0, true};
    int rc = emit(layers, count, s);
    if (rc != TBL_OK) return rc;
    const uint64_t payload = s.pos;
    char hex[65];
    tbl_sha256_hex(out, payload, hex);
    s.pod<uint32_t>(kTrailerMagic);
    s.pod<uint64_t>(payload);
    s.put(hex, 64);
    if (!s.ok) return TBL_ERR_WORKSPACE;
    // what is written must load: the same validation a reader applies (finite values, codes, scale)
    int version = 0, n = 0;
    rc = tbl_edge_pack_open(out, s.pos, &version, &n);
    if (rc != TBL_OK) return rc;
    if (written) *written = s.pos;
    return TBL_OK;
}

}  // extern "C"
