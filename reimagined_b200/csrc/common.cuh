// Shared device helpers for the sm_100a ternary-linear kernels: PTX wrappers for mbarrier,
// bulk (TMA) copies and dp4a, the sticky device status word, and launch bookkeeping.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ternary_b200.h"

namespace tbl {

// Sticky per-device status word; kernels OR a TBL_DEV_* code into it when a bounded wait
// gives up.  Read and cleared by tbl_device_status().  The word is a __device__ variable of one
// translation unit; launchers fetch its device address once per device and pass it to kernels.
int* device_status_ptr();
int read_and_clear_device_status(int* out);

// Host-side count of kernel launches issued by this library.
void note_launch(int n = 1);

// Upper bound on polls of one mbarrier phase before a kernel gives up (each poll is a
// try_wait with a hardware suspend window, so this is on the order of a second).
constexpr uint32_t kWaitSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait on an mbarrier phase.  Returns false (after recording the timeout in the
// device status word) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status,
                                                  uint32_t limit = kWaitSpinLimit) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicOr(status, TBL_DEV_WAIT_TIMEOUT);
    return false;
}

// 1-D bulk copy global -> shared (TMA engine), completion signalled on `bar` as bytes.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// The same copy for data that is read once (a weight stream): the lines are marked evict-first in L2, so that the
// stream does not push out the small buffers other CTAs are about to read.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// 128-bit load from a 32-bit shared-space address (keeps the access an LDS with 32-bit address
// arithmetic instead of a generic load the compiler cannot always prove to be shared).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// d = c + dot4(signed bytes of a, unsigned bytes of b)
__device__ __forceinline__ int dp4a_su(int a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// q_max of an activation width: 1 for <=2 bits, 2^(b-1)-1 otherwise (127 at 8 bits).
__host__ __device__ __forceinline__ float qmax_for_bits(int bits) {
    return bits <= 2 ? 1.0f : static_cast<float>((1 << (bits - 1)) - 1);
}

// Rounds v to an integer-valued float with the requested tie rule.
// Integer code of v (|v| < 2^22).  Ties-to-even is done on the FMA pipe: v + 1.5 * 2^23 rounds to
// nearest-even at integer granularity and leaves the integer in the low mantissa bits (float-to-int
// conversions run on the quarter-rate XU pipe, which bounds a quantiser that converts every element).
__device__ __forceinline__ int round_code(float v, bool away) {
    if (away) return static_cast<int>(roundf(v));
    return __float_as_int(__fadd_rn(v, 12582912.0f)) - 0x4B400000;
}

__device__ __forceinline__ float round_tie(float v, bool away) {
    return away ? roundf(v) : rintf(v);
}

// Programmatic dependent launch (both are no-ops in a kernel that was launched without the attribute).
// launch_dependents: the next kernel of the stream, if it was launched with the programmatic-stream-serialization
// attribute, may be scheduled once every CTA of this one has issued it (or exited).
// wait: blocks until the preceding kernel has completed and its writes are visible; a dependent kernel calls it
// before it touches anything that kernel writes and before its own first global write.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// The reference's epilogue, one separately rounded fp32 operation per step:
// float(acc) * (act_scale*weight_scale), then * magnitude, then + bias.
__device__ __forceinline__ float epilogue(int acc, float combined_scale, const float* magnitude,
                                          const float* bias, int n) {
    float v = __fmul_rn(static_cast<float>(acc), combined_scale);
    if (magnitude) v = __fmul_rn(v, __ldg(magnitude + n));
    if (bias) v = __fadd_rn(v, __ldg(bias + n));
    return v;
}

// 4x4 byte transpose of 16 consecutive int8 held in four words: out[j] byte e = in[e] byte j.
// Turns q[16w + 4e + j] (natural order) into the order the 2-bit extraction
// ((word >> 2j) & 0x03030303 -> weights 16w + {j, 4+j, 8+j, 12+j}) pairs them with.
__device__ __forceinline__ uint4 transpose4x4_bytes(uint4 v) {
    // first interleave bytes of (x,y) and (z,w), then 16-bit halves
    const uint32_t a0 = __byte_perm(v.x, v.y, 0x5140);  // x0 y0 x1 y1
    const uint32_t a1 = __byte_perm(v.x, v.y, 0x7362);  // x2 y2 x3 y3
    const uint32_t b0 = __byte_perm(v.z, v.w, 0x5140);  // z0 w0 z1 w1
    const uint32_t b1 = __byte_perm(v.z, v.w, 0x7362);  // z2 w2 z3 w3
    uint4 r;
    r.x = __byte_perm(a0, b0, 0x5410);  // x0 y0 z0 w0
    r.y = __byte_perm(a0, b0, 0x7632);  // x1 y1 z1 w1
    r.z = __byte_perm(a1, b1, 0x5410);  // x2 y2 z2 w2
    r.w = __byte_perm(a1, b1, 0x7632);  // x3 y3 z3 w3
    return r;
}

}  // namespace tbl
