// Shared host/device helpers of libhkb200: error plumbing, launch checks, small PTX wrappers.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/hkb200.h"

namespace hkb {

// Thread-local message behind hkb_last_error(); defined in runtime.cu.
int set_error(int code, const char* fmt, ...);

#define HKB_REQUIRE(cond, code, ...)                         \
    do {                                                     \
        if (!(cond)) return ::hkb::set_error((code), __VA_ARGS__); \
    } while (0)

#define HKB_CUDA(call)                                                              \
    do {                                                                            \
        cudaError_t e__ = (call);                                                   \
        if (e__ != cudaSuccess)                                                     \
            return ::hkb::set_error(HKB_ERR_CUDA, "%s failed: %s", #call,           \
                                    cudaGetErrorString(e__));                       \
    } while (0)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return set_error(HKB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return HKB_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Per-device, lazily grown scratch owned by the library (freed by hkb_release()).
// `slot` separates independent users so they do not overwrite each other.
enum ScratchSlot { SCRATCH_SFA = 0, SCRATCH_SFB = 1, SCRATCH_ROWS = 2, SCRATCH_SLOTS = 3 };
// Scratch is keyed by (device, stream): calls on different streams of one device get different
// blocks, so they may overlap on the GPU.  A device keeps blocks for up to kScratchStreams streams;
// when more streams than that use scratch, the least recently used stream's blocks are recycled
// (after a device-wide synchronisation, which cudaFree implies).
constexpr int kScratchStreams = 8;
int scratch_get(ScratchSlot slot, cudaStream_t stream, size_t bytes, void** out);
// Device status word (one uint32 per device): kernels OR an error bit in when a bounded
// wait runs out.  Zeroed at allocation.
int status_word(uint32_t** out);
// Name of the kernel variant the calling thread launched last (hkb_last_kernel()).
void note_kernel(const char* name);
// Status word of the allocation-free MXFP4 entry point on the current device, or null when that
// entry point has not run on it (gemm_mxfp4.cu).
uint32_t* static_status_peek();

}  // namespace hkb

// ---- device helpers -----------------------------------------------------------------------
namespace hkb {

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// 8 bf16 (one 16-byte chunk) -> 8 floats
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
    f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
    f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// max |.| over the 8 bf16 of a chunk, computed on the packed halves (exact: bf16 max).
__device__ __forceinline__ float amax8(const uint4& v) {
    const uint32_t m = 0x7FFF7FFFu;
    uint32_t x0 = v.x & m, x1 = v.y & m, x2 = v.z & m, x3 = v.w & m;
    __nv_bfloat162 b0 = *reinterpret_cast<__nv_bfloat162*>(&x0);
    __nv_bfloat162 b1 = *reinterpret_cast<__nv_bfloat162*>(&x1);
    __nv_bfloat162 b2 = *reinterpret_cast<__nv_bfloat162*>(&x2);
    __nv_bfloat162 b3 = *reinterpret_cast<__nv_bfloat162*>(&x3);
    __nv_bfloat162 mx = __hmax2(__hmax2(b0, b1), __hmax2(b2, b3));
    return fmaxf(__low2float(mx), __high2float(mx));
}

// Streaming 16-byte load that does not allocate in L1.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 16 bf16 = 32 bytes moved by one 256-bit load (sm_100+), as two 16-byte halves.
struct Wide { uint4 lo, hi; };
__device__ __forceinline__ Wide ld_stream32(const void* p) {
    Wide v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ Wide wide_zero() { Wide v; v.lo = make_uint4(0, 0, 0, 0); v.hi = v.lo; return v; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// Two floats -> two e4m3fn bytes (round-to-nearest-even, saturating to +-448), `lo` in bits 0-7.
__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// Exactly-rounded x / s for a divisor shared by many elements, given r = RN(1/s).
// q0 = RN(x*r) is within one ulp; the remainder e = x - q0*s is exact in an FMA; RN(q0 + e*r)
// is the correctly rounded quotient (Markstein) unless s has an all-ones mantissa or an
// intermediate leaves the normal range -- callers route those cases to a true division
// by passing exact = true.
struct Divider {
    float s, r;
    bool exact;
    __device__ __forceinline__ explicit Divider(float scale) {
        s = scale;
        r = __frcp_rn(scale);
        const uint32_t b = __float_as_uint(scale);
        const uint32_t ex = (b >> 23) & 0xFF;
        // keep clear of all-ones mantissas and of exponents where r or the remainder could
        // become subnormal / overflow
        exact = ((b & 0x7FFFFFu) == 0x7FFFFFu) || ex < 32 || ex > 222;
    }
    __device__ __forceinline__ float operator()(float x) const {
        if (exact) return __fdiv_rn(x, s);
        const float q0 = x * r;
        const float e = __fmaf_rn(-q0, s, x);
        return __fmaf_rn(e, r, q0);
    }
};

// bf16 pair -> (lo, hi) as fp32
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}

// Divider for two values at a time on the packed fp32 pipe (fmul2 / ffma2); same rounding.
struct Divider2 {
    float s, r;
    float2 r2, ns2;
    bool exact;
    __device__ __forceinline__ explicit Divider2(float scale) {
        const Divider d(scale);
        s = d.s; r = d.r; exact = d.exact;
        r2 = make_float2(r, r);
        ns2 = make_float2(-s, -s);
    }
    __device__ __forceinline__ float2 operator()(float2 x) const {
        if (exact) return make_float2(__fdiv_rn(x.x, s), __fdiv_rn(x.y, s));
        const float2 q0 = __fmul2_rn(x, r2);
        const float2 e = __ffma2_rn(q0, ns2, x);
        return __ffma2_rn(e, r2, q0);
    }
};

// max |.| over the 8 bf16 of a chunk as a packed bf16 pair (both halves hold partial maxima)
__device__ __forceinline__ __nv_bfloat162 amax8_packed(const uint4& v) {
    auto h2 = [](const uint32_t& w) { return __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w)); };
    return __hmax2(__hmax2(h2(v.x), h2(v.y)), __hmax2(h2(v.z), h2(v.w)));
}
__device__ __forceinline__ __nv_bfloat162 amax16_packed(const Wide& v) { return __hmax2(amax8_packed(v.lo), amax8_packed(v.hi)); }
__device__ __forceinline__ float hmax_halves(__nv_bfloat162 m) { return fmaxf(__low2float(m), __high2float(m)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}

}  // namespace hkb
