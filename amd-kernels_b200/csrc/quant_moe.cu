// MX down-/up-cast and static FP8 down-cast: the wire formats of quant_moe_tk.
//
//   downcast_to_static_fp8   y = e4m3fn( clamp(x / scale, +-448) ), one fp32 scale for the tensor
//   downcast_to_mxfp         per 32 contiguous elements: scale byte = biased exponent of
//                            amax / QMAX rounded UP to a power of two (QMAX = 448 for e4m3 codes,
//                            6 for e2m1 codes), codes = x * 2^(127 - byte) converted with
//                            round-to-nearest-even and saturation; all-zero blocks get byte 127
//   upcast_from_mxfp         out = bf16( decode(code) * float_from_bits(byte << 23) ); byte 255 -> NaN
//
// All three are pure streaming kernels (HBM-bound: 3, 3.03 / 2.53 and 3.03 / 2.53 bytes per
// element).  Two adjacent lanes own one 32-element block (16 elements = one 32-byte load each);
// scale bytes of four consecutive blocks leave as one word.
#include "common.cuh"

namespace hkb {
namespace {

// x * 2^(127 - e) for a biased exponent e in [0, 254], as two exact power-of-two factors (each a
// normal fp32, so that the product is exact whenever the result is representable).
struct Pow2 {
    float f1, f2;
    __device__ __forceinline__ explicit Pow2(uint32_t e) {
        const int d = 127 - (int)e;          // [-127, 127]
        const int d1 = d >> 1, d2 = d - d1;  // floor / ceil halves
        f1 = __uint_as_float((uint32_t)(127 + d1) << 23);
        f2 = __uint_as_float((uint32_t)(127 + d2) << 23);
    }
    __device__ __forceinline__ float operator()(float x) const { return x * f1 * f2; }
};

// biased exponent of amax / qmax rounded up to a power of two; 127 (scale 1.0) for amax == 0
__device__ __forceinline__ uint32_t mx_scale_byte(float amax, float qmax) {
    if (amax == 0.0f) return 127u;
    const uint32_t bits = __float_as_uint(__fdiv_rn(amax, qmax));
    return ((bits + 0x007FFFFFu) & 0x7F800000u) >> 23;
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
    return (uint32_t)cvt_e4m3x2(a, b) | ((uint32_t)cvt_e4m3x2(c, d) << 16);
}

__device__ __forceinline__ uint32_t e2m1x8(const float (&r)[8]) {
    uint32_t o;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}"
        : "=r"(o)
        : "f"(r[0]), "f"(r[1]), "f"(r[2]), "f"(r[3]), "f"(r[4]), "f"(r[5]), "f"(r[6]), "f"(r[7]));
    return o;
}

// ---- static FP8 -------------------------------------------------------------------------------
// 16 elements per thread; the division by the shared scale is the exact-quotient FMA form.
__global__ void __launch_bounds__(256)
static_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                  int64_t nchunks16, int64_t total) {
    const Divider2 div(__ldg(scale));
    const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (c >= nchunks16) return;
    const int64_t e0 = c * 16;
    if (e0 + 16 <= total) {
        const Wide v = ld_stream32(x + e0);
        const uint32_t w[8] = {v.lo.x, v.lo.y, v.lo.z, v.lo.w, v.hi.x, v.hi.y, v.hi.z, v.hi.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = div(bf16x2_to_f2(w[2 * j])), b = div(bf16x2_to_f2(w[2 * j + 1]));
            // the corrected quotient of x = -0.0 comes out as +0: take the sign bits from the input
            o[j] = e4m3x4(a.x, a.y, b.x, b.y) | (__byte_perm(w[2 * j], w[2 * j + 1], 0x7531) & 0x80808080u);
        }
        *reinterpret_cast<uint4*>(y + e0) = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        for (int64_t e = e0; e < total; ++e) {
            const float xe = __bfloat162float(x[e]);
            const float2 q = div(make_float2(xe, 0.0f));
            y[e] = (uint8_t)((cvt_e4m3x2(q.x, 0.0f) & 0xFF) | ((__float_as_uint(xe) >> 24) & 0x80u));
        }
    }
}

// ---- MX down-cast -----------------------------------------------------------------------------
template <bool kFp4, int ITER>
__global__ void __launch_bounds__(256)
downcast_mxfp_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                     int64_t total_blocks) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = lane & 1;
    const int64_t b0 = ((int64_t)blockIdx.x * 8 + warp) * (16 * ITER) + (lane >> 1);
    Wide v[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int64_t b = b0 + 16 * it;
        v[it] = (b < total_blocks) ? ld_stream32(x + (b * 2 + h) * 16) : wide_zero();
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int64_t b = b0 + 16 * it;
        float am = hmax_halves(amax16_packed(v[it]));
        am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 1));
        const uint32_t sb = mx_scale_byte(am, kFp4 ? 6.0f : 448.0f);
        const Pow2 scale(sb);
        const uint32_t w[8] = {v[it].lo.x, v[it].lo.y, v[it].lo.z, v[it].lo.w, v[it].hi.x, v[it].hi.y, v[it].hi.z, v[it].hi.w};
        if constexpr (kFp4) {
            uint32_t o[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float r[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = bf16x2_to_f2(w[4 * j + i]);
                    r[2 * i] = scale(f.x);
                    r[2 * i + 1] = scale(f.y);
                }
                o[j] = e2m1x8(r);
            }
            if (b < total_blocks) *reinterpret_cast<uint2*>(codes + (b * 2 + h) * 8) = make_uint2(o[0], o[1]);
        } else {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = bf16x2_to_f2(w[2 * j]), c = bf16x2_to_f2(w[2 * j + 1]);
                o[j] = e4m3x4(scale(a.x), scale(a.y), scale(c.x), scale(c.y));
            }
            if (b < total_blocks) *reinterpret_cast<uint4*>(codes + (b * 2 + h) * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        // scale bytes of 4 consecutive blocks (lanes 8j, 8j+2, 8j+4, 8j+6) go out as one word
        const int l8 = lane & 24;
        const uint32_t word = __shfl_sync(0xFFFFFFFFu, sb, l8) | (__shfl_sync(0xFFFFFFFFu, sb, l8 + 2) << 8) |
                              (__shfl_sync(0xFFFFFFFFu, sb, l8 + 4) << 16) | (__shfl_sync(0xFFFFFFFFu, sb, l8 + 6) << 24);
        const int64_t b4 = b & ~(int64_t)3;
        if (b4 + 4 <= total_blocks) {
            if ((lane & 7) == 0) *reinterpret_cast<uint32_t*>(scales + b) = word;
        } else if (b < total_blocks && h == 0) {
            scales[b] = (uint8_t)sb;
        }
    }
}

// ---- MX up-cast -------------------------------------------------------------------------------
__device__ __forceinline__ float2 e4m3x2_to_f2(uint16_t c) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(c));
    return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
// e2m1 nibble -> float: twice the magnitudes {0,.5,1,1.5,2,3,4,6} are the hex digits of 0xC8643210
__device__ __forceinline__ float e2m1_to_f(uint32_t nib) {
    const float mag = 0.5f * (float)((0xC8643210u >> ((nib & 7u) * 4)) & 0xFu);
    return (nib & 8u) ? -mag : mag;
}
__device__ __forceinline__ uint32_t bf16x2_from(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}

template <bool kFp4, int ITER>
__global__ void __launch_bounds__(256)
upcast_mxfp_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                   int64_t total_blocks) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = lane & 1;
    const int64_t b0 = ((int64_t)blockIdx.x * 8 + warp) * (16 * ITER) + (lane >> 1);
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int64_t b = b0 + 16 * it;
        if (b >= total_blocks) continue;
        const uint32_t sb = __ldg(scales + b);
        const float s = sb == 255u ? __uint_as_float(0x7FC00000u) : __uint_as_float(sb << 23);
        float f[16];
        if constexpr (kFp4) {
            const uint2 c = *reinterpret_cast<const uint2*>(codes + (b * 2 + h) * 8);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                f[i] = e2m1_to_f(c.x >> (4 * i));
                f[8 + i] = e2m1_to_f(c.y >> (4 * i));
            }
        } else {
            const uint4 c = ld_stream16(codes + (b * 2 + h) * 16);
            const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = e4m3x2_to_f2((uint16_t)(w[j] & 0xFFFF)), d = e4m3x2_to_f2((uint16_t)(w[j] >> 16));
                f[4 * j] = a.x; f[4 * j + 1] = a.y; f[4 * j + 2] = d.x; f[4 * j + 3] = d.y;
            }
        }
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = bf16x2_from(f[2 * i] * s, f[2 * i + 1] * s);
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"l"(out + (b * 2 + h) * 16), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                     : "memory");
    }
}

}  // namespace
}  // namespace hkb

extern "C" {

int hkb_moe_downcast_static_fp8(const void* x, void* y, const float* scale, int64_t M, int64_t N, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(x && y && scale, HKB_ERR_BAD_ARG, "downcast_to_static_fp8: null pointer");
    HKB_REQUIRE(M >= 0 && N >= 0, HKB_ERR_BAD_SHAPE, "downcast_to_static_fp8: negative size");
    HKB_REQUIRE(aligned32(x) && aligned16(y), HKB_ERR_BAD_ALIGN, "downcast_to_static_fp8: x must be 32-byte and y 16-byte aligned");
    const int64_t total = M * N;
    if (total == 0) return HKB_OK;
    const int64_t nchunks = (total + 15) / 16;
    const int64_t grid = (nchunks + 255) / 256;
    HKB_REQUIRE(grid <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "downcast_to_static_fp8: tensor too large");
    static_fp8_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (uint8_t*)y, scale, nchunks, total);
    return check_launch("static_fp8_kernel");
}

int hkb_moe_downcast_mxfp(void* codes, void* scales, const void* src, int64_t outer_dim, int64_t quant_dim, int is_fp4,
                          void* stream) {
    using namespace hkb;
    HKB_REQUIRE(codes && scales && src, HKB_ERR_BAD_ARG, "downcast_to_mxfp: null pointer");
    HKB_REQUIRE(outer_dim >= 0 && quant_dim > 0 && quant_dim % 32 == 0, HKB_ERR_BAD_SHAPE,
                "downcast_to_mxfp: quant_dim must be a positive multiple of 32, got outer_dim=%lld quant_dim=%lld",
                (long long)outer_dim, (long long)quant_dim);
    HKB_REQUIRE(aligned32(src) && aligned16(codes) && ((uintptr_t)scales & 3) == 0, HKB_ERR_BAD_ALIGN,
                "downcast_to_mxfp: src must be 32-byte, mx_tensor 16-byte, mx_scale 4-byte aligned");
    if (outer_dim == 0) return HKB_OK;
    constexpr int ITER = 4;
    const int64_t blocks = outer_dim * (quant_dim / 32);
    const int64_t grid = (blocks + 128 * ITER - 1) / (128 * ITER);
    HKB_REQUIRE(grid <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "downcast_to_mxfp: tensor too large");
    cudaStream_t st = (cudaStream_t)stream;
    if (is_fp4)
        downcast_mxfp_kernel<true, ITER><<<(unsigned)grid, 256, 0, st>>>((const __nv_bfloat16*)src, (uint8_t*)codes, (uint8_t*)scales, blocks);
    else
        downcast_mxfp_kernel<false, ITER><<<(unsigned)grid, 256, 0, st>>>((const __nv_bfloat16*)src, (uint8_t*)codes, (uint8_t*)scales, blocks);
    return check_launch("downcast_mxfp_kernel");
}

int hkb_moe_upcast_mxfp(void* out, const void* scales, const void* codes, int64_t outer_dim, int64_t quant_dim, int is_fp4,
                        void* stream) {
    using namespace hkb;
    HKB_REQUIRE(out && scales && codes, HKB_ERR_BAD_ARG, "upcast_from_mxfp: null pointer");
    HKB_REQUIRE(outer_dim >= 0 && quant_dim > 0 && quant_dim % 32 == 0, HKB_ERR_BAD_SHAPE,
                "upcast_from_mxfp: quant_dim must be a positive multiple of 32, got outer_dim=%lld quant_dim=%lld",
                (long long)outer_dim, (long long)quant_dim);
    HKB_REQUIRE(aligned32(out) && aligned16(codes), HKB_ERR_BAD_ALIGN, "upcast_from_mxfp: out must be 32-byte and mx_tensor 16-byte aligned");
    if (outer_dim == 0) return HKB_OK;
    constexpr int ITER = 4;
    const int64_t blocks = outer_dim * (quant_dim / 32);
    const int64_t grid = (blocks + 128 * ITER - 1) / (128 * ITER);
    HKB_REQUIRE(grid <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "upcast_from_mxfp: tensor too large");
    cudaStream_t st = (cudaStream_t)stream;
    if (is_fp4)
        upcast_mxfp_kernel<true, ITER><<<(unsigned)grid, 256, 0, st>>>((const uint8_t*)codes, (const uint8_t*)scales, (__nv_bfloat16*)out, blocks);
    else
        upcast_mxfp_kernel<false, ITER><<<(unsigned)grid, 256, 0, st>>>((const uint8_t*)codes, (const uint8_t*)scales, (__nv_bfloat16*)out, blocks);
    return check_launch("upcast_mxfp_kernel");
}

}  // extern "C"
