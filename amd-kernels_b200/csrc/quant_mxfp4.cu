// MXFP4 dynamic quantizer for sm_100a: e2m1 codes (two per byte, element 2i in the low
// nibble) with one e8m0 exponent byte per 32 contiguous elements.
//
// HBM-bound streaming kernel.  The [M, D] tensor is a flat sequence of 32-element blocks
// (D % 32 == 0) and the scale array [M, D/32] is the same sequence, so two adjacent lanes own
// one block (one 32-byte chunk each, a single 256-bit load; a warp reads 1 KB contiguous per
// load): one shuffle gives the block amax, the exponent is read from amax's bit pattern, each
// lane emits 8 code bytes and every 8th lane emits four scale bytes as one word.
//
// Rounding rule of mode 0: nearest E2M1 magnitude of x / 2^e with ties to the SMALLER
// magnitude, saturating at 6; sign nibble set iff x < 0.  For bf16 inputs q = x / 2^e carries at
// most 8 significant bits, so shrinking it by the factor (1 - 2^-10) turns every tie into a
// non-tie without moving any other value across a rounding boundary (a value above a boundary
// is at least one 8-bit grid step = |q| * 2^-8 away from it).  The hardware round-to-nearest
// conversion (cvt.rn.satfinite.e2m1x2.f32) of q' = fma(x, 2^-e * (1 - 2^-10), +0) then yields
// exactly that rule, sign included: the conversion keeps the sign of results that round to
// zero, and the "+0" addend turns the product of x = -0.0 into +0 ("x < 0" is false for it).
// fp32 inputs (the RMSNorm prologue) and mode 1 (truncation) use explicit threshold compares.
#include "common.cuh"

namespace hkb {
namespace {

// eight floats -> eight e2m1 nibbles in one word, element j in bits 4j..4j+3
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&r)[8]) {
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

__device__ __forceinline__ uint32_t nibble_compare(float q, int mode) {
    const float a = fabsf(q);
    uint32_t m;
    if (mode == HKB_MXFP4_MODE_KERNEL) {
        m = (a >= 0.5f) + (a >= 1.0f) + (a >= 1.5f) + (a >= 2.0f) + (a >= 3.0f) + (a >= 4.0f) + (a >= 6.0f);
        return m | ((__float_as_uint(q) >> 28) & 8u);
    }
    m = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    return m | (q < 0.0f ? 8u : 0u);
}

// block amax -> (scale byte, 2^-e as float)
template <int MODE>
__device__ __forceinline__ void block_exponent(float amax, uint32_t& scale_byte, float& inv) {
    uint32_t bits = __float_as_uint(amax);
    if (MODE == HKB_MXFP4_MODE_KERNEL) bits = (bits + 0x200000u) & 0xFF800000u;
    const int biased = (int)(bits >> 23) & 0xFF;
    int e = biased - 129;               // floor(log2 amax) - 2
    e = max(-127, min(127, e));         // subnormal or zero amax lands on -127
    if (biased == 255) e = 127;         // mode 1 can round amax up to infinity: exponent clamps to 127
    scale_byte = (uint32_t)(e + 127);
    // 2^-e: exponent field in [1, 254], or the subnormal 2^-127 for e = 127
    inv = e == 127 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(127 - e) << 23);
}

template <int MODE>
__device__ __forceinline__ uint32_t encode8_bf16(const uint4& v, float inv) {
    if constexpr (MODE == HKB_MXFP4_MODE_KERNEL) {
        float f[8];
        unpack8(v, f);
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) o |= nibble_compare(f[j] * inv, MODE) << (4 * j);
        return o;
    } else {
        // x * (2^-e * (1 - 2^-10)) + 0 on the packed fp32 pipe; `inv` already carries the factor
        const float2 inv2 = make_float2(inv, inv), z2 = make_float2(0.0f, 0.0f);
        const float2 m0 = __ffma2_rn(bf16x2_to_f2(v.x), inv2, z2);
        const float2 m1 = __ffma2_rn(bf16x2_to_f2(v.y), inv2, z2);
        const float2 m2 = __ffma2_rn(bf16x2_to_f2(v.z), inv2, z2);
        const float2 m3 = __ffma2_rn(bf16x2_to_f2(v.w), inv2, z2);
        const float r[8] = {m0.x, m0.y, m1.x, m1.y, m2.x, m2.y, m3.x, m3.y};
        return cvt_e2m1x8(r);
    }
}

// Two adjacent lanes own one 32-element block: lane (b, h) holds elements [16h, 16h+16) of
// block b.  A warp covers 16 blocks per iteration, a thread keeps ITER 32-byte chunks in flight.
// Where the four scale bytes of K atom `ka` of row `r` live in the tensor-core layout (see
// gemm_mxfp4.cu): atoms of 512 bytes, byte (r%32)*16 + ((r%128)/32)*4 + j inside an atom, atoms
// of a 128-row block consecutive along K (katoms_pad of them per block).
struct SfTc {
    uint8_t* base;        // null: no tensor-core-layout output
    uint32_t kgroups;     // D / 128: K atoms per row
    uint32_t katoms_pad;  // kgroups rounded up to even
};
__device__ __forceinline__ uint32_t* sf_tc_word(const SfTc& tc, uint32_t r, uint32_t ka) {
    return reinterpret_cast<uint32_t*>(tc.base + ((size_t)(r >> 7) * tc.katoms_pad + ka) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4);
}

// TC: also (or, with scales == null, only) write the scale bytes in the tensor-core layout; rows
// are then made of whole 128-element groups and total_blocks < 2^31.
template <int MODE, int ITER, bool TC = false>
__global__ void __launch_bounds__(256)
quant_mxfp4_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ codes,
                   uint8_t* __restrict__ scales, int64_t total_blocks, const SfTc tc = SfTc{}) {
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
        uint32_t sb;
        float inv;
        block_exponent<MODE>(am, sb, inv);
        if constexpr (MODE == HKB_MXFP4_MODE_DOC) inv *= (1.0f - 0x1p-10f);     // exact: inv is a power of two
        const uint32_t c0 = encode8_bf16<MODE>(v[it].lo, inv);
        const uint32_t c1 = encode8_bf16<MODE>(v[it].hi, inv);
        if (b < total_blocks) *reinterpret_cast<uint2*>(codes + (b * 2 + h) * 8) = make_uint2(c0, c1);
        // scale bytes of 4 consecutive blocks (lanes 8j, 8j+2, 8j+4, 8j+6) go out as one word
        const int l8 = lane & 24;
        const uint32_t word = __shfl_sync(0xFFFFFFFFu, sb, l8) | (__shfl_sync(0xFFFFFFFFu, sb, l8 + 2) << 8) |
                              (__shfl_sync(0xFFFFFFFFu, sb, l8 + 4) << 16) | (__shfl_sync(0xFFFFFFFFu, sb, l8 + 6) << 24);
        const int64_t b4 = b & ~(int64_t)3;
        if constexpr (TC) {
            if (b < total_blocks && (lane & 7) == 0) {       // D % 128 == 0: the four blocks are one K atom of one row
                if (scales) *reinterpret_cast<uint32_t*>(scales + b) = word;
                const uint32_t g = (uint32_t)b >> 2;
                const uint32_t r = g / tc.kgroups, ka = g - r * tc.kgroups;
                *sf_tc_word(tc, r, ka) = word;
                if (ka + 1 == tc.kgroups && tc.katoms_pad != tc.kgroups) *sf_tc_word(tc, r, ka + 1) = 0u;   // padding atom of an odd D/128
            }
        } else if (b4 + 4 <= total_blocks) {
            if ((lane & 7) == 0) *reinterpret_cast<uint32_t*>(scales + b) = word;
        } else if (b < total_blocks && h == 0) {
            scales[b] = (uint8_t)sb;
        }
    }
}

// Fused RMSNorm prologue: y = x * rsqrt(mean(x^2) + eps) * w in fp32, then the MXFP4 rule on y.
// Thread layout of the per-row FP8 quantizer: TPR threads share a row, each keeps NW 32-byte
// chunks (chunk index t + i*TPR) in registers between the sum-of-squares pass and the encode
// pass; the two chunks of a 32-element block sit in neighbouring lanes.  Rows of a CTA meet only
// on their own named barrier.  Mode "doc" converts with the hardware round-to-nearest-even after
// shrinking by (1 - 2^-22), which sends exact ties to the smaller magnitude (y is fp32 here, so
// unlike the bf16 path a value within four ulps above a tie point can also land below it).
template <int NW, int TPR, int MODE>
__global__ void __launch_bounds__(256, NW <= 4 ? 3 : 2)
rmsnorm_quant_mxfp4_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int64_t M, int nwide, float eps,
                           const SfTc tc) {
    constexpr int RPB = 256 / TPR;
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int r_in = tid / TPR;
    const int t = tid % TPR;
    const int64_t row = (int64_t)blockIdx.x * RPB + r_in;
    const bool live = row < M;
    const __nv_bfloat16* xr = x + row * ((int64_t)nwide * 16);

    Wide v[NW];
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const int c = t + i * TPR;
        v[i] = (live && c < nwide) ? ld_stream32(xr + (int64_t)c * 16) : wide_zero();
    }
    float2 ss2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const uint32_t xw[8] = {v[i].lo.x, v[i].lo.y, v[i].lo.z, v[i].lo.w, v[i].hi.x, v[i].hi.y, v[i].hi.z, v[i].hi.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float2 f = bf16x2_to_f2(xw[j]); ss2 = __ffma2_rn(f, f, ss2); }
    }
    float ss = ss2.x + ss2.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if constexpr (TPR > 32) {
        __shared__ float s_ss[8];
        if ((tid & 31) == 0) s_ss[tid >> 5] = ss;
        if constexpr (TPR == 256) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + r_in), "r"(TPR) : "memory");
        constexpr int WPR = TPR / 32;
        ss = 0.0f;
#pragma unroll
        for (int k = 0; k < WPR; ++k) ss += s_ss[r_in * WPR + k];
    }
    const float rinv = rsqrtf(ss / (float)(nwide * 16) + eps);
    uint8_t* cr = codes + row * ((int64_t)nwide * 8);
    uint8_t* sr = scales + row * (int64_t)(nwide / 2);
    const bool words = (nwide & 7) == 0;          // rows made of whole 128-element groups: scale bytes leave four at a time
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const int c = t + i * TPR;
        const bool ok = live && c < nwide;
        const uint4 w0 = ok ? __ldg(reinterpret_cast<const uint4*>(w + (int64_t)c * 16)) : make_uint4(0, 0, 0, 0);
        const uint4 w1 = ok ? __ldg(reinterpret_cast<const uint4*>(w + (int64_t)c * 16 + 8)) : make_uint4(0, 0, 0, 0);
        const uint32_t xw[8] = {v[i].lo.x, v[i].lo.y, v[i].lo.z, v[i].lo.w, v[i].hi.x, v[i].hi.y, v[i].hi.z, v[i].hi.w};
        const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float2 rinv2 = make_float2(rinv, rinv);
        float2 y[8];
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            y[j] = __fmul2_rn(__fmul2_rn(bf16x2_to_f2(xw[j]), rinv2), bf16x2_to_f2(ww[j]));
            am = fmaxf(am, fmaxf(fabsf(y[j].x), fabsf(y[j].y)));
        }
        am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 1));
        uint32_t sb;
        float inv;
        block_exponent<MODE>(am, sb, inv);
        uint32_t c0 = 0, c1 = 0;
        if constexpr (MODE == HKB_MXFP4_MODE_KERNEL) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                c0 |= (nibble_compare(y[j].x * inv, MODE) | (nibble_compare(y[j].y * inv, MODE) << 4)) << (8 * j);
                c1 |= (nibble_compare(y[4 + j].x * inv, MODE) | (nibble_compare(y[4 + j].y * inv, MODE) << 4)) << (8 * j);
            }
        } else {
            const float invs = inv * (1.0f - 0x1p-22f);
            const float2 invs2 = make_float2(invs, invs), z2 = make_float2(0.0f, 0.0f);
            float r[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 m = __ffma2_rn(y[j], invs2, z2); r[2 * j] = m.x; r[2 * j + 1] = m.y; }
            c0 = cvt_e2m1x8(r);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 m = __ffma2_rn(y[4 + j], invs2, z2); r[2 * j] = m.x; r[2 * j + 1] = m.y; }
            c1 = cvt_e2m1x8(r);
        }
        if (ok) *reinterpret_cast<uint2*>(cr + (int64_t)c * 8) = make_uint2(c0, c1);
        // scale bytes of the four blocks held by lanes 8k .. 8k+7
        const int l8 = lane & 24;
        const uint32_t word = __shfl_sync(0xFFFFFFFFu, sb, l8) | (__shfl_sync(0xFFFFFFFFu, sb, l8 + 2) << 8) |
                              (__shfl_sync(0xFFFFFFFFu, sb, l8 + 4) << 16) | (__shfl_sync(0xFFFFFFFFu, sb, l8 + 6) << 24);
        if (ok) {
            if (tc.base) {          // rows are whole 128-element groups here
                if ((t & 7) == 0) {
                    const uint32_t ka = (uint32_t)c >> 3;
                    if (scales) *reinterpret_cast<uint32_t*>(sr + (c >> 1)) = word;
                    *sf_tc_word(tc, (uint32_t)row, ka) = word;
                    if (ka + 1 == tc.kgroups && tc.katoms_pad != tc.kgroups) *sf_tc_word(tc, (uint32_t)row, ka + 1) = 0u;
                }
            } else if (words) { if ((t & 7) == 0) *reinterpret_cast<uint32_t*>(sr + (c >> 1)) = word; }
            else if ((t & 1) == 0) sr[c >> 1] = (uint8_t)sb;
        }
    }
}

template <int TPR, int MODE>
int launch_rms_mxfp4(int n, const void* x, const void* w, void* codes, void* scales, int64_t M, int nwide, float eps, const SfTc& tc, cudaStream_t st) {
    constexpr int RPB = 256 / TPR;
    const unsigned grid = (unsigned)((M + RPB - 1) / RPB);
#define HKB_RMS(NWV) rmsnorm_quant_mxfp4_kernel<NWV, TPR, MODE><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (uint8_t*)codes, (uint8_t*)scales, M, nwide, eps, tc)
    if (n <= 1) HKB_RMS(1); else if (n <= 2) HKB_RMS(2); else if (n <= 4) HKB_RMS(4); else HKB_RMS(8);
#undef HKB_RMS
    return check_launch("rmsnorm_quant_mxfp4_kernel");
}

template <int MODE>
int dispatch_rms_mxfp4(const void* x, const void* w, void* codes, void* scales, int64_t M, int nwide, float eps, const SfTc& tc, cudaStream_t st) {
    int tpr = 32;
    while (tpr < 256 && tpr * 4 < nwide) tpr *= 2;
    const int n = (nwide + tpr - 1) / tpr;
    switch (tpr) {
        case 32: return launch_rms_mxfp4<32, MODE>(n, x, w, codes, scales, M, nwide, eps, tc, st);
        case 64: return launch_rms_mxfp4<64, MODE>(n, x, w, codes, scales, M, nwide, eps, tc, st);
        case 128: return launch_rms_mxfp4<128, MODE>(n, x, w, codes, scales, M, nwide, eps, tc, st);
        default: return launch_rms_mxfp4<256, MODE>(n, x, w, codes, scales, M, nwide, eps, tc, st);
    }
}

}  // namespace
}  // namespace hkb

namespace hkb {
namespace {
int quant_mxfp4_impl(const void* x, const void* w, void* codes, void* scales, void* sf_tc,
                     int64_t M, int64_t D, float eps, int mode, void* stream) {
    HKB_REQUIRE(x && codes && (scales || sf_tc), HKB_ERR_BAD_ARG, "quant_mxfp4: null pointer");
    HKB_REQUIRE(mode == HKB_MXFP4_MODE_DOC || mode == HKB_MXFP4_MODE_KERNEL, HKB_ERR_BAD_ARG, "quant_mxfp4: unknown mode %d", mode);
    HKB_REQUIRE(M >= 0 && D > 0 && D % 32 == 0, HKB_ERR_BAD_SHAPE, "quant_mxfp4: need D %% 32 == 0, got M=%lld D=%lld", (long long)M, (long long)D);
    HKB_REQUIRE(aligned32(x) && ((uintptr_t)codes & 7) == 0 && ((uintptr_t)scales & 3) == 0 && (!w || aligned16(w)),
                HKB_ERR_BAD_ALIGN, "quant_mxfp4: x must be 32-byte, w 16-byte, codes 8-byte, scales 4-byte aligned");
    SfTc tc{};
    if (sf_tc) {
        HKB_REQUIRE(D % 128 == 0, HKB_ERR_BAD_SHAPE, "quant_mxfp4_tc: D=%lld must be a multiple of 128", (long long)D);
        HKB_REQUIRE(M * (D / 32) < (1LL << 31), HKB_ERR_BAD_SHAPE, "quant_mxfp4_tc: tensor too large");
        HKB_REQUIRE(aligned16(sf_tc), HKB_ERR_BAD_ALIGN, "quant_mxfp4_tc: sf_tc must be 16-byte aligned");
        tc.base = (uint8_t*)sf_tc;
        tc.kgroups = (uint32_t)(D / 128);
        tc.katoms_pad = (tc.kgroups + 1) & ~1u;
    }
    if (M == 0) return HKB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (w) {
        HKB_REQUIRE(D <= 32768 && M <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_mxfp4 with RMSNorm: D must be <= 32768");
        const int nwide = (int)(D / 16);
        if (mode == HKB_MXFP4_MODE_KERNEL) return dispatch_rms_mxfp4<HKB_MXFP4_MODE_KERNEL>(x, w, codes, scales, M, nwide, eps, tc, st);
        return dispatch_rms_mxfp4<HKB_MXFP4_MODE_DOC>(x, w, codes, scales, M, nwide, eps, tc, st);
    }
    constexpr int ITER = 4;
    const int64_t blocks = M * (D / 32);
    const int64_t grid = (blocks + 128 * ITER - 1) / (128 * ITER);
    HKB_REQUIRE(grid <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_mxfp4: tensor too large");
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    if (sf_tc) {
        if (mode == HKB_MXFP4_MODE_KERNEL)
            quant_mxfp4_kernel<HKB_MXFP4_MODE_KERNEL, ITER, true><<<(unsigned)grid, 256, 0, st>>>(xp, (uint8_t*)codes, (uint8_t*)scales, blocks, tc);
        else
            quant_mxfp4_kernel<HKB_MXFP4_MODE_DOC, ITER, true><<<(unsigned)grid, 256, 0, st>>>(xp, (uint8_t*)codes, (uint8_t*)scales, blocks, tc);
    } else if (mode == HKB_MXFP4_MODE_KERNEL)
        quant_mxfp4_kernel<HKB_MXFP4_MODE_KERNEL, ITER><<<(unsigned)grid, 256, 0, st>>>(xp, (uint8_t*)codes, (uint8_t*)scales, blocks);
    else
        quant_mxfp4_kernel<HKB_MXFP4_MODE_DOC, ITER><<<(unsigned)grid, 256, 0, st>>>(xp, (uint8_t*)codes, (uint8_t*)scales, blocks);
    return check_launch("quant_mxfp4_kernel");
}
}  // namespace
}  // namespace hkb

extern "C" int hkb_quant_mxfp4(const void* x, const void* w, void* codes, void* scales,
                               int64_t M, int64_t D, float eps, int mode, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(scales, HKB_ERR_BAD_ARG, "quant_mxfp4: null pointer");
    return quant_mxfp4_impl(x, w, codes, scales, nullptr, M, D, eps, mode, stream);
}

extern "C" int hkb_quant_mxfp4_tc(const void* x, const void* w, void* codes, void* scales, void* sf_tc,
                                  int64_t M, int64_t D, float eps, int mode, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(sf_tc, HKB_ERR_BAD_ARG, "quant_mxfp4_tc: null sf_tc");
    return quant_mxfp4_impl(x, w, codes, scales, sf_tc, M, D, eps, mode, stream);
}
