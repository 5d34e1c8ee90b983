// FP8 (e4m3fn) dynamic quantizers for sm_100a: per-row, 1x128 block and 128x128 block scales.
//
// All three are HBM-bound streaming kernels: every thread moves 32-byte chunks (16 bf16, one
// 256-bit no-allocate load), keeps them in registers between the amax pass and the convert
// pass (the input is read from HBM exactly once), reduces |x| maxima with warp shuffles and
// writes packed e4m3 bytes with 16-byte stores.  Arithmetic is IEEE fp32 and reproduces
//   scale = max(amax / 448, 1e-10);  q = e4m3fn_rne(clamp(x / scale, +-448))
// bit for bit (see hkb::Divider for the exactly rounded shared-divisor division).
#include "common.cuh"

namespace hkb {
namespace {

constexpr float kFp8Max = 448.0f;
constexpr float kInt8Max = 127.0f;
constexpr float kScaleFloor = 1e-10f;

// 8 bf16 (one chunk) -> 8 code bytes.  The e4m3 sign bit is taken from the input's own sign
// bit (the scale is positive), so quotients that underflow to zero keep their sign exactly as
// an IEEE division followed by a round-to-nearest cast does.
template <bool INT8>
__device__ __forceinline__ uint2 encode8(const uint4& v, const Divider2& div) {
    const float2 q0 = div(bf16x2_to_f2(v.x));
    const float2 q1 = div(bf16x2_to_f2(v.y));
    const float2 q2 = div(bf16x2_to_f2(v.z));
    const float2 q3 = div(bf16x2_to_f2(v.w));
    uint2 o;
    if constexpr (INT8) {
        auto b = [](float f) { return (uint32_t)max(-127, min(127, __float2int_rn(f))) & 0xFFu; };
        o.x = b(q0.x) | (b(q0.y) << 8) | (b(q1.x) << 16) | (b(q1.y) << 24);
        o.y = b(q2.x) | (b(q2.y) << 8) | (b(q3.x) << 16) | (b(q3.y) << 24);
    } else {
        // code pairs -> words; sign bytes (byte 1 and 3 of each bf16 pair) gathered with one permute
        o.x = __byte_perm(cvt_e4m3x2(q0.x, q0.y), cvt_e4m3x2(q1.x, q1.y), 0x5410) | (__byte_perm(v.x, v.y, 0x7531) & 0x80808080u);
        o.y = __byte_perm(cvt_e4m3x2(q2.x, q2.y), cvt_e4m3x2(q3.x, q3.y), 0x5410) | (__byte_perm(v.z, v.w, 0x7531) & 0x80808080u);
    }
    return o;
}

template <bool INT8>
__device__ __forceinline__ uint4 encode16(const Wide& v, const Divider2& div) {
    const uint2 a = encode8<INT8>(v.lo, div), b = encode8<INT8>(v.hi, div);
    return make_uint4(a.x, a.y, b.x, b.y);
}

// Same for eight fp32 values that are not bf16 images (RMSNorm prologue output).
__device__ __forceinline__ uint2 encode8_f32(const float (&f)[8], const Divider2& div) {
    uint32_t p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 q = div(make_float2(f[2 * j], f[2 * j + 1]));
        p[j] = cvt_e4m3x2(q.x, q.y) |
               ((__float_as_uint(f[2 * j]) >> 24) & 0x80u) | ((__float_as_uint(f[2 * j + 1]) >> 16) & 0x8000u);
    }
    uint2 o;
    o.x = p[0] | (p[1] << 16);
    o.y = p[2] | (p[3] << 16);
    return o;
}

// ---- per-row ---------------------------------------------------------------------------
// A CTA of 256 threads covers 256/TPR rows; TPR threads share a row and each holds NW 32-byte
// chunks (chunk index = t + i*TPR) in registers.  Needs D % 16 == 0 and 32-byte aligned rows.
template <int NW, int TPR, bool INT8>
__global__ void __launch_bounds__(256, NW <= 4 ? 4 : 2)
quant_row_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                 float* __restrict__ scales, int64_t M, int nwide, int64_t ldx) {
    constexpr int RPB = 256 / TPR;
    const int tid = threadIdx.x;
    const int r_in = tid / TPR;
    const int t = tid % TPR;
    const int64_t row = (int64_t)blockIdx.x * RPB + r_in;
    const bool live = row < M;
    const __nv_bfloat16* xr = x + row * ldx;

    Wide v[NW];
    float am = 0.0f;
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const int c = t + i * TPR;
        v[i] = (live && c < nwide) ? ld_stream32(xr + (int64_t)c * 16) : wide_zero();
    }
    {
        __nv_bfloat162 pm = amax16_packed(v[0]);
#pragma unroll
        for (int i = 1; i < NW; ++i) pm = __hmax2(pm, amax16_packed(v[i]));
        am = hmax_halves(pm);
    }
    am = warp_max(am);
    if constexpr (TPR > 32) {
        __shared__ float s_am[8];
        if ((tid & 31) == 0) s_am[tid >> 5] = am;
        // only the warps of this row wait for one another (named barrier 1 + row-in-CTA): rows of
        // one CTA stay independent, so a slow load of one row does not hold back the others
        if constexpr (TPR == 256) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(1 + r_in), "r"(TPR) : "memory");
        constexpr int WPR = TPR / 32;
        am = s_am[r_in * WPR];
#pragma unroll
        for (int w = 1; w < WPR; ++w) am = fmaxf(am, s_am[r_in * WPR + w]);
    }
    const float scale = fmaxf(__fdiv_rn(am, INT8 ? kInt8Max : kFp8Max), kScaleFloor);
    const Divider2 div(scale);
    if (live && t == 0) scales[row] = scale;
    uint8_t* qr = q + row * ((int64_t)nwide * 16);
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const int c = t + i * TPR;
        if (live && c < nwide) *reinterpret_cast<uint4*>(qr + (int64_t)c * 16) = encode16<INT8>(v[i], div);
    }
}

// Rows too long for registers, or not a multiple of 16 elements / not 32-byte aligned: two
// passes over global memory in 16-byte chunks (the second pass mostly hits L2).
template <bool INT8>
__global__ void __launch_bounds__(256)
quant_row_long_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                      float* __restrict__ scales, int64_t M, int nchunks, int64_t ldx) {
    const int64_t row = blockIdx.x;
    const __nv_bfloat16* xr = x + row * ldx;
    float am = 0.0f;
    for (int c = threadIdx.x; c < nchunks; c += 256) am = fmaxf(am, amax8(ld_stream16(xr + (int64_t)c * 8)));
    am = warp_max(am);
    __shared__ float s_am[8];
    if ((threadIdx.x & 31) == 0) s_am[threadIdx.x >> 5] = am;
    __syncthreads();
    am = s_am[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) am = fmaxf(am, s_am[w]);
    const float scale = fmaxf(__fdiv_rn(am, INT8 ? kInt8Max : kFp8Max), kScaleFloor);
    const Divider2 div(scale);
    if (threadIdx.x == 0) scales[row] = scale;
    uint8_t* qr = q + row * ((int64_t)nchunks * 8);
    for (int c = threadIdx.x; c < nchunks; c += 256)
        *reinterpret_cast<uint2*>(qr + (int64_t)c * 8) = encode8<INT8>(ld_stream16(xr + (int64_t)c * 8), div);
}

template <int NCHUNK, int TPR, bool INT8>
int launch_row(const void* x, void* q, float* scales, int64_t M, int nwide, int64_t ldx, cudaStream_t st) {
    constexpr int RPB = 256 / TPR;
    const int64_t grid = (M + RPB - 1) / RPB;
    quant_row_kernel<NCHUNK, TPR, INT8><<<(unsigned)grid, 256, 0, st>>>(
        (const __nv_bfloat16*)x, (uint8_t*)q, scales, M, nwide, ldx);
    return check_launch("quant_row_kernel");
}

template <int TPR, bool INT8>
int dispatch_nchunk(int n, const void* x, void* q, float* scales, int64_t M, int nchunks, int64_t ldx, cudaStream_t st) {
    switch (n) {
        case 1: return launch_row<1, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        case 2: return launch_row<2, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        case 4: return launch_row<4, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        default: return launch_row<8, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
    }
}

template <bool INT8>
int quant_per_token(const void* x, void* q, float* scales, int64_t M, int64_t D, int64_t ldx, void* stream) {
    HKB_REQUIRE(x && q && scales, HKB_ERR_BAD_ARG, "quant_per_token: null pointer");
    HKB_REQUIRE(M >= 0 && D > 0 && D % 8 == 0, HKB_ERR_BAD_SHAPE,
                "quant_per_token: need D %% 8 == 0 and D > 0, got M=%lld D=%lld", (long long)M, (long long)D);
    HKB_REQUIRE(D <= ((int64_t)1 << 30) && M <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_per_token: size too large");
    HKB_REQUIRE(ldx >= D && ldx % 8 == 0, HKB_ERR_BAD_ALIGN, "quant_per_token: row pitch %lld must be >= D and a multiple of 8", (long long)ldx);
    HKB_REQUIRE(aligned16(x) && ((uintptr_t)q & 7) == 0 && ((uintptr_t)scales & 3) == 0, HKB_ERR_BAD_ALIGN,
                "quant_per_token: x must be 16-byte, q 8-byte, scales 4-byte aligned");
    if (M == 0) return HKB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int nchunks = (int)(D / 8);
    // wide path: rows made of whole 32-byte chunks, held in registers (<= 8 chunks = 256 B per thread)
    const bool wide_ok = D % 16 == 0 && ldx % 16 == 0 && aligned32(x) && aligned16(q);
    const int nwide = (int)(D / 16);
    int tpr = 32;
    while (tpr < 256 && tpr * 4 < nwide) tpr *= 2;    // aim at 4 chunks (128 B in flight) per thread; 2 and 8 measured slower
    const int n = (nwide + tpr - 1) / tpr;
    if (!wide_ok || n > 8) {
        quant_row_long_kernel<INT8><<<(unsigned)M, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, scales, M, nchunks, ldx);
        return check_launch("quant_row_long_kernel");
    }
    int np = 1;
    while (np < n) np *= 2;
    switch (tpr) {
        case 32: return dispatch_nchunk<32, INT8>(np, x, q, scales, M, nwide, ldx, st);
        case 64: return dispatch_nchunk<64, INT8>(np, x, q, scales, M, nwide, ldx, st);
        case 128: return dispatch_nchunk<128, INT8>(np, x, q, scales, M, nwide, ldx, st);
        default: return dispatch_nchunk<256, INT8>(np, x, q, scales, M, nwide, ldx, st);
    }
}

// ---- 1x128 -----------------------------------------------------------------------------
// The [M, D] tensor is a flat sequence of 128-element groups (D % 128 == 0) and the scale
// array [M, D/128] is the same sequence, so no row structure is needed.  Four lanes own one
// group: lane (g, s) holds the 32-byte chunks s and s+4 of group g, so that every load
// instruction of a warp covers eight full 128-byte lines and the per-group work (amax shuffles,
// the divisions that produce scale and reciprocal) is amortised over 32 elements per thread.
template <int ITER>
__global__ void __launch_bounds__(256)
quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                   float* __restrict__ scales, int64_t total_groups) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane & 3;
    const int64_t g0 = ((int64_t)blockIdx.x * 8 + warp) * (8 * ITER) + (lane >> 2);
    Wide v[ITER][2];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int64_t g = g0 + 8 * it;
        const __nv_bfloat16* src = x + (g * 8 + sub) * 16;
#pragma unroll
        for (int k = 0; k < 2; ++k) v[it][k] = (g < total_groups) ? ld_stream32(src + k * 64) : wide_zero();
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
        const int64_t g = g0 + 8 * it;
        float am = hmax_halves(__hmax2(amax16_packed(v[it][0]), amax16_packed(v[it][1])));
        am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 1));
        am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, 2));
        const float scale = fmaxf(__fdiv_rn(am, kFp8Max), kScaleFloor);
        const Divider2 div(scale);
        if (g < total_groups) {
            uint8_t* dst = q + (g * 8 + sub) * 16;
#pragma unroll
            for (int k = 0; k < 2; ++k) *reinterpret_cast<uint4*>(dst + k * 64) = encode16<false>(v[it][k], div);
            if (sub == 0) scales[g] = scale;
        }
    }
}

// Fused RMSNorm prologue: y = x * rsqrt(mean(x^2) + eps) * w in fp32, then the 1x128 rule on y.
// Fused RMSNorm prologue: y = x * rsqrt(mean(x^2) + eps) * w in fp32, then the 1x128 rule on y.
// Same thread layout as quant_row_kernel: TPR threads share a row, each keeps NW 32-byte chunks
// (chunk index t + i*TPR) in registers between the sum-of-squares pass and the encode pass; the
// eight chunks of a 128-element group sit in eight neighbouring lanes, so the group maximum is
// three shuffles.  Rows of a CTA meet only on their own named barrier.
template <int NW, int TPR>
__global__ void __launch_bounds__(256, NW <= 4 ? 3 : 2)
rmsnorm_quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           uint8_t* __restrict__ q, float* __restrict__ scales, int64_t M, int nwide, float eps) {
    constexpr int RPB = 256 / TPR;
    const int tid = threadIdx.x;
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
    uint8_t* qr = q + row * ((int64_t)nwide * 16);
    float* sr = scales + row * (int64_t)(nwide / 8);
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
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, o));
        const float scale = fmaxf(__fdiv_rn(am, kFp8Max), kScaleFloor);
        // y is only defined up to the order of the sum of squares, so the quotient is taken as
        // y * RN(1/scale) (within one fp32 ulp of the true division) and the sign of a zero is
        // left to the conversion: the exactly rounded division of the other quantizers buys
        // nothing here and costs two more packed FMAs per pair.
        const float rs = __frcp_rn(scale);
        const float2 rs2 = make_float2(rs, rs);
        if (ok) {
            uint32_t o4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 qa = __fmul2_rn(y[2 * j], rs2), qb = __fmul2_rn(y[2 * j + 1], rs2);
                o4[j] = (uint32_t)cvt_e4m3x2(qa.x, qa.y) | ((uint32_t)cvt_e4m3x2(qb.x, qb.y) << 16);
            }
            *reinterpret_cast<uint4*>(qr + (int64_t)c * 16) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
            if ((t & 7) == 0) sr[c >> 3] = scale;
        }
    }
}

template <int TPR>
int launch_rms_1x128(int n, const void* x, const void* w, void* q, float* scales, int64_t M, int nwide, float eps, cudaStream_t st) {
    constexpr int RPB = 256 / TPR;
    const unsigned grid = (unsigned)((M + RPB - 1) / RPB);
#define HKB_RMS(NWV) rmsnorm_quant_1x128_kernel<NWV, TPR><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (uint8_t*)q, scales, M, nwide, eps)
    if (n <= 1) HKB_RMS(1); else if (n <= 2) HKB_RMS(2); else if (n <= 4) HKB_RMS(4); else HKB_RMS(8);
#undef HKB_RMS
    return check_launch("rmsnorm_quant_1x128_kernel");
}

// ---- 128x128 ---------------------------------------------------------------------------
// One CTA per weight tile; a thread keeps four 32-byte chunks (64 elements) of the 128x128 tile.
__global__ void __launch_bounds__(256)
quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                     float* __restrict__ scales, int64_t K, int n_tiles) {
    const int kb = blockIdx.x, nb = blockIdx.y;
    const int t = threadIdx.x;
    Wide v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = t + i * 256;
        const int64_t off = ((int64_t)nb * 128 + (j >> 3)) * K + (int64_t)kb * 128 + (j & 7) * 16;
        v[i] = ld_stream32(w + off);
    }
    float am = hmax_halves(__hmax2(__hmax2(amax16_packed(v[0]), amax16_packed(v[1])),
                                   __hmax2(amax16_packed(v[2]), amax16_packed(v[3]))));
    am = warp_max(am);
    __shared__ float s_am[8];
    if ((t & 31) == 0) s_am[t >> 5] = am;
    __syncthreads();
    am = s_am[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) am = fmaxf(am, s_am[k]);
    const float scale = fmaxf(__fdiv_rn(am, kFp8Max), kScaleFloor);
    const Divider2 div(scale);
    if (t == 0) scales[(int64_t)kb * n_tiles + nb] = scale;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = t + i * 256;
        const int64_t off = ((int64_t)nb * 128 + (j >> 3)) * K + (int64_t)kb * 128 + (j & 7) * 16;
        *reinterpret_cast<uint4*>(q + off) = encode16<false>(v[i], div);
    }
}

}  // namespace
}  // namespace hkb

extern "C" {

int hkb_quant_fp8_per_token(const void* x, void* q, float* scales, int64_t M, int64_t D, int64_t ldx, void* stream) {
    return hkb::quant_per_token<false>(x, q, scales, M, D, ldx, stream);
}

int hkb_quant_int8_per_token(const void* x, void* q, float* scales, int64_t M, int64_t D, int64_t ldx, void* stream) {
    return hkb::quant_per_token<true>(x, q, scales, M, D, ldx, stream);
}

int hkb_quant_fp8_1x128(const void* x, const void* w, void* q, float* scales, int64_t M, int64_t D, float eps, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(x && q && scales, HKB_ERR_BAD_ARG, "quant_fp8_1x128: null pointer");
    HKB_REQUIRE(M >= 0 && D > 0 && D % 128 == 0, HKB_ERR_BAD_SHAPE, "quant_fp8_1x128: need D %% 128 == 0, got M=%lld D=%lld", (long long)M, (long long)D);
    HKB_REQUIRE(aligned32(x) && aligned16(q) && ((uintptr_t)scales & 3) == 0 && (!w || aligned16(w)),
                HKB_ERR_BAD_ALIGN, "quant_fp8_1x128: x must be 32-byte, q and w 16-byte, scales 4-byte aligned");
    if (M == 0) return HKB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (w) {
        HKB_REQUIRE(D <= 32768 && M <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_fp8_1x128 with RMSNorm: D must be <= 32768");
        const int nwide = (int)(D / 16);
        int tpr = 32;
        while (tpr < 256 && tpr * 4 < nwide) tpr *= 2;       // 4 chunks per thread, as in the per-row quantizer
        const int n = (nwide + tpr - 1) / tpr;
        switch (tpr) {
            case 32: return launch_rms_1x128<32>(n, x, w, q, scales, M, nwide, eps, st);
            case 64: return launch_rms_1x128<64>(n, x, w, q, scales, M, nwide, eps, st);
            case 128: return launch_rms_1x128<128>(n, x, w, q, scales, M, nwide, eps, st);
            default: return launch_rms_1x128<256>(n, x, w, q, scales, M, nwide, eps, st);
        }
    }
    constexpr int ITER = 2;
    const int64_t groups = M * (D / 128);
    const int64_t grid = (groups + 64 * ITER - 1) / (64 * ITER);
    HKB_REQUIRE(grid <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_fp8_1x128: tensor too large");
    quant_1x128_kernel<ITER><<<(unsigned)grid, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, scales, groups);
    return check_launch("quant_1x128_kernel");
}

int hkb_quant_fp8_128x128(const void* w, void* q, float* scales, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(w && q && scales, HKB_ERR_BAD_ARG, "quant_fp8_128x128: null pointer");
    HKB_REQUIRE(N > 0 && K > 0 && N % 128 == 0 && K % 128 == 0, HKB_ERR_BAD_SHAPE,
                "quant_fp8_128x128: need N %% 128 == 0 and K %% 128 == 0, got N=%lld K=%lld", (long long)N, (long long)K);
    HKB_REQUIRE(N / 128 <= 65535, HKB_ERR_BAD_SHAPE, "quant_fp8_128x128: N too large");
    HKB_REQUIRE(aligned32(w) && aligned16(q) && ((uintptr_t)scales & 3) == 0, HKB_ERR_BAD_ALIGN,
                "quant_fp8_128x128: w must be 32-byte, q 16-byte, scales 4-byte aligned");
    dim3 grid((unsigned)(K / 128), (unsigned)(N / 128));
    quant_128x128_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q, scales, K, (int)(N / 128));
    return check_launch("quant_128x128_kernel");
}

}  // extern "C"
