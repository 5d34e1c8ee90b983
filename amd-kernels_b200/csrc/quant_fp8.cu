// FP8 (e4m3fn) dynamic quantizers for sm_100a: per-row, 1x128 block and 128x128 block scales.
//
// All three are HBM-bound streaming kernels: every thread moves 16-byte chunks (8 bf16) with
// coalesced no-allocate loads, keeps them in registers between the amax pass and the convert
// pass (the input is read from HBM exactly once), reduces |x| maxima with warp shuffles and
// writes packed e4m3 bytes with 8-byte stores.  Arithmetic is IEEE fp32 and reproduces
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
__device__ __forceinline__ uint2 encode8(const uint4& v, const Divider& div) {
    float f[8];
    unpack8(v, f);
    uint2 o;
    if constexpr (INT8) {
        uint32_t b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int q = __float2int_rn(div(f[j]));
            q = max(-127, min(127, q));
            b[j] = (uint32_t)q & 0xFFu;
        }
        o.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
        o.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
    } else {
        // sign bits of a bf16 pair (bits 15 and 31) moved to bits 7 and 15 of a code pair
        auto sgn = [](uint32_t w) { return ((w >> 8) & 0x80u) | ((w >> 16) & 0x8000u); };
        const uint32_t p0 = cvt_e4m3x2(div(f[0]), div(f[1])) | sgn(v.x);
        const uint32_t p1 = cvt_e4m3x2(div(f[2]), div(f[3])) | sgn(v.y);
        const uint32_t p2 = cvt_e4m3x2(div(f[4]), div(f[5])) | sgn(v.z);
        const uint32_t p3 = cvt_e4m3x2(div(f[6]), div(f[7])) | sgn(v.w);
        o.x = p0 | (p1 << 16);
        o.y = p2 | (p3 << 16);
    }
    return o;
}

// Same for eight fp32 values that are not bf16 images (RMSNorm prologue output).
__device__ __forceinline__ uint2 encode8_f32(const float (&f)[8], const Divider& div) {
    uint32_t p[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        p[j] = cvt_e4m3x2(div(f[2 * j]), div(f[2 * j + 1])) |
               ((__float_as_uint(f[2 * j]) >> 24) & 0x80u) | ((__float_as_uint(f[2 * j + 1]) >> 16) & 0x8000u);
    }
    uint2 o;
    o.x = p[0] | (p[1] << 16);
    o.y = p[2] | (p[3] << 16);
    return o;
}

// ---- per-row ---------------------------------------------------------------------------
// A CTA of 256 threads covers 256/TPR rows; TPR threads share a row and each holds NCHUNK
// chunks (chunk index = t + i*TPR) in registers.
template <int NCHUNK, int TPR, bool INT8>
__global__ void __launch_bounds__(256)
quant_row_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                 float* __restrict__ scales, int64_t M, int nchunks, int64_t ldx) {
    constexpr int RPB = 256 / TPR;
    const int tid = threadIdx.x;
    const int r_in = tid / TPR;
    const int t = tid % TPR;
    const int64_t row = (int64_t)blockIdx.x * RPB + r_in;
    const bool live = row < M;
    const __nv_bfloat16* xr = x + row * ldx;

    uint4 v[NCHUNK];
    float am = 0.0f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        v[i] = (live && c < nchunks) ? ld_stream16(xr + (int64_t)c * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) am = fmaxf(am, amax8(v[i]));
    am = warp_max(am);
    if constexpr (TPR > 32) {
        __shared__ float s_am[8];
        if ((tid & 31) == 0) s_am[tid >> 5] = am;
        __syncthreads();
        constexpr int WPR = TPR / 32;
        am = s_am[r_in * WPR];
#pragma unroll
        for (int w = 1; w < WPR; ++w) am = fmaxf(am, s_am[r_in * WPR + w]);
    }
    const float scale = fmaxf(__fdiv_rn(am, INT8 ? kInt8Max : kFp8Max), kScaleFloor);
    const Divider div(scale);
    if (live && t == 0) scales[row] = scale;
    uint8_t* qr = q + row * ((int64_t)nchunks * 8);
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        if (live && c < nchunks) *reinterpret_cast<uint2*>(qr + (int64_t)c * 8) = encode8<INT8>(v[i], div);
    }
}

// Rows too long for registers: two passes over global memory (second pass mostly hits L2).
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
    const Divider div(scale);
    if (threadIdx.x == 0) scales[row] = scale;
    uint8_t* qr = q + row * ((int64_t)nchunks * 8);
    for (int c = threadIdx.x; c < nchunks; c += 256)
        *reinterpret_cast<uint2*>(qr + (int64_t)c * 8) = encode8<INT8>(ld_stream16(xr + (int64_t)c * 8), div);
}

template <int NCHUNK, int TPR, bool INT8>
int launch_row(const void* x, void* q, float* scales, int64_t M, int nchunks, int64_t ldx, cudaStream_t st) {
    constexpr int RPB = 256 / TPR;
    const int64_t grid = (M + RPB - 1) / RPB;
    quant_row_kernel<NCHUNK, TPR, INT8><<<(unsigned)grid, 256, 0, st>>>(
        (const __nv_bfloat16*)x, (uint8_t*)q, scales, M, nchunks, ldx);
    return check_launch("quant_row_kernel");
}

template <int TPR, bool INT8>
int dispatch_nchunk(int n, const void* x, void* q, float* scales, int64_t M, int nchunks, int64_t ldx, cudaStream_t st) {
    switch (n) {
        case 1: return launch_row<1, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        case 2: return launch_row<2, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        case 4: return launch_row<4, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        case 8: return launch_row<8, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
        default: return launch_row<16, TPR, INT8>(x, q, scales, M, nchunks, ldx, st);
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
    // threads per row: aim at 4 chunks (64 B in flight) per thread
    int tpr = 32;
    while (tpr < 256 && tpr * 4 < nchunks) tpr *= 2;
    int n = (nchunks + tpr - 1) / tpr;
    if (n > 16) {
        quant_row_long_kernel<INT8><<<(unsigned)M, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, scales, M, nchunks, ldx);
        return check_launch("quant_row_long_kernel");
    }
    int np = 1;
    while (np < n) np *= 2;
    switch (tpr) {
        case 32: return dispatch_nchunk<32, INT8>(np, x, q, scales, M, nchunks, ldx, st);
        case 64: return dispatch_nchunk<64, INT8>(np, x, q, scales, M, nchunks, ldx, st);
        case 128: return dispatch_nchunk<128, INT8>(np, x, q, scales, M, nchunks, ldx, st);
        default: return dispatch_nchunk<256, INT8>(np, x, q, scales, M, nchunks, ldx, st);
    }
}

// ---- 1x128 -----------------------------------------------------------------------------
// The [M, D] tensor is a flat sequence of 128-element groups (D % 128 == 0) and the scale
// array [M, D/128] is the same sequence, so no row structure is needed: 16 consecutive lanes
// own one group, every thread keeps UNROLL chunks in flight.
template <int UNROLL>
__global__ void __launch_bounds__(256)
quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                   float* __restrict__ scales, int64_t total_chunks) {
    const int64_t base = (int64_t)blockIdx.x * (256 * UNROLL) + threadIdx.x;
    uint4 v[UNROLL];
#pragma unroll
    for (int i = 0; i < UNROLL; ++i) {
        const int64_t c = base + i * 256;
        v[i] = (c < total_chunks) ? ld_stream16(x + c * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < UNROLL; ++i) {
        const int64_t c = base + i * 256;
        float am = amax8(v[i]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, o));
        const float scale = fmaxf(__fdiv_rn(am, kFp8Max), kScaleFloor);
        const Divider div(scale);
        if (c < total_chunks) {
            *reinterpret_cast<uint2*>(q + c * 8) = encode8<false>(v[i], div);
            if ((threadIdx.x & 15) == 0) scales[c >> 4] = scale;
        }
    }
}

// Fused RMSNorm prologue: y = x * rsqrt(mean(x^2) + eps) * w in fp32, then the 1x128 rule on y.
// One CTA per row; the row stays in registers as bf16 chunks.
template <int NCHUNK>
__global__ void __launch_bounds__(256)
rmsnorm_quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           uint8_t* __restrict__ q, float* __restrict__ scales, int nchunks, float eps) {
    const int64_t row = blockIdx.x;
    const int t = threadIdx.x;
    const __nv_bfloat16* xr = x + row * (int64_t)nchunks * 8;
    uint4 v[NCHUNK];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * 256;
        v[i] = (c < nchunks) ? ld_stream16(xr + (int64_t)c * 8) : make_uint4(0, 0, 0, 0);
        float f[8];
        unpack8(v[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = __fmaf_rn(f[j], f[j], ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    __shared__ float s_ss[8];
    if ((t & 31) == 0) s_ss[t >> 5] = ss;
    __syncthreads();
    ss = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += s_ss[k];
    const float rinv = rsqrtf(ss / (float)(nchunks * 8) + eps);
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * 256;
        const bool ok = c < nchunks;
        float f[8], g[8];
        unpack8(v[i], f);
        const uint4 wv = ok ? *reinterpret_cast<const uint4*>(w + (int64_t)c * 8) : make_uint4(0, 0, 0, 0);
        unpack8(wv, g);
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            f[j] = f[j] * rinv * g[j];
            am = fmaxf(am, fabsf(f[j]));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xFFFFFFFFu, am, o));
        const float scale = fmaxf(__fdiv_rn(am, kFp8Max), kScaleFloor);
        const Divider div(scale);
        if (ok) {
            *reinterpret_cast<uint2*>(q + (row * nchunks + c) * 8) = encode8_f32(f, div);
            if ((t & 15) == 0) scales[(row * nchunks + c) >> 4] = scale;
        }
    }
}

// ---- 128x128 ---------------------------------------------------------------------------
// One CTA per weight tile; a thread keeps 8 chunks (64 elements) of the 128x128 tile.
__global__ void __launch_bounds__(256)
quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q,
                     float* __restrict__ scales, int64_t K, int n_tiles) {
    const int kb = blockIdx.x, nb = blockIdx.y;
    const int t = threadIdx.x;
    uint4 v[8];
    float am = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int j = t + i * 256;
        const int64_t off = ((int64_t)nb * 128 + (j >> 4)) * K + (int64_t)kb * 128 + (j & 15) * 8;
        v[i] = ld_stream16(w + off);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) am = fmaxf(am, amax8(v[i]));
    am = warp_max(am);
    __shared__ float s_am[8];
    if ((t & 31) == 0) s_am[t >> 5] = am;
    __syncthreads();
    am = s_am[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) am = fmaxf(am, s_am[k]);
    const float scale = fmaxf(__fdiv_rn(am, kFp8Max), kScaleFloor);
    const Divider div(scale);
    if (t == 0) scales[(int64_t)kb * n_tiles + nb] = scale;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int j = t + i * 256;
        const int64_t off = ((int64_t)nb * 128 + (j >> 4)) * K + (int64_t)kb * 128 + (j & 15) * 8;
        *reinterpret_cast<uint2*>(q + off) = encode8<false>(v[i], div);
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
    HKB_REQUIRE(aligned16(x) && ((uintptr_t)q & 7) == 0 && ((uintptr_t)scales & 3) == 0 && (!w || aligned16(w)),
                HKB_ERR_BAD_ALIGN, "quant_fp8_1x128: x/w must be 16-byte, q 8-byte, scales 4-byte aligned");
    if (M == 0) return HKB_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (w) {
        const int nchunks = (int)(D / 8);
        HKB_REQUIRE(D <= 32768 && M <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_fp8_1x128 with RMSNorm: D must be <= 32768");
        const int n = (nchunks + 255) / 256;
#define HKB_RMS(NC) rmsnorm_quant_1x128_kernel<NC><<<(unsigned)M, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (uint8_t*)q, scales, nchunks, eps)
        if (n <= 1) HKB_RMS(1); else if (n <= 2) HKB_RMS(2); else if (n <= 4) HKB_RMS(4); else if (n <= 8) HKB_RMS(8); else HKB_RMS(16);
#undef HKB_RMS
        return check_launch("rmsnorm_quant_1x128_kernel");
    }
    constexpr int UNROLL = 4;
    const int64_t total = M * D / 8;
    const int64_t grid = (total + 256 * UNROLL - 1) / (256 * UNROLL);
    HKB_REQUIRE(grid <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "quant_fp8_1x128: tensor too large");
    quant_1x128_kernel<UNROLL><<<(unsigned)grid, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, scales, total);
    return check_launch("quant_1x128_kernel");
}

int hkb_quant_fp8_128x128(const void* w, void* q, float* scales, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(w && q && scales, HKB_ERR_BAD_ARG, "quant_fp8_128x128: null pointer");
    HKB_REQUIRE(N > 0 && K > 0 && N % 128 == 0 && K % 128 == 0, HKB_ERR_BAD_SHAPE,
                "quant_fp8_128x128: need N %% 128 == 0 and K %% 128 == 0, got N=%lld K=%lld", (long long)N, (long long)K);
    HKB_REQUIRE(N / 128 <= 65535, HKB_ERR_BAD_SHAPE, "quant_fp8_128x128: N too large");
    HKB_REQUIRE(aligned16(w) && ((uintptr_t)q & 7) == 0 && ((uintptr_t)scales & 3) == 0, HKB_ERR_BAD_ALIGN,
                "quant_fp8_128x128: w must be 16-byte, q 8-byte, scales 4-byte aligned");
    dim3 grid((unsigned)(K / 128), (unsigned)(N / 128));
    quant_128x128_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)w, (uint8_t*)q, scales, K, (int)(N / 128));
    return check_launch("quant_128x128_kernel");
}

}  // extern "C"
