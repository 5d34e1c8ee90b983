// Batched FP8 GEMM with the activation quantizer inside the main loop ("per-token-group
// pre-quantization"): A arrives as bf16 and is quantized per row and per 64-wide K group while the
// tile is being staged; the weights are e4m3fn codes with one scalar scale; bias optional.
//
//   per 64-K group g:  m = max(|A[m, g]|, 1e-10);  a_scale = m * (1/448);  q = e4m3(A * (1 / a_scale))
//                      acc[m, n] += (q @ Wq[n, g]^T) * a_scale[m]
//   C[m, n] = bf16(acc * b_scale + bias[n])
//
// Roles (512 threads, one CTA per SM, persistent over 128 x 256 tiles):
//   warp 0        TMA producer of the weight tiles (256 rows x 128 bytes per stage)
//   warp 1        TMEM allocator + MMA issuer: two tcgen05.mma (K = 32) per 64-K group into one of two
//                 TMEM buffers, one commit per group
//   warp 2        TMA producer of the bf16 activations: one 128-row x 64-element box (128-byte rows,
//                 128-byte swizzle) per group into a ring of four slots, so that several groups are in
//                 flight (a converter that fetched its row from global memory itself, one group ahead,
//                 was bound by the round trip: 1230 clocks per group)
//   warps 4-7     converter: thread r owns row r of the tile; it reads the row's 64 bf16 of a group from
//                 the ring (the swizzle makes the 16-byte reads of neighbouring rows hit different banks),
//                 takes the amax, converts to e4m3 and writes the codes into the operand tile of the stage
//                 in the 128-byte-swizzle layout the tensor core reads; the group's scale goes into a
//                 ring in shared memory for the epilogue
//   warps 8-15    epilogue: promote every group's partial product from TMEM with the row's scale
//                 (packed FMAs, 128 accumulators per thread), then scale, add the bias and store
// The activations never exist as FP8 in global memory: this removes the quantizer pass and the
// round trip of its codes and scales.  Promotion per 64 K means the CUDA cores do one FMA per 64
// tensor-core MACs, which is what bounds this kernel (the packed-FMA pipe needs as long for a group as
// the tensor core).
//
// Every mbarrier wait is bounded (tc_common.cuh).
#include "tc_common.cuh"

namespace hkb {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BKS = 128;             // K per stage (bytes of e4m3 = one swizzle row)
constexpr int GK = 64;               // K per quantization group
constexpr int STAGES = 3;
constexpr int ASLOTS = 4;            // ring of bf16 activation groups (16 KB each)
constexpr int GROUP_M = 8;
constexpr int RING = 16;             // scale ring, in groups: the converter runs at most 2*STAGES + 2 groups ahead of the epilogue
constexpr int THREADS = 512;
// Registers per thread after setmaxnreg: first warpgroup (producers, MMA issuer), converter warpgroup, the two
// epilogue warpgroups.  The sum must stay within the CTA's allocation at launch (512 x 128): an increase beyond it
// never returns.
constexpr int kRegsWg0 = 40, kRegsConv = 104, kRegsEpi = 184;
static_assert(128 * (kRegsWg0 + kRegsConv + 2 * kRegsEpi) <= THREADS * 128, "setmaxnreg budget exceeds the CTA's registers");

struct PtgqParams {
    int M, N, K, batch;
    int m_blks, n_blks;
    const __nv_bfloat16* A;      // [batch, M, K]
    const float* b_scale;        // one float
    const __nv_bfloat16* bias;   // [batch, N] or null
    __nv_bfloat16* C;            // [batch, M, N]
    uint32_t* status;
};

struct Smem {
    static constexpr int kABytes = BM * BKS;          // 16 KB of codes
    static constexpr int kBBytes = BN * BKS;          // 32 KB
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kASlotBytes = BM * GK * 2;   // 16 KB of bf16
    static constexpr int kASlotOffset = STAGES * kStageBytes;
    static constexpr int kRingOffset = kASlotOffset + ASLOTS * kASlotBytes;
    static constexpr int kRingBytes = RING * BM * 4;
    static constexpr int kBarOffset = kRingOffset + kRingBytes;
    static constexpr int kNumBars = 2 * STAGES + 4 + 2 * ASLOTS;
    static constexpr int kDynamic = kBarOffset + kNumBars * 8 + 16 + 1024;
    static_assert(kDynamic <= 232448, "shared memory budget");
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ float2 ffma2(uint32_t a0, uint32_t a1, float2 s, float2 c) {
    return __ffma2_rn(make_float2(__uint_as_float(a0), __uint_as_float(a1)), s, c);
}
// 8 bf16 (one 16-byte chunk) * r -> 8 e4m3 bytes
__device__ __forceinline__ uint2 quant8(const uint4& v, float2 r2) {
    const float2 a = __fmul2_rn(bf16x2_to_f2(v.x), r2), b = __fmul2_rn(bf16x2_to_f2(v.y), r2);
    const float2 c = __fmul2_rn(bf16x2_to_f2(v.z), r2), d = __fmul2_rn(bf16x2_to_f2(v.w), r2);
    uint2 o;
    o.x = (uint32_t)cvt_e4m3x2(a.x, a.y) | ((uint32_t)cvt_e4m3x2(b.x, b.y) << 16);
    o.y = (uint32_t)cvt_e4m3x2(c.x, c.y) | ((uint32_t)cvt_e4m3x2(d.x, d.y) << 16);
    return o;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_ptgq_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PtgqParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + Smem::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    auto afull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 4 + a); };
    auto aempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 4 + ASLOTS + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::kBarOffset + Smem::kNumBars * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* const ring = reinterpret_cast<float*>(smem + Smem::kRingOffset);      // [RING][BM]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kstages = (p.K + BKS - 1) / BKS;      // a 64-wide tail group meets zero-filled weights
    const int tiles_per_batch = p.m_blks * p.n_blks;
    const int total_tiles = tiles_per_batch * p.batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 5);        // the producer's expect_tx arrive + four converter warps
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);
        }
        for (int a = 0; a < ASLOTS; ++a) {
            mbar_init(afull_bar(a), 1);
            mbar_init(aempty_bar(a), 4);      // the four converter warps
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        reg_dealloc<kRegsWg0>();
        if (warp == 0) {
            // ================= TMA producer (weights) =================
            if (elect_one()) {
                prefetch_tmap(&tmB);
                int s = 0;
                uint32_t ph = 0;
                bool ok = true;
                for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                    const int b = t / tiles_per_batch;
                    int mb, nb;
                    tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M, mb, nb);
                    for (int ks = 0; ks < kstages; ++ks) {
                        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, kErrWaitProducer)) { ok = false; break; }
                        mbar_arrive_expect_tx(full_bar(s), Smem::kBBytes);
                        tma_load_3d(smem_base + s * Smem::kStageBytes + Smem::kABytes, &tmB, full_bar(s), ks * BKS, nb * BN, b);
                        if (++s == STAGES) { s = 0; ph ^= 1; }
                    }
                }
            }
        } else if (warp == 1) {
            // ================= MMA issuer =================
            if (elect_one()) {
                constexpr uint32_t IDESC = idesc_f8(BM, BN);
                int s = 0;
                uint32_t ph = 0;
                int acc = 0;
                uint32_t acc_ph = 0;
                bool ok = true;
                for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                    for (int ks = 0; ks < kstages && ok; ++ks) {
                        if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                        tc_fence_after();
                        const uint32_t st = smem_base + s * Smem::kStageBytes;
                        const uint64_t da = smem_desc_sw128(st);
                        const uint64_t db = smem_desc_sw128(st + Smem::kABytes);
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                            tc_fence_after();
                            const uint32_t d_tmem = tmem_base + acc * BN;
#pragma unroll
                            for (int k = 0; k < 2; ++k)       // 32 bytes of K per MMA: +2 in the descriptor's address field
                                mma_f8(d_tmem, da + (uint64_t)((2 * g + k) * 2), db + (uint64_t)((2 * g + k) * 2), IDESC, k != 0);
                            tc_commit(tfull_bar(acc));
                            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                        }
                        if (ok) tc_commit(empty_bar(s));
                        if (++s == STAGES) { s = 0; ph ^= 1; }
                    }
                }
            }
        } else if (warp == 2) {
            // ================= TMA producer (bf16 activations, one 64-K group per slot) =================
            if (elect_one()) {
                prefetch_tmap(&tmA);
                int a = 0;
                uint32_t aph = 0;
                bool ok = true;
                for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                    const int b = t / tiles_per_batch;
                    int mb, nb;
                    tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M, mb, nb);
                    for (int g = 0; g < 2 * kstages; ++g) {
                        if (!mbar_wait(aempty_bar(a), aph ^ 1, abort_flag, p.status, kErrWaitProducer)) { ok = false; break; }
                        mbar_arrive_expect_tx(afull_bar(a), Smem::kASlotBytes);
                        // x in bytes of the bf16 row; a group past K (odd number of groups) reads as zeros
                        tma_load_3d(smem_base + Smem::kASlotOffset + a * Smem::kASlotBytes, &tmA, afull_bar(a), g * GK * 2, mb * BM, b);
                        if (++a == ASLOTS) { a = 0; aph ^= 1; }
                    }
                }
            }
        }
    } else if (warp < 8) {
        // ================= converter: bf16 rows -> e4m3 operand tile + scales =================
        reg_dealloc<kRegsConv>();
        const int r = (warp - 4) * 32 + lane;           // row of the tile
        const uint32_t sw = (uint32_t)(r & 7);          // 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r & 7)
        const float kInv448 = 1.0f / 448.0f;
        int s = 0;
        uint32_t ph = 0;
        int a = 0;
        uint32_t aph = 0;
        uint32_t gg = 0;                                // groups converted so far by this CTA
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            for (int ks = 0; ks < kstages && ok; ++ks) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, kErrWaitProducer))) { ok = false; break; }
                uint8_t* const arow_s = smem + s * Smem::kStageBytes + r * 128;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(afull_bar(a), aph, abort_flag, p.status, kErrWaitProducer))) { ok = false; break; }
                    const uint8_t* src = smem + Smem::kASlotOffset + a * Smem::kASlotBytes + r * 128;
                    uint4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = *reinterpret_cast<const uint4*>(src + (((uint32_t)j ^ sw) * 16));
                    __nv_bfloat162 mx = amax8_packed(v[0]);
#pragma unroll
                    for (int j = 1; j < 8; ++j) mx = __hmax2(mx, amax8_packed(v[j]));
                    const float m = fmaxf(hmax_halves(mx), 1e-10f);
                    const float a_scale = m * kInv448;
                    const float recip = __fdiv_rn(1.0f, a_scale);
                    const float2 r2 = make_float2(recip, recip);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint2 lo = quant8(v[2 * j], r2), hi = quant8(v[2 * j + 1], r2);
                        const uint32_t chunk = (uint32_t)(4 * g + j) ^ sw;
                        *reinterpret_cast<uint4*>(arow_s + chunk * 16) = make_uint4(lo.x, lo.y, hi.x, hi.y);
                    }
                    ring[((gg + g) % RING) * BM + r] = a_scale;
                    // The slot goes back to the TMA producer only now that every value read from it has been
                    // consumed: an arrive issued right behind the loads let the refill overtake them.
                    __syncwarp();
                    if (lane == 0) mbar_arrive(aempty_bar(a));
                    if (++a == ASLOTS) { a = 0; aph ^= 1; }
                }
                if (!ok) break;
                gg += 2;
                fence_proxy_async_smem();                  // the tensor core reads these generic-proxy writes
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar(s));
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else {
        // ================= epilogue =================
        reg_alloc<kRegsEpi>();
        const int ew = warp - 8;
        const int quarter = warp & 3;
        const int grp = ew >> 2;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float b_scale = __ldg(p.b_scale);
        const bool wide = (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 31) == 0;
        int acc = 0;
        uint32_t acc_ph = 0;
        uint32_t gg = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
            const int b = t / tiles_per_batch;
            int mb, nb;
            tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M, mb, nb);
            const int row = mb * BM + row_in_tile;
            const bool row_ok = row < p.M;
            const int col_base = nb * BN + grp * 128;
            float2 acc2[64];
#pragma unroll
            for (int j = 0; j < 64; ++j) acc2[j] = make_float2(0.0f, 0.0f);
            for (int g = 0; g < 2 * kstages; ++g, ++gg) {
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue))) { ok = false; break; }
                tc_fence_after();
                const float sc = ring[(gg % RING) * BM + row_in_tile];
                const float2 s2 = make_float2(sc, sc);
                const uint32_t t_addr = tmem_base + lane_addr + acc * BN + grp * 128;
                uint32_t ra[32], rb[32];
                tmem_ld32(t_addr, ra);
                tmem_ld_wait32(ra);
                tmem_ld32(t_addr + 32, rb);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc2[j] = ffma2(ra[2 * j], ra[2 * j + 1], s2, acc2[j]);
                tmem_ld_wait32(rb);
                tmem_ld32(t_addr + 64, ra);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc2[16 + j] = ffma2(rb[2 * j], rb[2 * j + 1], s2, acc2[16 + j]);
                tmem_ld_wait32(ra);
                tmem_ld32(t_addr + 96, rb);
#pragma unroll
                for (int j = 0; j < 16; ++j) acc2[32 + j] = ffma2(ra[2 * j], ra[2 * j + 1], s2, acc2[32 + j]);
                tmem_ld_wait32(rb);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(acc));
#pragma unroll
                for (int j = 0; j < 16; ++j) acc2[48 + j] = ffma2(rb[2 * j], rb[2 * j + 1], s2, acc2[48 + j]);
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
            if (ok && row_ok) {
                __nv_bfloat16* crow = p.C + ((int64_t)b * p.M + row) * p.N;
                const __nv_bfloat16* biasp = p.bias ? p.bias + (int64_t)b * p.N : nullptr;
#pragma unroll
                for (int c = 0; c < 128; c += 8) {            // N % 8 == 0: a group of 8 columns is all in or all out
                    const int col = col_base + c;
                    if (col < p.N) {
                        float bv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        if (biasp) unpack8(__ldg(reinterpret_cast<const uint4*>(biasp + col)), bv);
                        uint4 o;
                        o.x = pack_bf16(__fmaf_rn(acc2[c / 2 + 0].x, b_scale, bv[0]), __fmaf_rn(acc2[c / 2 + 0].y, b_scale, bv[1]));
                        o.y = pack_bf16(__fmaf_rn(acc2[c / 2 + 1].x, b_scale, bv[2]), __fmaf_rn(acc2[c / 2 + 1].y, b_scale, bv[3]));
                        o.z = pack_bf16(__fmaf_rn(acc2[c / 2 + 2].x, b_scale, bv[4]), __fmaf_rn(acc2[c / 2 + 2].y, b_scale, bv[5]));
                        o.w = pack_bf16(__fmaf_rn(acc2[c / 2 + 3].x, b_scale, bv[6]), __fmaf_rn(acc2[c / 2 + 3].y, b_scale, bv[7]));
                        *reinterpret_cast<uint4*>(crow + col) = o;
                    }
                }
            }
            (void)wide;
        }
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace
}  // namespace hkb

extern "C" int hkb_gemm_fp8_ptgq(const void* A, const void* B, const float* b_scale, void* C, const void* bias,
                                 int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(A && B && b_scale && C, HKB_ERR_BAD_ARG, "gemm_fp8_ptgq: null pointer");
    HKB_REQUIRE(batch >= 1 && M >= 1 && N >= 1 && K >= 1, HKB_ERR_BAD_SHAPE, "gemm_fp8_ptgq: empty problem");
    HKB_REQUIRE(K % GK == 0, HKB_ERR_BAD_SHAPE, "gemm_fp8_ptgq: K=%lld must be a multiple of %d", (long long)K, GK);
    HKB_REQUIRE(N % 8 == 0, HKB_ERR_BAD_SHAPE, "gemm_fp8_ptgq: N=%lld must be a multiple of 8", (long long)N);
    HKB_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31) && batch < 65536, HKB_ERR_BAD_SHAPE, "gemm_fp8_ptgq: dimension too large");
    HKB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && (!bias || aligned16(bias)) && ((uintptr_t)b_scale & 3) == 0,
                HKB_ERR_BAD_ALIGN, "gemm_fp8_ptgq: A, B, C and bias must be 16-byte aligned");
    PtgqParams p{};
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.m_blks = (int)((M + BM - 1) / BM);
    p.n_blks = (int)((N + BN - 1) / BN);
    p.A = (const __nv_bfloat16*)A;
    p.b_scale = b_scale;
    p.bias = (const __nv_bfloat16*)bias;
    p.C = (__nv_bfloat16*)C;
    int rc = status_word(&p.status);
    if (rc != HKB_OK) return rc;
    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, A, (uint64_t)K * 2, (uint64_t)M, (uint64_t)batch, BM);       // bf16 rows as bytes: a box is 64 elements wide
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)batch, BN);
    if (rc != HKB_OK) return rc;
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    HKB_CUDA(cudaFuncSetAttribute(gemm_fp8_ptgq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kDynamic));
    const int tiles = p.m_blks * p.n_blks * p.batch;
    gemm_fp8_ptgq_kernel<<<tiles < sms ? tiles : sms, THREADS, Smem::kDynamic, (cudaStream_t)stream>>>(tmA, tmB, p);
    note_kernel("gemm_fp8_ptgq_kernel");
    return check_launch("gemm_fp8_ptgq_kernel");
}
