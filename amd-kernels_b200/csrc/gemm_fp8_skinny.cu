// Per-token-scale FP8 GEMM for skinny M (decode shapes, M <= 64): C[M,N] = (A @ B^T) * sa * sb.
//
// The problem is HBM-bound on the weight stream B[N,K]; the TMA engine of an SM moves a bounded
// number of 128-byte lines per clock, so what matters is that every SM streams the same number
// of weight lines and as few other lines as possible:
//
//  * Balance.  N is cut into 16-column units and the units are dealt out as (rounds) x (number
//    of SMs) tiles whose widths differ by at most one unit.  N = 28672 on 148 SMs: one tile per
//    SM, 132 of 192 and 16 of 208 columns -- no partial last round.
//
//  * Wide tiles.  A tile takes all the columns its SM owns in that round (up to 256), so the A
//    block of a K step (M x 128 bytes, re-read from L2 every step) is fetched once per 192..256
//    weight rows instead of once per 64: A is 8 % of the lines moved instead of 20 %.
//
//  * Spread over the DRAM channels.  Consecutive CTAs start their walk over K at different
//    K blocks, so the SMs do not pull the same byte columns of the weight rows in lockstep.
//
// A tile of w units is staged with 128-, 64- and 16-row TMA boxes placed back to back in shared
// memory and multiplied by one tcgen05.mma of N = 16 w (the instruction descriptor is built per
// tile).  Only the rows of A that exist are staged (a_box_rows, rounded to 8); the MMA still reads
// 128 rows from the A base, i.e. runs on into what follows -- those rows only feed accumulator
// rows >= M, which are never stored (a 16 KB tail pad keeps the overrun of the last stage inside
// the allocation).  Stage size and stage count are run-time values.
//
// Roles, bounded waits and teardown as in gemm_fp8.cu: warp 0 TMA producer, warp 1 TMEM
// allocator + MMA issuer, warps 2-5 epilogue (two TMEM accumulators of 256 columns).
#include "tc_common.cuh"

namespace hkb {
namespace {

constexpr int kMaxStages = 24;
constexpr int kBarBytes = 1024;           // barriers + tmem slot + abort flag live in the first KB
constexpr int kTailPad = 16 * 1024;       // the MMA reads 128 rows x 128 B from every A base
constexpr int kSmemLimit = 232448;        // 227 KB

struct SkinnyParams {
    int M, N, K;
    int a_box_rows;       // rows of A fetched per stage (multiple of 8, <= 64)
    int a_bytes;          // smem reserved for A per stage (multiple of 1024)
    int tiles, base, rem; // tile t is base + (t < rem) units wide and starts at unit t*base + min(t, rem)
    int stages, stage_bytes;
    int rot;              // K blocks by which consecutive CTAs are offset in their walk over K
    const float* sa;
    const float* sb;
    const __nv_bfloat16* bias;
    __nv_bfloat16* C;
    uint32_t* status;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&p);
}

// Tile t of the schedule (base, rem): width in 16-column units and first column.  The kernel
// parameters are read field by field (never through a pointer or reference to the struct), which
// keeps them in the constant bank.
#define TILE_WIDTH(t) (p.base + ((t) < p.rem ? 1 : 0))
#define TILE_COL0(t) (((t) * p.base + min((t), p.rem)) * 16)

__global__ void __launch_bounds__(192, 1)
gemm_fp8_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB128,
                       const __grid_constant__ CUtensorMap tmB64, const __grid_constant__ CUtensorMap tmB16,
                       const SkinnyParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t bar_base = smem_u32(smem);
    const uint32_t ring_base = bar_base + kBarBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + 8 * (2 * kMaxStages + 4));
    volatile uint32_t* abort_flag = tmem_slot + 1;
    constexpr uint32_t TMEM_COLS = 512;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.K / 128;
    const int kb0 = (int)(((long long)blockIdx.x * p.rot) % kblocks);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            prefetch_tmap(&tmA);
            prefetch_tmap(&tmB128);
            prefetch_tmap(&tmB64);
            prefetch_tmap(&tmB16);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x) {
                const int w = TILE_WIDTH(t);
                const int n0 = TILE_COL0(t);
                const uint32_t stage_tx = (uint32_t)p.a_box_rows * 128 + (uint32_t)w * 2048;
                int kb = kb0;
                for (int i = 0; i < kblocks; ++i, kb = (kb + 1 == kblocks ? 0 : kb + 1)) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, kErrWaitProducer)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t st = ring_base + s * p.stage_bytes;
                    tma_load_3d(st, &tmA, full_bar(s), kb * 128, 0, 0);
                    const uint32_t sb = st + p.a_bytes;
                    int r = 0;
                    for (; r + 8 <= w; r += 8) tma_load_3d(sb + r * 2048, &tmB128, full_bar(s), kb * 128, n0 + r * 16, 0);
                    for (; r + 4 <= w; r += 4) tma_load_3d(sb + r * 2048, &tmB64, full_bar(s), kb * 128, n0 + r * 16, 0);
                    for (; r < w; ++r) tma_load_3d(sb + r * 2048, &tmB16, full_bar(s), kb * 128, n0 + r * 16, 0);
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x) {
                const int w = TILE_WIDTH(t);
                const uint32_t idesc = idesc_f8(128, 16 * w);
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int i = 0; i < kblocks; ++i) {     // accumulation order follows the producer's walk
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = ring_base + s * p.stage_bytes;
                    const uint64_t da = smem_desc_sw128(st);
                    const uint64_t db = smem_desc_sw128(st + p.a_bytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k) mma_f8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i | k) != 0);
                    tc_commit(empty_bar(s));
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
                if (ok) {
                    tc_commit(tfull_bar(acc));
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const bool warp_has_rows = quarter * 32 < p.M;       // warp-uniform: quarters past M read no TMEM
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float sa = row_ok ? __ldg(p.sa + row) : 0.0f;
        __nv_bfloat16* crow = p.C + (int64_t)(row_ok ? row : 0) * p.N;
        int acc = 0;
        uint32_t acc_ph = 0;
        for (int t = blockIdx.x; t < p.tiles; t += gridDim.x) {
            const int w = TILE_WIDTH(t);
            const int n0 = TILE_COL0(t);
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue))) break;
            tc_fence_after();
            if (warp_has_rows) {
                const uint32_t t_addr = tmem_base + lane_addr + acc * 256;
                for (int u = 0; u < w; ++u) {
                    uint32_t r[16];
                    tmem_ld16(t_addr + u * 16, r);
                    tmem_ld_wait();
                    const int col0 = n0 + u * 16;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.sb + col0 + j));
                        v[j] = __uint_as_float(r[j]) * sa * s4.x;
                        v[j + 1] = __uint_as_float(r[j + 1]) * sa * s4.y;
                        v[j + 2] = __uint_as_float(r[j + 2]) * sa * s4.z;
                        v[j + 3] = __uint_as_float(r[j + 3]) * sa * s4.w;
                    }
                    if (p.bias) {
                        float b[16];
                        unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + col0)), *reinterpret_cast<float(*)[8]>(b));
                        unpack8(__ldg(reinterpret_cast<const uint4*>(p.bias + col0 + 8)), *reinterpret_cast<float(*)[8]>(b + 8));
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] += b[j];
                    }
                    if (row_ok) {
                        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                                     ::"l"(crow + col0), "r"(pack2(v[0], v[1])), "r"(pack2(v[2], v[3])), "r"(pack2(v[4], v[5])),
                                       "r"(pack2(v[6], v[7])), "r"(pack2(v[8], v[9])), "r"(pack2(v[10], v[11])),
                                       "r"(pack2(v[12], v[13])), "r"(pack2(v[14], v[15])) : "memory");
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*abort_flag) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

#undef TILE_WIDTH
#undef TILE_COL0

}  // namespace

// Host side: called by hkb_gemm_fp8_pts for M <= 64, batch == 1, N % 16 == 0 (arguments already validated).
int launch_gemm_fp8_skinny(const void* A, const void* B, void* C, const float* sa, const float* sb, const void* bias,
                           int64_t M, int64_t N, int64_t K, uint32_t* status, cudaStream_t st) {
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    SkinnyParams p{};
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.sa = sa; p.sb = sb; p.bias = (const __nv_bfloat16*)bias; p.C = (__nv_bfloat16*)C; p.status = status;
    p.a_box_rows = (int)((M + 7) / 8 * 8);
    p.a_bytes = (p.a_box_rows * 128 + 1023) / 1024 * 1024;
    const int units = (int)(N / 16);
    // rounds of tiles of up to 256 columns over all SMs; the units are dealt out evenly
    const int rounds = (units + 16 * sms - 1) / (16 * sms);
    p.tiles = units < rounds * sms ? units : rounds * sms;
    p.base = units / p.tiles;
    p.rem = units % p.tiles;
    const int maxw = p.base + (p.rem ? 1 : 0);
    HKB_REQUIRE(maxw >= 1 && maxw <= 16, HKB_ERR_UNSUPPORTED, "gemm_fp8 (skinny): internal tile width %d out of range", maxw);
    p.stage_bytes = p.a_bytes + maxw * 2048;
    p.stages = (kSmemLimit - 1024 - kBarBytes - kTailPad) / p.stage_bytes;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    HKB_REQUIRE(p.stages >= 2, HKB_ERR_UNSUPPORTED, "gemm_fp8 (skinny): not enough shared memory for two stages");
    p.rot = 17;      // odd, so consecutive CTAs spread over all K blocks; measured best of {0, 1, 5, 17}
    const int smem = 1024 + kBarBytes + p.stages * p.stage_bytes + kTailPad;
    CUtensorMap tmA, tmB128, tmB64, tmB16;
    int rc = make_tmap_bytes(&tmA, A, (uint64_t)K, (uint64_t)M, 1, (uint32_t)p.a_box_rows);
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB128, B, (uint64_t)K, (uint64_t)N, 1, 128);
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB64, B, (uint64_t)K, (uint64_t)N, 1, 64);
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB16, B, (uint64_t)K, (uint64_t)N, 1, 16);
    if (rc != HKB_OK) return rc;
    const cudaError_t e = cudaFuncSetAttribute(gemm_fp8_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", smem, cudaGetErrorString(e));
    const int grid = p.tiles < sms ? p.tiles : sms;
    gemm_fp8_skinny_kernel<<<grid, 192, smem, st>>>(tmA, tmB128, tmB64, tmB16, p);
    return check_launch("gemm_fp8_skinny_kernel");
}

}  // namespace hkb
