// Tensor-core ceiling probe for sm_100a: every SM issues back-to-back tcgen05.mma instructions of
// the shapes the GEMMs use (128 x 256 per instruction; kind::f8f6f4 with K = 32, or
// kind::mxf4.block_scale with K = 64) on operand tiles that stay resident in shared memory.
// Nothing is loaded or stored in the loop, so the rate is what the tensor pipe delivers at the
// clock the power limit allows -- the denominator for "fraction of the FP8 / FP4 peak".
//
// One CTA per SM.  One thread issues MMAs in batches of four (one 128-byte swizzle row of K, as in
// the GEMM main loops) and commits each batch to one of four mbarriers; it runs three batches
// ahead of the oldest uncommitted one, which keeps the pipe fed while bounding what is in flight.
// The operand tiles hold pseudo-random bytes (no NaN codes), so the data paths toggle as they do
// in a real GEMM; the accumulator restarts with every batch.  Waits are bounded like everywhere else.
#include "tc_common.cuh"

namespace hkb {
namespace {

constexpr int kPeakTileA = 128 * 128;      // 128 rows x 128 bytes
constexpr int kPeakTileB = 256 * 128;      // 256 rows x 128 bytes
constexpr int kPeakSf = 3 * 1024;          // scale atoms for A (1 KB) and B (2 KB), FP4 only
constexpr int kPeakSmem = kPeakTileA + kPeakTileB + kPeakSf + 64 + 1024;

template <bool kFp4>
__global__ void __launch_bounds__(128, 1)
peak_mma_kernel(int64_t batches, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + kPeakTileA + kPeakTileB + kPeakSf;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + kPeakTileA + kPeakTileB + kPeakSf + 32);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int warp = threadIdx.x >> 5;

    // operand bytes: xorshift per word, top bit of each nibble pair cleared so that no e4m3 NaN (0x7F / 0xFF)
    // appears; FP4 scale bytes around 2^0
    uint32_t x = 0x9E3779B9u * (blockIdx.x * 128u + threadIdx.x + 1u);
    uint32_t* w = reinterpret_cast<uint32_t*>(smem);
    for (int i = threadIdx.x; i < (kPeakTileA + kPeakTileB) / 4; i += 128) {
        x ^= x << 13; x ^= x >> 17; x ^= x << 5;
        w[i] = x & 0xF7F7F7F7u;
    }
    for (int i = threadIdx.x; i < kPeakSf / 4; i += 128) w[(kPeakTileA + kPeakTileB) / 4 + i] = 0x7F7E7F80u;
    if (threadIdx.x == 0) {
        for (int b = 0; b < 4; ++b) mbar_init(bar_base + 8u * b, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();
    if (warp == 1) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 1 && elect_one()) {
        const uint64_t da = smem_desc_sw128(smem_base);
        const uint64_t db = smem_desc_sw128(smem_base + kPeakTileA);
        if constexpr (kFp4) {
            // scale atoms smem -> TMEM once (columns 480.. : A 8 columns, B 16 columns)
            for (int h = 0; h < 2; ++h) {
                tc_cp_sf(tmem_base + 480 + h * 4, smem_desc_sf(smem_base + kPeakTileA + kPeakTileB + h * 512));
                tc_cp_sf(tmem_base + 488 + h * 8, smem_desc_sf(smem_base + kPeakTileA + kPeakTileB + 1024 + h * 512));
                tc_cp_sf(tmem_base + 488 + h * 8 + 4, smem_desc_sf(smem_base + kPeakTileA + kPeakTileB + 2048 + h * 512));
            }
        }
        bool ok = true;
        for (int64_t i = 0; i < batches && ok; ++i) {
            const int b = (int)(i & 3);
            if (i >= 4) {
                // the batch that used this barrier four batches ago has retired
                ok = mbar_wait(bar_base + 8u * b, (uint32_t)(((i >> 2) - 1) & 1), abort_flag, status, kErrWaitMma);
                if (!ok) break;
            }
            const uint32_t d = tmem_base + (kFp4 ? 0u : (uint32_t)(i & 1) * 256u);   // FP4 keeps columns 480.. for its scale factors
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if constexpr (kFp4) {
                    const uint32_t h = k >> 1, sf_id = (k & 1) * 2;
                    mma_mxf4(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_mxf4(128, 256, sf_id, sf_id),
                             tmem_base + 480 + h * 4, tmem_base + 488 + h * 8, k != 0);
                } else {
                    mma_f8(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_f8(128, 256), k != 0);
                }
            }
            tc_commit(bar_base + 8u * b);
        }
        // drain: the last (up to four) batches
        for (int64_t i = batches > 4 ? batches - 4 : 0; i < batches && ok; ++i)
            ok = mbar_wait(bar_base + 8u * (uint32_t)(i & 3), (uint32_t)((i >> 2) & 1), abort_flag, status, kErrWaitMma);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace
}  // namespace hkb

extern "C" int hkb_debug_peak_mma(int kind, int64_t batches, double* flop_per_launch, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(kind == 0 || kind == 1, HKB_ERR_BAD_ARG, "peak_mma: kind must be 0 (FP8) or 1 (MXFP4)");
    HKB_REQUIRE(batches >= 1 && batches <= (1LL << 32), HKB_ERR_BAD_SHAPE, "peak_mma: batches out of range");
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    uint32_t* status = nullptr;
    int rc = status_word(&status);
    if (rc != HKB_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (kind == 0) {
        HKB_CUDA(cudaFuncSetAttribute(peak_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem));
        peak_mma_kernel<false><<<sms, 128, kPeakSmem, st>>>(batches, status);
        if (flop_per_launch) *flop_per_launch = 2.0 * 128 * 256 * 128 * (double)batches * sms;       // 4 x (128 x 256 x 32)
    } else {
        HKB_CUDA(cudaFuncSetAttribute(peak_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem));
        peak_mma_kernel<true><<<sms, 128, kPeakSmem, st>>>(batches, status);
        if (flop_per_launch) *flop_per_launch = 2.0 * 128 * 256 * 256 * (double)batches * sms;       // 4 x (128 x 256 x 64)
    }
    return check_launch("peak_mma_kernel");
}
