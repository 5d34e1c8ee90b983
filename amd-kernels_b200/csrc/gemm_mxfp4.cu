// MXFP4 x MXFP4 "NT" GEMM for sm_100a: e2m1 codes (two per byte, K-contiguous) with one e8m0
// scale per 32 K-elements on both operands, fp32 accumulation in TMEM, bf16 output.
//
// The tensor core applies the scales itself: tcgen05.mma kind::mxf4.block_scale.scale_vec::2X
// (K = 64 per instruction) reads the operand tiles from swizzled shared memory and the scale
// factors from tensor memory.  The scale factors arrive in the caller's row-major layout
// [rows, K/32]; a small pre-pass (sf_relayout_kernel) rewrites them into library scratch as
// 512-byte "atoms" (128 rows x 4 scale bytes = 128 rows x 128 K-elements; byte (r%32)*16 +
// (r/32)*4 + j for row r, scale j), atoms of one 128-row block consecutive along K.  A pipeline
// stage (256 K-elements) then needs one contiguous 1 KB bulk copy per 128 rows, and the MMA
// warp moves each atom smem -> TMEM with tcgen05.cp 32x128b.warpx4 right before the MMAs that
// use it.
//
// Roles, ring, bounded waits and teardown are those of the FP8 kernel (gemm_fp8.cu).
#include <cstdlib>

#include "tc_common.cuh"

#include <mutex>

namespace hkb {
namespace {

constexpr int BM = 128;
constexpr int BKB = 128;          // bytes of K per stage (= 256 e2m1 elements)
constexpr int GROUP_M = 8;
constexpr int SF_STAGE = 1024;    // scale bytes per 128 rows per stage (two atoms)

struct Mxfp4Params {
    int M, N, K, batch;
    int m_blks, n_blks;
    int katoms;                   // atoms per 128-row block in the scratch: K / 128 rounded up to even
    int sfa_rblks;                // 128-row blocks of A's scales per batch (incl. padding)
    int sfb_rblks;                // 128-row blocks of B's scales per batch (incl. padding)
    const uint8_t* sfa;           // re-laid-out scales of A: [batch, sfa_rblks, katoms, 512]
    const uint8_t* sfb;           // re-laid-out scales of B: [batch, sfb_rblks, katoms, 512]
    __nv_bfloat16* C;
    const __nv_bfloat16* c_a;     // fused multiply-add epilogue C = c_a * (A B^T) + c_b, both [batch, M, N]; null = plain
    const __nv_bfloat16* c_b;
    // grouped (MoE) mode, one-CTA kernels: M tile mb holds the sorted rows [mb*128, mb*128+128) of expert expert_ids[mb]
    // (-1: no expert, zeros are written); output row = sorted_ids[row] when < num_valid; B, its scales and b_scale_e per expert
    const int32_t* expert_ids;    // null = not grouped
    const int32_t* sorted_ids;
    int num_valid;
    const float* topk_w;          // per output row, or null
    const float* a_scale1;        // one float or null
    const float* b_scale_e;       // [E] or null
    __nv_bfloat16* c2;            // split-cat epilogue (sc_s1 > 0, one-CTA kernels, batch 1): column n = d*(s1+s2) + s goes to
    int sc_s1, sc_s2, sc_s3;      //   C[m, d, s] (row length s1+s3) when s < s1, else to c2[m, d, s-s1] (row length s2)
    uint32_t* status;
};

// Row-major e8m0 [batch, R, K/32] -> atoms [batch, ceil(R/128), katoms_pad, 512 B]; rows past R
// and atoms past K/128 are written as zero bytes (they meet zero-filled operand data).  One CTA
// moves 128 rows x 32 atoms through shared memory so that both the global reads (128 B per row)
// and writes (512 B per atom) are coalesced.
// Row indirection (MoE): with `ids`, row r of the output is source row ids[r] / ids_div when ids[r] < ids_valid and
// zero otherwise; R then counts output rows.
__global__ void __launch_bounds__(256)
sf_relayout_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int R, int katoms, int katoms_pad, int rblks,
                   const int32_t* __restrict__ ids = nullptr, int ids_div = 1, int ids_valid = 0) {
    __shared__ uint32_t tile[32][129];   // [atom in chunk][word in atom], padded
    const int b = blockIdx.z;
    const int rb = blockIdx.y;
    const int ka0 = blockIdx.x * 32;
    const int t = threadIdx.x;
    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(src) + (int64_t)b * R * katoms;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int idx = t + i * 256;
        const int r = idx >> 5, a = idx & 31;
        const int row = rb * 128 + r;
        uint32_t v = 0;
        if (row < R && ka0 + a < katoms) {
            int64_t srow = row;
            if (ids) { const int id = __ldg(ids + row); srow = id < ids_valid ? id / ids_div : -1; }
            if (srow >= 0) v = __ldg(s32 + srow * katoms + ka0 + a);
        }
        tile[a][(r & 31) * 4 + (r >> 5)] = v;
    }
    __syncthreads();
    uint32_t* d32 = reinterpret_cast<uint32_t*>(dst) + (((int64_t)b * rblks + rb) * katoms_pad + ka0) * 128;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int idx = t + i * 256;
        const int a = idx >> 7, w = idx & 127;
        if (ka0 + a < katoms_pad) d32[(int64_t)a * 128 + w] = tile[a][w];
    }
}

// Tile width.  The tensor core reads a K=64 slice of both operand tiles from shared memory per
// MMA, so a 128-wide tile saturates that path at ~63 % tensor activity; wider is better, but two
// accumulators of BN columns plus the scale factors must fit the 512 TMEM columns, which rules
// out 256.  192 = 6 x 32 columns works: 2 x 192 + 8 (SFA) + 16 (SFB) = 408.  A 192-wide tile
// starts 0 or 64 rows into a 128-row scale atom of B, so two atoms are staged per K atom and the
// MMA's scale-factor address is advanced by 0 or 2 TMEM columns (one column = 32 rows) to the
// tile's first row group.  (The offset has to stay even: a 224-wide tile, whose offsets are
// 0..3 columns, faulted with "misaligned address".)
template <int BN>
struct Cfg {
    static_assert(BN == 128 || BN == 192, "supported tile widths");
    static constexpr int kStages = BN == 128 ? 6 : 5;
    static constexpr int kSfbAtoms = BN == 128 ? 1 : 2;            // 128-row scale atoms staged per K atom
    static constexpr int kABytes = BM * BKB;
    static constexpr int kBBytes = BN * BKB;
    static constexpr int kSfaOff = kABytes + kBBytes;
    static constexpr int kSfbOff = kSfaOff + SF_STAGE;
    static constexpr int kStageBytes = kSfbOff + kSfbAtoms * SF_STAGE;   // 34 KB / 43 KB, multiples of 1024
    static constexpr int kBarOffset = kStages * kStageBytes;
    static constexpr int kNumBars = 2 * kStages + 4;
    static constexpr int kDynamic = kBarOffset + kNumBars * 8 + 16 + 1024;
    static constexpr uint32_t kTmemCols = 512;                     // power of two >= 2*BN + 8 + 8*kSfbAtoms
    static constexpr uint32_t kTmemSfa = 2 * BN;
    static constexpr uint32_t kTmemSfb = 2 * BN + 8;
    static_assert(kTmemSfb + 8 * kSfbAtoms <= 512, "TMEM budget");
    static_assert(kDynamic <= 232448, "shared memory budget");
};

template <int BN>
__global__ void __launch_bounds__(192, 1)
gemm_mxfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Mxfp4Params p) {
    using Smem = Cfg<BN>;
    constexpr int STAGES = Smem::kStages;
    constexpr uint32_t TMEM_COLS = Smem::kTmemCols, TMEM_SFA = Smem::kTmemSfa, TMEM_SFB = Smem::kTmemSfb;
    constexpr int SFB_ATOMS = Smem::kSfbAtoms;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + Smem::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::kBarOffset + Smem::kNumBars * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kstages = (p.K + 255) / 256;            // a 128-element tail reads zero-filled data and zero scales
    const int tiles_per_batch = p.m_blks * p.n_blks;
    const int total_tiles = tiles_per_batch * p.batch;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
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
            prefetch_tmap(&tmB);
            constexpr uint32_t stage_tx = Smem::kABytes + Smem::kBBytes + (1 + SFB_ATOMS) * SF_STAGE;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int b = t / tiles_per_batch;
                int mb, nb;
                tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M, mb, nb);
                int bb = b;                                   // batch coordinate of B and its scales: the expert in grouped mode
                if (p.expert_ids) {
                    bb = __ldg(p.expert_ids + mb);
                    if (bb < 0) continue;
                }
                const uint8_t* sfa_row = p.sfa + ((int64_t)b * p.sfa_rblks + mb) * p.katoms * 512;
                // first 128-row scale atom that the tile's B rows touch
                const int atom0 = (nb * BN) >> 7;
                const uint8_t* sfb_row = p.sfb + ((int64_t)bb * p.sfb_rblks + atom0) * p.katoms * 512;
                for (int ks = 0; ks < kstages; ++ks) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, kErrWaitProducer)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t st = smem_base + s * Smem::kStageBytes;
                    tma_load_3d(st, &tmA, full_bar(s), ks * BKB, mb * BM, b);
                    tma_load_3d(st + Smem::kABytes, &tmB, full_bar(s), ks * BKB, nb * BN, bb);
                    bulk_load(st + Smem::kSfaOff, sfa_row + (int64_t)ks * SF_STAGE, SF_STAGE, full_bar(s));
#pragma unroll
                    for (int r = 0; r < SFB_ATOMS; ++r)
                        bulk_load(st + Smem::kSfbOff + r * SF_STAGE, sfb_row + ((int64_t)r * p.katoms * 512) + (int64_t)ks * SF_STAGE,
                                  SF_STAGE, full_bar(s));
                    if (++s == STAGES) { s = 0; ph ^= 1; }
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
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                if (p.expert_ids) {
                    int mb_, nb_;
                    tile_coords(t, p.m_blks, p.n_blks, GROUP_M, mb_, nb_);
                    if (__ldg(p.expert_ids + mb_) < 0) continue;
                }
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                // 32-row group inside the first staged scale atom at which this tile's B rows start
                int sf_off = 0;
                if constexpr (SFB_ATOMS > 1) {
                    const int b_ = t / tiles_per_batch;
                    int mb_, nb_;
                    tile_coords(t - b_ * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M, mb_, nb_);
                    sf_off = ((nb_ * BN) >> 5) & 3;          // 0 or 2 for BN = 192
                }
                for (int ks = 0; ks < kstages; ++ks) {
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = smem_base + s * Smem::kStageBytes;
                    const uint64_t da = smem_desc_sw128(st);
                    const uint64_t db = smem_desc_sw128(st + Smem::kABytes);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {      // the two 128-K atoms of this stage
                        tc_cp_sf(tmem_base + TMEM_SFA + h * 4, smem_desc_sf(st + Smem::kSfaOff + h * 512));
#pragma unroll
                        for (int r = 0; r < SFB_ATOMS; ++r)
                            tc_cp_sf(tmem_base + TMEM_SFB + (h * SFB_ATOMS + r) * 4,
                                     smem_desc_sf(st + Smem::kSfbOff + r * SF_STAGE + h * 512));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {      // 4 x K=64 (32 bytes of each 128-byte row)
                        const uint32_t h = k >> 1, sf_id = (k & 1) * 2;
                        mma_mxf4(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_mxf4(BM, BN, sf_id, sf_id),
                                 tmem_base + TMEM_SFA + h * 4, tmem_base + TMEM_SFB + h * SFB_ATOMS * 4 + sf_off, (ks | k) != 0);
                    }
                    tc_commit(empty_bar(s));
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (ok) {
                    tc_commit(tfull_bar(acc));
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        int acc = 0;
        uint32_t acc_ph = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
            const int b = t / tiles_per_batch;
            int mb, nb;
            tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M, mb, nb);
            int row = mb * BM + row_in_tile;
            bool row_ok = row < p.M;
            float row_scale = 1.0f;
            if (p.expert_ids) {
                // grouped mode: this sorted row's output row and its scale (per-tensor x per-expert x routing weight)
                const int e = __ldg(p.expert_ids + mb);
                const int id = row_ok ? __ldg(p.sorted_ids + row) : p.num_valid;
                row_ok = id < p.num_valid;
                row = row_ok ? id : 0;
                if (e < 0) {
                    // no expert for this block: the rows it names get zeros (nothing was accumulated for them)
                    if (row_ok) {
                        for (int c = 0; c < BN; c += 8)
                            if (nb * BN + c < p.N) *reinterpret_cast<uint4*>(p.C + (int64_t)row * p.N + nb * BN + c) = make_uint4(0, 0, 0, 0);
                    }
                    continue;
                }
                row_scale = (p.a_scale1 ? __ldg(p.a_scale1) : 1.0f) * (p.b_scale_e ? __ldg(p.b_scale_e + e) : 1.0f);
                if (p.topk_w && row_ok) row_scale *= __ldg(p.topk_w + id);
            }
            const int64_t row_off = ((int64_t)b * p.M + (row_ok ? row : 0)) * p.N;
            __nv_bfloat16* crow = p.C + row_off;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue))) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + lane_addr + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(t_addr + c, r);
                tmem_ld_wait();
                if (row_ok) {
                    const int col0 = nb * BN + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col0 + j < p.N) {
                            if (p.c_a) {
                                float ca[8], cb[8];
                                unpack8(__ldg(reinterpret_cast<const uint4*>(p.c_a + row_off + col0 + j)), ca);
                                unpack8(__ldg(reinterpret_cast<const uint4*>(p.c_b + row_off + col0 + j)), cb);
#pragma unroll
                                for (int i = 0; i < 8; ++i) r[j + i] = __float_as_uint(__fmaf_rn(ca[i], __uint_as_float(r[j + i]), cb[i]));
                            }
                            if (p.expert_ids) {
#pragma unroll
                                for (int i = 0; i < 8; ++i) r[j + i] = __float_as_uint(__uint_as_float(r[j + i]) * row_scale);
                            }
                            uint4 o;
                            __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(r[j + 0]), __uint_as_float(r[j + 1]));
                            __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                            __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                            __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                            o.x = *reinterpret_cast<uint32_t*>(&q0);
                            o.y = *reinterpret_cast<uint32_t*>(&q1);
                            o.z = *reinterpret_cast<uint32_t*>(&q2);
                            o.w = *reinterpret_cast<uint32_t*>(&q3);
                            __nv_bfloat16* dst = crow + col0 + j;
                            if (p.sc_s1) {          // split-cat: 8 columns never straddle a boundary (sizes are multiples of 16)
                                const int per = p.sc_s1 + p.sc_s2, col = col0 + j;
                                const int d = col / per, sidx = col - d * per;
                                const int64_t rd = (int64_t)row * (p.N / per) + d;
                                dst = sidx < p.sc_s1 ? p.C + rd * (p.sc_s1 + p.sc_s3) + sidx : p.c2 + rd * p.sc_s2 + (sidx - p.sc_s1);
                            }
                            *reinterpret_cast<uint4*>(dst) = o;
                        }
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

// ---- CTA pairs -------------------------------------------------------------------------------
// Large problems: a cluster of two CTAs works on one 256 x 192 tile (tcgen05 cta_group::2).
// Each CTA stages its own 128 rows of A, its own half (96 rows) of the tile's B rows, the scale
// atoms of its own A rows and the scale atoms of ALL the tile's B rows: a third less operand
// traffic from L2 per SM, which is what bounds the single-CTA kernel (its 148 SMs together pull
// ~17.5 TB/s from L2).  The leader (even CTA) issues the scale copies and the MMAs for both CTAs;
// completion bytes of both CTAs' loads are credited to the leader's barriers (tensor-map loads
// in their cta_group::2 form, hence the scale atoms also travel through a -- linear -- tensor map);
// commits are multicast to both CTAs; both epilogues release the accumulator on the leader's
// barrier with a remote arrive.  No multicast loads anywhere.
struct PairCfg {
    static constexpr int BN = 192;
    static constexpr int kStages = 7;
    static constexpr int kABytes = BM * BKB;                  // 16 KB
    static constexpr int kBBytes = (BN / 2) * BKB;            // 12 KB: this CTA's half of the B rows
    static constexpr int kSfaOff = kABytes + kBBytes;
    static constexpr int kSfbOff = kSfaOff + SF_STAGE;
    static constexpr int kStageBytes = kSfbOff + 2 * SF_STAGE;   // 31 KB
    static constexpr int kBarOffset = kStages * kStageBytes;
    static constexpr int kNumBars = 2 * kStages + 4;
    static constexpr int kDynamic = kBarOffset + kNumBars * 8 + 16 + 1024;
    static constexpr uint32_t kTmemCols = 512;
    static constexpr uint32_t kTmemSfa = 2 * BN;
    static constexpr uint32_t kTmemSfb = 2 * BN + 8;
    static_assert(kStageBytes % 1024 == 0, "stages keep the 1024-byte swizzle alignment");
    static_assert(kDynamic <= 232448, "shared memory budget");
};

struct Mxfp4PairParams {
    Mxfp4Params g;                // m_blks counts 256-row blocks here; A's scale blocks are addressed as 2*mb + rank
};

__global__ void __launch_bounds__(192, 1)
gemm_mxfp4_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSfa, const __grid_constant__ CUtensorMap tmSfb,
                       const Mxfp4PairParams pp) {
    using Smem = PairCfg;
    constexpr int BN = Smem::BN;
    constexpr int STAGES = Smem::kStages;
    constexpr uint32_t TMEM_COLS = Smem::kTmemCols, TMEM_SFA = Smem::kTmemSfa, TMEM_SFB = Smem::kTmemSfb;
    const Mxfp4Params& p = pp.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + Smem::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::kBarOffset + Smem::kNumBars * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int kstages = (p.K + 255) / 256;
    const int tiles_per_batch = p.m_blks * p.n_blks;
    const int total_tiles = tiles_per_batch * p.batch;
    const int tile0 = (int)(blockIdx.x >> 1);
    const int tile_step = (int)(gridDim.x >> 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);          // the leader hears both CTAs' four epilogue warps
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();        // the partner's barriers and TMEM exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            prefetch_tmap(&tmA);
            prefetch_tmap(&tmB);
            prefetch_tmap(&tmSfa);
            prefetch_tmap(&tmSfb);
            // the leader's full barrier counts the bytes of both CTAs' loads
            constexpr uint32_t stage_tx = 2u * (Smem::kABytes + Smem::kBBytes + 3 * SF_STAGE);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step) {
                const int b = t / tiles_per_batch;
                int mb, nb;
                tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M / 2, mb, nb);
                // scratch rows (256 bytes each) of this CTA's A-scale block and of the tile's two B-scale atoms
                const int64_t sfa_row0 = (((int64_t)b * p.sfa_rblks + 2 * mb + (int)rank) * p.katoms) * 2;
                const int atom0 = (nb * BN) >> 7;
                const int64_t sfb_row0 = (((int64_t)b * p.sfb_rblks + atom0) * p.katoms) * 2;
                for (int ks = 0; ks < kstages; ++ks) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, kErrWaitProducer)) { ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t st = smem_base + s * Smem::kStageBytes;
                    tma_load_3d_pair(st, &tmA, full_bar(s), ks * BKB, mb * 2 * BM + (int)rank * BM, b);
                    tma_load_3d_pair(st + Smem::kABytes, &tmB, full_bar(s), ks * BKB, nb * BN + (int)rank * (BN / 2), b);
                    tma_load_3d_pair(st + Smem::kSfaOff, &tmSfa, full_bar(s), 0, (int32_t)(sfa_row0 + (int64_t)ks * 4), 0);
                    tma_load_3d_pair(st + Smem::kSfbOff, &tmSfb, full_bar(s), 0, (int32_t)(sfb_row0 + (int64_t)ks * 4), 0);
                    tma_load_3d_pair(st + Smem::kSfbOff + SF_STAGE, &tmSfb, full_bar(s), 0,
                                     (int32_t)(sfb_row0 + (int64_t)p.katoms * 2 + (int64_t)ks * 4), 0);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step) {
                if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int b_ = t / tiles_per_batch;
                int mb_, nb_;
                tile_coords(t - b_ * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M / 2, mb_, nb_);
                const int sf_off = ((nb_ * BN) >> 5) & 3;          // 0 or 2: first 32-row group of the tile inside its first atom
                for (int ks = 0; ks < kstages; ++ks) {
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kErrWaitMma)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t st = smem_base + s * Smem::kStageBytes;
                    const uint64_t da = smem_desc_sw128(st);
                    const uint64_t db = smem_desc_sw128(st + Smem::kABytes);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {      // the two 128-K atoms of this stage
                        tc_cp_sf_pair(tmem_base + TMEM_SFA + h * 4, smem_desc_sf(st + Smem::kSfaOff + h * 512));
#pragma unroll
                        for (int r = 0; r < 2; ++r)
                            tc_cp_sf_pair(tmem_base + TMEM_SFB + (h * 2 + r) * 4, smem_desc_sf(st + Smem::kSfbOff + r * SF_STAGE + h * 512));
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t h = k >> 1, sf_id = (k & 1) * 2;
                        mma_mxf4_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_mxf4(2 * BM, BN, sf_id, sf_id),
                                      tmem_base + TMEM_SFA + h * 4, tmem_base + TMEM_SFB + h * 2 * 4 + sf_off, (ks | k) != 0);
                    }
                    tc_commit_pair(empty_bar(s), 3);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (ok) {
                    tc_commit_pair(tfull_bar(acc), 3);
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    } else {
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        int acc = 0;
        uint32_t acc_ph = 0;
        for (int t = tile0; t < total_tiles; t += tile_step) {
            const int b = t / tiles_per_batch;
            int mb, nb;
            tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, GROUP_M / 2, mb, nb);
            const int row = mb * 2 * BM + (int)rank * BM + row_in_tile;
            const bool row_ok = row < p.M;
            const int64_t row_off = ((int64_t)b * p.M + (row_ok ? row : 0)) * p.N;
            __nv_bfloat16* crow = p.C + row_off;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue))) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + lane_addr + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(t_addr + c, r);
                tmem_ld_wait();
                if (row_ok) {
                    const int col0 = nb * BN + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col0 + j < p.N) {
                            if (p.c_a) {
                                float ca[8], cb[8];
                                unpack8(__ldg(reinterpret_cast<const uint4*>(p.c_a + row_off + col0 + j)), ca);
                                unpack8(__ldg(reinterpret_cast<const uint4*>(p.c_b + row_off + col0 + j)), cb);
#pragma unroll
                                for (int i = 0; i < 8; ++i) r[j + i] = __float_as_uint(__fmaf_rn(ca[i], __uint_as_float(r[j + i]), cb[i]));
                            }
                            uint4 o;
                            __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(r[j + 0]), __uint_as_float(r[j + 1]));
                            __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                            __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                            __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                            o.x = *reinterpret_cast<uint32_t*>(&q0);
                            o.y = *reinterpret_cast<uint32_t*>(&q1);
                            o.z = *reinterpret_cast<uint32_t*>(&q2);
                            o.w = *reinterpret_cast<uint32_t*>(&q3);
                            *reinterpret_cast<uint4*>(crow + col0 + j) = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_bar(acc), 0);
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();        // the partner is done with this CTA's shared memory, barriers and TMEM
    if (warp == 1) {
        if (*abort_flag) {
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// Rows of 128-row scale blocks that the tensor-core layout of an operand with R rows holds per
// batch: every block a kernel variant may address (CTA pairs address A's blocks as 2*mb + rank;
// 192-wide tiles stage up to two atoms past the last one).
inline int sf_tc_rblks(int64_t R) { return 2 * (int)((R + 255) / 256) + 2; }
inline int sf_tc_katoms(int64_t K) { return ((int)(K / 128) + 1) & ~1; }

int launch_sf_relayout(const void* src, void* dst, int64_t batch, int64_t R, int64_t K, cudaStream_t st) {
    const int katoms_src = (int)(K / 128), katoms = sf_tc_katoms(K), rblks = sf_tc_rblks(R);
    HKB_REQUIRE(rblks <= 65535 && batch <= 65535, HKB_ERR_BAD_SHAPE, "mxfp4 scale layout: too many row blocks");
    dim3 g((unsigned)((katoms + 31) / 32), (unsigned)rblks, (unsigned)batch);
    sf_relayout_kernel<<<g, 256, 0, st>>>((const uint8_t*)src, (uint8_t*)dst, (int)R, katoms_src, katoms, rblks);
    return check_launch("sf_relayout_kernel");
}

// MoE pre-pass: output row r <- source row ids[r] / div when ids[r] < valid, zeros otherwise.  One warp per row.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ ids, int div, int valid, uint8_t* __restrict__ xg,
                   int64_t rows, int row_bytes) {
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const int id = __ldg(ids + r);
    uint4* dst = reinterpret_cast<uint4*>(xg + r * row_bytes);
    if (id < valid && id >= 0) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)(id / div) * row_bytes);
        for (int i = lane; i < row_bytes / 16; i += 32) dst[i] = __ldg(src + i);
    } else {
        for (int i = lane; i < row_bytes / 16; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
    }
}

// sfa_tc / sfb_tc: the scale pointer already is in the tensor-core layout (hkb_mxfp4_sf_to_tc or
// hkb_quant_mxfp4_tc); otherwise it is row-major [batch, rows, K/32] and is re-laid-out into
// per-(device, stream) scratch first.
struct SplitCat { void* c2; int64_t s1, s2, s3; };      // C is c1 [M, D, s1+s3], c2 [M, D, s2], N = D*(s1+s2)

int gemm_mxfp4_impl(const void* A, const void* B, void* C, const void* sfa, const void* sfb, bool sfa_tc, bool sfb_tc,
                    const void* c_a, const void* c_b, int64_t batch, int64_t M, int64_t N, int64_t K, void* stream,
                    const SplitCat* sc = nullptr) {
    HKB_REQUIRE(A && B && C && sfa && sfb, HKB_ERR_BAD_ARG, "gemm_mxfp4: null pointer");
    HKB_REQUIRE(batch >= 1 && M >= 1 && N >= 1 && K >= 1, HKB_ERR_BAD_SHAPE, "gemm_mxfp4: empty problem");
    HKB_REQUIRE(K % 128 == 0, HKB_ERR_BAD_SHAPE, "gemm_mxfp4: K=%lld must be a multiple of 128", (long long)K);
    HKB_REQUIRE(N % 8 == 0, HKB_ERR_BAD_SHAPE, "gemm_mxfp4: N=%lld must be a multiple of 8", (long long)N);
    HKB_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31) && batch < 65536, HKB_ERR_BAD_SHAPE, "gemm_mxfp4: dimension too large");
    HKB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && ((uintptr_t)sfa & 3) == 0 && ((uintptr_t)sfb & 3) == 0,
                HKB_ERR_BAD_ALIGN, "gemm_mxfp4: A, B, C must be 16-byte and the scale arrays 4-byte aligned");
    HKB_REQUIRE((!sfa_tc || aligned16(sfa)) && (!sfb_tc || aligned16(sfb)), HKB_ERR_BAD_ALIGN,
                "gemm_mxfp4: scale factors in the tensor-core layout must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    Mxfp4Params p{};
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.m_blks = (int)((M + BM - 1) / BM);
    // wide tiles when there are enough of them to fill the SMs twice over
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    const bool wide = (int64_t)p.m_blks * ((N + 191) / 192) * batch >= 2LL * sms;
    const int bn = wide ? 192 : 128;
    p.n_blks = (int)((N + bn - 1) / bn);
    p.sfa_rblks = sf_tc_rblks(M);
    p.sfb_rblks = sf_tc_rblks(N);
    p.katoms = sf_tc_katoms(K);
    p.C = (__nv_bfloat16*)C;
    p.c_a = (const __nv_bfloat16*)c_a;
    p.c_b = (const __nv_bfloat16*)c_b;
    if (sc) {
        HKB_REQUIRE(batch == 1 && !c_a, HKB_ERR_UNSUPPORTED, "gemm_mxfp4_split_cat: 2-D operands, no other epilogue at the same time");
        HKB_REQUIRE(sc->c2 && aligned16(sc->c2), HKB_ERR_BAD_ALIGN, "gemm_mxfp4_split_cat: c2 must be 16-byte aligned");
        HKB_REQUIRE(sc->s1 > 0 && sc->s2 > 0 && sc->s3 >= 0 && sc->s1 % 16 == 0 && sc->s2 % 16 == 0 && sc->s3 % 16 == 0 &&
                    N % (sc->s1 + sc->s2) == 0 && sc->s1 + sc->s2 + sc->s3 < (1LL << 30),
                    HKB_ERR_BAD_SHAPE, "gemm_mxfp4_split_cat: S1, S2, S3 must be multiples of 16 and N a multiple of S1+S2");
        p.c2 = (__nv_bfloat16*)sc->c2; p.sc_s1 = (int)sc->s1; p.sc_s2 = (int)sc->s2; p.sc_s3 = (int)sc->s3;
    }
    int rc = status_word(&p.status);
    if (rc != HKB_OK) return rc;

    // CTA pairs on 256 x 192 tiles when there is at least half a wave of them (HKB_MXFP4_PAIRS=0: never)
    static const bool pairs_on = [] { const char* v = getenv("HKB_MXFP4_PAIRS"); return !(v && v[0] == '0'); }();
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 191) / 192) * batch;
    const bool pair = pairs_on && wide && M > 128 && pair_tiles >= sms / 2 && sms >= 2 && !sc;     // the split-cat store lives in the one-CTA kernels

    const size_t sfa_bytes = (size_t)batch * p.sfa_rblks * p.katoms * 512;
    const size_t sfb_bytes = (size_t)batch * p.sfb_rblks * p.katoms * 512;
    const void *sfa_sw = sfa, *sfb_sw = sfb;
    if (!sfa_tc) {
        void* buf = nullptr;
        rc = scratch_get(SCRATCH_SFA, st, sfa_bytes, &buf);
        if (rc != HKB_OK) return rc;
        rc = launch_sf_relayout(sfa, buf, batch, M, K, st);
        if (rc != HKB_OK) return rc;
        sfa_sw = buf;
    }
    if (!sfb_tc) {
        void* buf = nullptr;
        rc = scratch_get(SCRATCH_SFB, st, sfb_bytes, &buf);
        if (rc != HKB_OK) return rc;
        rc = launch_sf_relayout(sfb, buf, batch, N, K, st);
        if (rc != HKB_OK) return rc;
        sfb_sw = buf;
    }
    p.sfa = (const uint8_t*)sfa_sw;
    p.sfb = (const uint8_t*)sfb_sw;

    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, A, (uint64_t)K / 2, (uint64_t)M, (uint64_t)batch, BM);
    if (rc != HKB_OK) return rc;
    if (pair) {
        Mxfp4PairParams pp{};
        pp.g = p;
        pp.g.m_blks = (int)((M + 255) / 256);
        CUtensorMap tmSfa, tmSfb;
        rc = make_tmap_bytes(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)batch, PairCfg::BN / 2);
        if (rc != HKB_OK) return rc;
        rc = make_tmap_linear1k(&tmSfa, sfa_sw, sfa_bytes);
        if (rc != HKB_OK) return rc;
        rc = make_tmap_linear1k(&tmSfb, sfb_sw, sfb_bytes);
        if (rc != HKB_OK) return rc;
        cudaError_t e = cudaFuncSetAttribute(gemm_mxfp4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kDynamic);
        HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        int clusters = sms / 2;
        if (pair_tiles < clusters) clusters = (int)pair_tiles;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * clusters);
        cfg.blockDim = dim3(192);
        cfg.dynamicSmemBytes = PairCfg::kDynamic;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, gemm_mxfp4_pair_kernel, tmA, tmB, tmSfa, tmSfb, pp);
        HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "launch of gemm_mxfp4_pair_kernel failed: %s", cudaGetErrorString(e));
        note_kernel("gemm_mxfp4_pair_kernel<256x192>");
        return check_launch("gemm_mxfp4_pair_kernel");
    }
    rc = make_tmap_bytes(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)batch, (uint32_t)bn);
    if (rc != HKB_OK) return rc;
    const int tiles = p.m_blks * p.n_blks * p.batch;
    const int grid = tiles < sms ? tiles : sms;
    if (wide) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_mxfp4_kernel<192>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<192>::kDynamic);
        HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        gemm_mxfp4_kernel<192><<<grid, 192, Cfg<192>::kDynamic, st>>>(tmA, tmB, p);
        note_kernel("gemm_mxfp4_kernel<192>");
    } else {
        const cudaError_t e = cudaFuncSetAttribute(gemm_mxfp4_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::kDynamic);
        HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
        gemm_mxfp4_kernel<128><<<grid, 192, Cfg<128>::kDynamic, st>>>(tmA, tmB, p);
        note_kernel("gemm_mxfp4_kernel<128>");
    }
    return check_launch("gemm_mxfp4_kernel");
}

}  // namespace
}  // namespace hkb

extern "C" int hkb_gemm_mxfp4(const void* A, const void* B, void* C, const void* sfa, const void* sfb,
                              int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
    return hkb::gemm_mxfp4_impl(A, B, C, sfa, sfb, false, false, nullptr, nullptr, batch, M, N, K, stream);
}

extern "C" int hkb_moe_gemm_mxfp4(const void* A, const void* B, void* C, const void* A_mx_scale, const void* B_mx_scale,
                                  const float* A_scale, const float* B_scale, const float* topk_weights,
                                  const int32_t* sorted_token_ids, const int32_t* expert_ids, int64_t tokens, int64_t num_padded,
                                  int64_t E, int64_t N, int64_t K, int64_t num_valid_tokens, int64_t top_k, int mul_routed_weight,
                                  void* stream) {
    using namespace hkb;
    HKB_REQUIRE(A && B && C && A_mx_scale && B_mx_scale && sorted_token_ids && expert_ids, HKB_ERR_BAD_ARG, "moe_gemm_mxfp4: null pointer");
    HKB_REQUIRE(!mul_routed_weight || topk_weights, HKB_ERR_BAD_ARG, "moe_gemm_mxfp4: mul_routed_weight needs topk_weights");
    HKB_REQUIRE(tokens >= 1 && num_padded >= 1 && num_padded % BM == 0 && E >= 1 && E < 65536 && top_k >= 1 && num_valid_tokens >= 0 &&
                num_padded < (1LL << 31) && tokens < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31),
                HKB_ERR_BAD_SHAPE, "moe_gemm_mxfp4: bad problem size (the sorted row list is padded to multiples of %d)", BM);
    HKB_REQUIRE(K % 128 == 0 && N % 8 == 0, HKB_ERR_BAD_SHAPE, "moe_gemm_mxfp4: K must be a multiple of 128 and N of 8");
    HKB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && ((uintptr_t)A_mx_scale & 3) == 0 && ((uintptr_t)B_mx_scale & 3) == 0,
                HKB_ERR_BAD_ALIGN, "moe_gemm_mxfp4: A, B, C must be 16-byte and the scale arrays 4-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    Mxfp4Params p{};
    p.M = (int)num_padded; p.N = (int)N; p.K = (int)K; p.batch = 1;
    p.m_blks = (int)(num_padded / BM);
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    const bool wide = (int64_t)p.m_blks * ((N + 191) / 192) >= 2LL * sms;
    const int bn = wide ? 192 : 128;
    p.n_blks = (int)((N + bn - 1) / bn);
    p.sfa_rblks = sf_tc_rblks(num_padded);
    p.sfb_rblks = sf_tc_rblks(N);
    p.katoms = sf_tc_katoms(K);
    p.C = (__nv_bfloat16*)C;
    p.expert_ids = expert_ids; p.sorted_ids = sorted_token_ids; p.num_valid = (int)num_valid_tokens;
    p.topk_w = mul_routed_weight ? topk_weights : nullptr;
    p.a_scale1 = A_scale; p.b_scale_e = B_scale;
    int rc = status_word(&p.status);
    if (rc != HKB_OK) return rc;
    // expert-sorted copy of the activation codes, and both operands' scales in the tensor core's layout (per-stream scratch)
    void *ag = nullptr, *sfa_sw = nullptr, *sfb_sw = nullptr;
    rc = scratch_get(SCRATCH_ROWS, st, (size_t)num_padded * (K / 2), &ag);
    if (rc != HKB_OK) return rc;
    rc = scratch_get(SCRATCH_SFA, st, (size_t)p.sfa_rblks * p.katoms * 512, &sfa_sw);
    if (rc != HKB_OK) return rc;
    rc = scratch_get(SCRATCH_SFB, st, (size_t)E * p.sfb_rblks * p.katoms * 512, &sfb_sw);
    if (rc != HKB_OK) return rc;
    gather_rows_kernel<<<(unsigned)((num_padded + 7) / 8), 256, 0, st>>>((const uint8_t*)A, sorted_token_ids, (int)top_k, (int)num_valid_tokens,
                                                                         (uint8_t*)ag, num_padded, (int)(K / 2));
    {
        const int katoms_src = (int)(K / 128);
        dim3 ga((unsigned)((p.katoms + 31) / 32), (unsigned)p.sfa_rblks, 1);
        sf_relayout_kernel<<<ga, 256, 0, st>>>((const uint8_t*)A_mx_scale, (uint8_t*)sfa_sw, (int)num_padded, katoms_src, p.katoms, p.sfa_rblks,
                                               sorted_token_ids, (int)top_k, (int)num_valid_tokens);
    }
    rc = check_launch("moe_gemm_mxfp4 pre-pass");
    if (rc != HKB_OK) return rc;
    rc = launch_sf_relayout(B_mx_scale, sfb_sw, E, N, K, st);
    if (rc != HKB_OK) return rc;
    p.sfa = (const uint8_t*)sfa_sw;
    p.sfb = (const uint8_t*)sfb_sw;
    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, ag, (uint64_t)K / 2, (uint64_t)num_padded, 1, BM);
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)E, (uint32_t)bn);
    if (rc != HKB_OK) return rc;
    const int tiles = p.m_blks * p.n_blks;
    const int grid = tiles < sms ? tiles : sms;
    if (wide) {
        HKB_CUDA(cudaFuncSetAttribute(gemm_mxfp4_kernel<192>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<192>::kDynamic));
        gemm_mxfp4_kernel<192><<<grid, 192, Cfg<192>::kDynamic, st>>>(tmA, tmB, p);
        note_kernel("gemm_mxfp4_kernel<192> (grouped)");
    } else {
        HKB_CUDA(cudaFuncSetAttribute(gemm_mxfp4_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::kDynamic));
        gemm_mxfp4_kernel<128><<<grid, 192, Cfg<128>::kDynamic, st>>>(tmA, tmB, p);
        note_kernel("gemm_mxfp4_kernel<128> (grouped)");
    }
    return check_launch("gemm_mxfp4_kernel");
}

extern "C" int hkb_gemm_mxfp4_split_cat(const void* A, const void* B, const void* sfa, const void* sfb, const void* y,
                                        void* c1, void* c2, int64_t M, int64_t N, int64_t K, int64_t S1, int64_t S2,
                                        int64_t S3, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(c1 && c2 && (S3 == 0 || y), HKB_ERR_BAD_ARG, "gemm_mxfp4_split_cat: null pointer");
    const SplitCat sc{c2, S1, S2, S3};
    int rc = gemm_mxfp4_impl(A, B, c1, sfa, sfb, false, false, nullptr, nullptr, 1, M, N, K, stream, &sc);
    if (rc != HKB_OK || S3 == 0) return rc;
    return launch_concat_cols(y, c1, M * (N / (S1 + S2)), S3, S1 + S3, S1, (cudaStream_t)stream);
}

extern "C" int64_t hkb_mxfp4_sf_tc_bytes(int64_t batch, int64_t rows, int64_t K) {
    if (batch < 1 || rows < 1 || K < 128 || K % 128) return 0;
    return batch * (int64_t)hkb::sf_tc_rblks(rows) * hkb::sf_tc_katoms(K) * 512;
}

extern "C" int hkb_mxfp4_sf_to_tc(const void* sf, void* sf_tc, int64_t batch, int64_t rows, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(sf && sf_tc, HKB_ERR_BAD_ARG, "mxfp4_sf_to_tc: null pointer");
    HKB_REQUIRE(batch >= 1 && rows >= 1 && K >= 128 && K % 128 == 0 && rows < (1LL << 31) && K < (1LL << 31), HKB_ERR_BAD_SHAPE,
                "mxfp4_sf_to_tc: need batch, rows >= 1 and K a positive multiple of 128");
    HKB_REQUIRE(((uintptr_t)sf & 3) == 0 && aligned16(sf_tc), HKB_ERR_BAD_ALIGN,
                "mxfp4_sf_to_tc: sf must be 4-byte and sf_tc 16-byte aligned");
    return launch_sf_relayout(sf, sf_tc, batch, rows, K, (cudaStream_t)stream);
}

extern "C" int hkb_gemm_mxfp4_tc(const void* A, const void* B, void* C, const void* sfa, int sfa_is_tc, const void* sfb,
                                 int sfb_is_tc, int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
    return hkb::gemm_mxfp4_impl(A, B, C, sfa, sfb, sfa_is_tc != 0, sfb_is_tc != 0, nullptr, nullptr, batch, M, N, K, stream);
}

extern "C" int hkb_gemm_mxfp4_mul_add(const void* A, const void* B, void* C, const void* sfa, const void* sfb,
                                      const void* c_a, const void* c_b, int64_t M, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(c_a && c_b, HKB_ERR_BAD_ARG, "gemm_mxfp4_mul_add: null c_a / c_b");
    HKB_REQUIRE(aligned16(c_a) && aligned16(c_b), HKB_ERR_BAD_ALIGN, "gemm_mxfp4_mul_add: c_a and c_b must be 16-byte aligned");
    return gemm_mxfp4_impl(A, B, C, sfa, sfb, false, false, c_a, c_b, 1, M, N, K, stream);
}


// ---------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some callers must not trigger a device allocation at call time: code that runs inside a
// memory-pool or arena discipline where every byte is accounted for up front, latency-critical
// serving loops where cudaMalloc's implicit device synchronisation is unacceptable, and hosts
// that hand this library a device on which they have already claimed all memory.  For them the
// re-laid-out scale factors live in a fixed array that is part of the library image: every GPU
// that loads libhkb200.so reserves it until the process exits.
//
//   * Limit: the scales of both operands, padded to 128-row blocks and an even number of
//     128-wide K atoms, must fit kStaticSfBytes (8 MiB); e.g. M + N <= 32768 rows at K = 8192.
//     Larger problems are refused with HKB_ERR_BAD_SHAPE; nothing is launched.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and sets the kernel's shared-memory attribute.  Make that first call
//     outside any stream capture.
//   * Every call on a device shares the one array, which keeps the previous call's contents.
//     Nothing in it has to start at zero: the re-layout pass rewrites every byte the GEMM reads,
//     including the zero padding of partial row blocks and of an odd K atom.  Two calls that can
//     overlap on the GPU (different streams, or different host threads) race on the array; run
//     them in one stream or order them with events.
//   * Bounded-wait timeouts of this variant are recorded in a word of the same image
//     (g_static_status); hkb_check_status() reads and clears it together with the ordinary one,
//     without allocating.
//   * It always runs the one-CTA kernel on 128 x 128 tiles (the 192-wide and CTA-pair kernels of
//     hkb_gemm_mxfp4 address padded scale blocks that would cut the size limit further), so on
//     large problems it is the slower of the two entry points.
namespace hkb {
namespace {

constexpr size_t kStaticSfBytes = (size_t)8 << 20;
static __device__ __align__(256) uint8_t g_static_sf[kStaticSfBytes];
static __device__ __align__(256) uint32_t g_static_status[1];

struct StaticSlot {
    uint8_t* sf = nullptr;       // device address of g_static_sf on this device
    uint32_t* status = nullptr;  // device address of g_static_status on this device
};
StaticSlot g_static_slot[64];
std::mutex g_static_mu;

// Device addresses of the static arrays for the CURRENT device (looked up once per device).
int static_addresses(StaticSlot* out) {
    int dev = 0;
    HKB_CUDA(cudaGetDevice(&dev));
    HKB_REQUIRE(dev >= 0 && dev < 64, HKB_ERR_CUDA, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    StaticSlot& s = g_static_slot[dev];
    if (!s.sf) {
        void* p = nullptr;
        void* q = nullptr;
        // In host code the array names are host-side handles, not device addresses: ask the runtime.
        HKB_CUDA(cudaGetSymbolAddress(&p, g_static_sf));
        HKB_CUDA(cudaGetSymbolAddress(&q, g_static_status));
        HKB_CUDA(cudaFuncSetAttribute(gemm_mxfp4_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::kDynamic));
        s.status = static_cast<uint32_t*>(q);
        s.sf = static_cast<uint8_t*>(p);
    }
    *out = s;
    return HKB_OK;
}

}  // namespace

uint32_t* static_status_peek() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_static_mu);
    return g_static_slot[dev].status;
}

}  // namespace hkb

extern "C" int hkb_gemm_mxfp4_static(const void* A, const void* B, void* C, const void* sfa, const void* sfb,
                                     int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(A && B && C && sfa && sfb, HKB_ERR_BAD_ARG, "gemm_mxfp4_static: null pointer");
    HKB_REQUIRE(batch >= 1 && M >= 1 && N >= 1 && K >= 1, HKB_ERR_BAD_SHAPE, "gemm_mxfp4_static: empty problem");
    HKB_REQUIRE(K % 128 == 0, HKB_ERR_BAD_SHAPE, "gemm_mxfp4_static: K=%lld must be a multiple of 128", (long long)K);
    HKB_REQUIRE(N % 8 == 0, HKB_ERR_BAD_SHAPE, "gemm_mxfp4_static: N=%lld must be a multiple of 8", (long long)N);
    HKB_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31) && batch < 65536, HKB_ERR_BAD_SHAPE,
                "gemm_mxfp4_static: dimension too large");
    HKB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && ((uintptr_t)sfa & 3) == 0 && ((uintptr_t)sfb & 3) == 0,
                HKB_ERR_BAD_ALIGN, "gemm_mxfp4_static: A, B, C must be 16-byte and the scale arrays 4-byte aligned");
    Mxfp4Params p{};
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.m_blks = (int)((M + BM - 1) / BM);
    p.n_blks = (int)((N + 127) / 128);
    p.sfa_rblks = p.m_blks;
    p.sfb_rblks = p.n_blks;
    const int katoms_src = (int)(K / 128);
    p.katoms = (katoms_src + 1) & ~1;
    p.C = (__nv_bfloat16*)C;
    const size_t sfa_bytes = (size_t)batch * p.m_blks * p.katoms * 512;
    const size_t sfb_bytes = (size_t)batch * p.n_blks * p.katoms * 512;
    HKB_REQUIRE(sfa_bytes + sfb_bytes <= kStaticSfBytes, HKB_ERR_BAD_SHAPE,
                "gemm_mxfp4_static: the scale factors need %zu bytes of scratch but the built-in array holds %zu "
                "(limit: batch * (ceil(M/128) + ceil(N/128)) * ceil(K/256) * 1024 <= 8 MiB); use hkb_gemm_mxfp4",
                sfa_bytes + sfb_bytes, kStaticSfBytes);
    HKB_REQUIRE(p.m_blks <= 65535 && p.n_blks <= 65535, HKB_ERR_BAD_SHAPE, "gemm_mxfp4_static: too many row blocks");
    StaticSlot slot;
    int rc = static_addresses(&slot);
    if (rc != HKB_OK) return rc;
    p.status = slot.status;
    uint8_t* sfa_sw = slot.sf;
    uint8_t* sfb_sw = slot.sf + sfa_bytes;          // sfa_bytes is a multiple of 1024
    p.sfa = sfa_sw;
    p.sfb = sfb_sw;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 ga((unsigned)((p.katoms + 31) / 32), (unsigned)p.m_blks, (unsigned)batch);
    sf_relayout_kernel<<<ga, 256, 0, st>>>((const uint8_t*)sfa, sfa_sw, (int)M, katoms_src, p.katoms, p.m_blks);
    dim3 gb((unsigned)((p.katoms + 31) / 32), (unsigned)p.n_blks, (unsigned)batch);
    sf_relayout_kernel<<<gb, 256, 0, st>>>((const uint8_t*)sfb, sfb_sw, (int)N, katoms_src, p.katoms, p.n_blks);
    rc = check_launch("sf_relayout_kernel");
    if (rc != HKB_OK) return rc;
    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, A, (uint64_t)K / 2, (uint64_t)M, (uint64_t)batch, BM);
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)batch, 128);
    if (rc != HKB_OK) return rc;
    const int tiles = p.m_blks * p.n_blks * p.batch;
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    gemm_mxfp4_kernel<128><<<tiles < sms ? tiles : sms, 192, Cfg<128>::kDynamic, st>>>(tmA, tmB, p);
    note_kernel("gemm_mxfp4_kernel<128> (static scratch)");
    return check_launch("gemm_mxfp4_kernel");
}
