// FP8 (e4m3fn x e4m3fn -> fp32 -> bf16) "NT" GEMMs for sm_100a on the 5th-generation tensor
// cores: tcgen05.mma kind::f8f6f4 with the accumulator in tensor memory (TMEM), operands
// staged by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a multi-stage shared-memory
// ring, warp-specialised roles and a persistent tile loop.
//
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + MMA issuer (one elected lane)
//   warps 2..   epilogue: TMEM -> registers (tcgen05.ld) -> scale -> bf16 -> global
//               (block-scale kernels start the epilogue at warp 4, so that the first warpgroup
//               can hand registers to the epilogue warpgroups, which keep 128 fp32 accumulators
//               per thread)
//
// Two scale schemes share the pipeline:
//   * per-token / per-channel (kBlockScale = false): the whole K extent accumulates in TMEM
//     (two accumulator buffers, so the epilogue of tile i overlaps the main loop of tile i+1);
//     the epilogue multiplies by sa[m] * sb[n] and adds the optional bias.
//   * block scales (kBlockScale = true): scales are arbitrary fp32 per 128-wide K block, which
//     the tensor core cannot apply, so every K block is a fresh 128 x BN partial product in one
//     of two TMEM buffers and the epilogue warps promote it: acc += partial * (sa[m,kb] * sb[kb,n])
//     in registers, while the tensor core already works on the next K block.
//
// Every mbarrier wait is bounded (tc_common.cuh): on a timeout the CTA records an error bit in
// the device status word (read by hkb_check_status), stops issuing work, and still frees TMEM.
#include "tc_common.cuh"

#include <cstdlib>
#include <mutex>

namespace hkb {

// ---- host: tensor-map encoder -----------------------------------------------------------------
namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_encode_once;
void load_encoder() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeFn>(fn);
    });
}
}  // namespace

int make_tmap_bytes(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                    uint64_t batch, uint32_t box_rows) {
    load_encoder();
    HKB_REQUIRE(g_encode != nullptr, HKB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    HKB_REQUIRE(aligned16(base) && row_bytes % 16 == 0, HKB_ERR_BAD_ALIGN,
                "TMA operands need a 16-byte aligned base and row pitch (pitch %llu bytes)", (unsigned long long)row_bytes);
    const cuuint64_t dims[3] = {row_bytes, rows, batch};
    const cuuint64_t strides[2] = {row_bytes, row_bytes * rows};
    const cuuint32_t box[3] = {128, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HKB_REQUIRE(r == CUDA_SUCCESS, HKB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return HKB_OK;
}

int make_tmap_linear1k(CUtensorMap* map, const void* base, uint64_t bytes) {
    load_encoder();
    HKB_REQUIRE(g_encode != nullptr, HKB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    HKB_REQUIRE(aligned16(base) && bytes % 1024 == 0 && bytes > 0, HKB_ERR_BAD_ALIGN, "linear TMA view needs a 16-byte aligned base and a multiple of 1 KB");
    const cuuint64_t dims[3] = {256, bytes / 256, 1};
    const cuuint64_t strides[2] = {256, bytes};
    const cuuint32_t box[3] = {256, 4, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HKB_REQUIRE(r == CUDA_SUCCESS, HKB_ERR_CUDA, "cuTensorMapEncodeTiled (linear) failed with CUresult %d", (int)r);
    return HKB_OK;
}

namespace {

constexpr int BM = 128;        // tile rows = TMEM lanes
constexpr int BK = 128;        // bytes (= e4m3 elements) of K per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;     // K per tcgen05.mma for 8-bit operands
#define GROUP_M (p.group_m)     /* M blocks per group of the tile order (runtime: 8 by default) */

struct GemmParams {
    int M, N, K, batch;
    int m_blks, n_blks;
    int a_box_rows;            // rows of A that TMA actually fetches per tile (<= BM)
    const float* sa;           // pts: [batch, M]      blockscale: [M, K/128]
    const float* sb;           // pts: [batch, N]      blockscale: [K/128, N/gn]
    const __nv_bfloat16* bias; // pts only: [batch, N] or null
    __nv_bfloat16* C;          // [batch, M, N]
    int gn;                    // blockscale: 1 or 128
    const __nv_bfloat16* c_a;  // blockscale only: fused epilogue C = c_a * gemm + c_b, both [M, N]; null = plain
    const __nv_bfloat16* c_b;
    int64_t ldc;               // row pitch of C in elements (N unless the result goes into a slab of a wider matrix)
    __nv_bfloat16* peer[7];    // blockscale, gn = 128 only: further copies of the result (same pitch), e.g. the
    int n_peer;                //   same slab of the other GPUs' matrices, written with plain stores from the epilogue
    const int32_t* expt_data;  // grouped (MoE) mode (kOut == 3): per M tile (expert | block << 16) or -1; rows of expert e are
    const int32_t* expt_hist;  //   [expt_offs[e], expt_offs[e] + expt_hist[e]) of A / a_scale / C; B, sb and bias_f32 are per expert
    const int32_t* expt_offs;
    const float* bias_f32;     //   [E, N] or null
    __nv_bfloat16* c2;         // split-cat epilogue (kOut == 2): column n = d*(s1+s2) + s of the result goes to
    int sc_s1, sc_s2, sc_s3;   //   C[m, d, s] (row length s1+s3) when s < s1, else to c2[m, d, s-s1] (row length s2)
    int group_m;               // tile order: walk N inside groups of this many M blocks
    uint32_t* status;
    uint64_t wait_ns;          // limit of every mbarrier wait (kWaitLimitNs in production)
    int skip_kblock;           // >= 0: the producer leaves this K block of its first tile unloaded (wait-limit probe only)
    unsigned long long* trace; // timeline build (kOut == 4) only: [grid][kTraceEvents][kTraceKb] SM clock readings
};

// Timeline build of the block-scale kernel: every CTA records, for the first kTraceKb K blocks of its third tile,
// when (SM clock) the MMA thread saw the operands (event 0), issued the MMAs (1) and had them issued (3), when the
// producer got the stage back (2), and when each of the eight epilogue warps released the accumulator buffer
// (4 + warp) and saw the partial product (12 + warp).
constexpr int kTraceEvents = 20;
constexpr int kTraceKb = 64;

// kPair: two CTAs (a cluster of 2) share one 256 x BN tile; each stages its own 128 rows of A
// and its own half of B's BN rows.
// AROWS < 128 (skinny-M problems): only AROWS rows of A are staged per stage, which frees smem
// for more stages (more weight bytes in flight).  The MMA still reads 128 rows from the A base,
// i.e. it runs on into whatever follows; those rows only feed accumulator rows >= M, which are
// never stored.  kTailPad keeps that overrun of the last stage inside the allocation.
// SCALE_THREADS > 0 (block-scale epilogue with one weight scale per 128 columns): a scale area
// behind the barriers holds, per epilogue thread and for two chunks of kScaleChunk K blocks, the
// activation scales of the thread's row (thread-private float4 slots) and, per epilogue warp, the
// chunk's weight scales.
// kScaleChunk: K blocks per chunk of staged scales (at most 32: one lane per K block; 32 by default, 8 measured
// slower and 16 equal; the scatter kernels take 16 to make room for their output staging).
// kStageOut: bytes behind the scales in which the epilogue warps transpose their output block (scatter mode).
template <int BN, int STAGES, bool kPair = false, int AROWS = BM, int SCALE_THREADS = 0, int kScaleChunk = 32, int kStageOut = 0>
struct SmemLayout {
    static constexpr int kABytes = AROWS * BK;
    static constexpr int kTailPad = (BM - AROWS) * BK;
    static constexpr int kBRows = kPair ? BN / 2 : BN;
    static constexpr int kBBytes = kBRows * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOffset = STAGES * kStageBytes;
    // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], relay[2] (CTA pairs with block scales), then tmem base + abort flag
    static constexpr int kNumBars = 2 * STAGES + 6;
    static constexpr int kScaleOffset = kBarOffset + ((kNumBars * 8 + 16 + 15) / 16) * 16;
    static constexpr int kSaBytes = 2 * (kScaleChunk / 4) * SCALE_THREADS * 16;     // [2][chunk/4][thread] float4
    static constexpr int kSbBytes = 2 * (SCALE_THREADS / 32) * kScaleChunk * 4;     // [2][warp][chunk] float
    static constexpr int kScaleBytes = kSaBytes + kSbBytes;
    static constexpr int kStageOutOffset = ((kScaleOffset + kScaleBytes + 127) / 128) * 128;
    static constexpr int kTotal = kStageOut > 0 ? kStageOutOffset + kStageOut : SCALE_THREADS > 0 ? kScaleOffset + kScaleBytes
                                                    : kBarOffset + (kNumBars * 8 + 16 > kTailPad ? kNumBars * 8 + 16 : kTailPad);
    static constexpr int kDynamic = kTotal + 1024;   // slack for the manual 1024-byte alignment
    static_assert(kDynamic <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
};

__device__ __forceinline__ void store_bf16x8(__nv_bfloat16* dst, const float* v) {
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(v[6], v[7]);
    o.x = *reinterpret_cast<uint32_t*>(&p0);
    o.y = *reinterpret_cast<uint32_t*>(&p1);
    o.z = *reinterpret_cast<uint32_t*>(&p2);
    o.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(dst) = o;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&p);
}
// 16 bf16 (32 bytes) with one 256-bit store: a warp whose lanes write different rows pays one
// L1 wavefront per row and per instruction, so wider stores halve that cost.
__device__ __forceinline__ void store_bf16x16(__nv_bfloat16* dst, const float* v) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(dst), "r"(pack_bf16(v[0], v[1])), "r"(pack_bf16(v[2], v[3])), "r"(pack_bf16(v[4], v[5])),
                   "r"(pack_bf16(v[6], v[7])), "r"(pack_bf16(v[8], v[9])), "r"(pack_bf16(v[10], v[11])),
                   "r"(pack_bf16(v[12], v[13])), "r"(pack_bf16(v[14], v[15])) : "memory");
}
// v[0..NV) (consecutive columns of one row, starting at element offset `off` of the [M,N] arrays)
// -> c_a * v + c_b in fp32: the fused multiply-add epilogue.
template <int NV>
__device__ __forceinline__ void mul_add_cols(const __nv_bfloat16* c_a, const __nv_bfloat16* c_b, int64_t off, float* v) {
#pragma unroll
    for (int j = 0; j < NV; j += 8) {
        float ca[8], cb[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(c_a + off + j)), ca);
        unpack8(__ldg(reinterpret_cast<const uint4*>(c_b + off + j)), cb);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j + i] = __fmaf_rn(ca[i], v[j + i], cb[i]);
    }
}

// Split-cat epilogue: where 16 consecutive result columns starting at `col` (a multiple of 16; s1, s2 and
// s3 are multiples of 16, so a chunk never straddles a boundary) of row `row` go.
__device__ __forceinline__ __nv_bfloat16* split_cat_ptr(const GemmParams& p, int row, int col) {
    const int per = p.sc_s1 + p.sc_s2;
    const int d = col / per, s = col - d * per;
    const int64_t rd = (int64_t)row * (p.N / per) + d;
    return s < p.sc_s1 ? p.C + rd * (p.sc_s1 + p.sc_s3) + s : p.c2 + rd * p.sc_s2 + (s - p.sc_s1);
}

// Grouped (MoE) mode: M tile `mt` of the tile list -> its expert, first row and row count.
struct GroupedTile { int e, row0, rows; bool skip; };
__device__ __forceinline__ GroupedTile grouped_tile(const GemmParams& p, int mt) {
    const int ed = __ldg(p.expt_data + mt);
    GroupedTile g;
    g.skip = ed < 0;
    g.e = g.skip ? 0 : (ed & 0xFFFF);
    const int blk = g.skip ? 0 : (ed >> 16);
    g.row0 = g.skip ? 0 : __ldg(p.expt_offs + g.e) + blk * BM;
    g.rows = g.skip ? 0 : min(BM, __ldg(p.expt_hist + g.e) - blk * BM);
    if (g.rows <= 0 || g.row0 >= p.M) g.skip = true;
    return g;
}

// Writes 32 consecutive columns of one output row.  `wide` = rows are 32-byte aligned (N % 16 == 0);
// otherwise 16-byte stores (N % 8 == 0 is guaranteed).
__device__ __forceinline__ void store_row32(__nv_bfloat16* crow, int col0, int N, const float* v, bool wide) {
    if (wide) {
#pragma unroll
        for (int j = 0; j < 32; j += 16)
            if (col0 + j < N) store_bf16x16(crow + col0 + j, v + j);
    } else {
#pragma unroll
        for (int j = 0; j < 32; j += 8)
            if (col0 + j < N) store_bf16x8(crow + col0 + j, v + j);
    }
}

template <int BN, bool kBlockScale, bool kPair = false>
constexpr int gemm_threads() { return ((kBlockScale || kPair) ? 128 : 64) + 128 * (BN == 256 ? 2 : 1); }

__device__ __forceinline__ float2 ffma2(uint32_t a0, uint32_t a1, float2 s, float2 c) {
    return __ffma2_rn(make_float2(__uint_as_float(a0), __uint_as_float(a1)), s, c);
}

// kOut (block-scale): 0 = plain [M, N] result; 1 = the result also goes to p.n_peer further destinations
// (the other GPUs' copies of the assembled output; 128-column weight-scale groups only); 2 = split-cat;
// 3 = grouped (MoE): the M tiles come from a device-side list (expert, block), weights, weight scales and the
// fp32 bias are per expert, rows of A / C are sorted by expert (128-column weight-scale groups only);
// 4 = plain result plus the hand-off timeline in p.trace (diagnostic build, same code otherwise).
template <int BN, int STAGES, bool kBlockScale, bool kGn128, bool kPair = false, int AROWS = BM, int kOut = 0>
__global__ void __launch_bounds__(gemm_threads<BN, kBlockScale, kPair>(), 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    constexpr int EPI_GROUPS = (BN == 256) ? 2 : 1;     // groups of 4 warps; each owns BN/EPI_GROUPS columns
    constexpr int kScaleChunk = kOut == 1 ? 16 : 32;
    constexpr int kStageOut = kOut == 1 ? 4 * EPI_GROUPS * 4096 : 0;       // 32 rows x 128 bytes per epilogue warp
    using L = SmemLayout<BN, STAGES, kPair, AROWS, (kBlockScale && kGn128) ? 128 * EPI_GROUPS : 0, kScaleChunk, kStageOut>;
    constexpr bool kGrouped = kOut == 3;
    constexpr bool kTrace = kOut == 4;
    static_assert(!kGrouped || (kBlockScale && kGn128 && !kPair), "grouped mode: block scales, 128-column groups, one CTA");
    static_assert(!kPair || BN == 256, "CTA pairs work on 256 x 256 tiles");
    constexpr int EPI_WARPS = 4 * EPI_GROUPS;
    constexpr int COLS_PER_GROUP = BN / EPI_GROUPS;
    constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
    constexpr uint32_t IDESC = idesc_f8(kPair ? 2 * BM : BM, BN);
    constexpr int EPI_WARP0 = (kBlockScale || kPair) ? 4 : 2;      // first epilogue warp
    constexpr bool kRegSplit = kBlockScale && BN == 256; // 3 warpgroups: trade registers between them
    constexpr int kRegsWg0 = 128, kRegsEpi = 184;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    auto relay_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 4 + a); };
    // CTA pairs with block scales: the eight epilogue warps of a CTA release a TMEM buffer on a local barrier and
    // warp 2 forwards ONE arrive per CTA to the leader's barrier, instead of sixteen arrives crossing the cluster
    constexpr bool kRelay = kPair && kBlockScale;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.K / BK;
    auto trace_at = [&](int ev, int kb, bool on, long long clk) {
        if constexpr (kTrace) {
            if (on && kb < kTraceKb) p.trace[((size_t)blockIdx.x * kTraceEvents + ev) * kTraceKb + kb] = (unsigned long long)clk;
        }
    };
    // pair mode: p.m_blks counts 256-row blocks, a "tile" belongs to the cluster, CTA `rank` owns
    // rows [rank*128, rank*128+128) of it and stages rows [rank*128, ..) of the tile's B block
    const uint32_t rank = kPair ? cluster_ctarank() : 0u;
    const int tiles_per_batch = p.m_blks * p.n_blks;
    const int total_tiles = tiles_per_batch * p.batch;
    const int tile0 = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tile_step = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int TILE_M = kPair ? 2 * BM : BM;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kRelay ? 2 : kPair ? 2 * EPI_WARPS : EPI_WARPS);   // the leader hears both CTAs' epilogues
            mbar_init(relay_bar(a), EPI_WARPS);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (kPair) tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        else tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) { __syncwarp(); cluster_sync_all(); }   // the partner's barriers and TMEM exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < EPI_WARP0) {
    // First warpgroup (producer, MMA issuer, two idle warps): 168 -> 128 registers.  Fewer costs throughput: with
    // 96 the kernel was 2 % slower, with 56 13 % (the MMA issuer's loop is on the critical path of every K block).
    // The sum after re-allocation must stay within the CTA's allocation at launch (threads x 168): an increase
    // beyond it never returns.
    static_assert(!kRegSplit || 128 * kRegsWg0 + 256 * kRegsEpi <= 384 * 168, "setmaxnreg budget exceeds the CTA's registers");
    if constexpr (kRegSplit) reg_dealloc<kRegsWg0>();   // first warpgroup: producer, MMA issuer, two idle warps
    if (warp == 0) {
        // ================= TMA producer =================
        if (elect_one()) {
            prefetch_tmap(&tmA);
            prefetch_tmap(&tmB);
            // pair mode: the leader's full barrier counts the bytes of both CTAs' loads
            const uint32_t stage_tx = ((uint32_t)p.a_box_rows * BK + (uint32_t)L::kBBytes) * (kPair ? 2u : 1u);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step) {
                const int b = t / tiles_per_batch;
                int mb, nb;
                tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, kPair ? GROUP_M / 2 : GROUP_M, mb, nb);
                int a_row = mb * BM, a_z = b, b_z = b;
                if constexpr (kGrouped) {
                    const GroupedTile g = grouped_tile(p, mb);
                    if (g.skip) continue;
                    a_row = g.row0; a_z = 0; b_z = g.e;
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status, kErrWaitProducer, p.wait_ns)) { ok = false; break; }
                    if constexpr (kTrace) trace_at(2, kb, t == tile0 + 2 * tile_step, clock64());
                    const uint32_t sa = smem_base + s * L::kStageBytes;
                    if (p.skip_kblock == kb && t == tile0) {
                        // wait-limit probe: nothing is loaded and nothing will arrive on this stage's barrier
                        if (++s == STAGES) { s = 0; ph ^= 1; }
                        continue;
                    }
                    if constexpr (kPair) {
                        if (rank == 0) mbar_arrive_expect_tx(full_bar(s), stage_tx);
                        tma_load_3d_pair(sa, &tmA, full_bar(s), kb * BK, mb * TILE_M + (int)rank * BM, b);
                        tma_load_3d_pair(sa + L::kABytes, &tmB, full_bar(s), kb * BK, nb * BN + (int)rank * L::kBRows, b);
                    } else {
                        mbar_arrive_expect_tx(full_bar(s), stage_tx);
                        tma_load_3d(sa, &tmA, full_bar(s), kb * BK, a_row, a_z);
                        tma_load_3d(sa + L::kABytes, &tmB, full_bar(s), kb * BK, nb * BN, b_z);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer (pair mode: the leader CTA only) =================
        if ((!kPair || rank == 0) && elect_one()) {
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step) {
                if constexpr (kGrouped) {
                    int mb, nb;
                    tile_coords(t, p.m_blks, p.n_blks, GROUP_M, mb, nb);
                    if (grouped_tile(p, mb).skip) continue;
                }
                if (!kBlockScale) {
                    if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, kErrWaitMma, p.wait_ns)) { ok = false; break; }
                    tc_fence_after();
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    // The operands usually landed long ago; the accumulator buffer coming back from the epilogue is
                    // what this thread really waits for.  So: operands first, descriptors ready, then the buffer, and
                    // the MMAs go out right behind it.
                    if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kErrWaitMma, p.wait_ns)) { ok = false; break; }
                    // timeline: the readings stay in registers until the MMAs are out (a store here would sit in front of them)
                    const long long tr_full = kTrace ? clock64() : 0;
                    const uint32_t sa = smem_base + s * L::kStageBytes;
                    const uint64_t da = smem_desc_sw128(sa);
                    const uint64_t db = smem_desc_sw128(sa + L::kABytes);
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    if (kBlockScale) {
                        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, abort_flag, p.status, kErrWaitMma, p.wait_ns)) { ok = false; break; }
                    }
                    tc_fence_after();
                    const long long tr_issue = kTrace ? clock64() : 0;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint32_t accumulate = kBlockScale ? (k != 0) : ((kb | k) != 0);
                        // advancing K by 32 bytes inside the 128-byte swizzle row = +2 in the address field
                        if constexpr (kPair) mma_f8_pair(d_tmem, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), IDESC, accumulate);
                        else mma_f8(d_tmem, da + (uint64_t)(k * (UMMA_K >> 4)), db + (uint64_t)(k * (UMMA_K >> 4)), IDESC, accumulate);
                    }
                    if (kBlockScale) {
                        // partial product ready for promotion (the epilogue waits for this one: it goes first)
                        if constexpr (kPair) tc_commit_pair(tfull_bar(acc), 3); else tc_commit(tfull_bar(acc));
                        if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                    }
                    // smem stage free once these MMAs retire (pair mode: in both CTAs)
                    if constexpr (kPair) tc_commit_pair(empty_bar(s), 3); else tc_commit(empty_bar(s));
                    if constexpr (kTrace) {
                        const bool on = t == tile0 + 2 * tile_step;
                        trace_at(0, kb, on, tr_full);
                        trace_at(1, kb, on, tr_issue);
                        trace_at(3, kb, on, clock64());
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!kBlockScale && ok) {
                    if constexpr (kPair) tc_commit_pair(tfull_bar(acc), 3); else tc_commit(tfull_bar(acc));
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    } else if (kRelay && warp == 2) {
        // ================= release relay (CTA pairs with block scales) =================
        if (elect_one()) {
            int acc = 0;
            uint32_t acc_ph = 0;
            bool ok = true;
            for (int t = tile0; t < total_tiles && ok; t += tile_step) {
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(relay_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue, p.wait_ns)) { ok = false; break; }
                    mbar_arrive_cluster(tempty_bar(acc), 0);
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
            }
        }
    }
    } else {
        // ================= epilogue =================
        if constexpr (kRegSplit) reg_alloc<kRegsEpi>();   // epilogue warpgroups take the registers WG0 gave up
        const int ew = warp - EPI_WARP0;         // 0 .. EPI_WARPS-1
        const int quarter = warp & 3;            // TMEM lane quarter this warp may read
        const int grp = ew >> 2;                 // column group
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        int acc = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        const bool wide = (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 31) == 0;
        // staged scales (block-scale epilogue with 128-column weight-scale groups only)
        constexpr int EPI_THREADS = 32 * EPI_WARPS;
        float4* const sa_slots = reinterpret_cast<float4*>(smem + L::kScaleOffset) + (threadIdx.x - EPI_WARP0 * 32);
        float* const sb_slots = reinterpret_cast<float*>(smem + L::kScaleOffset + L::kSaBytes) + ew * kScaleChunk;
        int sbuf = 0;
        // cp.async the scales of (tile, chunk) into buffer `buf`: this thread's row of a_scale as
        // float4 slots [kb/4][thread], and lane l of each warp the weight scale of K block l of the
        // warp's column group.  Completion is awaited by the same thread (sa) / warp (sb) only.
        auto stage_scales = [&](int buf, int tile, int chunk) {
            const int tb = tile / tiles_per_batch;
            int tmb, tnb;
            tile_coords(tile - tb * tiles_per_batch, p.m_blks, p.n_blks, kPair ? GROUP_M / 2 : GROUP_M, tmb, tnb);
            int r = tmb * TILE_M + (int)rank * BM + row_in_tile;
            const float* sb_base = p.sb;
            if constexpr (kGrouped) {
                const GroupedTile g = grouped_tile(p, tmb);        // never called for a skipped tile
                r = g.row0 + row_in_tile;
                sb_base += (int64_t)g.e * kblocks * (p.N / 128);
            }
            if (r >= p.M) r = p.M - 1;
            const int kb0 = chunk * kScaleChunk;
            const float* src = p.sa + (int64_t)r * kblocks + kb0;
            const uint32_t dst = smem_u32(sa_slots + (size_t)buf * (kScaleChunk / 4) * EPI_THREADS);
            const bool vec = (kblocks % 4) == 0 && (reinterpret_cast<uintptr_t>(p.sa) & 15) == 0;
#pragma unroll
            for (int j = 0; j < kScaleChunk / 4; ++j) {
                const int kb = kb0 + 4 * j;
                const uint32_t d = dst + (uint32_t)j * EPI_THREADS * 16;
                if (vec) {
                    if (kb < kblocks) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + 4 * j) : "memory");
                } else {
                    for (int i = 0; i < 4; ++i)
                        if (kb + i < kblocks) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d + 4 * i), "l"(src + 4 * j + i) : "memory");
                }
            }
            const int nsb = p.N / 128;
            const int cg = min((tnb * BN + grp * COLS_PER_GROUP) / 128, nsb - 1);
            const int kb = kb0 + lane;
            if (lane < kScaleChunk && kb < kblocks)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;"
                             ::"r"(smem_u32(sb_slots + (size_t)buf * EPI_WARPS * kScaleChunk + lane)), "l"(sb_base + (int64_t)kb * nsb + cg) : "memory");
        };
        // grouped mode: the first tile at or after `t` (in this CTA's walk) that the tile list does not mark as empty
        auto next_live_tile = [&](int t) {
            if constexpr (kGrouped) {
                while (t < total_tiles) {
                    int mb_, nb_;
                    tile_coords(t, p.m_blks, p.n_blks, GROUP_M, mb_, nb_);
                    if (!grouped_tile(p, mb_).skip) break;
                    t += tile_step;
                }
            }
            return t;
        };
        if constexpr (kBlockScale && kGn128) {
            const int first = next_live_tile(tile0);
            if (first < total_tiles) stage_scales(0, first, 0);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (int t = next_live_tile(tile0); t < total_tiles && ok; t = next_live_tile(t + tile_step)) {
            const int b = t / tiles_per_batch;
            int mb, nb;
            tile_coords(t - b * tiles_per_batch, p.m_blks, p.n_blks, kPair ? GROUP_M / 2 : GROUP_M, mb, nb);
            int row = mb * TILE_M + (int)rank * BM + row_in_tile;
            bool row_ok = row < p.M;
            int expert = 0;
            if constexpr (kGrouped) {
                const GroupedTile g = grouped_tile(p, mb);
                row = g.row0 + row_in_tile;
                row_ok = row_in_tile < g.rows && row < p.M;
                expert = g.e;
            }
            const int col_base = nb * BN + grp * COLS_PER_GROUP;
            __nv_bfloat16* crow = p.C + ((int64_t)b * p.M + (row_ok ? row : 0)) * p.ldc;

            if constexpr (!kBlockScale) {
                const float sa = row_ok ? __ldg(p.sa + (int64_t)b * p.M + row) : 0.0f;
                const float* sbp = p.sb + (int64_t)b * p.N;
                const __nv_bfloat16* biasp = p.bias ? p.bias + (int64_t)b * p.N : nullptr;
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue, p.wait_ns))) { ok = false; break; }
                tc_fence_after();
                const uint32_t t_addr = tmem_base + lane_addr + acc * BN + grp * COLS_PER_GROUP;
#pragma unroll 1
                for (int c = 0; c < COLS_PER_GROUP; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(t_addr + c, r);
                    tmem_ld_wait();
                    const int col0 = col_base + c;
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {          // N % 8 == 0: a group of 8 columns is all in or all out
                        const bool in = col0 + j < p.N;
                        const float4 s0 = in ? __ldg(reinterpret_cast<const float4*>(sbp + col0 + j)) : make_float4(0, 0, 0, 0);
                        const float4 s1 = in ? __ldg(reinterpret_cast<const float4*>(sbp + col0 + j + 4)) : make_float4(0, 0, 0, 0);
                        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                        float bv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        if (biasp && in) {
                            const uint4 bw = __ldg(reinterpret_cast<const uint4*>(biasp + col0 + j));
                            unpack8(bw, bv);
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[j + i] = __uint_as_float(r[j + i]) * sa * sv[i] + bv[i];
                    }
                    if (row_ok) store_row32(crow, col0, p.N, v, wide);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { if constexpr (kPair) mbar_arrive_cluster(tempty_bar(acc), 0); else mbar_arrive(tempty_bar(acc)); }
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            } else if constexpr (kGn128) {
                // one scale per (row, K block) and per (K block, 128 columns): a single fp32 factor
                // per thread and K block.  128 accumulators per thread as 64 float2 (packed FMA).
                static_assert(COLS_PER_GROUP == 128, "block-scale epilogue groups own 128 columns");
                float2 acc2[64];
#pragma unroll
                for (int j = 0; j < 64; ++j) acc2[j] = make_float2(0.0f, 0.0f);
                const int kbs = kblocks;
                // Scales come from shared memory: a global load in this loop, even one issued a K
                // block ahead, returns after an L2 round trip that is as long as the K block itself
                // and sets the pace of the whole MMA <-> epilogue hand-off.  cp.async stages the
                // scales of the next chunk (32 K blocks; the next tile's first chunk at a tile's end)
                // while this one is processed.
                const int nchunks = (kbs + kScaleChunk - 1) / kScaleChunk;
                for (int ch = 0; ch < nchunks && ok; ++ch) {
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncwarp();
                    {   // stage the scales that follow this chunk
                        int nt = t, nch = ch + 1;
                        if (nch == nchunks) { nt = next_live_tile(t + tile_step); nch = 0; }
                        if (nt < total_tiles) stage_scales(sbuf ^ 1, nt, nch);
                        asm volatile("cp.async.commit_group;" ::: "memory");
                    }
                    const float4* sa_s = sa_slots + (size_t)sbuf * (kScaleChunk / 4) * EPI_THREADS;
                    const float* sb_s = sb_slots + (size_t)sbuf * EPI_WARPS * kScaleChunk;
                    const int kb_end = min(kbs - ch * kScaleChunk, kScaleChunk);
                    float4 sa4 = sa_s[0];
                for (int kk = 0; kk < kb_end; ++kk) {
                    const int sub = kk & 3;
                    const float sa_k = sub == 0 ? sa4.x : sub == 1 ? sa4.y : sub == 2 ? sa4.z : sa4.w;
                    const float sc = sa_k * sb_s[kk];
                    const float2 s2 = make_float2(sc, sc);
                    if (sub == 3 && kk + 1 < kb_end) sa4 = sa_s[(size_t)((kk + 1) >> 2) * EPI_THREADS];
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue, p.wait_ns))) { ok = false; break; }
                    tc_fence_after();
                    if constexpr (kTrace) trace_at(12 + ew, ch * kScaleChunk + kk, lane == 0 && t == tile0 + 2 * tile_step, clock64());
                    const uint32_t t_addr = tmem_base + lane_addr + acc * BN + grp * COLS_PER_GROUP;
                    uint32_t ra[32], rb[32];
                    // the partial product lives in registers after the fourth load: the TMEM buffer goes back
                    // to the MMA thread before the last FMAs
                    auto release = [&]() {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (kRelay) mbar_arrive(relay_bar(acc));
                            else if constexpr (kPair) mbar_arrive_cluster(tempty_bar(acc), 0);
                            else mbar_arrive(tempty_bar(acc));
                        }
                    };
                    tmem_ld32(t_addr, ra);
                    tmem_ld_wait32(ra);
                    tmem_ld32(t_addr + 32, rb);               // in flight during the FMAs on ra
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
                    release();
                    if constexpr (kTrace) trace_at(4 + ew, ch * kScaleChunk + kk, lane == 0 && t == tile0 + 2 * tile_step, clock64());
#pragma unroll
                    for (int j = 0; j < 16; ++j) acc2[48 + j] = ffma2(rb[2 * j], rb[2 * j + 1], s2, acc2[48 + j]);
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
                    sbuf ^= 1;
                }
                if constexpr (kOut == 1) {
                    // Scatter mode: the copies in the other GPUs' memory travel over NVLink, where a 32-byte store per
                    // lane and row wastes most of every packet.  The warp transposes its 32 x 128 block through shared
                    // memory, 64 columns at a time, so that eight lanes write 128 contiguous bytes of one row.
                    if (ok) {
                        uint8_t* const stg = smem + L::kStageOutOffset + ew * 4096;
                        const int wrow0 = (row - row_in_tile) + quarter * 32;          // first row of this warp's block
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                const float2 a0 = acc2[32 * h + 4 * c], a1 = acc2[32 * h + 4 * c + 1], a2 = acc2[32 * h + 4 * c + 2], a3 = acc2[32 * h + 4 * c + 3];
                                *reinterpret_cast<uint4*>(stg + lane * 128 + ((c ^ (lane & 7)) * 16)) =
                                    make_uint4(pack_bf16(a0.x, a0.y), pack_bf16(a1.x, a1.y), pack_bf16(a2.x, a2.y), pack_bf16(a3.x, a3.y));
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int rr = 4 * i + (lane >> 3), cc = lane & 7;
                                const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((cc ^ (rr & 7)) * 16));
                                const int grow = wrow0 + rr;
                                if (grow < p.M) {
                                    const int64_t off = (int64_t)grow * p.ldc + col_base + 64 * h + 8 * cc;
                                    *reinterpret_cast<uint4*>(p.C + off) = v;
                                    for (int d = 0; d < p.n_peer; ++d) *reinterpret_cast<uint4*>(p.peer[d] + off) = v;
                                }
                            }
                            __syncwarp();
                        }
                    }
                } else if (ok && row_ok) {
                    // N % 128 == 0 in block-scale mode: rows are 32-byte aligned, whole groups are in range
#pragma unroll
                    for (int c = 0; c < 128; c += 16) {
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 8; ++i) { v[2 * i] = acc2[c / 2 + i].x; v[2 * i + 1] = acc2[c / 2 + i].y; }
                        if (p.c_a) mul_add_cols<16>(p.c_a, p.c_b, (int64_t)row * p.N + col_base + c, v);
                        if constexpr (kGrouped) {
                            if (p.bias_f32) {
                                const float4* bp = reinterpret_cast<const float4*>(p.bias_f32 + (int64_t)expert * p.N + col_base + c);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float4 bv = __ldg(bp + i);
                                    v[4 * i] += bv.x; v[4 * i + 1] += bv.y; v[4 * i + 2] += bv.z; v[4 * i + 3] += bv.w;
                                }
                            }
                        }
                        if constexpr (kOut == 2) {
                            store_bf16x16(split_cat_ptr(p, row, col_base + c), v);
                        } else {
                            store_bf16x16(crow + col_base + c, v);
                        }
                    }
                }
            } else {
                // per-column weight scales (gn = 1): secondary mode, plain scalar code
                float accv[COLS_PER_GROUP];
#pragma unroll
                for (int j = 0; j < COLS_PER_GROUP; ++j) accv[j] = 0.0f;
                const int kbs = kblocks;
                const float* sarow = p.sa + (int64_t)(row_ok ? row : p.M - 1) * kbs;
                const int nsb = p.N;
                float sa_next = __ldg(sarow);
                for (int kb = 0; kb < kbs; ++kb) {
                    const float sa = sa_next;
                    if (kb + 1 < kbs) sa_next = __ldg(sarow + kb + 1);
                    const float* sbrow = p.sb + (int64_t)kb * nsb;
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kErrWaitEpilogue, p.wait_ns))) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t t_addr = tmem_base + lane_addr + acc * BN + grp * COLS_PER_GROUP;
#pragma unroll
                    for (int c = 0; c < COLS_PER_GROUP; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(t_addr + c, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = min(col_base + c + j, p.N - 1);
                            accv[c + j] = __fmaf_rn(__uint_as_float(r[j]), sa * __ldg(sbrow + col), accv[c + j]);
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { if constexpr (kPair) mbar_arrive_cluster(tempty_bar(acc), 0); else mbar_arrive(tempty_bar(acc)); }
                    if (++acc == 2) { acc = 0; acc_ph ^= 1; }
                }
                if (ok && row_ok) {
#pragma unroll
                    for (int c = 0; c < COLS_PER_GROUP; c += 32) {
                        if (p.c_a) mul_add_cols<32>(p.c_a, p.c_b, (int64_t)row * p.N + col_base + c, accv + c);
                        if constexpr (kOut == 2) {
                            store_bf16x16(split_cat_ptr(p, row, col_base + c), accv + c);
                            store_bf16x16(split_cat_ptr(p, row, col_base + c + 16), accv + c + 16);
                        } else {
                            store_row32(crow, col_base + c, p.N, accv + c, wide);
                        }
                    }
                }
            }
        }
    }

    // ---- teardown: every role is done (or has given up); free TMEM ----
    asm volatile("cp.async.wait_group 0;" ::: "memory");      // no staged-scale copy may outlive the CTA
    tc_fence_before();
    __syncthreads();
    if constexpr (kPair) { __syncwarp(); cluster_sync_all(); }   // the partner is done with this CTA's smem, barriers and TMEM
    if (warp == 1) {
        if (*abort_flag) {
            // give copies that may still be in flight time to land before the CTA exits
            const uint64_t t0 = globaltimer_ns();
            while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
        }
        tc_fence_after();
        if constexpr (kPair) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Grouped (MoE) pre-pass: rows of the token-major activations and their scales copied into expert-sorted order,
// row r <- token gather[r] / n_act.  One warp per row, 16-byte vectors for the codes.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint8_t* __restrict__ x, const float* __restrict__ xs, const int32_t* __restrict__ gather, int n_act,
                       uint8_t* __restrict__ xg, float* __restrict__ xsg, int64_t rows, int K, int kblocks, int64_t tokens) {
    const int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    int64_t tok = __ldg(gather + r) / n_act;
    tok = tok < 0 ? 0 : (tok >= tokens ? tokens - 1 : tok);
    const uint4* src = reinterpret_cast<const uint4*>(x + tok * K);
    uint4* dst = reinterpret_cast<uint4*>(xg + r * K);
    for (int i = lane; i < K / 16; i += 32) dst[i] = __ldg(src + i);
    for (int i = lane; i < kblocks; i += 32) xsg[r * kblocks + i] = __ldg(xs + tok * kblocks + i);
}

// dst[r, off + j] = src[r, j] for j < w: the concatenation half of the split-cat epilogues
// (rows of `w` bf16 copied into rows of pitch `ldd`), 16 bytes per thread.
__global__ void __launch_bounds__(256)
concat_cols_kernel(const uint4* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t rows, int w8, int64_t ldd, int64_t off) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= rows * w8) return;
    const int64_t r = i / w8;
    const int j = (int)(i - r * w8);
    *reinterpret_cast<uint4*>(dst + r * ldd + off + j * 8) = __ldg(src + i);
}
}  // namespace

int launch_concat_cols(const void* src, void* dst, int64_t rows, int64_t w, int64_t ldd, int64_t off, cudaStream_t st) {
    HKB_REQUIRE(aligned16(src) && aligned16(dst) && w % 8 == 0 && ldd % 8 == 0 && off % 8 == 0, HKB_ERR_BAD_ALIGN,
                "split-cat: y and c1 must be 16-byte aligned and the split sizes multiples of 8");
    const int64_t n = rows * (w / 8);
    if (n == 0) return HKB_OK;
    HKB_REQUIRE((n + 255) / 256 <= 0x7FFFFFFFLL, HKB_ERR_BAD_SHAPE, "split-cat: tensor too large");
    concat_cols_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const uint4*)src, (__nv_bfloat16*)dst, rows, (int)(w / 8), ldd, off);
    return check_launch("concat_cols_kernel");
}

namespace {
// CTA-pair launch: clusters of 2 along x, one cluster per pair of SMs, persistent over 256 x 256 tiles.
template <int STAGES, bool kBlockScale>
int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t st) {
    using L = SmemLayout<256, STAGES, true, BM, kBlockScale ? 256 : 0>;
    static_assert(L::kDynamic <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
    auto kern = gemm_fp8_kernel<256, STAGES, kBlockScale, true, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", L::kDynamic, cudaGetErrorString(e));
    const int sms = sm_count();
    HKB_REQUIRE(sms > 1, HKB_ERR_CUDA, "no CUDA device");
    const int tiles = p.m_blks * p.n_blks * p.batch;
    int clusters = sms / 2;
    if (tiles < clusters) clusters = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(gemm_threads<256, kBlockScale, true>());
    cfg.dynamicSmemBytes = L::kDynamic;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p);
    HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cluster launch of gemm_fp8_kernel failed: %s", cudaGetErrorString(e));
    note_kernel(kBlockScale ? "gemm_fp8_kernel<256,blockscale,pair>" : "gemm_fp8_kernel<256,pts,pair>");
    return check_launch("gemm_fp8_kernel (CTA pairs)");
}

inline int group_m_env() {
    static const int g = [] { const char* v = getenv("HKB_GROUP_M"); const int x = v ? atoi(v) : 0; return x >= 2 && x <= 64 ? x : 0; }();
    return g;
}
inline int group_m_default() { return group_m_env() ? group_m_env() : 8; }

// HKB_GEMM_PAIRS=0 in the environment forces the single-CTA kernels (for A/B measurements).
inline bool pairs_enabled() {
    static const bool on = [] { const char* v = getenv("HKB_GEMM_PAIRS"); return !(v && v[0] == '0'); }();
    return on;
}

inline bool skinny_enabled() {
    static const bool on = [] { const char* v = getenv("HKB_GEMM_SKINNY"); return !(v && v[0] == '0'); }();
    return on;
}

template <int BN, int STAGES, bool kBlockScale, bool kGn128 = false, int AROWS = BM, int kOut = 0>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, cudaStream_t st) {
    using L = SmemLayout<BN, STAGES, false, AROWS, (kBlockScale && kGn128) ? (BN == 256 ? 256 : 128) : 0, kOut == 1 ? 16 : 32,
                         kOut == 1 ? (BN == 256 ? 8 : 4) * 4096 : 0>;
    static_assert(L::kDynamic <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
    auto kern = gemm_fp8_kernel<BN, STAGES, kBlockScale, kGn128, false, AROWS, kOut>;
    // the attribute is per device; set it on every call (cheap) so multi-device processes work
    const cudaError_t attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    HKB_REQUIRE(attr_err == cudaSuccess, HKB_ERR_CUDA, "cudaFuncSetAttribute(smem=%d) failed: %s", L::kDynamic, cudaGetErrorString(attr_err));
    const int tiles = p.m_blks * p.n_blks * p.batch;
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, gemm_threads<BN, kBlockScale>(), L::kDynamic, st>>>(tmA, tmB, p);
    note_kernel(kOut == 1 ? (BN == 256 ? "gemm_fp8_kernel<256,blockscale,scatter>" : "gemm_fp8_kernel<128,blockscale,scatter>") :
                kOut == 2 ? (kGn128 ? "gemm_fp8_kernel<128,blockscale,split_cat>" : "gemm_fp8_kernel<128,blockscale,gn1,split_cat>") :
                kOut == 3 ? (BN == 256 ? "gemm_fp8_kernel<256,blockscale,grouped>" : "gemm_fp8_kernel<128,blockscale,grouped>") :
                kOut == 4 ? "gemm_fp8_kernel<256,blockscale,timeline>" :
                kBlockScale ? (BN == 256 ? "gemm_fp8_kernel<256,blockscale>" : kGn128 ? "gemm_fp8_kernel<128,blockscale>" : "gemm_fp8_kernel<128,blockscale,gn1>")
                            : (BN == 256 ? "gemm_fp8_kernel<256,pts>" : BN == 128 ? "gemm_fp8_kernel<128,pts>" : "gemm_fp8_kernel<64,pts>"));
    return check_launch("gemm_fp8_kernel");
}

int common_checks(const char* who, const void* A, const void* B, const void* C, int64_t batch, int64_t M, int64_t N, int64_t K) {
    HKB_REQUIRE(A && B && C, HKB_ERR_BAD_ARG, "%s: null pointer", who);
    HKB_REQUIRE(batch >= 1 && M >= 1 && N >= 1 && K >= 1, HKB_ERR_BAD_SHAPE, "%s: empty problem (batch=%lld M=%lld N=%lld K=%lld)", who,
                (long long)batch, (long long)M, (long long)N, (long long)K);
    HKB_REQUIRE(K % BK == 0, HKB_ERR_BAD_SHAPE, "%s: K=%lld must be a multiple of %d", who, (long long)K, BK);
    HKB_REQUIRE(N % 8 == 0, HKB_ERR_BAD_SHAPE, "%s: N=%lld must be a multiple of 8", who, (long long)N);
    HKB_REQUIRE(M < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31) && batch < 65536, HKB_ERR_BAD_SHAPE, "%s: dimension too large", who);
    HKB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C), HKB_ERR_BAD_ALIGN, "%s: A, B and C must be 16-byte aligned", who);
    return HKB_OK;
}

}  // namespace

struct SplitCat { void* c2; int64_t s1, s2, s3; };      // C is c1 [M, D, s1+s3], c2 [M, D, s2], N = D*(s1+s2)
int gemm_fp8_blockscale_impl(const void* A, const void* B, void* C, const float* sa, const float* sb, int64_t gn,
                             const void* c_a, const void* c_b, int64_t M, int64_t N, int64_t K, void* stream,
                             int64_t ldc = 0, void* const* peers = nullptr, int n_peer = 0, const SplitCat* sc = nullptr,
                             unsigned long long* trace = nullptr);

// wait_ns / skip_kblock: production passes kWaitLimitNs / -1; the wait-limit probe a short limit
// and a K block that the producer leaves unloaded.
int gemm_fp8_pts_impl(const void* A, const void* B, void* C, const float* sa, const float* sb, const void* bias,
                      int64_t batch, int64_t M, int64_t N, int64_t K, void* stream, uint64_t wait_ns, int skip_kblock) {
    int rc = common_checks("gemm_fp8_pts", A, B, C, batch, M, N, K);
    if (rc != HKB_OK) return rc;
    HKB_REQUIRE(sa && sb, HKB_ERR_BAD_ARG, "gemm_fp8_pts: null scale pointer");
    // the epilogues read b_scale four floats and the bias eight bf16 at a time
    HKB_REQUIRE((reinterpret_cast<uintptr_t>(sa) & 3) == 0 && aligned16(sb) && (!bias || aligned16(bias)), HKB_ERR_BAD_ALIGN,
                "gemm_fp8_pts: a_scale must be 4-byte, b_scale and bias 16-byte aligned");
    GemmParams p{};
    p.group_m = group_m_default();
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
    p.sa = sa; p.sb = sb; p.bias = (const __nv_bfloat16*)bias; p.C = (__nv_bfloat16*)C; p.gn = 0;
    p.ldc = N; p.n_peer = 0;
    p.wait_ns = wait_ns; p.skip_kblock = skip_kblock;
    rc = status_word(&p.status);
    if (rc != HKB_OK) return rc;
    // Decode shapes: HBM-bound on the weight stream; a kernel that deals the columns out evenly
    // over the SMs (gemm_fp8_skinny.cu).  HKB_GEMM_SKINNY=0 keeps the fixed-width tiles below.
    if (M <= 64 && batch == 1 && N % 16 == 0 && aligned32(C) && skip_kblock < 0 && skinny_enabled()) {
        note_kernel("gemm_fp8_skinny_kernel");
        return launch_gemm_fp8_skinny(A, B, C, sa, sb, bias, M, N, K, p.status, (cudaStream_t)stream);
    }
    p.m_blks = (int)((M + BM - 1) / BM);
    // Skinny M: fetch only the rows that exist (rounded up to 8); the remaining rows of the
    // smem tile hold stale bytes that only reach accumulator rows >= M, which are never stored.
    p.a_box_rows = M >= BM ? BM : (int)((M + 7) / 8 * 8);
    // Tile width: small problems (few tiles per SM) take narrower tiles so that the SMs stay busy;
    // skinny-M (decode) shapes are HBM-bound on B and want many independent B streams.
    const int sms = sm_count();
    int bn = 256;
    if (N % 256 != 0 && N < 4096) bn = 128;
    if ((int64_t)p.m_blks * ((N + 255) / 256) * batch < 2LL * sms) bn = 128;
    if ((int64_t)p.m_blks * ((N + 127) / 128) * batch < 2LL * sms) bn = 64;
    p.n_blks = (int)((N + bn - 1) / bn);
    cudaStream_t st = (cudaStream_t)stream;
    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)batch, (uint32_t)p.a_box_rows);
    if (rc != HKB_OK) return rc;
    // Large problems: CTA pairs on 256 x 256 tiles (a third less operand traffic per SM).
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256) * batch;
    if (bn == 256 && M > 128 && pair_tiles >= sms / 2 && pairs_enabled()) {
        p.m_blks = (int)((M + 255) / 256);
        rc = make_tmap_bytes(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)batch, 128);
        if (rc != HKB_OK) return rc;
        return launch_gemm_pair<7, false>(tmA, tmB, p, st);
    }
    rc = make_tmap_bytes(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)batch, (uint32_t)bn);
    if (rc != HKB_OK) return rc;
    if (bn == 256) return launch_gemm<256, 4, false>(tmA, tmB, p, st);
    if (bn == 128) return launch_gemm<128, 6, false>(tmA, tmB, p, st);
    // skinny M with narrow tiles (decode shapes): stage only the A rows that exist, deepen the ring
    if (p.a_box_rows <= 16) return launch_gemm<64, 19, false, false, 16>(tmA, tmB, p, st);
    if (p.a_box_rows <= 64) return launch_gemm<64, 12, false, false, 64>(tmA, tmB, p, st);
    return launch_gemm<64, 8, false>(tmA, tmB, p, st);
}
}  // namespace hkb

extern "C" {

int hkb_gemm_fp8_pts(const void* A, const void* B, void* C, const float* sa, const float* sb, const void* bias,
                     int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
    return hkb::gemm_fp8_pts_impl(A, B, C, sa, sb, bias, batch, M, N, K, stream, hkb::kWaitLimitNs, -1);
}

int hkb_debug_gemm_fp8_wait_probe(const void* A, const void* B, void* C, const float* sa, const float* sb,
                                  int64_t M, int64_t N, int64_t K, uint64_t wait_limit_ns, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(wait_limit_ns >= 1000 && wait_limit_ns <= kWaitLimitNs, HKB_ERR_BAD_ARG,
                "gemm_fp8_wait_probe: the wait limit must lie between 1 us and 2 s");
    return gemm_fp8_pts_impl(A, B, C, sa, sb, nullptr, 1, M, N, K, stream, wait_limit_ns, 0);
}

int hkb_gemm_fp8_blockscale(const void* A, const void* B, void* C, const float* sa, const float* sb, int64_t gn,
                            int64_t M, int64_t N, int64_t K, void* stream) {
    return hkb::gemm_fp8_blockscale_impl(A, B, C, sa, sb, gn, nullptr, nullptr, M, N, K, stream);
}

int hkb_debug_gemm_fp8_blockscale_timeline(const void* A, const void* B, void* C, const float* sa, const float* sb,
                                           int64_t M, int64_t N, int64_t K, void* trace, int64_t trace_bytes, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(trace && (reinterpret_cast<uintptr_t>(trace) & 7) == 0, HKB_ERR_BAD_ARG, "gemm_fp8_blockscale timeline: trace buffer must be non-null and 8-byte aligned");
    const int sms = sm_count();
    HKB_REQUIRE(sms > 0, HKB_ERR_CUDA, "no CUDA device");
    const int64_t need = (int64_t)sms * kTraceEvents * kTraceKb * 8;
    HKB_REQUIRE(trace_bytes >= need, HKB_ERR_BAD_ARG, "gemm_fp8_blockscale timeline: trace buffer has %lld bytes, %lld needed", (long long)trace_bytes, (long long)need);
    const cudaError_t e = cudaMemsetAsync(trace, 0, (size_t)need, (cudaStream_t)stream);
    HKB_REQUIRE(e == cudaSuccess, HKB_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
    return gemm_fp8_blockscale_impl(A, B, C, sa, sb, 128, nullptr, nullptr, M, N, K, stream, 0, nullptr, 0, nullptr, (unsigned long long*)trace);
}

int hkb_gemm_fp8_blockscale_scatter(const void* A, const void* B, void* const* C_dst, int n_dst, int64_t ldc,
                                    const float* sa, const float* sb, int64_t M, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(C_dst && n_dst >= 1 && n_dst <= 8, HKB_ERR_BAD_ARG, "gemm_fp8_blockscale_scatter: 1 to 8 destinations");
    return gemm_fp8_blockscale_impl(A, B, C_dst[0], sa, sb, 128, nullptr, nullptr, M, N, K, stream, ldc, C_dst + 1, n_dst - 1);
}

int hkb_moe_gemm_fp8_blockscale(const void* X, const void* W, void* Y, const float* X_scale, const float* W_scale,
                                const float* bias, const int32_t* GatherIndx, const int32_t* ExptHist, const int32_t* ExptOffs,
                                const int32_t* ExptData, int64_t tokens, int64_t rows, int64_t E, int64_t N, int64_t K,
                                int64_t grid_m, int64_t n_expts_act, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(X && W && Y && X_scale && W_scale && ExptHist && ExptOffs && ExptData, HKB_ERR_BAD_ARG, "moe_gemm_fp8_blockscale: null pointer");
    HKB_REQUIRE(tokens >= 1 && rows >= 1 && E >= 1 && E <= 65535 && N >= 128 && K >= 128 && grid_m >= 1 && n_expts_act >= 1 &&
                rows < (1LL << 31) && tokens < (1LL << 31) && N < (1LL << 31) && K < (1LL << 31) && grid_m < (1LL << 24),
                HKB_ERR_BAD_SHAPE, "moe_gemm_fp8_blockscale: bad problem size");
    HKB_REQUIRE(K % 128 == 0 && N % 128 == 0, HKB_ERR_BAD_SHAPE, "moe_gemm_fp8_blockscale: K and N must be multiples of 128 (the scale group)");
    HKB_REQUIRE(GatherIndx || tokens == rows, HKB_ERR_BAD_SHAPE, "moe_gemm_fp8_blockscale: without GatherIndx X holds one row per output row");
    HKB_REQUIRE(aligned16(X) && aligned16(W) && aligned32(Y) && (!bias || aligned16(bias)), HKB_ERR_BAD_ALIGN,
                "moe_gemm_fp8_blockscale: X, W and bias must be 16-byte, Y 32-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int kblocks = (int)(K / 128);
    const void* A = X;
    const float* sa = X_scale;
    int rc;
    if (GatherIndx) {
        // expert-sorted copy of the activations and their scales (per-stream scratch), so that a tile's rows are contiguous for TMA
        void *xg = nullptr, *xsg = nullptr;
        rc = scratch_get(SCRATCH_SFA, st, (size_t)rows * K, &xg);
        if (rc != HKB_OK) return rc;
        rc = scratch_get(SCRATCH_SFB, st, (size_t)rows * kblocks * 4, &xsg);
        if (rc != HKB_OK) return rc;
        moe_gather_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const uint8_t*)X, X_scale, GatherIndx, (int)n_expts_act,
                                                                             (uint8_t*)xg, (float*)xsg, rows, (int)K, kblocks, tokens);
        rc = check_launch("moe_gather_rows_kernel");
        if (rc != HKB_OK) return rc;
        A = xg;
        sa = (const float*)xsg;
    }
    GemmParams p{};
    p.group_m = group_m_default();
    p.M = (int)rows; p.N = (int)N; p.K = (int)K; p.batch = 1;
    p.sa = sa; p.sb = W_scale; p.C = (__nv_bfloat16*)Y; p.gn = 128;
    p.ldc = N; p.wait_ns = kWaitLimitNs; p.skip_kblock = -1;
    p.expt_data = ExptData; p.expt_hist = ExptHist; p.expt_offs = ExptOffs; p.bias_f32 = bias;
    rc = status_word(&p.status);
    if (rc != HKB_OK) return rc;
    p.m_blks = (int)grid_m;
    p.a_box_rows = BM;
    const int sms = sm_count();
    const int bn = (N % 256 == 0 && grid_m * (N / 256) >= 2LL * sms) ? 256 : 128;
    p.n_blks = (int)(N / bn);
    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, A, (uint64_t)K, (uint64_t)rows, 1, BM);
    if (rc != HKB_OK) return rc;
    rc = make_tmap_bytes(&tmB, W, (uint64_t)K, (uint64_t)N, (uint64_t)E, (uint32_t)bn);
    if (rc != HKB_OK) return rc;
    if (bn == 256) return launch_gemm<256, 3, true, true, BM, 3>(tmA, tmB, p, st);
    return launch_gemm<128, 5, true, true, BM, 3>(tmA, tmB, p, st);
}

int hkb_gemm_fp8_blockscale_split_cat(const void* A, const void* B, const float* sa, const float* sb, int64_t gn,
                                      const void* y, void* c1, void* c2, int64_t M, int64_t N, int64_t K,
                                      int64_t S1, int64_t S2, int64_t S3, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(c1 && c2 && (S3 == 0 || y), HKB_ERR_BAD_ARG, "gemm_fp8_blockscale_split_cat: null pointer");
    const SplitCat sc{c2, S1, S2, S3};
    int rc = gemm_fp8_blockscale_impl(A, B, c1, sa, sb, gn, nullptr, nullptr, M, N, K, stream, 0, nullptr, 0, &sc);
    if (rc != HKB_OK || S3 == 0) return rc;
    return launch_concat_cols(y, c1, M * (N / (S1 + S2)), S3, S1 + S3, S1, (cudaStream_t)stream);
}

int hkb_gemm_fp8_blockscale_mul_add(const void* A, const void* B, void* C, const float* sa, const float* sb, int64_t gn,
                                    const void* c_a, const void* c_b, int64_t M, int64_t N, int64_t K, void* stream) {
    using namespace hkb;
    HKB_REQUIRE(c_a && c_b, HKB_ERR_BAD_ARG, "gemm_fp8_blockscale_mul_add: null c_a / c_b");
    HKB_REQUIRE(aligned16(c_a) && aligned16(c_b), HKB_ERR_BAD_ALIGN, "gemm_fp8_blockscale_mul_add: c_a and c_b must be 16-byte aligned");
    return gemm_fp8_blockscale_impl(A, B, C, sa, sb, gn, c_a, c_b, M, N, K, stream);
}

}  // extern "C"

namespace hkb {

int gemm_fp8_blockscale_impl(const void* A, const void* B, void* C, const float* sa, const float* sb, int64_t gn,
                             const void* c_a, const void* c_b, int64_t M, int64_t N, int64_t K, void* stream,
                             int64_t ldc, void* const* peers, int n_peer, const SplitCat* sc, unsigned long long* trace) {
    int rc = common_checks("gemm_fp8_blockscale", A, B, C, 1, M, N, K);
    if (rc != HKB_OK) return rc;
    if (sc) {
        HKB_REQUIRE(sc->c2 && aligned32(sc->c2) && aligned32(C), HKB_ERR_BAD_ALIGN, "gemm_fp8_blockscale_split_cat: c1 and c2 must be 32-byte aligned");
        HKB_REQUIRE(sc->s1 > 0 && sc->s2 > 0 && sc->s3 >= 0 && sc->s1 % 16 == 0 && sc->s2 % 16 == 0 && sc->s3 % 16 == 0 &&
                    N % (sc->s1 + sc->s2) == 0 && sc->s1 + sc->s2 + sc->s3 < (1LL << 30),
                    HKB_ERR_BAD_SHAPE, "gemm_fp8_blockscale_split_cat: S1, S2, S3 must be multiples of 16 and N a multiple of S1+S2");
        HKB_REQUIRE(!c_a && n_peer == 0 && ldc == 0, HKB_ERR_UNSUPPORTED, "gemm_fp8_blockscale_split_cat: no other epilogue at the same time");
    }
    if (ldc == 0) ldc = N;
    HKB_REQUIRE(ldc >= N && ldc % 16 == 0, HKB_ERR_BAD_SHAPE, "gemm_fp8_blockscale: row pitch %lld must be >= N and a multiple of 16", (long long)ldc);
    HKB_REQUIRE(n_peer >= 0 && n_peer <= 7 && (n_peer == 0 || peers), HKB_ERR_BAD_ARG, "gemm_fp8_blockscale: at most 8 destinations");
    HKB_REQUIRE((n_peer == 0 && ldc == N) || gn == 128, HKB_ERR_UNSUPPORTED,
                "gemm_fp8_blockscale: a pitched or replicated result needs 128-column weight-scale groups");
    for (int d = 0; d < n_peer; ++d)
        HKB_REQUIRE(peers[d] && aligned32(peers[d]), HKB_ERR_BAD_ALIGN, "gemm_fp8_blockscale: destination %d must be non-null and 32-byte aligned", d + 1);
    HKB_REQUIRE(gn != 128 || aligned32(C), HKB_ERR_BAD_ALIGN, "gemm_fp8_blockscale: C must be 32-byte aligned");
    HKB_REQUIRE(sa && sb, HKB_ERR_BAD_ARG, "gemm_fp8_blockscale: null scale pointer");
    HKB_REQUIRE(gn == 1 || gn == 128, HKB_ERR_UNSUPPORTED, "gemm_fp8_blockscale: weight scale group along N must be 1 or 128, got %lld", (long long)gn);
    HKB_REQUIRE(N % 128 == 0, HKB_ERR_BAD_SHAPE, "gemm_fp8_blockscale: N=%lld must be a multiple of 128", (long long)N);
    GemmParams p{};
    p.group_m = group_m_env() ? group_m_env() : 16;      // 16 M blocks per group: +2.3 % on 16384 x 57344 x 8192, +0.8 % on 4096 x 14336 x 4096 over 8
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = 1;
    p.sa = sa; p.sb = sb; p.bias = nullptr; p.C = (__nv_bfloat16*)C; p.gn = (int)gn;
    p.c_a = (const __nv_bfloat16*)c_a; p.c_b = (const __nv_bfloat16*)c_b;
    p.ldc = ldc; p.n_peer = n_peer;
    for (int d = 0; d < n_peer; ++d) p.peer[d] = (__nv_bfloat16*)peers[d];
    if (sc) { p.c2 = (__nv_bfloat16*)sc->c2; p.sc_s1 = (int)sc->s1; p.sc_s2 = (int)sc->s2; p.sc_s3 = (int)sc->s3; }
    p.wait_ns = kWaitLimitNs; p.skip_kblock = -1;
    rc = status_word(&p.status);
    if (rc != HKB_OK) return rc;
    p.m_blks = (int)((M + BM - 1) / BM);
    p.a_box_rows = BM;
    const int sms = sm_count();
    int bn = 256;
    if (gn != 128 || sc || N % 256 != 0 || (int64_t)p.m_blks * (N / 256) < 2LL * sms) bn = 128;
    p.n_blks = (int)(N / bn);
    cudaStream_t st = (cudaStream_t)stream;
    CUtensorMap tmA, tmB;
    rc = make_tmap_bytes(&tmA, A, (uint64_t)K, (uint64_t)M, 1, BM);
    if (rc != HKB_OK) return rc;
    if (trace) {
        HKB_REQUIRE(bn == 256 && !c_a && n_peer == 0 && ldc == N, HKB_ERR_UNSUPPORTED,
                    "gemm_fp8_blockscale timeline: needs the 256-wide kernel (gn = 128, N %% 256 == 0, at least two tiles per SM) and the plain epilogue");
        p.trace = trace;
        rc = make_tmap_bytes(&tmB, B, (uint64_t)K, (uint64_t)N, 1, 256);
        if (rc != HKB_OK) return rc;
        return launch_gemm<256, 3, true, true, BM, 4>(tmA, tmB, p, st);
    }
    // CTA pairs: the per-K-block accumulator hand-off crosses the cluster.  With a relaxed remote arrive it runs within
    // 2-3 % of the single-CTA kernel (with a release at cluster scope it was 1.9x slower), never ahead of it: kept
    // reachable for experiments only.
    static const bool bs_pairs = [] { const char* v = getenv("HKB_BLOCKSCALE_PAIRS"); return v && v[0] == '1'; }();
    const int64_t pair_tiles = ((M + 255) / 256) * (N / 256);
    if (bs_pairs && bn == 256 && M > 128 && pair_tiles >= sms / 2) {
        p.m_blks = (int)((M + 255) / 256);
        rc = make_tmap_bytes(&tmB, B, (uint64_t)K, (uint64_t)N, 1, 128);
        if (rc != HKB_OK) return rc;
        return launch_gemm_pair<4, true>(tmA, tmB, p, st);
    }
    rc = make_tmap_bytes(&tmB, B, (uint64_t)K, (uint64_t)N, 1, (uint32_t)bn);
    if (rc != HKB_OK) return rc;
    if (sc) {
        if (gn == 128) return launch_gemm<128, 5, true, true, BM, 2>(tmA, tmB, p, st);
        return launch_gemm<128, 6, true, false, BM, 2>(tmA, tmB, p, st);
    }
    if (gn == 128 && n_peer > 0) {
        if (bn == 256) return launch_gemm<256, 3, true, true, BM, 1>(tmA, tmB, p, st);
        return launch_gemm<128, 5, true, true, BM, 1>(tmA, tmB, p, st);
    }
    if (gn == 128) {
        if (bn == 256) return launch_gemm<256, 3, true, true>(tmA, tmB, p, st);
        return launch_gemm<128, 5, true, true>(tmA, tmB, p, st);
    }
    return launch_gemm<128, 6, true, false>(tmA, tmB, p, st);
}

}  // namespace hkb
