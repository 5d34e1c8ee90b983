/*
 * hkb200.h -- C ABI of libhkb200.so: the quantized-GEMM path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain DEVICE pointers and sizes, launches asynchronously on the
 * given CUDA stream (a cudaStream_t passed as void*, NULL = default stream), allocates no
 * caller-visible memory, and returns 0 on success or a negative hkb_status.  After a
 * failure hkb_last_error() returns a thread-local message.  Nothing here has a CPU
 * fallback: without a CUDA device every compute entry point returns HKB_ERR_CUDA.
 *
 * Each declaration cites the interface of the reference project (m8than/amd-kernels)
 * that it replaces, as <path>:<lines> inside that project.
 */
#ifndef HKB200_H
#define HKB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    HKB_OK = 0,
    HKB_ERR_BAD_ARG = -1,     /* null pointer, bad enum value */
    HKB_ERR_BAD_SHAPE = -2,   /* dimension not supported (divisibility, zero, too large) */
    HKB_ERR_BAD_ALIGN = -3,   /* pointer or pitch not aligned as required */
    HKB_ERR_UNSUPPORTED = -4, /* combination not implemented */
    HKB_ERR_CUDA = -5,        /* CUDA runtime / driver error, message has the detail */
    HKB_ERR_TIMEOUT = -6      /* a bounded device-side wait gave up (see hkb_check_status) */
} hkb_status;

#define HKB_MXFP4_MODE_DOC 0    /* e = floor(log2 amax) - 2, nearest value, ties to smaller */
#define HKB_MXFP4_MODE_KERNEL 1 /* the reference device code's variant (rounded amax, truncation) */

/* ---- library ------------------------------------------------------------------------- */
int hkb_version(void);
const char* hkb_last_error(void);
/* Frees the per-device workspace (scale re-layout scratch, status word). */
int hkb_release(void);
/* Synchronises `stream` and returns HKB_ERR_TIMEOUT if any GEMM launched so far on the
 * current device abandoned a bounded wait (it then left its output incomplete); the failure is
 * cleared by the call.  Covers every entry point, hkb_gemm_mxfp4_static included, and allocates
 * nothing. */
int hkb_check_status(void* stream);
/* Name of the kernel variant that the calling thread's last GEMM call launched (tile width, scale
 * scheme, CTA pairs), e.g. "gemm_fp8_kernel<256,pts,pair>".  For tests and tuning: the variant is
 * chosen from the problem size and the SM count. */
const char* hkb_last_kernel(void);
/* Test hook for the bounded waits: hkb_gemm_fp8_pts (batch 1, no bias) whose producer leaves the
 * first K block of its first tile unloaded and whose waits give up after wait_limit_ns instead of
 * 2 s.  The kernel winds down by itself, frees its tensor memory and records the failure, which
 * hkb_check_status() then reports as HKB_ERR_TIMEOUT; C is left incomplete.  The device stays
 * usable.  No counterpart in the reference project. */
int hkb_debug_gemm_fp8_wait_probe(const void* A, const void* B, void* C, const float* sa,
                                  const float* sb, int64_t M, int64_t N, int64_t K,
                                  uint64_t wait_limit_ns, void* stream);

/* Timeline of the block-scale GEMM's per-K-block hand-off: hkb_gemm_fp8_blockscale (gn = 128, a problem
 * that takes the 256-wide kernel: N % 256 == 0 and at least two tiles per SM) run from a build of the same
 * kernel in which every CTA records SM-clock readings for the first 64 K blocks of its third tile into
 * trace, a device array u64 [SMs][20][64] (zeroed by the call; trace_bytes >= SMs * 20 * 64 * 8):
 * event 0 MMA thread saw the operands, 1 issued the K block's MMAs, 3 had them issued, 2 the producer got the
 * stage back, 4 + w epilogue warp w released the accumulator buffer, 12 + w epilogue warp w saw the partial
 * product.  C receives the same result as hkb_gemm_fp8_blockscale.  For tuning; no counterpart in the
 * reference project. */
int hkb_debug_gemm_fp8_blockscale_timeline(const void* A, const void* B, void* C, const float* sa,
                                           const float* sb, int64_t M, int64_t N, int64_t K,
                                           void* trace, int64_t trace_bytes, void* stream);

/* Tensor-core ceiling probe: every SM issues `batches` x 4 back-to-back tcgen05.mma instructions
 * (kind 0: FP8 e4m3, 128 x 256 x 32 each; kind 1: MXFP4 block-scaled, 128 x 256 x 64 each) on
 * operand tiles resident in shared memory; no loads or stores in the loop.  The caller times the
 * launch (CUDA events on `stream`); *flop_per_launch receives the flops it performs.  Used by the
 * benchmark as the measured FP8 / FP4 denominator.  No counterpart in the reference project. */
int hkb_debug_peak_mma(int kind, int64_t batches, double* flop_per_launch, void* stream);

/* ---- quantizers ---------------------------------------------------------------------- */

/* Per-row dynamic FP8: scales[m] = max(amax_m / 448, 1e-10), q = e4m3fn(clamp(x / scale)).
 * x bf16 [M, D] with row pitch ldx elements; q u8 [M, D]; scales f32 [M].  D % 8 == 0; x 16-byte
 * and q 8-byte aligned (fast path: D % 16 == 0, ldx % 16 == 0, x 32-byte and q 16-byte aligned).
 * Replaces per_token_quant_fwd(input, output, scales):
 *   kernels/quantization/quant/kernel.cpp:31-109,159-171 (re-targeted from INT8/127 to e4m3fn/448). */
int hkb_quant_fp8_per_token(const void* x, void* q, float* scales,
                            int64_t M, int64_t D, int64_t ldx, void* stream);

/* The reference kernel's own INT8 mode: scale = max(amax/127, 1e-10), q = rint(x/scale) in [-127,127].
 *   kernels/quantization/quant/kernel.cpp:92-107. */
int hkb_quant_int8_per_token(const void* x, void* q, float* scales,
                             int64_t M, int64_t D, int64_t ldx, void* stream);

/* 1x128 block FP8: one fp32 scale per 128 contiguous columns, scales f32 [M, D/128].
 * w (bf16 [D]) non-null selects the fused RMSNorm prologue y = x*rsqrt(mean x^2+eps)*w.
 * x 32-byte, q and w 16-byte aligned.
 * Replaces fused_rmsnorm_fp8_quant_fwd(input, weight, output, scales, eps):
 *   kernels/quantization/fused_fp8_quant/kernel.cpp:110-210,262-275. */
int hkb_quant_fp8_1x128(const void* x, const void* w_or_null, void* q, float* scales,
                        int64_t M, int64_t D, float eps, void* stream);

/* 128x128 block FP8 for weights: w bf16 [N, K] -> q u8 [N, K], scales f32 [K/128, N/128]
 * (transposed, the b_scale layout of the block-scale GEMM); w 32-byte, q 16-byte aligned.
 * No reference kernel; produces
 * the operand layout of kernels/gemm-basic/gemm_a8w8_blockscale/kernel.cpp:7,41,146. */
int hkb_quant_fp8_128x128(const void* w, void* q, float* scales,
                          int64_t N, int64_t K, void* stream);

/* MXFP4: e2m1 codes packed 2/byte (element 2i in the low nibble), one e8m0 byte per 32
 * contiguous elements.  codes u8 [M, D/2], scales u8 [M, D/32].  D % 32 == 0; x 32-byte,
 * codes 8-byte, scales 4-byte aligned.
 * Replaces fused_rmsnorm_mxfp4_quant_fwd(input, weight, output, scales, eps):
 *   kernels/quantization/fused_mxfp4_quant/kernel.cpp:71-169,172-249,301-314. */
int hkb_quant_mxfp4(const void* x, const void* w_or_null, void* codes, void* scales,
                    int64_t M, int64_t D, float eps, int mode, void* stream);

/* ---- GEMMs (all "NT": A [M,K] and B [N,K] are K-contiguous; C [M,N] bf16) ------------- */

/* C[b] = bf16( (A[b] @ B[b]^T) * sa[b][m] * sb[b][n] + bias[b][n] ), e4m3fn operands.
 * batch >= 1; tensors of consecutive batches are contiguous; bias (bf16 [batch, N]) may be NULL.
 * K % 128 == 0, N % 8 == 0; A, B, C, sb and bias 16-byte, sa 4-byte aligned.  Replaces
 *   gemm_a8w8_per_token_scale_tk.dispatch(A,B,C,a_scale,b_scale)
 *       kernels/gemm-basic/gemm_a8w8_per_token_scale/kernel.cpp:49-171
 *   gemm_a8w8_tk.dispatch(A,B,a_scale,b_scale,C)   kernels/gemm-basic/gemm_a8w8/kernel.cpp:46-175
 *   batched_gemm_a8w8_tk.dispatch(A,B,a_scale,b_scale,C,bias)
 *       kernels/gemm-batched/batched_gemm_a8w8/kernel.cpp:59-203 */
int hkb_gemm_fp8_pts(const void* A, const void* B, void* C, const float* sa, const float* sb,
                     const void* bias_or_null, int64_t batch, int64_t M, int64_t N, int64_t K,
                     void* stream);

/* Batched GEMM with the activation quantizer inside the main loop.  A bf16 [batch, M, K] is quantized
 * per row and per 64-wide K group while it is staged: m = max(|A_g|, 1e-10), a_scale = m * (1/448),
 * q = e4m3fn(clamp(A_g * (1/a_scale), +-448)); C[b] = bf16( (sum_g (q_g @ B_g^T) * a_scale_g) * b_scale
 * + bias[b] ), fp32 throughout.  B e4m3fn codes [batch, N, K], b_scale ONE float (per-tensor weight
 * scale, device memory), bias bf16 [batch, N] or NULL.  K % 64 == 0, N % 8 == 0; A 32-byte, B, C and
 * bias 16-byte aligned.  Replaces dispatch(a, b, b_scale, c, bias) of
 *   kernels/gemm-batched/batched_gemm_a8w8_ptgq/kernel.cpp:168-215,241-249
 * re-targeted from the INT8 range (127, no rounding of the quantized values in the reference's
 * arithmetic) to e4m3fn (448, round-to-nearest-even), the expression order kept. */
int hkb_gemm_fp8_ptgq(const void* A, const void* B, const float* b_scale, void* C,
                      const void* bias_or_null, int64_t batch, int64_t M, int64_t N, int64_t K,
                      void* stream);

/* C = bf16( sum_kb (A_kb @ B_kb^T) * sa[m, kb] * sb[kb, n / gn] ), e4m3fn operands,
 * sa f32 [M, K/128], sb f32 [K/128, N/gn], gn in {1, 128}.  K % 128 == 0, N % 128 == 0.
 * Replaces gemm_a8w8_blockscale_tk.dispatch(A,B,C,a_scale,b_scale):
 *   kernels/gemm-basic/gemm_a8w8_blockscale/kernel.cpp:51-180. */
int hkb_gemm_fp8_blockscale(const void* A, const void* B, void* C, const float* sa,
                            const float* sb, int64_t gn, int64_t M, int64_t N, int64_t K,
                            void* stream);

/* The block-scale GEMM (gn = 128) whose [M, N] result is written into n_dst (1..8) destinations of
 * row pitch ldc elements (ldc >= N, ldc % 16 == 0): C_dst[i] points at the first element of the
 * result's column slab inside destination i (32-byte aligned).  This is the column-sharded GEMM
 * with its all-gather fused in: rank r of g passes, for every rank j, the address of columns
 * [r*N, (r+1)*N) of rank j's assembled [M, g*N] matrix (peer-mapped device memory, its own first);
 * the epilogue writes each finished tile to all of them with plain stores, so the transfer over
 * NVLink overlaps the main loop of the following tiles and no collective runs afterwards.  The
 * caller orders the readers behind every rank's launch (a barrier).  C_dst is a HOST array.
 * No counterpart in the reference project (it has no multi-GPU code). */
int hkb_gemm_fp8_blockscale_scatter(const void* A, const void* B, void* const* C_dst, int n_dst,
                                    int64_t ldc, const float* sa, const float* sb, int64_t M,
                                    int64_t N, int64_t K, void* stream);

/* The column partition of the N-sharded GEMM: rank `rank` of `world_size` owns output columns (= rows of
 * B and columns of b_scale / 128) [*n0, *n1): N is cut into 128-wide blocks which are dealt out as evenly
 * as possible, the first (N/128) % world_size ranks get one more.  Host arithmetic only; the same rule as
 * hipkittens.sharded.shard_bounds.  No counterpart in the reference project. */
int hkb_shard_bounds(int64_t N, int64_t world_size, int64_t rank, int64_t* n0, int64_t* n1);

/* The same GEMM with the multiply-add epilogue fused in: C = bf16( c_a * gemm + c_b ), c_a and
 * c_b bf16 [M, N] (16-byte aligned), evaluated in fp32 before the one rounding to bf16.  Replaces
 * fused_gemm_a8w8_blockscale_mul_add_tk.dispatch(a,b,c,a_scale,b_scale,c_a,c_b):
 *   kernels/gemm-fused/fused_gemm_a8w8_blockscale_mul_add/kernel.cpp:154-193
 * (the reference's b_scale there is [K/128, N], i.e. gn = 1; gn = 128 is accepted as well). */
int hkb_gemm_fp8_blockscale_mul_add(const void* A, const void* B, void* C, const float* sa,
                                    const float* sb, int64_t gn, const void* c_a, const void* c_b,
                                    int64_t M, int64_t N, int64_t K, void* stream);

/* C[b] = bf16( dq(A[b]) @ dq(B[b])^T ), dq(v)[i,k] = e2m1(v[i,k]) * 2^(s[i,k/32]-127).
 * A u8 [batch, M, K/2], B u8 [batch, N, K/2], sfa u8 [batch, M, K/32], sfb u8 [batch, N, K/32].
 * K % 128 == 0, N % 8 == 0.  The scales are first re-laid-out for the tensor core into
 * library-owned scratch that is kept per (device, stream): calls on different streams of a device
 * may overlap on the GPU (up to 8 streams per device keep their own scratch; beyond that the least
 * recently used stream's scratch is recycled behind a device-wide synchronisation).  A call that
 * has to allocate or grow its stream's scratch calls cudaMalloc / cudaFree, so the first call of a
 * size on a stream must come before any stream capture.  Replaces
 *   gemm_afp4wfp4_tk.dispatch           kernels/gemm-basic/gemm_afp4wfp4/kernel.cpp:1-12,48-159
 *   batched_gemm_afp4wfp4_tk.dispatch   kernels/gemm-batched/batched_gemm_afp4wfp4/kernel.cpp:3-7,52-168
 * (operand spec from those files' header comments; the reference kernels themselves take
 * host-dequantized bf16). */
int hkb_gemm_mxfp4(const void* A, const void* B, void* C, const void* sfa, const void* sfb,
                   int64_t batch, int64_t M, int64_t N, int64_t K, void* stream);

/* Scale factors in the layout the tensor core reads ("tc layout"): per batch and 128-row block,
 * 512-byte atoms of 128 rows x 4 scale bytes (128 K elements), byte (r%32)*16 + (r/32)*4 + j for
 * row r and scale j, atoms of a row block consecutive along K; row blocks and K atoms are padded
 * (2*ceil(rows/256) + 2 blocks, an even number of atoms).  hkb_mxfp4_sf_tc_bytes gives the size of
 * that array (0 for invalid arguments); hkb_mxfp4_sf_to_tc fills it from row-major e8m0
 * [batch, rows, K/32] (sf 4-byte, sf_tc 16-byte aligned), padding included.  Weights are converted
 * once and reused; activations can be quantized straight into this layout (hkb_quant_mxfp4_tc).
 * hkb_gemm_mxfp4_tc is hkb_gemm_mxfp4 where each of sfa / sfb is either row-major (flag 0, re-laid
 * out per call as above) or already in the tc layout (flag 1, used in place: no scratch, no extra
 * launch).  With both flags set the call allocates nothing.  No counterpart in the reference
 * project, whose FP4 kernels take host-dequantized operands. */
int64_t hkb_mxfp4_sf_tc_bytes(int64_t batch, int64_t rows, int64_t K);
int hkb_mxfp4_sf_to_tc(const void* sf, void* sf_tc, int64_t batch, int64_t rows, int64_t K,
                       void* stream);
int hkb_gemm_mxfp4_tc(const void* A, const void* B, void* C, const void* sfa, int sfa_is_tc,
                      const void* sfb, int sfb_is_tc, int64_t batch, int64_t M, int64_t N,
                      int64_t K, void* stream);
/* hkb_quant_mxfp4 that also (or only: scales may be NULL) writes the scales in the tc layout for
 * an [M, D] operand of batch 1 (sf_tc of hkb_mxfp4_sf_tc_bytes(1, M, D) bytes, 16-byte aligned).
 * D % 128 == 0.  Every byte of the real rows' atoms is written, the padding atom of an odd D/128
 * included; padding ROWS are left untouched (they only meet output rows that are never stored). */
int hkb_quant_mxfp4_tc(const void* x, const void* w_or_null, void* codes, void* scales_or_null,
                       void* sf_tc, int64_t M, int64_t D, float eps, int mode, void* stream);

/* hkb_gemm_mxfp4 (batch 1) with the multiply-add epilogue fused in: C = bf16( c_a * gemm + c_b ),
 * c_a and c_b bf16 [M, N] (16-byte aligned).  Replaces
 * fused_gemm_afp4wfp4_mul_add_tk.dispatch(a,b,c,a_scale,b_scale,c_a,c_b):
 *   kernels/gemm-fused/fused_gemm_afp4wfp4_mul_add/kernel.cpp:31-39,182-191
 * (packed e2m1 + e8m0 operands as for hkb_gemm_mxfp4; the reference kernel takes host-dequantized
 * bf16 and fp32 scales per 32). */
int hkb_gemm_mxfp4_mul_add(const void* A, const void* B, void* C, const void* sfa, const void* sfb,
                           const void* c_a, const void* c_b, int64_t M, int64_t N, int64_t K,
                           void* stream);

/* The block-scale FP8 and the MXFP4 GEMM with the split-concatenate epilogue: with N = D*(S1+S2), column
 * n = d*(S1+S2) + s of the [M, N] result goes to c1[m, d, s] when s < S1 and to c2[m, d, s-S1] otherwise;
 * y [M, D, S3] is copied behind the first part, c1[m, d, S1:S1+S3] = y[m, d, :].  c1 bf16 [M, D, S1+S3],
 * c2 bf16 [M, D, S2], written straight from the GEMMs' epilogues (no [M, N] intermediate).  S1, S2, S3
 * multiples of 16 (S3 may be 0); c1, c2 32-byte, y 16-byte aligned; other arguments as for
 * hkb_gemm_fp8_blockscale / hkb_gemm_mxfp4 (batch 1).  Replace
 *   dispatch_fused_gemm_a8w8_bs_split_cat   kernels/gemm-fused/fused_gemm_a8w8_blockscale_split_cat/kernel.cpp:34-50,168-247
 *   dispatch_fused_gemm_afp4wfp4_split_cat  kernels/gemm-fused/fused_gemm_afp4wfp4_split_cat/kernel.cpp:34-45
 * (the reference gives these two no Python binding; its b_scale there is [K/128, N], gn = 1). */
int hkb_gemm_fp8_blockscale_split_cat(const void* A, const void* B, const float* sa, const float* sb,
                                      int64_t gn, const void* y, void* c1, void* c2, int64_t M,
                                      int64_t N, int64_t K, int64_t S1, int64_t S2, int64_t S3,
                                      void* stream);
int hkb_gemm_mxfp4_split_cat(const void* A, const void* B, const void* sfa, const void* sfb,
                             const void* y, void* c1, void* c2, int64_t M, int64_t N, int64_t K,
                             int64_t S1, int64_t S2, int64_t S3, void* stream);

/* Grouped (MoE) block-scale FP8 GEMM: output row r (rows sorted by expert) is
 *   Y[r, n] = bf16( sum_kb (X[tok(r), kb] @ W[e, n, kb]) * X_scale[tok(r), kb] * W_scale[e, kb, n/128] + bias[e, n] )
 * with tok(r) = GatherIndx[r] / n_expts_act (GatherIndx NULL: tok(r) = r) and e the expert of r's tile.
 * X e4m3fn [tokens, K]; W e4m3fn [E, N, K] (K-contiguous, like every GEMM here); Y bf16 [rows, N];
 * X_scale f32 [tokens, K/128]; W_scale f32 [E, K/128, N/128]; bias f32 [E, N] or NULL; ExptHist[e] rows
 * of expert e, ExptOffs[e] their first row; ExptData[grid_m]: per 128-row tile (expert | block << 16),
 * -1 = no tile.  All index arrays int32 in device memory.  K, N multiples of 128.  With GatherIndx the
 * rows are first copied into expert-sorted order in per-(device, stream) scratch (allocated on first
 * use).  Replaces moe_a8w8_blockscale(X, W, Y, X_scale, W_scale, bias, GatherIndx, ExptHist, ExptOffs,
 * ExptData, N, K, group_k, group_n, grid_m, grid_n, n_expts_act, strides...):
 *   kernels/moe-gemm/moe_op_gemm_a8w8_blockscale/kernel.cpp:26-176,201-246
 * for group_k = group_n = 128 and e4m3fn codes instead of int8. */
int hkb_moe_gemm_fp8_blockscale(const void* X, const void* W, void* Y, const float* X_scale,
                                const float* W_scale, const float* bias_or_null,
                                const int32_t* GatherIndx_or_null, const int32_t* ExptHist,
                                const int32_t* ExptOffs, const int32_t* ExptData, int64_t tokens,
                                int64_t rows, int64_t E, int64_t N, int64_t K, int64_t grid_m,
                                int64_t n_expts_act, void* stream);

/* Grouped (MoE) MXFP4 GEMM over a padded, expert-sorted row list: block mb (128 rows) of the list belongs to
 * expert expert_ids[mb] (-1: no expert, zeros are written); sorted row r names the flat (token, k) index
 * id = sorted_token_ids[r] (id >= num_valid_tokens: padding, skipped), reads activation row id / top_k and
 * writes output row id:
 *   C[id, n] = bf16( dq(A[id/top_k]) . dq(B[e, n]) * A_scale[0] * B_scale[e] * (mul_routed_weight ? topk_weights[id] : 1) )
 * A u8 [tokens, K/2] + A_mx_scale u8 [tokens, K/32]; B u8 [E, N, K/2] + B_mx_scale u8 [E, N, K/32] (K-contiguous);
 * C bf16 [num_valid_tokens, N]; A_scale (1 float), B_scale ([E]) and topk_weights may be NULL.  num_padded (the
 * length of sorted_token_ids) is a multiple of 128; K % 128 == 0, N % 8 == 0.  Rows and scales are first brought
 * into expert-sorted order / the tensor core's layout in per-(device, stream) scratch.  Replaces
 * moe_mxfp4(A, B, C, A_mx_scale, B_mx_scale, A_scale, B_scale, topk_weights, sorted_token_ids, expert_ids, N, K,
 * num_valid_tokens, top_k, mul_routed_weight, strides..., grid_m, grid_n):
 *   kernels/moe-gemm/moe_op_mxfp4/kernel.cpp:38-66,90-238,262-349. */
int hkb_moe_gemm_mxfp4(const void* A, const void* B, void* C, const void* A_mx_scale,
                       const void* B_mx_scale, const float* A_scale_or_null,
                       const float* B_scale_or_null, const float* topk_weights_or_null,
                       const int32_t* sorted_token_ids, const int32_t* expert_ids, int64_t tokens,
                       int64_t num_padded, int64_t E, int64_t N, int64_t K,
                       int64_t num_valid_tokens, int64_t top_k, int mul_routed_weight, void* stream);

/* quant_moe_tk: wire formats of the MoE activation/weight casts.  Replace
 *   quant_moe_tk.downcast_to_static_fp8(x, y, scale, M, N)
 *   quant_moe_tk.downcast_to_mxfp(mx_tensor, mx_scale, src, outer_dim, quant_dim, is_fp4)
 *   quant_moe_tk.upcast_from_mxfp(out, mx_scale, mx_tensor, outer_dim, quant_dim, is_fp4)
 *       kernels/moe-misc/quant_moe/kernel.cpp:74-107, 143-231, 289-359, 392-476
 * x / src / out bf16 row-major; y and FP8 codes 1 byte per element (e4m3fn); FP4 codes e2m1, two per
 * byte, element 2i in the low nibble; mx_scale one byte per 32 elements of the last dimension.
 *  - static: y = e4m3fn(clamp(x / scale[0], +-448)), true division, round-to-nearest-even
 *    (tests/test_moe.py:997-999; the reference device code truncates instead, :56-71).
 *  - downcast: byte = biased exponent of amax / QMAX rounded up to a power of two (:155-158; QMAX 448,
 *    or 6 for FP4), codes = x * 2^(127 - byte) rounded to nearest even, saturating.  An all-zero block
 *    gets byte 127 (the reference's Python path, test_parity.py:116-117; its device code writes 255,
 *    which its own up-cast turns into NaN).  The reference leaves the FP4 codes unwritten (:214-217);
 *    here they follow the same rule with QMAX 6.
 *  - upcast: out = bf16(decode(code) * float_from_bits(byte << 23)); byte 255 gives NaN (:313-321),
 *    byte 0 gives 0.
 * quant_dim % 32 == 0; src/out 32-byte, codes 16-byte, scales 4-byte aligned. */
int hkb_moe_downcast_static_fp8(const void* x, void* y, const float* scale, int64_t M, int64_t N,
                                void* stream);
int hkb_moe_downcast_mxfp(void* mx_tensor, void* mx_scale, const void* src, int64_t outer_dim,
                          int64_t quant_dim, int is_fp4, void* stream);
int hkb_moe_upcast_mxfp(void* out, const void* mx_scale, const void* mx_tensor, int64_t outer_dim,
                        int64_t quant_dim, int is_fp4, void* stream);

/* hkb_gemm_mxfp4 for callers that must not allocate device memory at call time (arena / pool
 * disciplines that account for every byte up front, serving loops that cannot take cudaMalloc's
 * device-wide synchronisation, devices whose memory the host has already claimed in full).
 * Same arguments and results as hkb_gemm_mxfp4; the re-laid-out scale factors go into an 8 MiB
 * array built into the library image instead of grown scratch, so it calls no cudaMalloc/cudaFree.
 * Limit: batch * (ceil(M/128) + ceil(N/128)) * ceil(K/256) * 1024 bytes <= 8 MiB (e.g. M + N <=
 * 32768 at K = 8192); beyond it HKB_ERR_BAD_SHAPE is returned and nothing is launched.  The first
 * call on each device resolves the array's device address: make it outside stream capture.  All
 * calls on a device share the array; calls that may overlap on the GPU race on it and must be
 * ordered by the caller.  It always runs the one-CTA kernel on 128-wide tiles, so on large problems
 * it is slower than hkb_gemm_mxfp4 (which picks 192-wide tiles and CTA pairs).  Bounded-wait
 * failures are reported by hkb_check_status like those of every other entry point.
 * No counterpart in the reference project. */
int hkb_gemm_mxfp4_static(const void* A, const void* B, void* C, const void* sfa, const void* sfb,
                          int64_t batch, int64_t M, int64_t N, int64_t K, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HKB200_H */
