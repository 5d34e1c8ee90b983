"""CPU oracle for the quantized GEMMs: dequantize, then matmul in fp32 (torch CPU).
TEST INFRASTRUCTURE (see package docstring).

Expressions followed:
  per-token   tests/test_gemm.py:183; kernels/gemm-basic/gemm_a8w8_per_token_scale/test_parity.py:45-46
  block-scale tests/test_gemm.py:148-153; kernels/gemm-basic/gemm_a8w8_blockscale/test_parity.py:57-76
  mxfp4       kernels/gemm-basic/gemm_afp4wfp4/test_parity.py:30-31 on operands dequantized as
              kernels/moe-gemm/moe_op_mxfp4/test_parity.py:36-46
  batched     tests/test_gemm.py:366-367 (bias added in fp32 before the bf16 store)
  MoE grouped kernels/moe-gemm/moe_op_gemm_a8w8_blockscale/test_parity.py:58-99
  ptgq        kernels/gemm-batched/batched_gemm_a8w8_ptgq/test_parity.py:40-82 (in-loop re-quantization)
  metric      tests/test_gemm.py:190-192
"""
import numpy as np
import torch

from .codecs import e4m3fn_to_f32, e8m0_to_f32, unpack_e2m1


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def _codes(a):
    if hasattr(a, "detach"):
        a = a.detach().cpu()
        if a.dtype != torch.uint8:
            a = a.view(torch.uint8)
        a = a.numpy()
    return np.asarray(a, dtype=np.uint8)


def _f32(a):
    if hasattr(a, "detach"):
        a = a.detach().cpu().float().numpy()
    return np.asarray(a, dtype=np.float32)


def gemm_fp8_per_token(Aq, Bq, sa, sb, bias=None):
    """Per-token-scale GEMM on e4m3fn code bytes (see gemm_per_token_f32)."""
    return gemm_per_token_f32(e4m3fn_to_f32(_codes(Aq)), e4m3fn_to_f32(_codes(Bq)), sa, sb, bias)


def gemm_per_token_f32(A, B, sa, sb, bias=None):
    """C[m,n] = (sum_k A[m,k] B[n,k]) * sa[m] * sb[n] (+ bias[n]) on already-decoded operand
    values; fp32 result [.., M, N].  Leading batch dimensions broadcast through torch.matmul."""
    A = _t(_f32(A))
    B = _t(_f32(B))
    sa = _t(_f32(sa)).reshape(*A.shape[:-1], 1)
    sb = _t(_f32(sb)).reshape(*B.shape[:-2], 1, B.shape[-2])
    C = (A @ B.transpose(-1, -2)) * sa * sb
    if bias is not None:
        C = C + _t(_f32(bias)).reshape(*B.shape[:-2], 1, B.shape[-2])
    return C.numpy()


def gemm_fp8_blockscale(Aq, Bq, sa, sb, group_k=128):
    """Block-scale GEMM on e4m3fn code bytes (see gemm_blockscale_f32)."""
    return gemm_blockscale_f32(e4m3fn_to_f32(_codes(Aq)), e4m3fn_to_f32(_codes(Bq)), sa, sb, group_k)


def gemm_blockscale_f32(A, B, sa, sb, group_k=128):
    """C = sum_kb (A_kb @ B_kb^T) * sa[:, kb, None] * expand(sb[kb, :]) on decoded operand values;
    sa [M, K/128], sb [K/128, N/gn] with gn = N / sb.shape[1]."""
    A = _t(_f32(A))
    B = _t(_f32(B))
    sa = _t(_f32(sa))
    sb = _t(_f32(sb))
    M, K = A.shape
    N = B.shape[0]
    gn = N // sb.shape[1]
    C = torch.zeros(M, N, dtype=torch.float32)
    for kg in range(K // group_k):
        ks = slice(kg * group_k, (kg + 1) * group_k)
        partial = A[:, ks] @ B[:, ks].T
        b_s = sb[kg].repeat_interleave(gn)[:N]
        C += partial * sa[:, kg, None] * b_s[None, :]
    return C.numpy()


def dequant_mxfp4(codes, scale_bytes):
    """[.., R, K/2] packed e2m1 + [.., R, K/32] e8m0 -> fp32 [.., R, K]."""
    v = unpack_e2m1(_codes(codes))
    s = e8m0_to_f32(_codes(scale_bytes))
    return (v.reshape(*s.shape, 32) * s[..., None]).reshape(v.shape).astype(np.float32)


def gemm_mxfp4(Aq, Bq, sfa, sfb):
    """C = dq(A) @ dq(B)^T in fp32; batch dimensions broadcast."""
    A = _t(dequant_mxfp4(Aq, sfa))
    B = _t(dequant_mxfp4(Bq, sfb))
    return (A @ B.transpose(-1, -2)).numpy()


def gemm_group32_f32(A, B, sa, sb, group=32):
    """C = sum_kb (A_kb @ B_kb^T) * sa[:, kb, None] * sb[:, kb][None, :] on decoded operand values
    with fp32 scales per `group` K elements for both operands, sa [M, K/group], sb [N, K/group]
    (kernels/gemm-fused/fused_gemm_afp4wfp4_mul_add/test_parity.py:22-37; tests/test_gemm.py:601-606).
    With power-of-two scales this equals gemm_mxfp4 on the same codes."""
    A = _t(_f32(A))
    B = _t(_f32(B))
    sa = _t(_f32(sa))
    sb = _t(_f32(sb))
    M, K = A.shape
    N = B.shape[0]
    C = torch.zeros(M, N, dtype=torch.float32)
    for kb in range(K // group):
        ks = slice(kb * group, (kb + 1) * group)
        C += (A[:, ks] @ B[:, ks].T) * sa[:, kb, None] * sb[:, kb][None, :]
    return C.numpy()


def gemm_ptgq(A, B, b_scale, bias=None, group=64, qmax=448.0, qmin=-448.0, cast="e4m3"):
    """GEMM with per-row, per-`group`-K dynamic quantization of A inside the K loop, restating
    kernels/gemm-batched/batched_gemm_a8w8_ptgq/test_parity.py:56-77 line by line (all fp32):
        m = clamp(max|A_g|, min=1e-10); a_scale = m * (1/qmax); recip = 1 / a_scale
        A_q = clamp(A_g * recip, qmin, qmax)   [then `cast`]
        acc += (A_q @ B_g^T) * a_scale;  after the loop acc *= b_scale;  acc += bias
    A [.., M, K] (bf16 values), B [.., N, K] decoded weight values, bias [.., 1, N] or None.
    The reference's own arithmetic is qmax=127, qmin=-128, cast=None (its quantized values are never
    rounded); the B200 build's is the default: e4m3fn range and round-to-nearest-even cast."""
    from .codecs import f32_to_e4m3fn
    A = _f32(A)
    B = _f32(B)
    K = A.shape[-1]
    acc = torch.zeros(*A.shape[:-1], B.shape[-2], dtype=torch.float32)
    inv = np.float32(1.0 / qmax)
    for k0 in range(0, K, group):
        Ag = A[..., k0:k0 + group]
        m = np.maximum(np.abs(Ag).max(axis=-1, keepdims=True), np.float32(1e-10)).astype(np.float32)
        a_scale = (m * inv).astype(np.float32)
        recip = (np.float32(1.0) / a_scale).astype(np.float32)
        Aq = np.clip((Ag * recip).astype(np.float32), np.float32(qmin), np.float32(qmax))
        if cast == "e4m3":
            Aq = e4m3fn_to_f32(f32_to_e4m3fn(Aq))
        elif cast is not None:
            raise ValueError(cast)
        acc += (_t(Aq) @ _t(B[..., k0:k0 + group]).transpose(-1, -2)) * _t(a_scale)
    acc = acc * float(np.float32(b_scale))
    if bias is not None:
        acc = acc + _t(_f32(bias)).reshape(*B.shape[:-2], 1, B.shape[-2])
    return acc.numpy()


def mul_add(G, c_a, c_b):
    """Fused epilogue of the *_mul_add GEMMs: c_a.float() * gemm_out + c_b.float(), in fp32, the
    GEMM result not yet rounded (tests/test_gemm.py:527 and :608;
    kernels/gemm-fused/fused_gemm_a8w8_blockscale_mul_add/test_parity.py:36-38)."""
    return (_f32(c_a) * _f32(G) + _f32(c_b)).astype(np.float32)


def moe_gemm_blockscale(X, W, x_scale, w_scale, gather, hist, offs, expt_data, n_expts_act, bias=None, block_m=128, group=128):
    """Grouped (MoE) block-scale GEMM, restating kernels/moe-gemm/moe_op_gemm_a8w8_blockscale/test_parity.py:58-99
    (device code: kernel.cpp:60-176): for every tile (expert e, block) of the tile list and every row r of that
    expert, token = gather[r] // n_expts_act (r itself without gather) and
        Y[r, n] = sum_kg (X[token, kg] @ W[e, n, kg]) * x_scale[token, kg] * w_scale[e, kg, n // group] (+ bias[e, n]).
    X [tokens, K] and W [E, N, K] are decoded operand values; returns fp32 [rows, N] (rows no tile covers stay 0)."""
    X = _f32(X)
    W = _f32(W)
    xs = _f32(x_scale)
    ws = _f32(w_scale)
    E, N, K = W.shape
    rows = len(gather) if gather is not None else X.shape[0]
    Y = np.zeros((rows, N), dtype=np.float32)
    for ed in np.asarray(expt_data).tolist():
        if ed < 0:
            continue
        e, blk = ed & 0xFFFF, ed >> 16
        M = int(hist[e])
        r0 = int(offs[e]) + blk * block_m
        r1 = int(offs[e]) + min(M, (blk + 1) * block_m)
        if r1 <= r0:
            continue
        tok = (np.asarray(gather[r0:r1]) // n_expts_act) if gather is not None else np.arange(r0, r1)
        acc = torch.zeros(r1 - r0, N, dtype=torch.float32)
        for kg in range(K // group):
            ks = slice(kg * group, (kg + 1) * group)
            part = _t(X[tok][:, ks]) @ _t(W[e][:, ks]).T
            acc += part * _t(xs[tok, kg])[:, None] * _t(np.repeat(ws[e, kg], group)[:N])[None, :]
        if bias is not None:
            acc += _t(_f32(bias)[e])[None, :]
        Y[r0:r1] = acc.numpy()
    return Y


def moe_gemm_mxfp4(A, B, A_mx, B_mx, a_scale, b_scale, sorted_ids, expert_ids, topk_weights, num_valid, top_k,
                   mul_weight=True, index="token", block_m=128):
    """Grouped (MoE) MXFP4 GEMM over a padded, expert-sorted row list.  A u8 [tokens, K/2] + A_mx u8 [tokens, K/32];
    B u8 [E, N, K/2] + B_mx u8 [E, N, K/32].  For block b with expert e = expert_ids[b] != -1 and sorted row
    t = b*block_m + lm with id = sorted_ids[t] < num_valid:
        result = dq(A[id // top_k]) . dq(B[e])^T * a_scale * b_scale[e]   (* weight when mul_weight)
    index="token"  -- the reference device code (kernels/moe-gemm/moe_op_mxfp4/kernel.cpp:118-131,215-238): output row
                      and weight index are `id`;
    index="sorted" -- the reference's Python restatement (test_parity.py:79-115): both are the sorted position t.
    Returns fp32 [num_valid or num_padded, N]."""
    Adq = dequant_mxfp4(A, A_mx)
    E = np.asarray(B).shape[0]
    Bdq = [dequant_mxfp4(np.asarray(B)[e], np.asarray(B_mx)[e]) for e in range(E)]
    N = Bdq[0].shape[0]
    sorted_ids = np.asarray(sorted_ids)
    rows = num_valid if index == "token" else len(sorted_ids)
    C = np.zeros((rows, N), dtype=np.float32)
    for b, e in enumerate(np.asarray(expert_ids).tolist()):
        if e < 0:
            continue
        t = np.arange(b * block_m, min((b + 1) * block_m, len(sorted_ids)))
        ids = sorted_ids[t]
        ok = ids < num_valid
        t, ids = t[ok], ids[ok]
        if len(ids) == 0:
            continue
        res = (_t(Adq[ids // top_k]) @ _t(Bdq[e]).T).numpy() * np.float32(np.float32(a_scale) * np.float32(np.asarray(b_scale)[e]))
        out = ids if index == "token" else t
        if mul_weight:
            res = res * _f32(topk_weights)[out][:, None]
        C[out] = res
    return C


def split_cat(G, y, S1, S2):
    """Split-concatenate epilogue of the *_split_cat GEMMs on a GEMM result G [M, D*(S1+S2)] and
    y [M, D, S3] (kernels/gemm-fused/fused_gemm_a8w8_blockscale_split_cat/test_parity.py:45-56):
    c1[:, d, :S1] = G[:, d*(S1+S2) : +S1], c2[:, d, :] = the S2 columns behind them, c1[:, d, S1:] = y[:, d, :].
    Returns (c1 [M, D, S1+S3], c2 [M, D, S2]) in fp32."""
    G = _f32(G)
    y = _f32(y)
    M, D, S3 = y.shape
    g = G.reshape(M, D, S1 + S2)
    return np.concatenate([g[:, :, :S1], y], axis=2).astype(np.float32), g[:, :, S1:].astype(np.float32).copy()


def rel_err(C, C_ref):
    """max |C - C_ref| / (max |C_ref| + 1e-8), both fp32 (tests/test_gemm.py:190-192)."""
    C = _f32(C).astype(np.float64)
    R = _f32(C_ref).astype(np.float64)
    return float(np.abs(C - R).max() / (np.abs(R).max() + 1e-8))
