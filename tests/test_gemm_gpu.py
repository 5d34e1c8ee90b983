"""GPU tier: the tcgen05 GEMMs against the CPU oracle (dequantize-then-matmul in fp32),
through the reference-facing `hipkittens` modules.  Tolerance, as stated for this path:
max|C - C_ref| / max|C_ref| <= 1e-2 with both sides in fp32 (tests/test_gemm.py:190-192 of the
reference uses the same metric with looser bars)."""
import os

import numpy as np
import pytest
import torch

from oracle import codecs, gemm, inputs, quant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2


def _report(C, ref, what):
    """Error summary that localises layout bugs: worst element, per-128x128-block maxima."""
    C = np.asarray(C, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(C - ref)
    denom = np.abs(ref).max() + 1e-8
    idx = np.unravel_index(err.argmax(), err.shape)
    msg = [f"{what}: rel_err={err.max() / denom:.4g} worst at {idx}: got {C[idx]:.6g} want {ref[idx]:.6g}; "
           f"nan={np.isnan(C).sum()} zeros={int((C == 0).sum())}/{C.size}"]
    e2 = err.reshape(-1, err.shape[-2], err.shape[-1])[0]
    bm, bn = min(128, e2.shape[0]), min(128, e2.shape[1])
    blocks = [[e2[i:i + bm, j:j + bn].max() / denom for j in range(0, min(e2.shape[1], 1024), bn)]
              for i in range(0, min(e2.shape[0], 1024), bm)]
    msg.append("block maxima (rows=M blocks, cols=N blocks): " +
               "; ".join(" ".join(f"{v:.2g}" for v in row) for row in blocks))
    rows_bad = np.where((e2 / denom > TOL).any(axis=1))[0]
    cols_bad = np.where((e2 / denom > TOL).any(axis=0))[0]
    msg.append(f"bad rows {rows_bad[:16]} (n={len(rows_bad)}), bad cols {cols_bad[:16]} (n={len(cols_bad)})")
    return "\n".join(msg)


def _check(C, ref, what, tol=TOL):
    C = C.float().cpu().numpy() if hasattr(C, "cpu") else C
    r = gemm.rel_err(C, ref)
    assert r <= tol, _report(C, ref, what)
    return r


def _status_ok():
    import ctypes
    lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                   "amd-kernels_b200", "kernels", "libhkb200.so"))
    lib.hkb_last_error.restype = ctypes.c_char_p
    rc = lib.hkb_check_status(None)
    assert rc == 0, lib.hkb_last_error().decode()


def _fp8_operands(M, N, K, batch=1, seed=42):
    """e4m3fn-representable operands with the reference tests' scale distributions
    (rand*0.1+0.01, tests/test_gemm.py:179-180): randn -> per-row quantize."""
    g = torch.Generator().manual_seed(seed)
    shape_a = (batch, M, K) if batch > 1 else (M, K)
    shape_b = (batch, N, K) if batch > 1 else (N, K)
    A = torch.randn(shape_a, generator=g).bfloat16()
    B = torch.randn(shape_b, generator=g).bfloat16()
    aq, _ = quant.quant_fp8_per_token(A.reshape(-1, K))
    bq, _ = quant.quant_fp8_per_token(B.reshape(-1, K))
    sa = (torch.rand(shape_a[:-1], generator=g) * 0.1 + 0.01).float()
    sb = (torch.rand(shape_b[:-1], generator=g) * 0.1 + 0.01).float()
    return aq.reshape(shape_a), bq.reshape(shape_b), sa, sb


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    t = t.to(DEV)
    return t.view(dtype) if dtype is not None else t


# ---- per-token / per-channel scales ------------------------------------------------------------

@pytest.mark.parametrize("shape", [(128, 128, 128), (512, 512, 512), (2048, 2048, 2048),   # the reference's sizes
                                   (128, 1024, 1024), (200, 1032, 384), (16, 2048, 1024), (1, 256, 128),
                                   (48, 512, 2560), (72, 640, 256), (384, 4608, 512)])
def test_gemm_per_token_scale(hk, shape):
    M, N, K = shape
    aq, bq, sa, sb = _fp8_operands(M, N, K)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(_dev(aq), _dev(bq), C, _dev(sa), _dev(sb))
    torch.cuda.synchronize()
    _status_ok()
    _check(C, gemm.gemm_fp8_per_token(aq, bq, sa, sb), f"per-token {shape}")


def test_gemm_a8w8_module_takes_scales_before_C(hk):
    aq, bq, sa, sb = _fp8_operands(256, 256, 256)
    C = torch.zeros(256, 256, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8.dispatch(_dev(aq, torch.float8_e4m3fn), _dev(bq, torch.float8_e4m3fn), _dev(sa), _dev(sb), C)
    torch.cuda.synchronize()
    _check(C, gemm.gemm_fp8_per_token(aq, bq, sa, sb), "a8w8 order")


def test_config1_quantize_then_gemm_end_to_end(hk):
    """Config 1: A [128,1024] ~N(0,1), W [1024,1024] ~N(0,0.02), both quantized per row on the
    GPU, GEMM on the GPU; everything compared with the oracle on the same inputs."""
    A, W = inputs.make_config("c1")
    M, K = A.shape
    N = W.shape[0]
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, 1, device=DEV)
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(N, 1, device=DEV)
    hk.per_token_quant_fwd(A.to(DEV), aq, sa)
    hk.per_token_quant_fwd(W.to(DEV), wq, sw)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(aq, wq, C, sa, sw)
    torch.cuda.synchronize()
    raq, rsa = quant.quant_fp8_per_token(A)
    rwq, rsw = quant.quant_fp8_per_token(W)
    assert np.array_equal(aq.cpu().numpy(), raq) and np.array_equal(wq.cpu().numpy(), rwq)
    Adq = torch.from_numpy(codecs.e4m3fn_to_f32(raq) * rsa)
    Wdq = torch.from_numpy(codecs.e4m3fn_to_f32(rwq) * rsw)
    _check(C, (Adq @ Wdq.T).numpy(), "config 1 vs (Aq*sa)(Wq*sw)^T")


@pytest.mark.parametrize("with_bias", [False, True])
def test_batched_gemm_a8w8(hk, with_bias):
    """B=4, 128^3 as in tests/test_gemm.py:349-390 of the reference, 4-D tensors with a leading 1."""
    Bn, M, N, K = 4, 128, 128, 128
    aq, bq, sa, sb = _fp8_operands(M, N, K, batch=Bn)
    bias = (torch.randn(Bn, N, generator=torch.Generator().manual_seed(5))).bfloat16() if with_bias else None
    C = torch.zeros(1, Bn, M, N, dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.a8w8.dispatch(_dev(aq).view(1, Bn, M, K), _dev(bq).view(1, Bn, N, K), _dev(sa).view(1, Bn, 1, M),
                                  _dev(sb).view(1, Bn, 1, N), C, None if bias is None else _dev(bias).view(1, Bn, 1, N))
    torch.cuda.synchronize()
    ref = gemm.gemm_fp8_per_token(aq, bq, sa, sb, None if bias is None else bias.float().numpy())
    _check(C[0], ref, f"batched bias={with_bias}")


def test_batched_gemm_ragged_sizes(hk):
    Bn, M, N, K = 3, 200, 264, 256
    aq, bq, sa, sb = _fp8_operands(M, N, K, batch=Bn)
    C = torch.zeros(Bn, M, N, dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.a8w8.dispatch(_dev(aq), _dev(bq), _dev(sa), _dev(sb), C)
    torch.cuda.synchronize()
    _check(C, gemm.gemm_fp8_per_token(aq, bq, sa, sb), "batched ragged")


def test_reference_golden_shapes_with_int_valued_operands(hk, golden_dir):
    """The reference's own case (int8 values, seed 42) restricted to values e4m3 holds exactly:
    operands are clamped to [-16, 16], where every integer is an e4m3 value, so the GEMM must
    reproduce the oracle's exact-integer accumulation."""
    g = np.load(os.path.join(golden_dir, "gemm_per_token_128x128x128.npz"))
    A = np.clip(g["A"], -16, 16).astype(np.float32)
    B = np.clip(g["B"], -16, 16).astype(np.float32)
    aq, bq = codecs.f32_to_e4m3fn(A), codecs.f32_to_e4m3fn(B)
    assert np.array_equal(codecs.e4m3fn_to_f32(aq), A)
    C = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(_dev(aq), _dev(bq), C, _dev(g["a_scale"]), _dev(g["b_scale"]))
    ref = torch.from_numpy(gemm.gemm_per_token_f32(A, B, g["a_scale"], g["b_scale"])).bfloat16()
    assert torch.equal(C.cpu(), ref), _report(C.float().cpu().numpy(), ref.float().numpy(), "int-valued golden")


def test_decode_shape_sampled_columns(hk):
    """Config 4a: M=16, N=28672, K=8192.  The oracle checks 1024 sampled output columns."""
    M, N, K = 16, 28672, 8192
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, 1, device=DEV)
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(N, 1, device=DEV)
    hk.per_token_quant_fwd(A, aq, sa)
    hk.per_token_quant_fwd(W, wq, sw)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(aq, wq, C, sa, sw)
    torch.cuda.synchronize()
    _status_ok()
    cols = torch.randperm(N, generator=torch.Generator().manual_seed(0))[:1024].sort().values
    ref = gemm.gemm_fp8_per_token(aq.cpu(), wq[cols.to(DEV)].cpu(), sa.cpu(), sw[cols.to(DEV)].cpu())
    _check(C[:, cols.to(DEV)], ref, "decode sampled columns")
    # every column (all tile widths of the balanced schedule) against an fp32 product on the device
    full = (aq.view(torch.float8_e4m3fn).float() @ wq.view(torch.float8_e4m3fn).float().T) * sa * sw.T
    _check(C, full.cpu().numpy(), "decode all columns vs device fp32")


@pytest.mark.parametrize("shape", [(1, 48, 128), (7, 2000, 256), (16, 10064, 256), (33, 17600, 128), (64, 9488, 384),
                                   (8, 1032, 256), (64, 16, 1024), (16, 37888, 128), (8, 40000, 128), (24, 30000, 256)])
def test_gemm_per_token_skinny_tile_widths(hk, shape):
    """M <= 64: columns are dealt out in 16-column units as tiles of unequal width (1 to 16 units,
    one tile per SM and round); these sizes hit narrow and wide tiles, every box size, a
    single-unit problem, two rounds, and N % 16 != 0 (fixed-width fallback)."""
    M, N, K = shape
    aq, bq, sa, sb = _fp8_operands(M, N, K, seed=7)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(_dev(aq), _dev(bq), C, _dev(sa), _dev(sb))
    torch.cuda.synchronize()
    _status_ok()
    _check(C, gemm.gemm_fp8_per_token(aq, bq, sa, sb), f"skinny {shape}")


def test_gemm_per_token_skinny_with_bias(hk):
    M, N, K = 16, 2000, 256
    aq, bq, sa, sb = _fp8_operands(M, N, K, seed=9)
    bias = torch.randn(1, N, generator=torch.Generator().manual_seed(5)).bfloat16()
    C = torch.full((1, M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.a8w8.dispatch(_dev(aq).view(1, M, K), _dev(bq).view(1, N, K), _dev(sa).view(1, M), _dev(sb).view(1, N), C,
                                  _dev(bias))
    torch.cuda.synchronize()
    _status_ok()
    _check(C[0], gemm.gemm_fp8_per_token(aq, bq, sa, sb, bias.float().numpy()[0]), "skinny bias")


# ---- the per-token kernels that large problems dispatch to ------------------------------------
# Which kernel runs is decided from the tile counts and the SM count (148 on B200): 256-wide tiles
# when ceil(M/128) * ceil(N/256) * batch >= 2 * SMs, as CTA pairs on 256 x 256 tiles when M > 128 and
# at least SMs / 2 such tiles exist; else 128-wide tiles when twice the SM count of those exist;
# else 64-wide tiles.  Each case asserts the variant through hkb_last_kernel().

def _sampled_rows_check(C, aq, bq, sa, sb, what, nrows=128, bias=None):
    """Oracle on `nrows` sampled rows (all columns), plus every element against an fp32 product on the device."""
    M = aq.shape[-2]
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(3))[:min(nrows, M)].sort().values
    ref = gemm.gemm_fp8_per_token(aq[..., rows.numpy(), :], bq, sa[..., rows], sb, bias)
    _check(C[..., rows.to(DEV), :], ref, what + " (sampled rows vs oracle)")
    full = torch.matmul(_dev(aq, torch.float8_e4m3fn).float(), _dev(bq, torch.float8_e4m3fn).float().transpose(-1, -2))
    full = full * _dev(sa).unsqueeze(-1) * _dev(sb).unsqueeze(-2)
    if bias is not None:
        full = full + _dev(torch.from_numpy(bias)).unsqueeze(-2)
    _check(C, full.cpu().numpy(), what + " (all elements vs device fp32)")


@pytest.mark.parametrize("shape,kernel", [
    ((2432, 4864, 512), "gemm_fp8_kernel<256,pts,pair>"),     # last 256-row block half empty
    ((2400, 4864, 512), "gemm_fp8_kernel<256,pts,pair>"),     # last 256-row block: 96 rows, all in the leader CTA
    ((4096, 14336, 256), "gemm_fp8_kernel<256,pts,pair>"),    # config 2's M and N
    ((2048, 4608, 256), "gemm_fp8_kernel<128,pts>"),
    ((2048, 4360, 256), "gemm_fp8_kernel<128,pts>"),          # N % 128 != 0: ragged last tile
    ((2048, 2048, 2048), "gemm_fp8_kernel<64,pts>"),
])
def test_gemm_per_token_large_variants(hk, shape, kernel):
    M, N, K = shape
    aq, bq, sa, sb = _fp8_operands(M, N, K, seed=21)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(_dev(aq), _dev(bq), C, _dev(sa), _dev(sb))
    assert hk.last_kernel() == kernel
    torch.cuda.synchronize()
    _status_ok()
    _sampled_rows_check(C, aq, bq, sa, sb, f"per-token {shape} {kernel}", nrows=256)


def test_per_token_8192_cubed_every_element_vs_device_fp32_and_exact_properties(hk):
    """The CTA-pair per-token kernel on 8192^3 (the shape its throughput is quoted on): all 67 M outputs against an
    fp32 matmul of the dequantized operands on the device (torch, TF32 off: a checker); doubling a_scale doubles every
    output exactly; permuting the rows of A permutes the rows of C exactly."""
    M = N = K = 8192
    g = torch.Generator(device=DEV).manual_seed(61)
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, device=DEV)
    bq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sb = torch.empty(N, device=DEV)
    hk.per_token_quant_fwd(torch.randn(M, K, generator=g, device=DEV).bfloat16(), aq, sa)
    hk.per_token_quant_fwd((torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16(), bq, sb)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(aq, bq, C, sa, sb)
    assert hk.last_kernel() == "gemm_fp8_kernel<256,pts,pair>"
    C2 = torch.empty_like(C)
    hk.gemm.a8w8_per_token.dispatch(aq, bq, C2, sa * 2.0, sb)
    torch.cuda.synchronize()
    assert torch.equal(C2, C * 2.0)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(3)).to(DEV)
    hk.gemm.a8w8_per_token.dispatch(aq[perm].contiguous(), bq, C2, sa[perm].contiguous(), sb)
    torch.cuda.synchronize()
    _status_ok()
    assert torch.equal(C2, C[perm])
    del C2
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = (aq.view(torch.float8_e4m3fn).float() * sa[:, None]) @ (bq.view(torch.float8_e4m3fn).float() * sb[:, None]).t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
    err = float((C.float() - ref).abs().max() / ref.abs().max())
    assert err <= TOL, err


def test_ptgq_bench_size_every_element_vs_device_fp32(hk):
    """The in-loop re-quantizing GEMM at the bench's size (4096 x 14336 x 4096): the activations quantized per row and
    64-wide K group on the device with torch (amax / 448, e4m3 cast), dequantized, multiplied in fp32 (TF32 off) with the
    decoded weights, scaled by b_scale, plus bias -- all 59 M outputs."""
    M, N, K = 4096, 14336, 4096
    g = torch.Generator(device=DEV).manual_seed(62)
    A = torch.randn(1, M, K, generator=g, device=DEV).bfloat16()
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(N, device=DEV)
    hk.per_token_quant_fwd(torch.randn(N, K, generator=g, device=DEV).bfloat16(), wq, sw)      # any e4m3 codes will do
    bias = torch.randn(1, 1, N, generator=g, device=DEV).bfloat16()
    bs = torch.full((1,), 0.02, device=DEV)
    C = torch.empty(1, M, N, dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.a8w8_ptgq.dispatch(A, wq.view(1, N, K), bs, C, bias)
    torch.cuda.synchronize()
    _status_ok()
    Ag = A[0].float().view(M, K // 64, 64)
    a_scale = Ag.abs().amax(dim=2, keepdim=True).clamp_min(1e-10) * (1.0 / 448.0)
    a_deq = ((Ag * (1.0 / a_scale)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float() * a_scale).view(M, K)
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = (a_deq @ wq.view(torch.float8_e4m3fn).float().t()) * 0.02 + bias[0].float()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
    err = float((C[0].float() - ref).abs().max() / ref.abs().max())
    assert err <= TOL, err


_SUBPROCESS_CASE = r"""
import json, os, sys
import numpy as np, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "amd-kernels_b200"))
sys.path.insert(0, os.path.join({root!r}, "tests"))
import hipkittens as hk
import test_gemm_gpu as T
from oracle import gemm
kind, M, N, K, batch = {case!r}
if kind == "pts":
    aq, bq, sa, sb = T._fp8_operands(M, N, K, seed=22)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=T.DEV)
    hk.gemm.a8w8_per_token.dispatch(T._dev(aq), T._dev(bq), C, T._dev(sa), T._dev(sb))
    name = hk.last_kernel()
    torch.cuda.synchronize()
    err = gemm.rel_err(C.float().cpu().numpy(), gemm.gemm_fp8_per_token(aq, bq, sa, sb))
else:
    ac, wc, asc, wsc = T._mxfp4_operands(M, N, K, batch=batch, seed=23)
    C = torch.full((batch, M, N), float("nan"), dtype=torch.bfloat16, device=T.DEV)
    hk.batched_gemm.afp4wfp4.dispatch(T._dev(ac), T._dev(wc), C, T._dev(asc), T._dev(wsc))
    name = hk.last_kernel()
    torch.cuda.synchronize()
    err = max(gemm.rel_err(C[b].float().cpu().numpy(), gemm.gemm_mxfp4(ac[b], wc[b], asc[b], wsc[b])) for b in range(batch))
print(json.dumps({{"kernel": name, "rel_err": float(err)}}))
"""


def _run_case_in_subprocess(case, env_extra):
    """Kernel selection switches are read once per process, so variants that need one run in a child."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, **env_extra)
    r = subprocess.run([sys.executable, "-c", _SUBPROCESS_CASE.format(root=root, case=case)], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_gemm_per_token_256_wide_single_cta_kernel():
    """The 256-wide one-CTA kernel is what large problems get when CTA pairs are switched off."""
    out = _run_case_in_subprocess(("pts", 1024, 9728, 256, 1), {"HKB_GEMM_PAIRS": "0"})
    assert out["kernel"] == "gemm_fp8_kernel<256,pts>"
    assert out["rel_err"] <= TOL, out


def test_config4b_batched_full_size_with_bias(hk):
    """Config 4b: B=8, M=512, N=4096, K=4096 (the CTA-pair kernel with the batch in its tile loop), with
    the bias of the reference's batched test (tests/test_gemm.py:349-390 there)."""
    Bn, M, N, K = 8, 512, 4096, 4096
    aq, bq, sa, sb = _fp8_operands(M, N, K, batch=Bn, seed=24)
    bias = torch.randn(Bn, N, generator=torch.Generator().manual_seed(5)).bfloat16()
    C = torch.full((1, Bn, M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.a8w8.dispatch(_dev(aq).view(1, Bn, M, K), _dev(bq).view(1, Bn, N, K), _dev(sa).view(1, Bn, 1, M),
                                  _dev(sb).view(1, Bn, 1, N), C, _dev(bias).view(1, Bn, 1, N))
    assert hk.last_kernel() == "gemm_fp8_kernel<256,pts,pair>"
    torch.cuda.synchronize()
    _status_ok()
    _sampled_rows_check(C[0], aq, bq, sa, sb, "config 4b", nrows=64, bias=bias.float().numpy())


def test_unaligned_scale_and_bias_pointers_are_refused(hk):
    """The epilogues read b_scale and bias with vector loads: offset views are an error, not a fault."""
    aq, bq, sa, sb = _fp8_operands(128, 128, 128)
    C = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    sb_off = torch.zeros(129, device=DEV)[1:]
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        hk.gemm.a8w8_per_token.dispatch(_dev(aq), _dev(bq), C, _dev(sa), sb_off)
    bias_off = torch.zeros(129, dtype=torch.bfloat16, device=DEV)[1:]
    with pytest.raises(RuntimeError, match="16-byte aligned"):
        hk.batched_gemm.a8w8.dispatch(_dev(aq), _dev(bq), _dev(sa), _dev(sb), C, bias_off)


# ---- activation quantizer inside the GEMM's main loop ---------------------------------------------

def _ptgq_case(Bn, M, N, K, seed, with_bias=True):
    """bf16 activations ~ N(0,1); weights as e4m3 codes of N(0,1) draws scaled into the e4m3 range; a scalar
    weight scale; bias ~ N(0,1) (distributions of kernels/gemm-batched/batched_gemm_a8w8_ptgq/test_parity.py:40-52)."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(Bn, M, K, generator=g).bfloat16()
    W = torch.randn(Bn, N, K, generator=g) * 64.0
    wq = codecs.f32_to_e4m3fn(W.numpy().clip(-448, 448))
    bias = torch.randn(Bn, 1, N, generator=g).bfloat16() if with_bias else None
    return A, wq, np.float32(0.05), bias


@pytest.mark.parametrize("case", [(4, 128, 128, 128, True),        # the reference's own size (B=4, 128^3, bias)
                                  (1, 200, 264, 192, False),       # ragged M and N, K = 3 groups (a half-filled stage)
                                  (2, 384, 512, 1024, True),
                                  (1, 2048, 4096, 2048, True)])    # several tiles per SM
def test_batched_gemm_a8w8_ptgq(hk, case):
    Bn, M, N, K, with_bias = case
    A, wq, b_scale, bias = _ptgq_case(Bn, M, N, K, seed=61, with_bias=with_bias)
    C = torch.full((1, Bn, M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    bs = torch.full((1, 1, 1, 1), float(b_scale), device=DEV)
    hk.batched_gemm.a8w8_ptgq.dispatch(A.to(DEV).view(1, Bn, M, K), _dev(wq).view(1, Bn, N, K), bs, C,
                                       None if bias is None else bias.to(DEV).view(1, Bn, 1, N))
    assert hk.last_kernel() == "gemm_fp8_ptgq_kernel"
    torch.cuda.synchronize()
    _status_ok()
    ref = gemm.gemm_ptgq(A.float().numpy(), codecs.e4m3fn_to_f32(wq), b_scale, None if bias is None else bias.float().numpy())
    _check(C[0], ref, f"ptgq {case}")


def test_batched_gemm_a8w8_ptgq_reference_golden(hk, golden_dir):
    """The reference's own case (its A, bias and scale; its int8 weights clipped to +-16, where every
    integer is an e4m3 value): the kernel follows the e4m3 oracle to 1e-2 and stays within the
    quantization noise of the reference's unrounded arithmetic."""
    g = np.load(os.path.join(golden_dir, "gemm_ptgq.npz"))
    A = torch.from_numpy(g["A_bf16"].view(np.int16).copy()).view(torch.bfloat16)
    bias = torch.from_numpy(g["bias_bf16"].view(np.int16).copy()).view(torch.bfloat16)
    Bc = np.clip(g["B_nk"].astype(np.float32), -16, 16)
    wq = codecs.f32_to_e4m3fn(Bc)
    Bn, M, K = A.shape
    N = Bc.shape[1]
    C = torch.zeros(Bn, M, N, dtype=torch.bfloat16, device=DEV)
    bs = torch.full((1,), float(g["b_scale"]), device=DEV)
    hk.batched_gemm.a8w8_ptgq.dispatch(A.to(DEV), _dev(wq), bs, C, bias.to(DEV))
    torch.cuda.synchronize()
    _status_ok()
    _check(C, gemm.gemm_ptgq(A.float().numpy(), Bc, g["b_scale"], bias.float().numpy()), "ptgq golden, e4m3 oracle")
    unrounded = gemm.gemm_ptgq(A.float().numpy(), Bc, g["b_scale"], bias.float().numpy(), qmax=127.0, qmin=-128.0, cast=None)
    assert gemm.rel_err(C.float().cpu().numpy(), unrounded) < 3e-2


# ---- grouped (MoE) block-scale GEMM -----------------------------------------------------------------

def _routing(tokens, E, top_k, seed, block_m=128):
    """Expert-sorted routing tables in the form of kernels/moe-gemm/moe_op_gemm_a8w8_blockscale/test_parity.py:29-58."""
    rng = np.random.RandomState(seed)
    assigns = rng.randint(0, E, (tokens, top_k))
    hist = np.bincount(assigns.ravel(), minlength=E).astype(np.int32)
    offs = np.concatenate([[0], np.cumsum(hist)[:-1]]).astype(np.int32)
    order = np.argsort(assigns.ravel(), kind="stable")
    gather = order.astype(np.int32)                        # flat (token * top_k + k) index of each sorted row
    tiles = [e | (b << 16) for e in range(E) for b in range((hist[e] + block_m - 1) // block_m)]
    return hist, offs, gather, np.array(tiles + [-1], dtype=np.int32)      # one empty entry at the end of the tile list


def _moe_call(hk, X, W_nk, Y, xs, ws, bias, gather, hist, offs, data, top_k):
    E, N, K = W_nk.shape
    kb, nb = K // 128, N // 128
    hk.moe_gemm.a8w8_blockscale.moe_a8w8_blockscale(
        X, W_nk.transpose(1, 2), Y, xs, ws, bias, gather, hist, offs, data, N, K, 128, 128, data.numel(), (N + 63) // 64, top_k,
        N, 1, K, 1, N * K, 1, K, kb, 1, kb * nb, nb, 1)


@pytest.mark.parametrize("tokens,E,top_k,K,N,with_bias", [(96, 4, 2, 256, 256, False), (700, 8, 2, 512, 1024, True),
                                                          (4096, 16, 4, 1024, 4096, True)])      # the last one takes the 256-wide tiles
def test_moe_gemm_blockscale(hk, tokens, E, top_k, K, N, with_bias):
    g = torch.Generator().manual_seed(81)
    X = torch.randn(tokens, K, generator=g).bfloat16()
    W = (torch.randn(E * N, K, generator=g) * 0.02).bfloat16()
    xq, xs = quant.quant_fp8_1x128(X)
    wq = np.empty((E, N, K), dtype=np.uint8); ws = np.empty((E, K // 128, N // 128), dtype=np.float32)
    for e in range(E):
        wq[e], ws[e] = quant.quant_fp8_128x128(W[e * N:(e + 1) * N])
    bias = torch.randn(E, N, generator=g) if with_bias else None
    hist, offs, gather, data = _routing(tokens, E, top_k, seed=5)
    rows = tokens * top_k
    Y = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _moe_call(hk, _dev(xq), _dev(wq), Y, _dev(xs), _dev(ws), None if bias is None else bias.to(DEV), _dev(gather), _dev(hist), _dev(offs),
              _dev(data), top_k)
    assert "grouped" in hk.last_kernel()
    torch.cuda.synchronize()
    _status_ok()
    ref = gemm.moe_gemm_blockscale(codecs.e4m3fn_to_f32(xq), codecs.e4m3fn_to_f32(wq), xs, ws, gather, hist, offs, data, top_k,
                                   None if bias is None else bias.numpy())
    _check(Y, ref, f"moe blockscale tokens={tokens} E={E}")


def test_moe_gemm_blockscale_bench_size_equals_the_dense_kernel_expert_by_expert(hk):
    """The grouped GEMM at the bench's size (8192 tokens x top-2 of 8 experts, N = 14336, K = 4096): every output row
    must equal, bit for bit, what the dense block-scale GEMM gives for that expert's rows and weights (same tile
    width, same K order) -- all 235 M outputs, ragged expert row counts included."""
    tokens, E, top_k, K, N = 8192, 8, 2, 4096, 14336
    g = torch.Generator(device=DEV).manual_seed(91)
    X = torch.randn(tokens, K, generator=g, device=DEV).bfloat16()
    xq = torch.empty(tokens, K, dtype=torch.uint8, device=DEV); xs = torch.empty(tokens, K // 128, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(X, None, xq, xs, 1e-6)
    wq = torch.empty(E, N, K, dtype=torch.uint8, device=DEV); ws = torch.empty(E, K // 128, N // 128, device=DEV)
    for e in range(E):
        W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
        hk.weight_quant_128x128(W, wq[e], ws[e])
    hist, offs, gather, data = _routing(tokens, E, top_k, seed=9)
    assert (hist % 128 != 0).any()
    rows = tokens * top_k
    Y = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    gd = _dev(gather)
    _moe_call(hk, xq, wq, Y, xs, ws, None, gd, _dev(hist), _dev(offs), _dev(data), top_k)
    assert hk.last_kernel() == "gemm_fp8_kernel<256,blockscale,grouped>"
    torch.cuda.synchronize()
    _status_ok()
    for e in range(E):
        r0, r1 = int(offs[e]), int(offs[e] + hist[e])
        tok = (gd[r0:r1] // top_k).long()
        Ce = torch.empty(r1 - r0, N, dtype=torch.bfloat16, device=DEV)
        hk.gemm.a8w8_blockscale.dispatch(xq[tok].contiguous(), wq[e], Ce, xs[tok].contiguous(), ws[e])
        assert hk.last_kernel() == "gemm_fp8_kernel<256,blockscale>"
        assert torch.equal(Y[r0:r1], Ce), f"expert {e}: grouped and dense results differ"
    _status_ok()


def test_moe_gemm_blockscale_reference_golden(hk, golden_dir):
    """The reference's own routing generator and reference function (group 128) on integer operands e4m3 holds exactly."""
    g = np.load(os.path.join(golden_dir, "moe_gemm_blockscale.npz"))
    xq = codecs.f32_to_e4m3fn(g["X"].astype(np.float32)); wq = codecs.f32_to_e4m3fn(g["W_nk"].astype(np.float32))
    rows, N = g["Y"].shape
    Y = torch.zeros(rows, N, dtype=torch.bfloat16, device=DEV)
    data = torch.from_numpy(g["expt_data"]).to(DEV)
    _moe_call(hk, _dev(xq), _dev(wq), Y, _dev(g["x_scale"]), _dev(g["w_scale"]), None, _dev(g["gather"]), _dev(g["hist"]), _dev(g["offs"]),
              data, int(g["top_k"]))
    torch.cuda.synchronize()
    _status_ok()
    _check(Y, g["Y"], "moe blockscale golden")


def test_moe_gemm_blockscale_without_gather_and_layout_check(hk):
    """GatherIndx=None: X already holds one row per sorted output row; an N-contiguous weight tensor is refused."""
    tokens, E, K, N = 300, 3, 256, 384
    g = torch.Generator().manual_seed(82)
    xq, xs = quant.quant_fp8_1x128(torch.randn(tokens, K, generator=g).bfloat16())
    wq = np.empty((E, N, K), dtype=np.uint8); ws = np.empty((E, K // 128, N // 128), dtype=np.float32)
    for e in range(E):
        wq[e], ws[e] = quant.quant_fp8_128x128((torch.randn(N, K, generator=g) * 0.02).bfloat16())
    hist = np.array([100, 0, 200], dtype=np.int32); offs = np.array([0, 100, 100], dtype=np.int32)       # an expert without rows
    data = np.array([0, 2, 2 | (1 << 16)], dtype=np.int32)
    Y = torch.full((tokens, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _moe_call(hk, _dev(xq), _dev(wq), Y, _dev(xs), _dev(ws), None, None, _dev(hist), _dev(offs), _dev(data), 1)
    torch.cuda.synchronize()
    _status_ok()
    ref = gemm.moe_gemm_blockscale(codecs.e4m3fn_to_f32(xq), codecs.e4m3fn_to_f32(wq), xs, ws, None, hist, offs, data, 1)
    _check(Y, ref, "moe blockscale, no gather")
    with pytest.raises(RuntimeError, match="K-contiguous"):
        Wkn = _dev(wq).transpose(1, 2).contiguous()         # physically [E, K, N]
        hk.moe_gemm.a8w8_blockscale.moe_a8w8_blockscale(_dev(xq), Wkn, Y, _dev(xs), _dev(ws), None, None, _dev(hist), _dev(offs), _dev(data),
                                                        N, K, 128, 128, 3, 6, 1, N, 1, K, 1, K * N, N, 1, 2, 1, 6, 3, 1)


def _moe_mxfp4_routing(tokens, E, top_k, seed, block_m=128):
    """Padded expert-sorted row list with every expert's rows padded to whole blocks (the form fused-MoE
    routing produces): sorted_ids (padding = tokens*top_k), expert per block, routing weight per flat index."""
    rng = np.random.RandomState(seed)
    assigns = rng.randint(0, E, (tokens, top_k))
    total = tokens * top_k
    ids, experts = [], []
    for e in range(E):
        mine = np.nonzero(assigns.ravel() == e)[0].astype(np.int32)
        pad = (-len(mine)) % block_m
        ids.append(np.concatenate([mine, np.full(pad, total, dtype=np.int32)]))
        experts += [e] * ((len(mine) + pad) // block_m)
    ids.append(np.full(block_m, total, dtype=np.int32))          # one block without an expert
    experts.append(-1)
    w = rng.rand(total).astype(np.float32)
    return np.concatenate(ids), np.array(experts, dtype=np.int32), w, total


def _moe_mxfp4_call(hk, A, B_nk, C, A_mx, B_mx_nk, a_scale, b_scale, w, ids, eids, num_valid, top_k, mul):
    E, N, K2 = B_nk.shape
    K = K2 * 2
    hk.moe_gemm.mxfp4.moe_mxfp4(A, B_nk.transpose(1, 2), C, A_mx, B_mx_nk.transpose(1, 2), a_scale, b_scale, w, ids, eids, N, K,
                                num_valid, top_k, mul, K // 2, 1, N * K // 2, 1, K // 2, N, 1, K // 32, 1, N * K // 32, 1, K // 32,
                                eids.numel(), (N + 127) // 128)


@pytest.mark.parametrize("tokens,E,top_k,K,N,mul", [(80, 3, 2, 128, 64, True), (600, 8, 2, 512, 1024, True), (5000, 8, 4, 1024, 3072, False)])
def test_moe_gemm_mxfp4(hk, tokens, E, top_k, K, N, mul):
    g = torch.Generator().manual_seed(91)
    ac, asc = quant.quant_mxfp4(torch.randn(tokens, K, generator=g).bfloat16())
    wc = np.empty((E, N, K // 2), dtype=np.uint8); wsc = np.empty((E, N, K // 32), dtype=np.uint8)
    for e in range(E):
        wc[e], wsc[e] = quant.quant_mxfp4((torch.randn(N, K, generator=g) * 0.02).bfloat16())
    ids, eids, w, total = _moe_mxfp4_routing(tokens, E, top_k, seed=6)
    a_scale = np.float32(0.5)
    b_scale = (np.random.RandomState(1).rand(E).astype(np.float32) + 0.5)
    C = torch.full((total, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _moe_mxfp4_call(hk, _dev(ac), _dev(wc), C, _dev(asc), _dev(wsc), torch.full((1,), float(a_scale), device=DEV), _dev(b_scale), _dev(w),
                    _dev(ids), _dev(eids), total, top_k, mul)
    assert "grouped" in hk.last_kernel()
    torch.cuda.synchronize()
    _status_ok()
    ref = gemm.moe_gemm_mxfp4(ac, wc, asc, wsc, a_scale, b_scale, ids, eids, w, total, top_k, mul_weight=mul, index="token")
    assert not torch.isnan(C.float()).any()               # every (token, k) row is named by the list
    _check(C, ref, f"moe mxfp4 tokens={tokens} E={E}")


def test_moe_gemm_mxfp4_bench_size_equals_the_dense_kernel_expert_by_expert(hk):
    """The grouped MXFP4 GEMM at the bench's size (8192 tokens x top-2 of 8 experts, N = K = 8192) with unit global
    scales and no routing-weight multiply: every output row must equal, bit for bit, the dense MXFP4 GEMM of that
    token's codes with its expert's weights (the dense call runs the CTA-pair kernel, the grouped one single CTAs:
    the order of the K steps is the same)."""
    tokens, E, top_k, K, N = 8192, 8, 2, 8192, 8192
    g = torch.Generator(device=DEV).manual_seed(92)
    X = torch.randn(tokens, K, generator=g, device=DEV).bfloat16()
    ac = torch.empty(tokens, K // 2, dtype=torch.uint8, device=DEV); asc = torch.empty(tokens, K // 32, dtype=torch.uint8, device=DEV)
    hk.fused_rmsnorm_mxfp4_quant_fwd(X, None, ac, asc, 1e-6)
    wc = torch.empty(E, N, K // 2, dtype=torch.uint8, device=DEV); wsc = torch.empty(E, N, K // 32, dtype=torch.uint8, device=DEV)
    for e in range(E):
        W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
        hk.fused_rmsnorm_mxfp4_quant_fwd(W, None, wc[e], wsc[e], 1e-6)
    ids, eids, w, total = _moe_mxfp4_routing(tokens, E, top_k, seed=8)
    C = torch.full((total, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    one = torch.ones(1, device=DEV)
    _moe_mxfp4_call(hk, ac, wc, C, asc, wsc, one, torch.ones(E, device=DEV), _dev(w), _dev(ids), _dev(eids), total, top_k, False)
    assert "grouped" in hk.last_kernel()
    torch.cuda.synchronize()
    _status_ok()
    assert not torch.isnan(C.float()).any()
    blocks = ids.reshape(-1, 128)
    for e in range(E):
        flat = blocks[eids == e].ravel()
        flat = torch.from_numpy(flat[flat < total]).long().to(DEV)
        tok = flat // top_k
        Ce = torch.empty(flat.numel(), N, dtype=torch.bfloat16, device=DEV)
        hk.gemm.afp4wfp4.dispatch(ac[tok].contiguous(), wc[e], Ce, asc[tok].contiguous(), wsc[e])
        assert torch.equal(C[flat], Ce), f"expert {e}: grouped and dense results differ"
    _status_ok()


def test_moe_gemm_mxfp4_reference_golden(hk, golden_dir):
    """The reference's own routing generator (blocks take the expert of their first row) and data; its Python
    restatement indexes output rows and weights by sorted position, its device code by flat (token, k) index:
    the kernel follows the device code, the same numbers land in other rows."""
    g = np.load(os.path.join(golden_dir, "moe_gemm_mxfp4.npz"))
    nv, tk = int(g["num_valid"]), int(g["top_k"])
    valid = g["sorted_ids"] < nv
    w_by_id = np.zeros(nv, dtype=np.float32)
    w_by_id[g["sorted_ids"][valid]] = g["weights_sorted"][valid]
    N = g["B_nk"].shape[1]
    C = torch.zeros(nv, N, dtype=torch.bfloat16, device=DEV)
    _moe_mxfp4_call(hk, _dev(g["A"]), _dev(g["B_nk"]), C, _dev(g["A_mx"]), _dev(g["B_mx_nk"]), torch.full((1,), float(g["a_scale"]), device=DEV),
                    _dev(g["b_scale"]), _dev(w_by_id), _dev(g["sorted_ids"]), _dev(g["expert_ids"]), nv, tk, True)
    torch.cuda.synchronize()
    _status_ok()
    _check(C[torch.from_numpy(g["sorted_ids"][valid]).long().to(DEV)], g["C_sorted"][valid], "moe mxfp4 golden")


# ---- bounded waits -----------------------------------------------------------------------------

def test_bounded_wait_gives_up_by_itself_and_the_device_stays_usable(hk):
    """A wait that nothing will ever satisfy: the probe's producer leaves the only K block of a 128^3
    problem unloaded and the waits are limited to 2 ms.  The MMA role gives up, raises the CTA's abort
    flag, every role winds down, tensor memory is freed, the kernel returns; hkb_check_status() reports
    the timeout once; an ordinary GEMM right after is correct."""
    import ctypes
    lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                   "amd-kernels_b200", "kernels", "libhkb200.so"))
    lib.hkb_last_error.restype = ctypes.c_char_p
    assert lib.hkb_check_status(None) == 0
    aq, bq, sa, sb = _fp8_operands(128, 128, 128)
    d = [_dev(aq), _dev(bq), _dev(sa), _dev(sb)]
    C = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    vp = ctypes.c_void_p
    i64 = ctypes.c_int64
    stream = vp(torch.cuda.current_stream().cuda_stream)
    rc = lib.hkb_debug_gemm_fp8_wait_probe(vp(d[0].data_ptr()), vp(d[1].data_ptr()), vp(C.data_ptr()), vp(d[2].data_ptr()),
                                           vp(d[3].data_ptr()), i64(128), i64(128), i64(128), ctypes.c_uint64(2_000_000), stream)
    assert rc == 0, lib.hkb_last_error().decode()
    rc = lib.hkb_check_status(stream)
    assert rc == -6, f"expected HKB_ERR_TIMEOUT, got {rc}: {lib.hkb_last_error().decode()}"
    assert b"bounded wait" in lib.hkb_last_error()
    assert lib.hkb_check_status(stream) == 0            # reported once, then cleared
    C2 = torch.full((128, 128), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_per_token.dispatch(d[0], d[1], C2, d[2], d[3])
    torch.cuda.synchronize()
    _status_ok()
    _check(C2, gemm.gemm_fp8_per_token(aq, bq, sa, sb), "GEMM after an abandoned wait")


# ---- block scales ---------------------------------------------------------------------------------

@pytest.mark.parametrize("shape,gn", [((128, 128, 256), 1), ((128, 128, 128), 128), ((256, 256, 512), 128),
                                      ((512, 512, 512), 1), ((200, 384, 1024), 128), ((1024, 4096, 2048), 128),
                                      # more than one 32-K-block chunk of staged scales: 36, 65 (odd) and 96 K blocks
                                      ((128, 256, 4608), 128), ((256, 128, 8320), 128), ((384, 512, 12288), 128)])
def test_gemm_blockscale_reference_scale_distribution(hk, shape, gn):
    """Shapes and scale distributions of the reference (tests/test_gemm.py:128-162: 128x128x256, gn=1;
    per-directory reference with generic gn), operands e4m3-representable."""
    M, N, K = shape
    aq, bq, _, _ = _fp8_operands(M, N, K)
    g = torch.Generator().manual_seed(7)
    sa = torch.rand(M, K // 128, generator=g) * 0.1 + 0.01
    sb = torch.rand(K // 128, N // gn, generator=g) * 0.1 + 0.01
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(_dev(aq), _dev(bq), C, _dev(sa), _dev(sb))
    torch.cuda.synchronize()
    _status_ok()
    _check(C, gemm.gemm_fp8_blockscale(aq, bq, sa, sb), f"blockscale {shape} gn={gn}")


def test_config2_shrunk_quantize_then_blockscale_gemm(hk):
    """Config 2 distributions (outlier channels x20, 1x128 / 128x128 scales) at M=512, N=2048, K=4096:
    quantizers and GEMM on the GPU, oracle on the same inputs."""
    A, W = inputs.make_inputs(512, 2048, 4096, outliers=True)
    M, K = A.shape
    N = W.shape[0]
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, K // 128, device=DEV)
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(K // 128, N // 128, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(A.to(DEV), None, aq, sa, 1e-6)
    hk.weight_quant_128x128(W.to(DEV), wq, sw)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(aq, wq, C, sa, sw)
    torch.cuda.synchronize()
    raq, rsa = quant.quant_fp8_1x128(A)
    rwq, rsw = quant.quant_fp8_128x128(W)
    assert np.array_equal(aq.cpu().numpy(), raq) and np.array_equal(wq.cpu().numpy(), rwq)
    ref = gemm.gemm_fp8_blockscale(raq, rwq, rsa, rsw)
    _check(C, ref, "config 2 (shrunk)")
    # quantization error against the unquantized bf16 product stays small despite the outliers
    assert gemm.rel_err(C.float().cpu().numpy(), (A.float() @ W.float().T).numpy()) < 0.05


def test_config2_full_size_sampled_rows(hk):
    """Config 2 at full size (4096 x 14336 x 4096); the oracle checks 96 sampled rows of C."""
    M, N, K = 4096, 14336, 4096
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    idx = torch.randperm(K, generator=torch.Generator().manual_seed(42))[:41].to(DEV)
    A[:, idx] = (A[:, idx].float() * 20).bfloat16()
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, K // 128, device=DEV)
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(K // 128, N // 128, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(A, None, aq, sa, 1e-6)
    hk.weight_quant_128x128(W, wq, sw)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(aq, wq, C, sa, sw)
    torch.cuda.synchronize()
    _status_ok()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:96].sort().values.to(DEV)
    ref = gemm.gemm_fp8_blockscale(aq[rows].cpu(), wq.cpu(), sa[rows].cpu(), sw.cpu())
    _check(C[rows], ref, "config 2 full size, sampled rows")


def _blockscale_all_elements_vs_device_fp32(hk, M, N, K, what, col_chunk):
    """Every element of the block-scale GEMM against an fp32 evaluation on the device (torch matmul with TF32 off,
    a checker only): C = (codes_a * sa per 128-K block) @ (codes_w * sb per 128 x 128 block)^T, N in chunks.
    Also the exact property that doubling a_scale doubles every bf16 output bit for bit."""
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, K // 128, device=DEV)
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(K // 128, N // 128, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(A, None, aq, sa, 1e-6)
    hk.weight_quant_128x128(W, wq, sw)
    del A, W
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(aq, wq, C, sa, sw)
    assert hk.last_kernel() == "gemm_fp8_kernel<256,blockscale>"
    C2 = torch.empty_like(C)
    hk.gemm.a8w8_blockscale.dispatch(aq, wq, C2, sa * 2.0, sw)
    torch.cuda.synchronize()
    _status_ok()
    assert torch.equal(C2, C * 2.0), f"{what}: doubling a_scale must double every output exactly"
    del C2
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        a_deq = aq.view(torch.float8_e4m3fn).float() * sa.repeat_interleave(128, dim=1)
        worst, peak = 0.0, 0.0
        for n0 in range(0, N, col_chunk):
            n1 = min(N, n0 + col_chunk)
            w_deq = wq[n0:n1].view(torch.float8_e4m3fn).float()
            w_deq *= sw[:, n0 // 128:(n1 + 127) // 128].repeat_interleave(128, dim=1)[:, :n1 - n0].t().repeat_interleave(128, dim=1)
            ref = a_deq @ w_deq.t()
            worst = max(worst, float((C[:, n0:n1].float() - ref).abs().max()))
            peak = max(peak, float(ref.abs().max()))
            del w_deq, ref
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
    assert worst / peak <= TOL, f"{what}: max |C - ref| / max |ref| = {worst / peak:.3e}"


def test_config2_full_size_every_element_vs_device_fp32(hk):
    _blockscale_all_elements_vs_device_fp32(hk, 4096, 14336, 4096, "config 2", 14336)


def test_config5_full_size_every_element_vs_device_fp32(hk):
    """Config 5 on one GPU (16384 x 57344 x 8192, 0.94 G outputs), the reference matmul in eight column chunks."""
    _blockscale_all_elements_vs_device_fp32(hk, 16384, 57344, 8192, "config 5", 7168)


@pytest.mark.parametrize("shape", [(384, 512, 512), (2304, 4608, 256)])      # 128-wide and 256-wide tile kernels
def test_blockscale_result_scattered_into_column_slabs_of_wider_matrices(hk, shape):
    """The multi-GPU form of the GEMM on one device: the [M, N] result goes into columns [col0, col0+N)
    of three wider row-major matrices (stand-ins for three GPUs' assembled outputs); every copy must
    equal the plain GEMM bit for bit and nothing outside the slab may be touched."""
    M, N, K = shape
    aq, bq, _, _ = _fp8_operands(M, N, K, seed=51)
    g = torch.Generator().manual_seed(7)
    sa = torch.rand(M, K // 128, generator=g) * 0.1 + 0.01
    sb = torch.rand(K // 128, N // 128, generator=g) * 0.1 + 0.01
    d = [_dev(aq), _dev(bq), _dev(sa), _dev(sb)]
    plain = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(d[0], d[1], plain, d[2], d[3])
    ldc, col0 = 3 * N + 256, N + 128
    outs = [torch.full((M, ldc), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    hk.gemm.a8w8_blockscale.dispatch_scatter(d[0], d[1], [o.data_ptr() + col0 * 2 for o in outs], ldc, d[2], d[3])
    assert "scatter" in hk.last_kernel()
    torch.cuda.synchronize()
    _status_ok()
    for o in outs:
        assert torch.equal(o[:, col0:col0 + N], plain)
        assert bool((o[:, :col0] == 7.0).all()) and bool((o[:, col0 + N:] == 7.0).all())
    _check(plain, gemm.gemm_fp8_blockscale(aq, bq, sa, sb), f"blockscale scatter {shape}")


def test_blockscale_timeline_build_gives_the_same_result_and_ordered_clock_readings(hk):
    """The diagnostic build of the 256-wide block-scale kernel: bit-equal output, and for every CTA's third
    tile the per-K-block readings come in the order the hand-off imposes: operands seen <= MMAs issued <
    first epilogue warp sees the partial < that warp releases the buffer; a buffer's next MMAs are issued
    after its last release."""
    M, N, K = 2048, 7168, 1024                   # 16 x 28 = 448 tiles: three per CTA on 148 SMs
    aq, bq, _, _ = _fp8_operands(M, N, K, seed=77)
    g = torch.Generator().manual_seed(3)
    sa = torch.rand(M, K // 128, generator=g) * 0.1 + 0.01
    sb = torch.rand(K // 128, N // 128, generator=g) * 0.1 + 0.01
    d = [_dev(aq), _dev(bq), _dev(sa), _dev(sb)]
    plain = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(d[0], d[1], plain, d[2], d[3])
    assert hk.last_kernel() == "gemm_fp8_kernel<256,blockscale>"
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    traced = torch.empty_like(plain)
    trace = torch.full((sms, 20, 64), -1, dtype=torch.int64, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch_timeline(d[0], d[1], traced, d[2], d[3], trace)
    assert "timeline" in hk.last_kernel()
    torch.cuda.synchronize()
    _status_ok()
    assert torch.equal(traced, plain)
    t = trace.cpu().numpy()
    kbs = K // 128
    ctas = [c for c in range(sms) if c + 2 * sms < 448]
    assert len(ctas) >= 100
    for c in ctas:
        full, issue, issued = t[c, 0, :kbs], t[c, 1, :kbs], t[c, 3, :kbs]
        rel, seen = t[c, 4:12, :kbs], t[c, 12:20, :kbs]
        assert (t[c, :, :kbs] > 0).all() and (t[c, :, kbs:] == 0).all()
        assert (full <= issue).all() and (issue < issued).all()
        assert (issue < seen.min(0)).all() and (seen < rel).all()
        assert (issue[2:] > rel.max(0)[:-2]).all()          # two accumulator buffers
    with pytest.raises(RuntimeError):                        # a problem that takes the 128-wide kernel has no timeline build
        small = torch.empty(256, 512, dtype=torch.bfloat16, device=DEV)
        hk.gemm.a8w8_blockscale.dispatch_timeline(d[0][:256], d[1][:512], small, d[2][:256], _dev(sb[:, :4].contiguous()), trace)


def test_config5_single_gpu_shard_shape_sampled_rows(hk):
    """Config 5's per-GPU problem at 8 GPUs (16384 x 7168 x 8192: one rank's column shard), config 5's
    distributions; the oracle checks 64 sampled rows."""
    M, N, K = 16384, 7168, 8192
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    idx = torch.randperm(K, generator=torch.Generator().manual_seed(42))[:K // 100].to(DEV)
    A[:, idx] = (A[:, idx].float() * 20).bfloat16()
    aq = torch.empty(M, K, dtype=torch.uint8, device=DEV); sa = torch.empty(M, K // 128, device=DEV)
    wq = torch.empty(N, K, dtype=torch.uint8, device=DEV); sw = torch.empty(K // 128, N // 128, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(A, None, aq, sa, 1e-6)
    hk.weight_quant_128x128(W, wq, sw)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(aq, wq, C, sa, sw)
    assert hk.last_kernel() == "gemm_fp8_kernel<256,blockscale>"
    torch.cuda.synchronize()
    _status_ok()
    assert not torch.isnan(C.float()).any()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:64].sort().values.to(DEV)
    ref = gemm.gemm_fp8_blockscale(aq[rows].cpu(), wq.cpu(), sa[rows].cpu(), sw.cpu())
    _check(C[rows], ref, "config 5 shard shape, sampled rows")


# ---- MXFP4 ----------------------------------------------------------------------------------------

def _mxfp4_operands(M, N, K, batch=1, seed=42):
    g = torch.Generator().manual_seed(seed)
    sa = (batch, M, K) if batch > 1 else (M, K)
    sb = (batch, N, K) if batch > 1 else (N, K)
    A = torch.randn(sa, generator=g).bfloat16()
    W = (torch.randn(sb, generator=g) * 0.02).bfloat16()
    ac, asc = quant.quant_mxfp4(A.reshape(-1, K))
    wc, wsc = quant.quant_mxfp4(W.reshape(-1, K))
    return (ac.reshape(*sa[:-1], K // 2), wc.reshape(*sb[:-1], K // 2),
            asc.reshape(*sa[:-1], K // 32), wsc.reshape(*sb[:-1], K // 32))


@pytest.mark.parametrize("shape", [(128, 128, 256), (128, 128, 128), (256, 256, 256), (1024, 1024, 1024),
                                   (200, 264, 512), (128, 128, 384), (512, 2048, 8192),
                                   (2304, 3264, 256), (4096, 4680, 512),         # wide (192-column) tiles, ragged N
                                   (2400, 3072, 256), (2432, 3080, 384)])        # CTA pairs whose last row block is partial / half empty
def test_gemm_mxfp4(hk, shape):
    M, N, K = shape
    ac, wc, asc, wsc = _mxfp4_operands(M, N, K)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.afp4wfp4.dispatch(_dev(ac), _dev(wc), C, _dev(asc), _dev(wsc))
    torch.cuda.synchronize()
    _status_ok()
    _check(C, gemm.gemm_mxfp4(ac, wc, asc, wsc), f"mxfp4 {shape}")


def test_gemm_mxfp4_rejects_host_dequantized_form(hk):
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="packed e2m1"):
        hk.gemm.afp4wfp4.dispatch(x, x, x)


def test_batched_gemm_mxfp4_reference_golden(hk, golden_dir):
    """The reference's batched FP4 case (B=4, 128^3, seed 42; kernels/gemm-batched/
    batched_gemm_afp4wfp4/test_parity.py:27-63) as packed codes + e8m0 bytes."""
    g = np.load(os.path.join(golden_dir, "gemm_afp4_batched.npz"))
    Bn, M, _ = g["A"].shape
    N = g["B"].shape[1]
    C = torch.zeros(1, Bn, M, N, dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.afp4wfp4.dispatch(_dev(g["A"]), _dev(g["B"]), C, _dev(g["a_scales"]), _dev(g["b_scales"]))
    torch.cuda.synchronize()
    ref = torch.from_numpy(g["C_bf16"].view(np.int16).copy()).view(torch.bfloat16).float().numpy()
    _check(C[0], ref, "batched mxfp4 golden")


def test_config3_quantize_then_mxfp4_gemm_sampled(hk):
    """Config 3 distributions at 2048 x 8192 x 8192: MXFP4 quantizers and GEMM on the GPU; the oracle
    re-derives 128 sampled rows from the GPU codes (which are themselves checked bit-exact elsewhere)."""
    M, N, K = 2048, 8192, 8192
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    ac = torch.empty(M, K // 2, dtype=torch.uint8, device=DEV); asc = torch.empty(M, K // 32, dtype=torch.uint8, device=DEV)
    wc = torch.empty(N, K // 2, dtype=torch.uint8, device=DEV); wsc = torch.empty(N, K // 32, dtype=torch.uint8, device=DEV)
    hk.fused_rmsnorm_mxfp4_quant_fwd(A, None, ac, asc, 1e-6)
    hk.fused_rmsnorm_mxfp4_quant_fwd(W, None, wc, wsc, 1e-6)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.afp4wfp4.dispatch(ac, wc, C, asc, wsc)
    torch.cuda.synchronize()
    _status_ok()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(2))[:128].sort().values.to(DEV)
    ref = gemm.gemm_mxfp4(ac[rows].cpu(), wc.cpu(), asc[rows].cpu(), wsc.cpu())
    _check(C[rows], ref, "config 3 (M=2048) sampled rows")


def test_config3_full_size_sampled_rows(hk):
    """Config 3 at full size (8192^3, the CTA-pair kernel on 256 x 192 tiles); 96 sampled rows vs the oracle."""
    M = N = K = 8192
    g = torch.Generator(device=DEV).manual_seed(42)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    ac = torch.empty(M, K // 2, dtype=torch.uint8, device=DEV); asc = torch.empty(M, K // 32, dtype=torch.uint8, device=DEV)
    wc = torch.empty(N, K // 2, dtype=torch.uint8, device=DEV); wsc = torch.empty(N, K // 32, dtype=torch.uint8, device=DEV)
    hk.fused_rmsnorm_mxfp4_quant_fwd(A, None, ac, asc, 1e-6)
    hk.fused_rmsnorm_mxfp4_quant_fwd(W, None, wc, wsc, 1e-6)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.gemm.afp4wfp4.dispatch(ac, wc, C, asc, wsc)
    assert hk.last_kernel() == "gemm_mxfp4_pair_kernel<256x192>"
    torch.cuda.synchronize()
    _status_ok()
    assert not torch.isnan(C.float()).any()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(2))[:96].sort().values.to(DEV)
    ref = gemm.gemm_mxfp4(ac[rows].cpu(), wc.cpu(), asc[rows].cpu(), wsc.cpu())
    _check(C[rows], ref, "config 3 full size, sampled rows")


def test_config3_full_size_every_element_and_exact_scale_doubling(hk):
    """Config 3 at full size: raising every activation scale byte by one (x2 in e8m0) must double all 67 M bf16
    outputs of the CTA-pair kernel bit for bit; and all of them against an fp32 matmul on the device."""
    M = N = K = 8192
    g = torch.Generator(device=DEV).manual_seed(43)
    A = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    W = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    ac = torch.empty(M, K // 2, dtype=torch.uint8, device=DEV); asc = torch.empty(M, K // 32, dtype=torch.uint8, device=DEV)
    wc = torch.empty(N, K // 2, dtype=torch.uint8, device=DEV); wsc = torch.empty(N, K // 32, dtype=torch.uint8, device=DEV)
    hk.fused_rmsnorm_mxfp4_quant_fwd(A, None, ac, asc, 1e-6)
    hk.fused_rmsnorm_mxfp4_quant_fwd(W, None, wc, wsc, 1e-6)
    C1 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    C2 = torch.empty_like(C1)
    hk.gemm.afp4wfp4.dispatch(ac, wc, C1, asc, wsc)
    assert hk.last_kernel() == "gemm_mxfp4_pair_kernel<256x192>"
    hk.gemm.afp4wfp4.dispatch(ac, wc, C2, asc + 1, wsc)
    torch.cuda.synchronize()
    _status_ok()
    assert int(asc.max()) < 254
    assert torch.equal(C2, C1 * 2.0)
    del C2
    # every element against an fp32 matmul of the decoded operands on the device (torch, TF32 off: a checker)
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], device=DEV)

    def decode(codes, sbytes):
        v = torch.stack([lut[(codes & 0xF).long()], lut[(codes >> 4).long()]], dim=-1).view(codes.shape[0], -1)
        return v * torch.ldexp(torch.ones_like(sbytes, dtype=torch.float32), sbytes.int() - 127).repeat_interleave(32, dim=1)

    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = decode(ac, asc) @ decode(wc, wsc).t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = tf32
    err = float((C1.float() - ref).abs().max() / ref.abs().max())
    assert err <= TOL, err


def test_batched_gemm_mxfp4_wide_and_pair_kernels(hk):
    """A batch > 1 through the CTA-pair kernel (and, with pairs switched off in a child process, through
    the 192-wide one-CTA kernel): B=2, 2304 x 3264 x 256."""
    Bn, M, N, K = 2, 2304, 3264, 256
    ac, wc, asc, wsc = _mxfp4_operands(M, N, K, batch=Bn, seed=23)
    C = torch.full((Bn, M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.batched_gemm.afp4wfp4.dispatch(_dev(ac), _dev(wc), C, _dev(asc), _dev(wsc))
    assert hk.last_kernel() == "gemm_mxfp4_pair_kernel<256x192>"
    torch.cuda.synchronize()
    _status_ok()
    for b in range(Bn):
        _check(C[b], gemm.gemm_mxfp4(ac[b], wc[b], asc[b], wsc[b]), f"batched mxfp4 pairs, batch {b}")
    out = _run_case_in_subprocess(("mxfp4", M, N, K, Bn), {"HKB_MXFP4_PAIRS": "0"})
    assert out["kernel"] == "gemm_mxfp4_kernel<192>"
    assert out["rel_err"] <= TOL, out


def test_mxfp4_scales_in_tensor_core_layout(hk):
    """Scale factors handed over in the tensor core's layout (weights converted once, activations
    quantized straight into it) give the same bits as the row-major form, with no re-layout launch."""
    M, N, K = 2304, 3264, 384            # CTA pairs, ragged N, odd number of 128-wide K atoms
    g = torch.Generator().manual_seed(31)
    A = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    W = (torch.randn(N, K, generator=g) * 0.02).bfloat16().to(DEV)
    mod = hk.gemm.afp4wfp4
    ac = torch.empty(M, K // 2, dtype=torch.uint8, device=DEV); asc = torch.empty(M, K // 32, dtype=torch.uint8, device=DEV)
    wc = torch.empty(N, K // 2, dtype=torch.uint8, device=DEV); wsc = torch.empty(N, K // 32, dtype=torch.uint8, device=DEV)
    a_tc = torch.zeros(mod.sf_tc_bytes(1, M, K), dtype=torch.uint8, device=DEV)
    w_tc = torch.full((mod.sf_tc_bytes(1, N, K),), 0xAB, dtype=torch.uint8, device=DEV)
    hk.fused_rmsnorm_mxfp4_quant_fwd(W, None, wc, wsc, 1e-6)
    mod.sf_to_tc(wsc, w_tc, K)                                              # weights: converted once
    hk.fused_rmsnorm_mxfp4_quant_tc_fwd(A, None, ac, asc, a_tc, 1e-6)       # activations: written by the quantizer
    # the quantizer's layout equals the converter's (which also zeroes the padding the quantizer leaves alone)
    a_tc_ref = torch.full_like(a_tc, 0xCD)
    mod.sf_to_tc(asc, a_tc_ref, K)
    assert torch.equal(a_tc, a_tc_ref)
    # row-major scales of the tc quantizer equal the plain quantizer's
    ac2 = torch.empty_like(ac); asc2 = torch.empty_like(asc)
    hk.fused_rmsnorm_mxfp4_quant_fwd(A, None, ac2, asc2, 1e-6)
    assert torch.equal(ac, ac2) and torch.equal(asc, asc2)
    C_ref = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    mod.dispatch(ac, wc, C_ref, asc, wsc)
    for a_is_tc, b_is_tc in [(True, True), (False, True), (True, False)]:
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        mod.dispatch_tc(ac, wc, C, a_tc if a_is_tc else asc, w_tc if b_is_tc else wsc, a_is_tc, b_is_tc)
        torch.cuda.synchronize()
        assert torch.equal(C, C_ref), (a_is_tc, b_is_tc)
    _status_ok()
    _check(C_ref, gemm.gemm_mxfp4(ac.cpu().numpy(), wc.cpu().numpy(), asc.cpu().numpy(), wsc.cpu().numpy()), "mxfp4 tc layout")
    # the RMSNorm form of the quantizer writes the same layout
    w_norm = torch.ones(K, dtype=torch.bfloat16, device=DEV)
    a_tc3 = torch.zeros_like(a_tc); asc3 = torch.empty_like(asc); ac3 = torch.empty_like(ac)
    hk.fused_rmsnorm_mxfp4_quant_tc_fwd(A, w_norm, ac3, asc3, a_tc3, 1e-6)
    a_tc3_ref = torch.empty_like(a_tc)
    mod.sf_to_tc(asc3, a_tc3_ref, K)
    assert torch.equal(a_tc3, a_tc3_ref)


def test_mxfp4_gemms_on_two_streams_do_not_share_scratch(hk):
    """Two different MXFP4 GEMMs issued alternately on two streams (their scale re-layout scratch is
    kept per stream) must both give the result they give when run alone."""
    shapes = [(1024, 1536, 2048), (768, 2048, 2048)]
    cases = []
    for i, (M, N, K) in enumerate(shapes):
        ac, wc, asc, wsc = _mxfp4_operands(M, N, K, seed=40 + i)
        t = [_dev(x) for x in (ac, wc, asc, wsc)]
        C_alone = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        hk.gemm.afp4wfp4.dispatch(t[0], t[1], C_alone, t[2], t[3])
        cases.append((t, C_alone, torch.empty(M, N, dtype=torch.bfloat16, device=DEV)))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for rep in range(20):
        for (t, _, C), st in zip(cases, streams):
            with torch.cuda.stream(st):
                hk.gemm.afp4wfp4.dispatch(t[0], t[1], C, t[2], t[3])
    torch.cuda.synchronize()
    _status_ok()
    for t, C_alone, C in cases:
        assert torch.equal(C, C_alone)


# ---- fused multiply-add epilogue (C = c_a * gemm + c_b) ---------------------------------------------

def _ca_cb(M, N, seed=11):
    """c_a, c_b ~ N(0, 0.5) bf16 [M, N], as in the reference's tests (tests/test_gemm.py:516-517)."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, N, generator=g) * 0.5).bfloat16(), (torch.randn(M, N, generator=g) * 0.5).bfloat16()


@pytest.mark.parametrize("shape,gn", [((256, 256, 256), 1),            # the reference's case: b_scale [K/128, N]
                                      ((256, 256, 256), 128), ((512, 1024, 512), 128),
                                      ((200, 384, 256), 128), ((2304, 4608, 256), 128)])   # 256-wide tiles
def test_fused_blockscale_mul_add(hk, shape, gn):
    """fused_gemm_a8w8_blockscale_mul_add (reference test: tests/test_gemm.py:498-533): scales
    rand*2.0 as there, operands e4m3-representable."""
    M, N, K = shape
    aq, bq, _, _ = _fp8_operands(M, N, K)
    g = torch.Generator().manual_seed(7)
    sa = torch.rand(M, K // 128, generator=g) * 2.0
    sb = torch.rand(K // 128, N // gn, generator=g) * 2.0
    c_a, c_b = _ca_cb(M, N)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.fused_gemm.a8w8_blockscale_mul_add.dispatch(_dev(aq), _dev(bq), C, _dev(sa), _dev(sb), _dev(c_a), _dev(c_b))
    torch.cuda.synchronize()
    _status_ok()
    ref = gemm.mul_add(gemm.gemm_fp8_blockscale(aq, bq, sa, sb), c_a, c_b)
    _check(C, ref, f"blockscale mul_add {shape} gn={gn}")
    # and the epilogue really is applied to the unrounded GEMM of the plain entry point
    P = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    hk.gemm.a8w8_blockscale.dispatch(_dev(aq), _dev(bq), P, _dev(sa), _dev(sb))
    two_step = (c_a.float() * P.float().cpu() + c_b.float()).numpy()
    assert gemm.rel_err(C.float().cpu().numpy(), two_step) < 2 ** -7


@pytest.mark.parametrize("shape", [(256, 256, 256), (200, 264, 512), (2304, 3264, 256)])
def test_fused_mxfp4_mul_add(hk, shape):
    """fused_gemm_afp4wfp4_mul_add (reference test: tests/test_gemm.py:579-614) on packed e2m1 codes
    and e8m0 scales."""
    M, N, K = shape
    ac, wc, asc, wsc = _mxfp4_operands(M, N, K)
    c_a, c_b = _ca_cb(M, N)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.fused_gemm.afp4wfp4_mul_add.dispatch(_dev(ac), _dev(wc), C, _dev(asc), _dev(wsc), _dev(c_a), _dev(c_b))
    torch.cuda.synchronize()
    _status_ok()
    _check(C, gemm.mul_add(gemm.gemm_mxfp4(ac, wc, asc, wsc), c_a, c_b), f"mxfp4 mul_add {shape}")


# ---- split-concatenate epilogue ------------------------------------------------------------------------

@pytest.mark.parametrize("M,K,D,S1,S2,S3,gn", [(128, 256, 2, 64, 64, 32, 1),        # the reference's sizes
                                               (200, 512, 3, 128, 64, 16, 128), (384, 256, 4, 96, 32, 0, 1)])
def test_fused_blockscale_split_cat(hk, M, K, D, S1, S2, S3, gn):
    N = D * (S1 + S2)
    if gn == 128 and N % 128:
        pytest.skip("N must be a multiple of 128 for 128-column scale groups")
    aq, bq, _, _ = _fp8_operands(M, N, K, seed=71)
    g = torch.Generator().manual_seed(7)
    sa = torch.rand(M, K // 128, generator=g) * 0.1 + 0.01
    sb = torch.rand(K // 128, N // gn, generator=g) * 0.1 + 0.01
    y = torch.randn(M, D, max(S3, 1), generator=g).bfloat16()[:, :, :S3].contiguous()
    c1 = torch.full((M, D, S1 + S3), float("nan"), dtype=torch.bfloat16, device=DEV)
    c2 = torch.full((M, D, S2), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.fused_gemm.a8w8_blockscale_split_cat.dispatch(_dev(aq), _dev(bq), _dev(sa), _dev(sb), _dev(y), c1, c2)
    assert "split_cat" in hk.last_kernel()
    torch.cuda.synchronize()
    _status_ok()
    r1, r2 = gemm.split_cat(gemm.gemm_fp8_blockscale(aq, bq, sa, sb), y, S1, S2)
    _check(c1[:, :, :S1], r1[:, :, :S1], "split-cat c1 (GEMM part)")
    _check(c2, r2, "split-cat c2")
    assert torch.equal(c1[:, :, S1:].cpu(), y)              # the concatenated part is a copy


def test_fused_blockscale_split_cat_reference_golden(hk, golden_dir):
    g = np.load(os.path.join(golden_dir, "fused_blockscale_split_cat.npz"))
    aq, bq = codecs.f32_to_e4m3fn(g["a"]), codecs.f32_to_e4m3fn(g["b"])        # integers up to 8: exact in e4m3
    assert np.array_equal(codecs.e4m3fn_to_f32(aq), g["a"])
    y = torch.from_numpy(g["y"]).bfloat16()
    M, D, S1, S2, S3 = g["a"].shape[0], int(g["D"]), int(g["S1"]), int(g["S2"]), int(g["S3"])
    c1 = torch.zeros(M, D, S1 + S3, dtype=torch.bfloat16, device=DEV)
    c2 = torch.zeros(M, D, S2, dtype=torch.bfloat16, device=DEV)
    hk.fused_gemm.a8w8_blockscale_split_cat.dispatch(_dev(aq), _dev(bq), _dev(g["a_scale"]), _dev(g["b_scale"]), _dev(y), c1, c2)
    torch.cuda.synchronize()
    _check(c1[:, :, :S1], g["c1"][:, :, :S1], "split-cat golden c1")
    _check(c2, g["c2"], "split-cat golden c2")
    assert torch.equal(c1[:, :, S1:].cpu(), y)


@pytest.mark.parametrize("M,K,D,S1,S2,S3", [(128, 256, 2, 64, 64, 32), (2304, 256, 17, 128, 64, 16)])   # 128-wide and 192-wide tiles
def test_fused_mxfp4_split_cat(hk, M, K, D, S1, S2, S3):
    N = D * (S1 + S2)
    ac, wc, asc, wsc = _mxfp4_operands(M, N, K, seed=72)
    y = torch.randn(M, D, S3, generator=torch.Generator().manual_seed(3)).bfloat16()
    c1 = torch.full((M, D, S1 + S3), float("nan"), dtype=torch.bfloat16, device=DEV)
    c2 = torch.full((M, D, S2), float("nan"), dtype=torch.bfloat16, device=DEV)
    hk.fused_gemm.afp4wfp4_split_cat.dispatch(_dev(ac), _dev(wc), _dev(asc), _dev(wsc), _dev(y), c1, c2)
    torch.cuda.synchronize()
    _status_ok()
    r1, r2 = gemm.split_cat(gemm.gemm_mxfp4(ac, wc, asc, wsc), y, S1, S2)
    _check(c1[:, :, :S1], r1[:, :, :S1], "mxfp4 split-cat c1")
    _check(c2, r2, "mxfp4 split-cat c2")
    assert torch.equal(c1[:, :, S1:].cpu(), y)


def test_fused_mul_add_validates_its_operands(hk):
    x8 = torch.zeros(128, 128, dtype=torch.uint8, device=DEV)
    c = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    s = torch.ones(128, 1, device=DEV)
    with pytest.raises(RuntimeError, match="c_a and c_b must be"):
        hk.fused_gemm.a8w8_blockscale_mul_add.dispatch(x8, x8, c, s, s.view(1, 128), c[:64], c)
    with pytest.raises(RuntimeError, match="c_a"):
        hk.fused_gemm.a8w8_blockscale_mul_add.dispatch(x8, x8, c, s, s.view(1, 128), c.float(), c)
