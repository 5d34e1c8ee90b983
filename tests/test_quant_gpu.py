"""GPU tier: the CUDA quantizers against the CPU oracle, bit for bit, through the
reference-facing `hipkittens` functions (pybind shim -> C ABI -> kernels)."""
import numpy as np
import pytest
import torch

from oracle import codecs, inputs, quant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _diff_report(got, ref, what):
    bad = np.argwhere(got != ref)
    head = ", ".join(f"{tuple(i)}: got {got[tuple(i)]} want {ref[tuple(i)]}" for i in bad[:8])
    return f"{what}: {len(bad)} of {ref.size} differ; first: {head}"


def _run_per_token(hk, x, int8=False):
    M, D = x.shape
    q = torch.full((M, D), 0x55, dtype=torch.int8 if int8 else torch.uint8, device=DEV)
    s = torch.full((M, 1), -1.0, dtype=torch.float32, device=DEV)
    hk.per_token_quant_fwd(x.to(DEV), q, s)
    torch.cuda.synchronize()
    return q.cpu().numpy(), s.cpu().numpy()


def _all_bf16_values():
    """Every finite bf16 bit pattern, as rows of 128 so that every row mixes magnitudes."""
    bits = np.arange(65536, dtype=np.uint32)
    f = (bits << 16).view(np.float32)
    bits = bits[np.isfinite(f)].astype(np.uint16)
    rng = np.random.default_rng(7)
    rng.shuffle(bits)
    bits = bits[: len(bits) // 128 * 128].reshape(-1, 128)
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


@pytest.mark.parametrize("shape", [(128, 1024), (16, 8192), (4096, 4096), (37, 136), (5, 16384), (3, 40000), (1, 8)])
def test_fp8_per_token_bit_exact(hk, shape):
    x = torch.randn(shape, generator=torch.Generator().manual_seed(42)).bfloat16()
    q, s = _run_per_token(hk, x)
    rq, rs = quant.quant_fp8_per_token(x)
    assert np.array_equal(s, rs), _diff_report(s, rs, "scales")
    assert np.array_equal(q, rq), _diff_report(q, rq, "codes")


def test_fp8_per_token_every_bf16_value_and_many_scales(hk):
    """Exhaustive sweep: all finite bf16 values, with row maxima spread over many exponents and
    mantissas so that the shared-divisor division is exercised against true IEEE division."""
    base = _all_bf16_values().float()
    base = base.clamp(-3e4, 3e4)
    rows = []
    rng = np.random.default_rng(3)
    for k in range(24):
        sc = float(np.float32(2.0 ** rng.integers(-20, 10)) * np.float32(1 + rng.random()))
        rows.append((base * sc).bfloat16())
    x = torch.cat(rows)
    q, s = _run_per_token(hk, x)
    rq, rs = quant.quant_fp8_per_token(x)
    assert np.array_equal(s, rs), _diff_report(s, rs, "scales")
    assert np.array_equal(q, rq), _diff_report(q, rq, "codes")


def test_fp8_per_token_edge_rows(hk):
    x = torch.zeros(6, 256).bfloat16()
    x[1, 3] = 1e-30                       # scale floor 1e-10 applies
    x[2] = -0.0
    x[3, :4] = torch.tensor([448.0, -448.0, 224.0, 1.0]).bfloat16()
    x[4, 0] = 3.3e38                      # near bf16 max
    x[4, 1] = -1.0
    x[5] = torch.linspace(-1, 1, 256).bfloat16()
    q, s = _run_per_token(hk, x)
    rq, rs = quant.quant_fp8_per_token(x)
    assert np.array_equal(s, rs) and np.array_equal(q, rq), _diff_report(q, rq, "codes")


def test_int8_mode_matches_reference_golden(hk, golden_dir):
    import os
    g = np.load(os.path.join(golden_dir, "quant_int8_per_token.npz"))
    x = torch.from_numpy(g["x_bf16"].view(np.int16).copy()).view(torch.bfloat16)
    q, s = _run_per_token(hk, x, int8=True)
    assert np.array_equal(s, g["scales"])
    assert np.array_equal(q, g["q"]), _diff_report(q, g["q"], "int8 codes")


@pytest.mark.parametrize("shape", [(4096, 4096), (256, 4096), (7, 128), (33, 8192)])
def test_fp8_1x128_bit_exact(hk, shape):
    M, D = shape
    A, _ = inputs.make_inputs(M, 128, D, outliers=True)
    q = torch.zeros(M, D, dtype=torch.uint8, device=DEV)
    s = torch.zeros(M, D // 128, dtype=torch.float32, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(A.to(DEV), None, q, s, 1e-6)
    torch.cuda.synchronize()
    rq, rs = quant.quant_fp8_1x128(A)
    assert np.array_equal(s.cpu().numpy(), rs), _diff_report(s.cpu().numpy(), rs, "scales")
    assert np.array_equal(q.cpu().numpy(), rq), _diff_report(q.cpu().numpy(), rq, "codes")


def test_fp8_1x128_accepts_float8_output_tensor(hk):
    A, _ = inputs.make_inputs(64, 128, 1024)
    q = torch.zeros(64, 1024, dtype=torch.float8_e4m3fn, device=DEV)
    s = torch.zeros(64, 8, dtype=torch.float32, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(A.to(DEV), None, q, s, 1e-6)
    rq, _ = quant.quant_fp8_1x128(A)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), rq)


@pytest.mark.parametrize("shape", [(1024, 4096), (128, 128), (384, 2048)])
def test_fp8_128x128_weight_quant_bit_exact(hk, shape):
    N, K = shape
    _, W = inputs.make_inputs(128, N, K)
    q = torch.zeros(N, K, dtype=torch.uint8, device=DEV)
    s = torch.zeros(K // 128, N // 128, dtype=torch.float32, device=DEV)
    hk.weight_quant_128x128(W.to(DEV), q, s)
    torch.cuda.synchronize()
    rq, rs = quant.quant_fp8_128x128(W)
    assert np.array_equal(s.cpu().numpy(), rs), _diff_report(s.cpu().numpy(), rs, "scales")
    assert np.array_equal(q.cpu().numpy(), rq), _diff_report(q.cpu().numpy(), rq, "codes")


def _run_mxfp4(hk, x, mode=None, weight=None, eps=1e-6):
    M, D = x.shape
    codes = torch.full((M, D // 2), 0x55, dtype=torch.uint8, device=DEV)
    sc = torch.full((M, D // 32), 0x55, dtype=torch.uint8, device=DEV)
    w = None if weight is None else weight.to(DEV)
    if mode is None:
        hk.fused_rmsnorm_mxfp4_quant_fwd(x.to(DEV), w, codes, sc, eps)
    else:
        hk.fused_rmsnorm_mxfp4_quant_fwd(x.to(DEV), w, codes, sc, eps, mode)
    torch.cuda.synchronize()
    return codes.cpu().numpy(), sc.cpu().numpy()


@pytest.mark.parametrize("shape", [(1024, 4096), (256, 4096), (8192, 1024), (3, 32), (5, 96), (1, 64)])
@pytest.mark.parametrize("mode", ["doc", "kernel"])
def test_mxfp4_bit_exact(hk, shape, mode):
    x = torch.randn(shape, generator=torch.Generator().manual_seed(42)).bfloat16()
    codes, sc = _run_mxfp4(hk, x, mode)
    rc, rs = quant.quant_mxfp4(x, mode=quant.MODE_DOC if mode == "doc" else quant.MODE_KERNEL)
    assert np.array_equal(sc, rs), _diff_report(sc, rs, "scale bytes")
    assert np.array_equal(codes, rc), _diff_report(codes, rc, "packed codes")


@pytest.mark.parametrize("mode", ["doc", "kernel"])
def test_mxfp4_every_bf16_value_ties_and_signed_zero(hk, mode):
    base = _all_bf16_values()
    # blocks made of exact tie points times powers of two, with a block maximum that fixes e
    ties = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0,
                         0.0, -0.0, 7.5, -7.5, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 4.5, 5.5, 0.125, -0.125, 1e-30, -1e-30, 5.0])
    rows = [(ties * (2.0 ** e)).bfloat16().repeat(4)[None, :] for e in range(-30, 31, 3)]
    x = torch.cat([base] + rows)
    codes, sc = _run_mxfp4(hk, x, mode)
    rc, rs = quant.quant_mxfp4(x, mode=quant.MODE_DOC if mode == "doc" else quant.MODE_KERNEL)
    assert np.array_equal(sc, rs), _diff_report(sc, rs, "scale bytes")
    assert np.array_equal(codes, rc), _diff_report(codes, rc, "packed codes")


def test_mxfp4_default_mode_is_doc(hk):
    x = torch.randn(64, 512, generator=torch.Generator().manual_seed(1)).bfloat16()
    codes, sc = _run_mxfp4(hk, x)
    rc, rs = quant.quant_mxfp4(x, mode=quant.MODE_DOC)
    assert np.array_equal(sc, rs) and np.array_equal(codes, rc)


def test_rmsnorm_prologue_close_to_oracle(hk):
    """With a weight the fused quantizers apply RMSNorm first; the fp32 reduction order is not
    pinned, so compare dequantized values with a tolerance (shape of tests/test_misc.py:556-567)."""
    g = torch.Generator().manual_seed(42)
    x = torch.randn(256, 4096, generator=g).bfloat16()
    w = torch.randn(4096, generator=g).bfloat16()
    y = quant.rmsnorm(x, w, 1e-6)
    q = torch.zeros(256, 4096, dtype=torch.uint8, device=DEV)
    s = torch.zeros(256, 32, dtype=torch.float32, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(x.to(DEV), w.to(DEV), q, s, 1e-6)
    dq = codecs.e4m3fn_to_f32(q.cpu().numpy()).reshape(256, 32, 128) * s.cpu().numpy()[:, :, None]
    err = np.abs(dq.reshape(256, 4096) - y)
    assert (err <= np.abs(y) * 0.0626 + 1e-3 * np.abs(y).max()).all()       # e4m3 half-ulp = 2^-4
    rs = quant.quant_fp8_1x128(x, w, 1e-6)[1]
    assert np.allclose(s.cpu().numpy(), rs, rtol=1e-5)
    codes, sc = _run_mxfp4(hk, x, None, w)
    rc, rsb = quant.quant_mxfp4(x, w, 1e-6)
    assert (sc != rsb).mean() < 1e-3            # exponent bytes can flip only when amax sits on a power of two
    assert (codes != rc).mean() < 1e-3


def test_round_trip_property_at_full_size(hk):
    """Size-independent property at the bandwidth-benchmark size: dequantized codes stay within
    half an e4m3 step of the input, and every row's maximum maps to code 0x7E (448)."""
    M, D = 16384, 8192
    x = torch.randn(M, D, device=DEV, dtype=torch.bfloat16)
    q = torch.empty(M, D, dtype=torch.uint8, device=DEV)
    s = torch.empty(M, 1, dtype=torch.float32, device=DEV)
    hk.per_token_quant_fwd(x, q, s)
    dq = q.view(torch.float8_e4m3fn).float() * s
    xf = x.float()
    assert ((dq - xf).abs() <= xf.abs() * 0.0626 + s * 2 ** -10).all()
    assert ((q & 0x7F).amax(dim=1) == 0x7E).all()
    assert torch.equal(s.flatten(), (xf.abs().amax(1) / torch.tensor(448.0, device=DEV)).clamp(min=1e-10))


def test_block_quantizers_bit_exact_at_the_bandwidth_benchmark_size(hk):
    """1x128 FP8 and MXFP4 (default mode) on 16384 x 8192 -- the size their GB/s is quoted on -- against the same
    rules evaluated with torch on the device (a checker; IEEE fp32 division and torch's e4m3fn cast, which the CPU
    tier pins against the oracle's): every code and every scale of all 134 M elements."""
    M, D = 16384, 8192
    x = torch.randn(M, D, device=DEV, dtype=torch.bfloat16)
    x[:, 7] *= 37.0
    x[5] = 0.0                                                  # an all-zero row: floor scale, zero codes / byte 0
    xf = x.float()
    # 1 x 128 FP8
    q = torch.empty(M, D, dtype=torch.uint8, device=DEV); s = torch.empty(M, D // 128, device=DEV)
    hk.fused_rmsnorm_fp8_quant_fwd(x, None, q, s, 1e-6)
    g = xf.view(M, D // 128, 128)
    scale = (g.abs().amax(dim=2, keepdim=True) / torch.tensor(448.0, device=DEV)).clamp_min(oracle_floor())    # tensor / tensor: a true division
    ref = (g / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).view(M, D)
    assert torch.equal(s, scale.view(M, D // 128))
    assert torch.equal(q, ref)
    del q, s, ref, scale, g
    # MXFP4, mode "doc": e = floor(log2 amax) - 2, nearest E2M1 magnitude with ties to the smaller one
    c = torch.empty(M, D // 2, dtype=torch.uint8, device=DEV); sb = torch.empty(M, D // 32, dtype=torch.uint8, device=DEV)
    hk.fused_rmsnorm_mxfp4_quant_fwd(x, None, c, sb, 1e-6)
    g = xf.view(M, D // 32, 32)
    amax = g.abs().amax(dim=2)
    e = torch.where(amax > 0, torch.frexp(amax)[1] - 1 - 2, torch.full_like(amax, -127, dtype=torch.int32)).clamp(-127, 127)
    assert torch.equal(sb, (e + 127).to(torch.uint8))
    a = (g * torch.ldexp(torch.ones_like(amax), -e)[..., None]).abs()          # exact: power-of-two scaling
    mag = torch.zeros_like(a, dtype=torch.uint8)
    for mid in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        mag += (a > mid).to(torch.uint8)
    nib = (mag | ((g < 0).to(torch.uint8) << 3)).view(M, D)
    assert torch.equal(c, nib[:, 0::2] | (nib[:, 1::2] << 4))


def test_weight_quantizer_bit_exact_at_config5_size(hk):
    """128 x 128 block FP8 weight quantizer on config 5's weight (57344 x 8192): every code and scale against the rule
    evaluated with torch on the device (true division, torch's e4m3fn cast)."""
    N, K = 57344, 8192
    w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
    w[130:200, 4096:4100] = 0.0
    q = torch.empty(N, K, dtype=torch.uint8, device=DEV); s = torch.empty(K // 128, N // 128, device=DEV)
    hk.weight_quant_128x128(w, q, s)
    t = w.float().view(N // 128, 128, K // 128, 128)
    scale = (t.abs().amax(dim=(1, 3), keepdim=True) / torch.tensor(448.0, device=DEV)).clamp_min(oracle_floor())
    assert torch.equal(s, scale.view(N // 128, K // 128).t())
    for n0 in range(0, N // 128, 64):                    # the fp32 temporaries of 64 row blocks at a time
        ref = (t[n0:n0 + 64] / scale[n0:n0 + 64]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        assert torch.equal(q[n0 * 128:(n0 + 64) * 128], ref.view(-1, K))


def oracle_floor():
    from oracle import quant
    return float(quant.SCALE_FLOOR)
