"""GPU parity of quant_moe_tk (static FP8, MX down-/up-cast) against the oracle: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import quant_moe as qm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf16(bits):
    return torch.from_numpy(np.asarray(bits, dtype=np.uint16).view(np.int16).copy()).view(torch.bfloat16)


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def test_static_fp8_reference_case(hk, golden_dir):
    """The reference's own case: 256 x 128 randn, scale 0.5 (tests/test_moe.py:984-999)."""
    g = np.load(os.path.join(golden_dir, "quant_static_fp8.npz"))
    x = _bf16(g["x_bf16"]).to(DEV)
    y = torch.empty(256, 128, dtype=torch.uint8, device=DEV)
    hk.moe_routing.quant.downcast_to_static_fp8(x, y, torch.tensor([0.5], device=DEV), 256, 128)
    assert np.array_equal(y.cpu().numpy(), g["bytes"])


@pytest.mark.parametrize("shape,scale", [((64, 96), 0.37), ((7, 33), 1.0 / 3.0), ((1, 5), 2.0), ((512, 1024), 0.011)])
def test_static_fp8_bit_exact(hk, shape, scale):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(shape, generator=g) * 50).bfloat16()
    x.view(-1)[0] = -0.0
    x.view(-1)[-1] = 1e30                       # saturates to 448
    y = torch.full(shape, 0xAA, dtype=torch.uint8, device=DEV)
    hk.moe_routing.quant.downcast_to_static_fp8(x.to(DEV), y, torch.tensor([scale], device=DEV), *shape)
    assert np.array_equal(y.cpu().numpy(), qm.downcast_to_static_fp8(x, np.float32(scale)))


def _all_bf16_blocks():
    """Every finite bf16 value, laid out so that blocks of 32 hold neighbouring magnitudes, plus
    blocks that mix the extremes, all-zero blocks and signed zeros."""
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite = bits[((bits >> 7) & 0xFF) != 0xFF]
    finite = finite[np.argsort(finite & 0x7FFF, kind="stable")]
    n = (len(finite) // 32) * 32
    a = finite[:n].reshape(-1, 32)
    rng = np.random.default_rng(0)
    mixed = rng.choice(finite[(finite & 0x7FFF) < 0x7000], size=(512, 32))
    zeros = np.zeros((4, 32), dtype=np.uint16); zeros[1, ::2] = 0x8000
    blocks = np.concatenate([a, mixed, zeros])
    pad = (-len(blocks)) % 8
    blocks = np.concatenate([blocks, np.zeros((pad, 32), dtype=np.uint16)])
    return _bf16(blocks.reshape(-1, 256))          # rows of 8 blocks


@pytest.mark.parametrize("is_fp4", [False, True])
def test_downcast_mxfp_bit_exact_on_every_bf16_value(hk, is_fp4):
    src = _all_bf16_blocks()
    outer, Q = src.shape
    t = torch.full((outer, Q // (2 if is_fp4 else 1)), 0xAA, dtype=torch.uint8, device=DEV)
    s = torch.full((outer, Q // 32), 0xAA, dtype=torch.uint8, device=DEV)
    hk.moe_routing.quant.downcast_to_mxfp(t, s, src.to(DEV), outer, Q, is_fp4)
    rc, rs = qm.downcast_to_mxfp(src, is_fp4)
    assert np.array_equal(s.cpu().numpy(), rs)
    got = t.cpu().numpy()
    bad = np.argwhere(got != rc)
    assert len(bad) == 0, f"{len(bad)} code bytes differ, first at {bad[0]}: got {got[tuple(bad[0])]:#x} want {rc[tuple(bad[0])]:#x}"


@pytest.mark.parametrize("is_fp4", [False, True])
@pytest.mark.parametrize("shape", [(128, 256), (3, 32), (257, 4096)])
def test_downcast_mxfp_random(hk, shape, is_fp4):
    g = torch.Generator().manual_seed(42)
    src = torch.randn(shape, generator=g).bfloat16()
    src[:, :32] *= 100
    outer, Q = shape
    t = torch.empty(outer, Q // (2 if is_fp4 else 1), dtype=torch.uint8, device=DEV)
    s = torch.empty(outer, Q // 32, dtype=torch.uint8, device=DEV)
    hk.moe_routing.quant.downcast_to_mxfp(t, s, src.to(DEV), outer, Q, is_fp4)
    rc, rs = qm.downcast_to_mxfp(src, is_fp4)
    assert np.array_equal(s.cpu().numpy(), rs) and np.array_equal(t.cpu().numpy(), rc)


@pytest.mark.parametrize("is_fp4", [False, True])
def test_upcast_every_code_and_scale_byte(hk, is_fp4):
    """Row r is decoded with scale byte r; an FP8 row holds all 256 code bytes, an FP4 row 128
    bytes that change with r so that every byte value (both nibbles) meets many scale bytes."""
    if is_fp4:
        codes = ((np.arange(128, dtype=np.int64)[None, :] * 37 + np.arange(256, dtype=np.int64)[:, None] * 11) % 256).astype(np.uint8)
    else:
        codes = np.tile(np.arange(256, dtype=np.uint8), (256, 1))
    sb = np.repeat(np.arange(256, dtype=np.uint8)[:, None], 8, axis=1)      # row r uses scale byte r
    out = torch.full((256, 256), 7.0, dtype=torch.bfloat16, device=DEV)
    hk.moe_routing.quant.upcast_from_mxfp(out, torch.from_numpy(sb).to(DEV), torch.from_numpy(codes).to(DEV), 256, 256, is_fp4)
    ref = qm.upcast_from_mxfp(codes, sb, is_fp4)
    got = _bits(out)
    nan_ref = (ref & 0x7FFF) > 0x7F80
    nan_got = (got & 0x7FFF) > 0x7F80
    assert np.array_equal(nan_ref, nan_got)
    assert np.array_equal(got[~nan_ref], ref[~nan_ref])


@pytest.mark.parametrize("is_fp4", [False, True])
def test_round_trip_as_in_the_reference_test(hk, is_fp4):
    """tests/test_moe.py:1027-1052: 128 x 256 randn, down-cast then up-cast, mean error < 0.5."""
    torch.manual_seed(42)
    src = torch.randn(128, 256, dtype=torch.bfloat16, device=DEV)
    t = torch.empty(128, 256 // (2 if is_fp4 else 1), dtype=torch.uint8, device=DEV)
    s = torch.empty(128, 8, dtype=torch.uint8, device=DEV)
    q = hk.moe_routing.quant
    q.downcast_to_mxfp(t, s, src, 128, 256, is_fp4)
    out = torch.empty(128, 256, dtype=torch.bfloat16, device=DEV)
    q.upcast_from_mxfp(out, s, t, 128, 256, is_fp4)
    err = (src.float() - out.float()).abs().mean().item()
    assert err < (0.12 if is_fp4 else 0.03)
    ref = qm.upcast_from_mxfp(*qm.downcast_to_mxfp(src.cpu(), is_fp4), is_fp4)
    assert np.array_equal(_bits(out), ref)


def test_shapes_are_validated(hk):
    q = hk.moe_routing.quant
    x = torch.zeros(4, 48, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="multiple of 32"):
        q.downcast_to_mxfp(torch.zeros(4, 48, dtype=torch.uint8, device=DEV), torch.zeros(4, 1, dtype=torch.uint8, device=DEV), x, 4, 48, False)
    with pytest.raises(RuntimeError, match="outer_dim\\*quant_dim"):
        q.downcast_to_mxfp(torch.zeros(4, 64, dtype=torch.uint8, device=DEV), torch.zeros(4, 2, dtype=torch.uint8, device=DEV), x, 4, 64, False)


@pytest.mark.parametrize("is_fp4", [False, True])
def test_casts_at_the_bandwidth_benchmark_size_sampled_rows_bit_exact(hk, is_fp4):
    """16384 x 8192, the size the casts' GB/s is quoted on: 128 sampled rows of the down-cast (codes and scale bytes)
    and of the up-cast of the whole result against the oracle, bit for bit."""
    M, D = 16384, 8192
    g = torch.Generator(device=DEV).manual_seed(17)
    src = torch.randn(M, D, generator=g, device=DEV).bfloat16()
    src[:, 5] *= 100.0
    src[3] = 0.0
    q = hk.moe_routing.quant
    t = torch.empty(M, D // (2 if is_fp4 else 1), dtype=torch.uint8, device=DEV); s = torch.empty(M, D // 32, dtype=torch.uint8, device=DEV)
    q.downcast_to_mxfp(t, s, src, M, D, is_fp4)
    out = torch.empty(M, D, dtype=torch.bfloat16, device=DEV)
    q.upcast_from_mxfp(out, s, t, M, D, is_fp4)
    torch.cuda.synchronize()
    rows = torch.cat([torch.tensor([0, 3, M - 1]), torch.randperm(M, generator=torch.Generator().manual_seed(4))[:125]]).to(DEV)
    rc, rs = qm.downcast_to_mxfp(src[rows].cpu(), is_fp4)
    assert np.array_equal(t[rows].cpu().numpy(), rc) and np.array_equal(s[rows].cpu().numpy(), rs)
    assert np.array_equal(_bits(out[rows]), qm.upcast_from_mxfp(rc, rs, is_fp4))
