"""Oracle of the MoE casts (quant_moe_tk) against the reference's pinned case and its own rules."""
import os

import numpy as np
import torch

from oracle import codecs, quant_moe as qm


def _bf16(bits):
    return torch.from_numpy(np.asarray(bits, dtype=np.uint16).view(np.int16).copy()).view(torch.bfloat16)


def test_static_fp8_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_static_fp8.npz"))
    assert np.array_equal(qm.downcast_to_static_fp8(_bf16(g["x_bf16"]), 0.5), g["bytes"])


def test_static_fp8_is_the_torch_expression():
    x = torch.randn(64, 96, generator=torch.Generator().manual_seed(1)).bfloat16() * 300
    ref = (x.float() / 0.37).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(qm.downcast_to_static_fp8(x, 0.37), ref)


def test_mx_scale_is_the_rounded_up_exponent():
    amax = np.array([448.0, 449.0, 224.0, 1.0, 0.0, 6.0, 6.5, 3.0], dtype=np.float32)
    assert list(qm.mx_scale_bytes(amax, 448.0)) == [127, 128, 126, 127 - 8, 127, 127 - 6, 127 - 6, 127 - 7]
    assert list(qm.mx_scale_bytes(amax[5:], 6.0)) == [127, 128, 126]
    # codes never saturate: the scale covers the block maximum
    x = (torch.randn(32, 64, generator=torch.Generator().manual_seed(2)) * 1000).bfloat16()
    c, s = qm.downcast_to_mxfp(x)
    assert np.abs(codecs.e4m3fn_to_f32(c)).max() <= 448


def test_e2m1_rne_ties_go_to_the_even_code():
    q = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -0.0, 0.26], dtype=np.float32)
    assert list(qm.f32_to_e2m1_rne(q)) == [0, 2, 2, 4, 4, 6, 6, 7, 8, 8, 1]


def test_mx_round_trip_error_is_within_the_reference_bound():
    """tests/test_moe.py:1046-1052 of the reference: mean |src - roundtrip| < 0.5 on randn 128x256."""
    torch.manual_seed(42)
    src = torch.randn(128, 256).bfloat16()
    for fp4, bound in ((False, 0.03), (True, 0.12)):
        c, s = qm.downcast_to_mxfp(src, fp4)
        out = _bf16(qm.upcast_from_mxfp(c, s, fp4)).float()
        assert (src.float() - out).abs().mean().item() < bound < 0.5


def test_upcast_special_bytes():
    codes = np.full((1, 32), 0x38, dtype=np.uint8)                      # 1.0
    assert np.all(_bf16(qm.upcast_from_mxfp(codes, np.array([[130]], dtype=np.uint8))).float().numpy() == 8.0)
    assert np.all(_bf16(qm.upcast_from_mxfp(codes, np.array([[0]], dtype=np.uint8))).float().numpy() == 0.0)
    assert np.all(np.isnan(_bf16(qm.upcast_from_mxfp(codes, np.array([[255]], dtype=np.uint8))).float().numpy()))
