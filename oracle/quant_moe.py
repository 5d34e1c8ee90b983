"""CPU oracle for the MoE casts of quant_moe_tk.  TEST INFRASTRUCTURE (see package docstring).

Rules restated (paths inside the reference project):
  * static FP8: ``(x.float() / scale).clamp(-448, 448).to(torch.float8_e4m3fn)``
    (tests/test_moe.py:997-999; pinned by tests/golden/quant_static_fp8.npz).
  * MX down-cast: per 32 elements of the last dimension the scale byte is the biased exponent of
    ``amax / QMAX`` rounded up to a power of two, ``((bits + 0x007FFFFF) & 0x7F800000) >> 23``
    (kernels/moe-misc/quant_moe/kernel.cpp:143-161); codes = x / 2**(byte-127), rounded to nearest
    even (:173-176 computes the power-of-two quantisation scale the same way).  An all-zero block
    takes byte 127 (scale 1.0), the reference's Python path (kernels/moe-misc/quant_moe/
    test_parity.py:116-117); the device code's 0xFF would make the block NaN on the way back.
    The reference leaves the FP4 codes unwritten (kernel.cpp:214-217); here the same rule with
    QMAX = 6 and round-to-nearest-even E2M1 codes, element 2i in the low nibble.
  * MX up-cast: decode(code) * float_from_bits(byte << 23), byte 255 -> NaN, result rounded to
    bf16 (kernel.cpp:313-357).
Parity of the two MX casts is unpinned: the reference's tests only bound the round-trip error
(tests/test_moe.py:1046-1052), which tests/ also checks.
"""
import numpy as np
import torch

from .codecs import as_f32, f32_to_e4m3fn, e4m3fn_to_f32, pack_e2m1, unpack_e2m1


def downcast_to_static_fp8(x, scale):
    q = as_f32(x) / np.float32(scale)
    return f32_to_e4m3fn(np.clip(q, -448.0, 448.0))


def mx_scale_bytes(amax, qmax):
    amax = np.asarray(amax, dtype=np.float32)
    with np.errstate(under="ignore"):
        ds = (amax / np.float32(qmax)).astype(np.float32)
    e = ((ds.view(np.uint32) + np.uint32(0x007FFFFF)) & np.uint32(0x7F800000)) >> np.uint32(23)
    return np.where(amax == 0, 127, e).astype(np.uint8)


def f32_to_e2m1_rne(q):
    """fp32 -> e2m1 nibble, round-to-nearest-even on the code grid {0,.5,1,1.5,2,3,4,6}, saturating
    at 6; the sign bit follows the sign bit of q (also for zeros)."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    a = np.abs(q)
    code = ((a > 0.25).astype(np.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5) + (a > 5.0))
    return (code | ((q.view(np.uint32) >> np.uint32(28)) & np.uint32(8))).astype(np.uint8)


def downcast_to_mxfp(src, is_fp4=False):
    """src [outer, Q] (Q % 32 == 0) -> (codes uint8 [outer, Q] or [outer, Q/2], scale bytes [outer, Q/32])."""
    x = as_f32(src)
    outer, Q = x.shape
    blk = x.reshape(outer, Q // 32, 32)
    amax = np.abs(blk).max(axis=2)
    sb = mx_scale_bytes(amax, 6.0 if is_fp4 else 448.0)
    scale = np.ldexp(np.float64(1.0), sb.astype(np.int32) - 127)[..., None]
    with np.errstate(under="ignore"):
        q = (blk.astype(np.float64) / scale).astype(np.float32).reshape(outer, Q)
    if is_fp4:
        return pack_e2m1(f32_to_e2m1_rne(q)), sb
    return f32_to_e4m3fn(np.clip(q, -448.0, 448.0)), sb


def upcast_from_mxfp(codes, scale_bytes, is_fp4=False):
    """-> bf16 bit patterns (uint16) [outer, Q]."""
    codes = np.asarray(codes, dtype=np.uint8)
    sb = np.asarray(scale_bytes, dtype=np.uint8)
    v = unpack_e2m1(codes) if is_fp4 else e4m3fn_to_f32(codes)
    outer, Q = v.shape
    s = (sb.astype(np.uint32) << np.uint32(23)).view(np.float32)
    s = np.where(sb == 255, np.float32(np.nan), s).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore", under="ignore"):
        r = (v.reshape(outer, Q // 32, 32) * s[..., None]).astype(np.float32).reshape(outer, Q)
    return torch.from_numpy(r).bfloat16().view(torch.int16).numpy().view(np.uint16)
