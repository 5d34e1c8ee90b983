"""Number formats of the quantized-GEMM path, restated with NumPy bit arithmetic.

TEST INFRASTRUCTURE (see the package docstring).  Formats:

  * e4m3fn (OCP FP8, bias 7, no infinities, 0x7F/0xFF = NaN, max 448):
    the cast the reference pins is ``x.clamp(-448, 448).to(torch.float8_e4m3fn)``
    (tests/test_moe.py:997-999) = round-to-nearest-even from fp32.
  * e2m1 (FP4): magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}, bit 3 = sign; element
    ``k`` of a row lives in byte ``k // 2`` at shift ``(k & 1) * 4``
    (kernels/moe-gemm/moe_op_mxfp4/test_parity.py:30-40,
    kernels/quantization/fused_mxfp4_quant/kernel.cpp:154-162).
  * e8m0 scale byte: ``2 ** (byte - 127)``; the reference decodes byte 0 as 0.0
    (kernels/moe-gemm/moe_op_mxfp4/test_parity.py:43-46).
"""
import numpy as np

E4M3_MAX = 448.0

# kernels/moe-gemm/moe_op_mxfp4/test_parity.py:30-34
E2M1_LUT = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def as_f32(x):
    """Accept a torch tensor (any float dtype) or array-like; return a float32 ndarray."""
    if hasattr(x, "detach"):
        return np.ascontiguousarray(x.detach().cpu().float().numpy())
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def f32_to_e4m3fn(x):
    """fp32 -> e4m3fn byte, round-to-nearest-even; |x| >= 464 or NaN -> 0x7F|sign (NaN).

    Same result as ``torch.tensor(x).to(torch.float8_e4m3fn).view(torch.uint8)``;
    callers clamp to +-448 first, as the reference expression does.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    b = x.view(np.uint32)
    sign = ((b >> 24) & 0x80).astype(np.uint8)
    a = b & np.uint32(0x7FFFFFFF)
    out = np.empty(x.shape, dtype=np.uint8)
    # normal e4m3 range: 2**-6 <= |x|
    odd = (a >> 20) & 1
    rounded = a + np.uint32(0x7FFFF) + odd
    normal = ((rounded >> 20).astype(np.int64) - ((127 - 7) << 3))
    # e4m3 subnormals: quantum 2**-9, RNE on the integer grid
    with np.errstate(invalid="ignore", over="ignore"):
        sub = np.rint(np.abs(x).astype(np.float64) * 512.0)
    is_sub = a < np.uint32(0x3C800000)           # |x| < 2**-6
    code = np.where(is_sub, np.nan_to_num(sub, nan=0.0, posinf=0.0), normal)
    code = np.where(code > 0x7E, 0x7F, code)      # past 448 (after rounding) or inf/NaN
    code = np.where(a > np.uint32(0x7F800000), 0x7F, code)
    out[...] = code.astype(np.uint8)
    return out | sign


def _build_e4m3_table():
    t = np.zeros(256, dtype=np.float32)
    for c in range(256):
        s = -1.0 if c & 0x80 else 1.0
        e = (c >> 3) & 0xF
        m = c & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[c] = s * v
    return t


E4M3_TABLE = _build_e4m3_table()


def e4m3fn_to_f32(codes):
    return E4M3_TABLE[np.asarray(codes, dtype=np.uint8)]


def e8m0_to_f32(b, zero_is_zero=True):
    """Scale byte -> 2**(b-127).  ``zero_is_zero`` follows the reference decoder
    (byte 0 -> 0.0); the tensor-core hardware reads byte 0 as 2**-127.  The
    quantizer only emits byte 0 for all-zero blocks, where both agree on the product."""
    b = np.asarray(b, dtype=np.uint8)
    v = np.ldexp(np.float64(1.0), b.astype(np.int32) - 127)
    if zero_is_zero:
        v = np.where(b == 0, 0.0, v)
    return v.astype(np.float32)


def unpack_e2m1(packed):
    """[..., K/2] bytes -> [..., K] float32 magnitudes with sign (low nibble = even index)."""
    p = np.asarray(packed, dtype=np.uint8)
    lo = E2M1_LUT[p & 0xF]
    hi = E2M1_LUT[p >> 4]
    return np.stack([lo, hi], axis=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def pack_e2m1(nibbles):
    n = np.asarray(nibbles, dtype=np.uint8)
    return (n[..., 0::2] | (n[..., 1::2] << 4)).astype(np.uint8)
