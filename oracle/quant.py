"""CPU oracle for the dynamic quantizers.  TEST INFRASTRUCTURE (see package docstring).

All arithmetic is IEEE fp32 in NumPy with true division, exactly as the
reference's PyTorch expressions evaluate on the CPU:

    xf = x.float(); amax = xf.abs().amax(...); scale = (amax / QMAX).clamp(min=1e-10)
    q  = (xf / scale)                                   # tests/test_misc.py:531-536
    q.clamp(-448, 448).to(torch.float8_e4m3fn)          # tests/test_moe.py:997-999
"""
import numpy as np

from .codecs import as_f32, f32_to_e4m3fn, E4M3_MAX

SCALE_FLOOR = np.float32(1e-10)   # kernels/quantization/quant/kernel.cpp:93; fused_fp8_quant/kernel.cpp:190


def rmsnorm(x, weight, eps):
    """fp32 RMSNorm prologue of the fused quantizers: y = x * rsqrt(mean(x^2)+eps) * w
    (kernels/quantization/fused_fp8_quant/kernel.cpp:38-66; test_parity.py:51-53).
    Not bit-pinned: the reduction order is implementation-defined; tests use a tolerance."""
    x = as_f32(x)
    w = as_f32(weight)
    ms = np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    return (x * (1.0 / np.sqrt(ms + eps)).astype(np.float32) * w).astype(np.float32)


def _scale_from_amax(amax, qmax):
    return np.maximum(amax / np.float32(qmax), SCALE_FLOOR).astype(np.float32)


def quant_fp8_per_token(x):
    """[M, D] -> (codes u8 [M, D], scales f32 [M, 1]); one scale per row.
    Rule: tests/test_misc.py:531-536 with QMAX 448 and the e4m3fn cast."""
    x = as_f32(x)
    amax = np.abs(x).max(axis=1, keepdims=True)
    scale = _scale_from_amax(amax, E4M3_MAX)
    q = np.clip(x / scale, -E4M3_MAX, E4M3_MAX).astype(np.float32)
    return f32_to_e4m3fn(q), scale


def quant_int8_per_token(x):
    """The reference kernel's own INT8 mode (kernels/quantization/quant/kernel.cpp:92-107;
    tests/test_misc.py:531-536): scale = amax/127, q = round-half-even(x/scale) clamped to +-127."""
    x = as_f32(x)
    amax = np.abs(x).max(axis=1, keepdims=True)
    scale = _scale_from_amax(amax, 127.0)
    q = np.clip(np.rint(x / scale), -127, 127).astype(np.int8)
    return q, scale


def quant_fp8_1x128(x, weight=None, eps=1e-6):
    """[M, D] -> (codes u8 [M, D], scales f32 [M, D/128]); one scale per 128 contiguous
    columns (kernels/quantization/fused_fp8_quant/test_parity.py:55-67, kernel.cpp:147-199).
    ``weight`` given -> RMSNorm prologue first."""
    y = as_f32(x) if weight is None else rmsnorm(x, weight, eps)
    M, D = y.shape
    assert D % 128 == 0
    g = y.reshape(M, D // 128, 128)
    amax = np.abs(g).max(axis=2, keepdims=True)
    scale = _scale_from_amax(amax, E4M3_MAX)
    q = np.clip(g / scale, -E4M3_MAX, E4M3_MAX).astype(np.float32)
    return f32_to_e4m3fn(q).reshape(M, D), scale.reshape(M, D // 128)


def quant_fp8_128x128(w):
    """Weight [N, K] -> (codes u8 [N, K], b_scale f32 [K/128, N/128]).
    One scale per 128x128 tile, stored transposed: the layout the block-scale GEMM consumes
    (kernels/gemm-basic/gemm_a8w8_blockscale/kernel.cpp:7,41,146; test_parity.py:49-54,70-72)."""
    w = as_f32(w)
    N, K = w.shape
    assert N % 128 == 0 and K % 128 == 0
    t = w.reshape(N // 128, 128, K // 128, 128)
    amax = np.abs(t).max(axis=(1, 3), keepdims=True)
    scale = _scale_from_amax(amax, E4M3_MAX)
    q = np.clip(t / scale, -E4M3_MAX, E4M3_MAX).astype(np.float32)
    codes = f32_to_e4m3fn(q).reshape(N, K)
    return codes, np.ascontiguousarray(scale.reshape(N // 128, K // 128).T)


# ---------------------------------------------------------------------------------------
# MXFP4: e2m1 codes, one e8m0 exponent byte per 32 contiguous elements.
# ---------------------------------------------------------------------------------------
_E2M1_MAG = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
# midpoints between neighbouring magnitudes; a tie stays on the smaller one (argmin takes
# the first minimum, kernels/quantization/fused_mxfp4_quant/test_parity.py:89)
_E2M1_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float64)
# lower bounds used by the reference KERNEL (truncation), fused_mxfp4_quant/kernel.cpp:127-143
_E2M1_LOW = np.array([0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float64)

MODE_DOC = 0      # the Python path printed in fused_mxfp4_quant/test_parity.py:63-96
MODE_KERNEL = 1   # the device code in fused_mxfp4_quant/kernel.cpp:96-152


def _floor_log2(a):
    """floor(log2(a)) for positive finite fp32 (incl. subnormals), exact."""
    m, e = np.frexp(a.astype(np.float64))
    return e.astype(np.int32) - 1


def quant_mxfp4(x, weight=None, eps=1e-6, mode=MODE_DOC):
    """[M, D] -> (packed codes u8 [M, D/2], scale bytes u8 [M, D/32]).

    mode 0 (default): exponent e = floor(log2(amax)) - 2, value = nearest E2M1 magnitude of
      x / 2**e with ties to the smaller magnitude, saturating at 6, sign set iff x < 0
      (fused_mxfp4_quant/test_parity.py:75-93).  Completed where that text is undefined
      with the kernel's conventions: e clamped to [-127, 127]; amax == 0 -> byte 0.
    mode 1: the reference kernel's variant: amax first rounded with
      (bits + 0x200000) & 0xFF800000, thresholds by >= (truncation), sign = sign bit
      of the scaled value (fused_mxfp4_quant/kernel.cpp:96-152).
    """
    y = as_f32(x) if weight is None else rmsnorm(x, weight, eps)
    M, D = y.shape
    assert D % 32 == 0
    g = y.reshape(M, D // 32, 32)
    amax = np.abs(g).max(axis=2)
    if mode == MODE_KERNEL:
        bits = (amax.view(np.uint32) + np.uint32(0x200000)) & np.uint32(0xFF800000)
        amax_e = bits.view(np.float32)
    else:
        amax_e = amax
    safe = np.where((amax_e > 0) & np.isfinite(amax_e), amax_e, np.float32(1.0))
    e = _floor_log2(safe) - 2
    e = np.where(amax_e > 0, e, -127)
    e = np.where(np.isinf(amax_e), 127, e)     # mode 1 only: amax rounded up past the largest finite value
    e = np.clip(e, -127, 127).astype(np.int32)
    scale_byte = (e + 127).astype(np.uint8)
    q = g.astype(np.float64) * np.ldexp(1.0, -e)[..., None]
    a = np.abs(q)
    if mode == MODE_KERNEL:
        mag = (a[..., None] >= _E2M1_LOW).sum(axis=-1).astype(np.uint8)
        sign = np.signbit(q)
    else:
        mag = (a[..., None] > _E2M1_MID).sum(axis=-1).astype(np.uint8)
        sign = q < 0
    nib = (mag | (sign.astype(np.uint8) << 3)).reshape(M, D)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    return packed, scale_byte


def quant_mxfp4_literal(row):
    """The reference text, transcribed as a scalar loop for ONE row (small inputs only):
    kernels/quantization/fused_mxfp4_quant/test_parity.py:67-96.  Returns
    (dequantized-in-block-units values, scale bytes).  Used to pin quant_mxfp4(mode=0)."""
    row = np.asarray(row, dtype=np.float64)
    vals, scales = [], []
    for i in range(len(row) // 32):
        block = row[i * 32:(i + 1) * 32]
        block_max = np.abs(block).max()
        exp = int(np.floor(np.log2(block_max))) - 2
        scaled = block / (2.0 ** exp)
        for v in scaled:
            sign = 1 if v >= 0 else -1
            idx = int(np.argmin([abs(abs(v) - m) for m in _E2M1_MAG]))
            vals.append(sign * _E2M1_MAG[idx])
        scales.append(exp + 127)
    return np.array(vals), np.array(scales)
