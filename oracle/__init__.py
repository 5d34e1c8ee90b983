"""CPU oracle for the quantized-GEMM path.  TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU, the arithmetic that the reference project
defines for its quantizers and quantized GEMMs (in the PyTorch/NumPy
expressions of its tests).  It exists to check the CUDA kernels; it is never a
fallback.  Only the test-suite, the smoke check and the benchmark's
``cpu_baseline`` / ``--impl reference`` legs may import it.

Parity status of each piece (pinned = checked against a vector or expression
that the reference's own tests hold):

  * e4m3fn cast ............. pinned  (tests/test_moe.py:997-999 cast expression)
  * per-token scale rule .... pinned  (tests/test_misc.py:531-536, INT8 variant)
  * E2M1 LUT / nibble order / E8M0 decode ... pinned
        (kernels/moe-gemm/moe_op_mxfp4/test_parity.py:30-46)
  * GEMM expressions ........ pinned  (kernels/gemm-basic/*/test_parity.py
        reference_* functions, imported to make tests/golden/*.npz)
  * 1x128 / 128x128 FP8 block quantizers, MXFP4 encoder ... parity unpinned:
        the reference tests only assert "some byte is non-zero"
        (tests/test_misc.py:569-571,597-599); the rule restated here is the one
        printed in kernels/quantization/fused_*_quant/test_parity.py.
"""
from . import codecs, quant, gemm, inputs  # noqa: F401
