"""hipkittens (B200 build) -- the quantized-GEMM path of the reference `hipkittens` package,
re-implemented for NVIDIA B200 (sm_100a) behind the same module and function names.

    import hipkittens as hk

    hk.per_token_quant_fwd(x, q, scales)                        # FP8 e4m3fn, one scale per row
    hk.fused_rmsnorm_fp8_quant_fwd(x, None, q, scales, eps)     # 1x128 block scales
    hk.fused_rmsnorm_mxfp4_quant_fwd(x, None, codes, scales, eps)
    hk.gemm.a8w8_per_token.dispatch(A, B, C, a_scale, b_scale)
    hk.gemm.a8w8.dispatch(A, B, a_scale, b_scale, C)
    hk.gemm.a8w8_blockscale.dispatch(A, B, C, a_scale, b_scale)
    hk.gemm.afp4wfp4.dispatch(A, B, C, a_scales, b_scales)
    hk.batched_gemm.a8w8.dispatch(A, B, a_scale, b_scale, C, bias)
    hk.batched_gemm.afp4wfp4.dispatch(A, B, C, a_scales, b_scales)
    hk.batched_gemm.a8w8_ptgq.dispatch(a_bf16, b, b_scale, c, bias)
    hk.modules['quant_tk'].per_token_quant_fwd(...)

The loader mirrors the reference's (hipkittens/__init__.py:31-111,209-304 there): compiled
extension modules named ``<module>_tk<EXT_SUFFIX>`` are discovered by file name under a
``kernels`` directory next to this package (or ``$HIPKITTENS_KERNELS_DIR``) and loaded lazily;
a missing module raises ``RuntimeError("Kernel module '<name>' not found. Did you compile
it?")``.  Namespaces of the reference that are outside the quantized-GEMM path keep their
attribute names and raise that same error on use.  There is no CPU fallback anywhere: the
extension modules call CUDA kernels through the C ABI of ``libhkb200.so`` only.
"""
import importlib.util
import os
import sysconfig

_THIS_DIR = os.path.dirname(os.path.abspath(__file__))
_KERNELS_DIR = os.path.join(_THIS_DIR, "kernels")
if not os.path.isdir(_KERNELS_DIR):
    _KERNELS_DIR = os.path.join(_THIS_DIR, "..", "kernels")
if not os.path.isdir(_KERNELS_DIR):
    _KERNELS_DIR = os.environ.get("HIPKITTENS_KERNELS_DIR", _KERNELS_DIR)

_EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".cpython-312-x86_64-linux-gnu.so"
_SKIP_PREFIXES = ("ds_read_test", "hk_", "mfma_", "gemm_debug", "test_")

_so_paths = {}   # module name -> path, filled at import
_loaded = {}     # module name -> module, filled on first use


def _discover():
    _so_paths.clear()
    if not os.path.isdir(_KERNELS_DIR):
        return
    for root, _dirs, files in os.walk(_KERNELS_DIR):
        for f in sorted(files):
            if not f.endswith(_EXT_SUFFIX):
                continue
            name = f[: -len(_EXT_SUFFIX)]
            if name.startswith(_SKIP_PREFIXES):
                continue
            _so_paths[name] = os.path.join(root, f)


_discover()


def _load(name):
    if name in _loaded:
        return _loaded[name]
    path = _so_paths.get(name)
    if path is None:
        raise RuntimeError(f"Kernel module '{name}' not found. Did you compile it?")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _loaded[name] = mod
    return mod


class _LazyModuleDict:
    """``hk.modules[name]``: dict-like view of the discovered extension modules."""

    def __getitem__(self, name):
        return _load(name)

    def __contains__(self, name):
        return name in _so_paths

    def __len__(self):
        return len(_so_paths)

    def keys(self):
        return _so_paths.keys()

    def items(self):
        for name in _so_paths:
            yield name, _load(name)

    def get(self, name, default=None):
        try:
            return _load(name)
        except RuntimeError:
            return default

    def __repr__(self):
        return f"<hipkittens.modules: {len(_so_paths)} available, {len(_loaded)} loaded>"


modules = _LazyModuleDict()


def _call(mod_name, func_name, *args, **kwargs):
    fn = getattr(_load(mod_name), func_name, None)
    if fn is None:
        raise RuntimeError(f"Function '{func_name}' not found in '{mod_name}'")
    return fn(*args, **kwargs)


# ---- quantizers (top-level convenience functions, as in the reference) --------------------

def per_token_quant_fwd(*args, **kwargs):
    """(input bf16 [M,D], output [M,D], scales f32 [M,1]).  output.dtype selects the code type:
    float8_e4m3fn / uint8 -> e4m3fn with scale amax/448; int8 -> the reference's INT8 mode."""
    return _call("quant_tk", "per_token_quant_fwd", *args, **kwargs)


def fused_rmsnorm_fp8_quant_fwd(*args, **kwargs):
    """(input, weight_or_None, output [M,D], scales f32 [M,D/128], eps)."""
    return _call("fused_fp8_quant_tk", "fused_rmsnorm_fp8_quant_fwd", *args, **kwargs)


def fused_rmsnorm_mxfp4_quant_fwd(*args, **kwargs):
    """(input, weight_or_None, output u8 [M,D/2], scales u8 [M,D/32], eps[, mode])."""
    return _call("fused_mxfp4_quant_tk", "fused_rmsnorm_mxfp4_quant_fwd", *args, **kwargs)


def fused_rmsnorm_mxfp4_quant_tc_fwd(*args, **kwargs):
    """(input, weight_or_None, output u8 [M,D/2], scales_or_None, sf_tc, eps[, mode]) -- not in the
    reference: also writes the scales in the MXFP4 GEMM's tensor-core layout (``sf_tc`` of
    ``hk.gemm.afp4wfp4.sf_tc_bytes(1, M, D)`` bytes) so that ``dispatch_tc`` needs no re-layout."""
    return _call("fused_mxfp4_quant_tk", "fused_rmsnorm_mxfp4_quant_tc_fwd", *args, **kwargs)


def last_kernel():
    """Name of the kernel variant the last GEMM call of this thread launched (tests, tuning)."""
    return _call("quant_tk", "hkb_last_kernel")


def weight_quant_128x128(*args, **kwargs):
    """(weight bf16 [N,K], output [N,K], scales f32 [K/128,N/128]) -- not in the reference;
    produces the block-scale GEMM's weight operand."""
    return _call("fused_fp8_quant_tk", "weight_quant_128x128", *args, **kwargs)


# ---- namespaces ---------------------------------------------------------------------------

class _SubModule:
    """Lazy handle on one extension module (loaded on first attribute access)."""

    def __init__(self, mod_name):
        self._mod_name = mod_name

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return getattr(_load(self._mod_name), name)

    def __repr__(self):
        return f"<hipkittens.{self._mod_name}>"


class _GemmNamespace:
    # on the quantized-GEMM path
    a8w8 = _SubModule("gemm_a8w8_tk")
    a8w8_blockscale = _SubModule("gemm_a8w8_blockscale_tk")
    a8w8_per_token = _SubModule("gemm_a8w8_per_token_scale_tk")
    afp4wfp4 = _SubModule("gemm_afp4wfp4_tk")
    # names kept for compatibility; not built here (bf16 / mixed-precision variants)
    a16w16 = _SubModule("gemm_a16w16_tk")
    a16w16_atomic = _SubModule("gemm_a16w16_atomic_tk")
    a16w16_gated = _SubModule("gemm_a16w16_gated_tk")
    a16w8_blockscale = _SubModule("gemm_a16w8_blockscale_tk")
    a16wfp4 = _SubModule("gemm_a16wfp4_tk")
    a8wfp4 = _SubModule("gemm_a8wfp4_tk")


class _BatchedGemmNamespace:
    a8w8 = _SubModule("batched_gemm_a8w8_tk")
    a8w8_ptgq = _SubModule("batched_gemm_a8w8_ptgq_tk")    # bf16 activations quantized per 64-K group inside the GEMM
    afp4wfp4 = _SubModule("batched_gemm_afp4wfp4_tk")
    bf16 = _SubModule("batched_gemm_bf16_tk")
    a16wfp4 = _SubModule("batched_gemm_a16wfp4_tk")


class _FusedGemmNamespace:
    # quantized GEMM + multiply-add epilogue (C = c_a * gemm + c_b)
    a8w8_blockscale_mul_add = _SubModule("fused_gemm_a8w8_blockscale_mul_add_tk")
    afp4wfp4_mul_add = _SubModule("fused_gemm_afp4wfp4_mul_add_tk")
    # quantized GEMM + split-concatenate epilogue (c1[:, d, :S1] | y, c2[:, d, :S2])
    a8w8_blockscale_split_cat = _SubModule("fused_gemm_a8w8_blockscale_split_cat_tk")
    afp4wfp4_split_cat = _SubModule("fused_gemm_afp4wfp4_split_cat_tk")
    # names kept for compatibility; not built here (each pairs the quantized GEMM with a bf16 GEMM)
    a8w8_blockscale_a16w16 = _SubModule("fused_gemm_a8w8_blockscale_a16w16_tk")
    afp4wfp4_a16w16 = _SubModule("fused_gemm_afp4wfp4_a16w16_tk")


class _MoeGemmNamespace:
    # grouped (per-expert) quantized GEMMs over expert-sorted rows
    a8w8_blockscale = _SubModule("moe_op_gemm_a8w8_blockscale_tk")
    mxfp4 = _SubModule("moe_op_mxfp4_tk")
    # names kept for compatibility; not built here (bf16 / int4 / fused-activation variants)
    gemm = _SubModule("moe_op_tk")
    e2e = _SubModule("moe_op_e2e_tk")
    gelu = _SubModule("moe_op_gelu_tk")
    silu_fused = _SubModule("moe_op_silu_fused_tk")
    a4w4 = _SubModule("moe_op_gemm_a4w4_tk")
    a8w4 = _SubModule("moe_op_gemm_a8w4_tk")
    a8w8 = _SubModule("moe_op_gemm_a8w8_tk")
    mxfp4_silu_fused = _SubModule("moe_op_mxfp4_silu_fused_tk")


class _MoeRoutingNamespace:
    # the MoE activation / weight casts (static FP8, MX FP8 / FP4 down- and up-cast)
    quant = _SubModule("quant_moe_tk")
    # names kept for compatibility; not built here (routing, not quantization)
    align_block_size = _SubModule("moe_align_block_size_tk")
    bitmatrix = _SubModule("moe_bitmatrix_tk")
    expt_data = _SubModule("moe_expt_data_tk")
    topk = _SubModule("moe_topk_tk")
    sigmoid_top1_fused = _SubModule("moe_routing_sigmoid_top1_fused_tk")


gemm = _GemmNamespace()
batched_gemm = _BatchedGemmNamespace()
fused_gemm = _FusedGemmNamespace()
moe_gemm = _MoeGemmNamespace()
moe_routing = _MoeRoutingNamespace()

from . import sharded  # noqa: E402,F401  (N-sharded block-scale GEMM over torch.distributed)
