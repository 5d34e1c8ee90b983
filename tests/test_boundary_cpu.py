"""CPU tier: the drop-in boundary without a GPU -- the C-ABI library loads and exports every
symbol the header declares, argument validation answers with error codes (never a crash, never a
CPU fallback), and the `hipkittens` loader behaves like the reference's."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "amd-kernels_b200", "kernels", "libhkb200.so")
HEADER = os.path.join(ROOT, "include", "hkb200.h")

i64 = ctypes.c_int64


@pytest.fixture(scope="module")
def lib():
    l = ctypes.CDLL(LIB)
    l.hkb_last_error.restype = ctypes.c_char_p
    return l


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hkb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_all_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/hkb200.h but not exported"


def test_version_and_error_string(lib):
    assert lib.hkb_version() >= 100
    assert isinstance(lib.hkb_last_error(), bytes)


def test_null_pointers_are_rejected(lib):
    assert lib.hkb_quant_fp8_per_token(None, None, None, i64(4), i64(128), i64(128), None) == -1
    assert b"null" in lib.hkb_last_error()
    assert lib.hkb_gemm_fp8_pts(None, None, None, None, None, None, i64(1), i64(128), i64(128), i64(128), None) == -1
    assert lib.hkb_gemm_mxfp4(None, None, None, None, None, i64(1), i64(128), i64(128), i64(128), None) == -1


def test_bad_shapes_and_alignment_are_rejected_before_any_cuda_call(lib):
    buf = ctypes.create_string_buffer(4096 + 64)
    base = (ctypes.addressof(buf) + 63) & ~63
    p = ctypes.c_void_p(base)
    f = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    # D not a multiple of 8 / 128 / 32
    assert lib.hkb_quant_fp8_per_token(p, p, f, i64(4), i64(100), i64(100), None) == -2
    assert lib.hkb_quant_fp8_1x128(p, None, p, f, i64(4), i64(192), ctypes.c_float(1e-6), None) == -2
    assert b"128" in lib.hkb_last_error()
    assert lib.hkb_quant_mxfp4(p, None, p, p, i64(4), i64(48), ctypes.c_float(1e-6), 0, None) == -2
    assert lib.hkb_quant_mxfp4(p, None, p, p, i64(4), i64(64), ctypes.c_float(1e-6), 7, None) == -1     # unknown mode
    assert lib.hkb_quant_fp8_128x128(p, p, f, i64(100), i64(128), None) == -2
    # misaligned input
    q = ctypes.c_void_p(base + 2)
    assert lib.hkb_quant_fp8_per_token(q, p, f, i64(4), i64(128), i64(128), None) == -3
    # pitch smaller than the row
    assert lib.hkb_quant_fp8_per_token(p, p, f, i64(4), i64(128), i64(64), None) == -3
    # GEMM: K not a multiple of 128, N not a multiple of 8, gn unsupported
    assert lib.hkb_gemm_fp8_pts(p, p, p, f, f, None, i64(1), i64(128), i64(128), i64(96), None) == -2
    assert lib.hkb_gemm_fp8_pts(p, p, p, f, f, None, i64(1), i64(128), i64(100), i64(128), None) == -2
    assert lib.hkb_gemm_fp8_blockscale(p, p, p, f, f, i64(64), i64(128), i64(128), i64(128), None) == -4
    assert lib.hkb_gemm_fp8_blockscale(p, p, p, f, f, i64(128), i64(128), i64(192), i64(128), None) == -2
    assert lib.hkb_gemm_mxfp4(p, p, p, p, p, i64(1), i64(128), i64(128), i64(64), None) == -2
    assert lib.hkb_gemm_fp8_pts(q, p, p, f, f, None, i64(1), i64(128), i64(128), i64(128), None) == -3


def test_offset_scale_and_bias_pointers_are_an_alignment_error(lib):
    """b_scale and bias are read with 16-byte vector loads by the per-token epilogues: an offset view
    must come back as HKB_ERR_BAD_ALIGN before any device is looked for."""
    buf = ctypes.create_string_buffer(4096 + 64)
    base = (ctypes.addressof(buf) + 63) & ~63
    p = ctypes.c_void_p(base)
    f = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    f_off = ctypes.cast(ctypes.c_void_p(base + 4), ctypes.POINTER(ctypes.c_float))
    args = (i64(1), i64(128), i64(128), i64(128), None)
    assert lib.hkb_gemm_fp8_pts(p, p, p, f, f_off, None, *args) == -3
    assert b"16-byte" in lib.hkb_last_error()
    assert lib.hkb_gemm_fp8_pts(p, p, p, f, f, ctypes.c_void_p(base + 2), *args) == -3
    assert lib.hkb_gemm_fp8_pts(p, p, p, ctypes.cast(ctypes.c_void_p(base + 2), ctypes.POINTER(ctypes.c_float)), f, None, *args) == -3
    # tensor-core-layout scale factors
    assert lib.hkb_mxfp4_sf_to_tc(p, ctypes.c_void_p(base + 4), i64(1), i64(128), i64(128), None) == -3
    assert lib.hkb_gemm_mxfp4_tc(p, p, p, ctypes.c_void_p(base + 4), 1, p, 1, i64(1), i64(128), i64(128), i64(128), None) == -3


def test_mxfp4_tensor_core_layout_size(lib):
    lib.hkb_mxfp4_sf_tc_bytes.restype = ctypes.c_int64
    # 2*ceil(rows/256)+2 row blocks, K/128 rounded up to even atoms of 512 bytes
    assert lib.hkb_mxfp4_sf_tc_bytes(i64(1), i64(8192), i64(8192)) == (2 * 32 + 2) * 64 * 512
    assert lib.hkb_mxfp4_sf_tc_bytes(i64(3), i64(100), i64(384)) == 3 * 4 * 4 * 512
    assert lib.hkb_mxfp4_sf_tc_bytes(i64(1), i64(128), i64(100)) == 0
    assert lib.hkb_mxfp4_sf_tc_bytes(i64(0), i64(128), i64(128)) == 0


def test_wait_probe_validates_its_limit(lib):
    buf = ctypes.create_string_buffer(4096 + 64)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)
    f = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    assert lib.hkb_debug_gemm_fp8_wait_probe(p, p, p, f, f, i64(128), i64(128), i64(128), ctypes.c_uint64(10), None) == -1
    assert lib.hkb_debug_gemm_fp8_wait_probe(p, p, p, f, f, i64(128), i64(128), i64(128), ctypes.c_uint64(10**10), None) == -1


def test_empty_input_is_a_no_op(lib):
    buf = ctypes.create_string_buffer(256)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)
    f = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    assert lib.hkb_quant_fp8_per_token(p, p, f, i64(0), i64(128), i64(128), None) == 0
    assert lib.hkb_quant_mxfp4(p, None, p, p, i64(0), i64(64), ctypes.c_float(1e-6), 0, None) == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_compute_without_a_gpu_fails_loudly_instead_of_falling_back(lib):
    buf = ctypes.create_string_buffer(1 << 16)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)
    f = ctypes.cast(p, ctypes.POINTER(ctypes.c_float))
    rc = lib.hkb_quant_fp8_per_token(p, p, f, i64(4), i64(128), i64(128), None)
    assert rc == -5, "a launch without a CUDA device must return HKB_ERR_CUDA"
    assert lib.hkb_release() == 0


# ---- the Python loader ----------------------------------------------------------------------------

HOT_MODULES = ["quant_tk", "fused_fp8_quant_tk", "fused_mxfp4_quant_tk", "gemm_a8w8_tk", "gemm_a8w8_per_token_scale_tk",
               "gemm_a8w8_blockscale_tk", "gemm_afp4wfp4_tk", "batched_gemm_a8w8_tk", "batched_gemm_afp4wfp4_tk",
               "fused_gemm_a8w8_blockscale_mul_add_tk", "fused_gemm_afp4wfp4_mul_add_tk", "quant_moe_tk",
               "batched_gemm_a8w8_ptgq_tk", "fused_gemm_a8w8_blockscale_split_cat_tk", "fused_gemm_afp4wfp4_split_cat_tk",
               "moe_op_gemm_a8w8_blockscale_tk", "moe_op_mxfp4_tk"]


def test_loader_discovers_the_reference_module_names(hk):
    for m in HOT_MODULES:
        assert m in hk.modules
    assert len(hk.modules) == len(HOT_MODULES)
    assert "available" in repr(hk.modules)
    assert hk.modules.get("no_such_tk") is None


def test_functions_and_argument_names_match_the_reference_bindings(hk):
    assert hk.modules["quant_tk"].per_token_quant_fwd.__doc__.startswith("per_token_quant_fwd(input: object, output: object, scales: object)")
    d = hk.gemm.a8w8_per_token.dispatch.__doc__
    assert d.startswith("dispatch(A: object, B: object, C: object, a_scale: object, b_scale: object)")
    d = hk.gemm.a8w8.dispatch.__doc__
    assert d.startswith("dispatch(A: object, B: object, a_scale: object, b_scale: object, C: object)")
    d = hk.gemm.a8w8_blockscale.dispatch.__doc__
    assert d.startswith("dispatch(A: object, B: object, C: object, a_scale: object, b_scale: object)")
    d = hk.batched_gemm.a8w8.dispatch.__doc__
    assert d.startswith("dispatch(A: object, B: object, a_scale: object, b_scale: object, C: object, bias: object")
    for mod in (hk.fused_gemm.a8w8_blockscale_mul_add, hk.fused_gemm.afp4wfp4_mul_add):
        assert mod.dispatch.__doc__.startswith(
            "dispatch(a: object, b: object, c: object, a_scale: object, b_scale: object, c_a: object, c_b: object)")
    d = hk.batched_gemm.a8w8_ptgq.dispatch.__doc__          # kernels/gemm-batched/batched_gemm_a8w8_ptgq/kernel.cpp:241-249
    assert d.startswith("dispatch(a: object, b: object, b_scale: object, c: object, bias: object")
    for mod in (hk.fused_gemm.a8w8_blockscale_split_cat, hk.fused_gemm.afp4wfp4_split_cat):
        assert mod.dispatch.__doc__.startswith(
            "dispatch(a: object, b: object, a_scale: object, b_scale: object, y: object, c1: object, c2: object)")
    q = hk.moe_routing.quant
    assert q.downcast_to_static_fp8.__doc__.startswith("downcast_to_static_fp8(x: object, y: object, scale: object, M: ")
    assert q.downcast_to_mxfp.__doc__.startswith("downcast_to_mxfp(mx_tensor: object, mx_scale: object, src: object, outer_dim: ")
    assert q.upcast_from_mxfp.__doc__.startswith("upcast_from_mxfp(out: object, mx_scale: object, mx_tensor: object, outer_dim: ")
    d = hk.modules["fused_fp8_quant_tk"].fused_rmsnorm_fp8_quant_fwd.__doc__
    assert d.startswith("fused_rmsnorm_fp8_quant_fwd(input: object, weight: object, output: object, scales: object, eps: ")
    d = hk.modules["fused_mxfp4_quant_tk"].fused_rmsnorm_mxfp4_quant_fwd.__doc__
    assert d.startswith("fused_rmsnorm_mxfp4_quant_fwd(input: object, weight: object, output: object, scales: object, eps: ")


def test_modules_off_the_path_raise_the_reference_error(hk):
    with pytest.raises(RuntimeError, match="Kernel module 'gemm_a16w16_tk' not found. Did you compile it?"):
        hk.gemm.a16w16.dispatch(None, None, None)
    with pytest.raises(RuntimeError, match="Kernel module 'fused_gemm_afp4wfp4_a16w16_tk' not found"):
        hk.fused_gemm.afp4wfp4_a16w16.dispatch(None)
    with pytest.raises(RuntimeError, match="not found"):
        hk.modules["rmsnorm_tk"]


def test_cpu_tensors_are_refused_there_is_no_cpu_path(hk):
    x = torch.randn(4, 128).bfloat16()
    q = torch.empty(4, 128, dtype=torch.uint8)
    s = torch.empty(4, 1)
    with pytest.raises(RuntimeError, match="CUDA device"):
        hk.per_token_quant_fwd(x, q, s)
    c = torch.empty(4, 4, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA device"):
        hk.gemm.a8w8_per_token.dispatch(q, q, c, s, s)


def test_shim_validates_dtype_and_contiguity_first(hk):
    x = torch.randn(4, 128)              # float32 instead of bf16
    q = torch.empty(4, 128, dtype=torch.uint8)
    s = torch.empty(4, 1)
    with pytest.raises(RuntimeError, match="dtype float32 not accepted"):
        hk.per_token_quant_fwd(x, q, s)
    xt = torch.randn(128, 4).bfloat16().t()
    with pytest.raises(RuntimeError, match="contiguous"):
        hk.per_token_quant_fwd(xt, q, s)


def test_mxfp4_gemm_refuses_the_host_dequantized_three_argument_form(hk):
    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="packed e2m1"):
        hk.gemm.afp4wfp4.dispatch(x, x, x)


def test_header_is_plain_c_and_a_c_program_links_against_the_library(tmp_path):
    """include/hkb200.h must compile as strict C99 (no C++ in the boundary) and a C caller must link and get error
    codes, not crashes, without a GPU: the form in which a cgo / JNI / ctypes binding sees the library."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "amd-kernels_b200", "kernels")
    src = tmp_path / "caller.c"
    src.write_text(r'''
#include "hkb200.h"
#include <stdio.h>
int main(void) {
    int64_t n0 = 0, n1 = 0;
    int rc = hkb_shard_bounds(57344, 8, 3, &n0, &n1);
    printf("%d %d %lld %lld\n", hkb_version(), rc, (long long)n0, (long long)n1);
    rc = hkb_gemm_fp8_blockscale(0, 0, 0, 0, 0, 128, 128, 128, 128, 0);
    printf("%d %s\n", rc, hkb_last_error());
    return 0;
}
''')
    exe = tmp_path / "caller"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(root, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-lhkb200", "-Wl,-rpath," + libdir], check=True, capture_output=True, text=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines()
    assert out[0].split() == ["200", "0", "21504", "28672"]
    assert out[1].startswith("-1 ") and "null pointer" in out[1]
