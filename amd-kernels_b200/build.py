"""Builds libhkb200.so (CUDA kernels + C ABI, sm_100a) and the pybind11 shim modules.

    python amd-kernels_b200/build.py [--force] [--verbose]

Outputs land in amd-kernels_b200/kernels/ (the directory the `hipkittens` loader walks):
    libhkb200.so
    <module>_tk<EXT_SUFFIX>      one per reference module name on the quantized-GEMM path
nvcc cross-compiles for sm_100a without a GPU present.  Objects are rebuilt only when a
source or header is newer than the object.
"""
import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "kernels")
OBJ = os.path.join(HERE, "build")
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"

CU_SOURCES = ["runtime.cu", "quant_fp8.cu", "quant_mxfp4.cu", "quant_moe.cu", "gemm_fp8.cu", "gemm_fp8_skinny.cu", "gemm_mxfp4.cu", "peak_mma.cu", "gemm_fp8_ptgq.cu"]

# module name -> selector macro of csrc/shim.cpp
SHIMS = {
    "quant_tk": "HKB_SHIM_QUANT",
    "fused_fp8_quant_tk": "HKB_SHIM_FUSED_FP8_QUANT",
    "fused_mxfp4_quant_tk": "HKB_SHIM_FUSED_MXFP4_QUANT",
    "gemm_a8w8_tk": "HKB_SHIM_GEMM_A8W8",
    "gemm_a8w8_per_token_scale_tk": "HKB_SHIM_GEMM_A8W8_PER_TOKEN_SCALE",
    "gemm_a8w8_blockscale_tk": "HKB_SHIM_GEMM_A8W8_BLOCKSCALE",
    "gemm_afp4wfp4_tk": "HKB_SHIM_GEMM_AFP4WFP4",
    "batched_gemm_a8w8_tk": "HKB_SHIM_BATCHED_GEMM_A8W8",
    "batched_gemm_afp4wfp4_tk": "HKB_SHIM_BATCHED_GEMM_AFP4WFP4",
    "batched_gemm_a8w8_ptgq_tk": "HKB_SHIM_BATCHED_GEMM_A8W8_PTGQ",
    "fused_gemm_a8w8_blockscale_mul_add_tk": "HKB_SHIM_FUSED_GEMM_A8W8_BLOCKSCALE_MUL_ADD",
    "fused_gemm_afp4wfp4_mul_add_tk": "HKB_SHIM_FUSED_GEMM_AFP4WFP4_MUL_ADD",
    "fused_gemm_a8w8_blockscale_split_cat_tk": "HKB_SHIM_FUSED_GEMM_A8W8_BLOCKSCALE_SPLIT_CAT",
    "fused_gemm_afp4wfp4_split_cat_tk": "HKB_SHIM_FUSED_GEMM_AFP4WFP4_SPLIT_CAT",
    "moe_op_gemm_a8w8_blockscale_tk": "HKB_SHIM_MOE_OP_GEMM_A8W8_BLOCKSCALE",
    "moe_op_mxfp4_tk": "HKB_SHIM_MOE_OP_MXFP4",
    "quant_moe_tk": "HKB_SHIM_QUANT_MOE",
}

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "hkb200.h"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(o, [s] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = os.path.join(OUT, "libhkb200.so")
    if force or jobs or _newer(lib, objs):
        _run([nvcc, "-shared", "-o", lib] + objs + ["-lcudart"], verbose)

    import pybind11
    shim_src = os.path.join(CSRC, "shim.cpp")
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"]]
    jobs = []
    for name, macro in SHIMS.items():
        so = os.path.join(OUT, name + EXT_SUFFIX)
        if force or _newer(so, [shim_src, os.path.join(ROOT, "include", "hkb200.h")]):
            jobs.append(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
                         "-Wno-unused-function", "-DHKB_SHIM_NAME=" + name, "-D" + macro] + inc +
                        [shim_src, "-o", so, "-L" + OUT, "-lhkb200", "-Wl,-rpath,$ORIGIN"])
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
