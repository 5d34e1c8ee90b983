"""GPU tier: a plain C program (gcc, CUDA runtime API, no Python, no torch) drives the library through
include/hkb200.h -- the way a cgo / JNI / FFI binding of the reference's host side would."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C_SOURCE = r'''
#include "hkb200.h"
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define CHECK(x) do { if ((x) != cudaSuccess) { printf("cuda error at line %d\n", __LINE__); return 2; } } while (0)

int main(void) {
    enum { M = 256, N = 384, K = 512 };
    /* activations: bf16 with one large value per row, so that the per-token quantizer's scale is row + 1 over 448 */
    unsigned short* hx = (unsigned short*)malloc(sizeof(unsigned short) * M * K);
    float* hs = (float*)malloc(sizeof(float) * M);
    unsigned char* hq = (unsigned char*)malloc(M * K);
    unsigned short* hc = (unsigned short*)malloc(sizeof(unsigned short) * M * N);
    unsigned char* hb = (unsigned char*)malloc(N * K);
    float* hsb = (float*)malloc(sizeof(float) * N);
    int i, j, bad = 0;
    for (i = 0; i < M; ++i)
        for (j = 0; j < K; ++j) hx[i * K + j] = 0x4000;          /* bf16 2.0 everywhere */
    memset(hb, 0x38, N * K);                                     /* e4m3fn 1.0 */
    for (j = 0; j < N; ++j) hsb[j] = 0.5f;
    void *dx, *dq, *ds, *db, *dsb, *dc;
    CHECK(cudaMalloc(&dx, sizeof(unsigned short) * M * K)); CHECK(cudaMalloc(&dq, M * K)); CHECK(cudaMalloc(&ds, sizeof(float) * M));
    CHECK(cudaMalloc(&db, N * K)); CHECK(cudaMalloc(&dsb, sizeof(float) * N)); CHECK(cudaMalloc(&dc, sizeof(unsigned short) * M * N));
    CHECK(cudaMemcpy(dx, hx, sizeof(unsigned short) * M * K, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(db, hb, N * K, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(dsb, hsb, sizeof(float) * N, cudaMemcpyHostToDevice));
    int rc = hkb_quant_fp8_per_token(dx, dq, (float*)ds, M, K, K, 0);
    if (rc != HKB_OK) { printf("quant rc %d: %s\n", rc, hkb_last_error()); return 3; }
    rc = hkb_gemm_fp8_pts(dq, db, dc, (const float*)ds, (const float*)dsb, 0, 1, M, N, K, 0);
    if (rc != HKB_OK) { printf("gemm rc %d: %s\n", rc, hkb_last_error()); return 4; }
    CHECK(cudaDeviceSynchronize());
    rc = hkb_check_status(0);
    if (rc != HKB_OK) { printf("status rc %d: %s\n", rc, hkb_last_error()); return 5; }
    CHECK(cudaMemcpy(hq, dq, M * K, cudaMemcpyDeviceToHost));
    CHECK(cudaMemcpy(hs, ds, sizeof(float) * M, cudaMemcpyDeviceToHost));
    CHECK(cudaMemcpy(hc, dc, sizeof(unsigned short) * M * N, cudaMemcpyDeviceToHost));
    /* every element 2.0 -> scale 2/448, code 0x7E (448); C = K * 448 * (2/448) * 1.0 * 0.5 = K = 512 = bf16 0x4400 */
    for (i = 0; i < M * K; ++i) bad += hq[i] != 0x7E;
    for (i = 0; i < M; ++i) bad += hs[i] != 2.0f / 448.0f;
    for (i = 0; i < M * N; ++i) bad += hc[i] != 0x4400;
    printf("version %d kernel %s mismatches %d\n", hkb_version(), hkb_last_kernel(), bad);
    return bad != 0;
}
'''


@pytest.mark.gpu
def test_c_program_quantizes_and_multiplies_through_the_c_abi(tmp_path):
    gcc = shutil.which("gcc")
    inc = "/usr/local/cuda/include"
    if gcc is None or not os.path.exists(os.path.join(inc, "cuda_runtime_api.h")):
        pytest.skip("no C compiler or CUDA runtime headers")
    libdir = os.path.join(ROOT, "amd-kernels_b200", "kernels")
    src = tmp_path / "caller.c"
    src.write_text(C_SOURCE)
    exe = tmp_path / "caller"
    subprocess.run([gcc, "-std=c99", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", inc, str(src), "-o", str(exe), "-L", libdir, "-lhkb200",
                    "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir + ":/usr/local/cuda/lib64"], check=True, capture_output=True, text=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "mismatches 0" in r.stdout and "gemm_fp8_kernel" in r.stdout
