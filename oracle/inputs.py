"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations.  TEST INFRASTRUCTURE (see package docstring).

Generated on the CPU with ``torch.Generator().manual_seed(42)`` (the reference tests' seed,
tests/test_gemm.py:176) in the order A, W, outlier indices, so that the oracle and the
device see identical bits.  Activations ~ N(0,1), weights ~ N(0,0.02); the block-scale
configurations multiply 1 % of A's channels by 20 (outlier channels).
"""
import torch

SEED = 42

# name -> (M, N, K, batch, outliers)
SHAPES = {
    "c1": (128, 1024, 1024, 1, False),        # per-token FP8 quant + per-token-scale GEMM
    "c2": (4096, 14336, 4096, 1, True),       # block-scale, Llama-3-8B MLP up-projection
    "c3": (8192, 8192, 8192, 1, False),       # MXFP4
    "c4a": (16, 28672, 8192, 1, False),       # decode-shaped per-token
    "c4b": (512, 4096, 4096, 8, False),       # batched per-token
    "c5": (16384, 57344, 8192, 1, True),      # N-sharded block-scale
}


def make_inputs(M, N, K, batch=1, outliers=False, seed=SEED, device="cpu"):
    """Returns (A bf16 [batch?, M, K], W bf16 [batch?, N, K])."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    a_shape = (M, K) if batch == 1 else (batch, M, K)
    w_shape = (N, K) if batch == 1 else (batch, N, K)
    A = torch.randn(a_shape, generator=g, dtype=torch.float32).to(torch.bfloat16)
    W = (torch.randn(w_shape, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    if outliers:
        idx = torch.randperm(K, generator=g)[: max(1, K // 100)]
        A[..., idx] = (A[..., idx].float() * 20.0).to(torch.bfloat16)
    return A.to(device), W.to(device)


def make_config(name, shrink=1, device="cpu"):
    """Inputs of a named configuration; ``shrink`` divides M and N (kept multiples of 128)
    to get a same-distribution case the CPU oracle finishes in seconds."""
    M, N, K, batch, outl = SHAPES[name]
    if shrink > 1:
        M = max(128 if M >= 128 else M, (M // shrink) // 128 * 128 or M)
        N = max(128, (N // shrink) // 128 * 128)
    return make_inputs(M, N, K, batch, outl, device=device)
