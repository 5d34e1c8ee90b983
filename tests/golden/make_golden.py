"""Generates tests/golden/*.npz by RUNNING the reference project's own Python reference
functions (CPU, torch) -- the closest thing it has to golden vectors for the quantized-GEMM
path.  Needs a checkout of the reference project (m8than/amd-kernels); the fixtures it writes are
committed so the test-suite never needs the checkout.

    python tests/golden/make_golden.py --ref <path to the reference checkout>

Fixtures (all seed 42, the reference tests' seed):
  gemm_per_token_{M}x{N}x{K}.npz   reference_gemm_a8w8_per_token_scale
      kernels/gemm-basic/gemm_a8w8_per_token_scale/test_parity.py:31-47
  gemm_blockscale_{M}x{N}x{K}_gn{g}.npz   reference_gemm_a8w8_blockscale
      kernels/gemm-basic/gemm_a8w8_blockscale/test_parity.py:36-78
  gemm_afp4_batched.npz   reference_torch of kernels/gemm-batched/batched_gemm_afp4wfp4/test_parity.py:27-63,
      re-expressed as packed e2m1 codes + e8m0 scale bytes that dequantize to exactly its operands
  quant_int8_per_token.npz   the expression of tests/test_misc.py:531-536 on its 1024x4096 input (first 64 rows)
  quant_static_fp8.npz       the expression of tests/test_moe.py:984-999 (256x128, scale 0.5)
  fused_blockscale_mul_add.npz   reference_blockscale_gemm_mul_add on generate_test_data()
      kernels/gemm-fused/fused_gemm_a8w8_blockscale_mul_add/test_parity.py:20-50 (output only; the inputs are
      np.random.seed(42) draws that the test regenerates, checked through a_sum / c_b_sum)
  fused_afp4_mul_add.npz         reference_fp4_gemm_mul_add on generate_test_data()
      kernels/gemm-fused/fused_gemm_afp4wfp4_mul_add/test_parity.py:22-51 (same form)
  fused_blockscale_split_cat.npz   reference_blockscale_gemm_split_cat
      kernels/gemm-fused/fused_gemm_a8w8_blockscale_split_cat/test_parity.py:28-57 on seeded integer-valued operands
      (its D, S1, S2, S3), inputs and outputs
  moe_gemm_blockscale.npz    generate_ogs_routing + reference_moe_a8w8_bs of
      kernels/moe-gemm/moe_op_gemm_a8w8_blockscale/test_parity.py:29-99 (96 tokens, 4 experts, top-2, K=N=256, group 128)
  moe_gemm_mxfp4.npz         generate_routing + reference_moe_mxfp4 of kernels/moe-gemm/moe_op_mxfp4/test_parity.py:49-115
      (80 tokens, 3 experts, top-2, K=128, N=64; output and weights indexed by sorted position, as that script does)
  gemm_ptgq.npz              reference_torch of kernels/gemm-batched/batched_gemm_a8w8_ptgq/test_parity.py:40-82
      (B=4, 128^3, bias; A bf16, int8 weights, scalar weight scale, output bf16)
  e2m1_lut.npz               FP4_LUT / decode_mx_scale of kernels/moe-gemm/moe_op_mxfp4/test_parity.py:30-46
"""
import argparse
import importlib.util
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="path of the reference project's checkout")
    ref = ap.parse_args().ref
    k = os.path.join(ref, "kernels")

    pt = _load(os.path.join(k, "gemm-basic/gemm_a8w8_per_token_scale/test_parity.py"), "ref_pt")
    for (M, N, K) in [(128, 128, 128), (512, 512, 512)]:
        A, B, sa, sb, C = pt.reference_gemm_a8w8_per_token_scale(M, N, K)
        np.savez_compressed(os.path.join(HERE, f"gemm_per_token_{M}x{N}x{K}.npz"),
                            A=A.numpy(), B=B.numpy(), a_scale=sa.numpy(), b_scale=sb.numpy(), C_bf16=_bf16_bits(C))

    bs = _load(os.path.join(k, "gemm-basic/gemm_a8w8_blockscale/test_parity.py"), "ref_bs")
    for (M, N, K, gn) in [(128, 128, 256, 1), (256, 256, 512, 128)]:
        A, B, sa, sb, C = bs.reference_gemm_a8w8_blockscale(M, N, K, group_k=128, group_n=gn)
        np.savez_compressed(os.path.join(HERE, f"gemm_blockscale_{M}x{N}x{K}_gn{gn}.npz"),
                            A=A.numpy(), B=B.numpy(), a_scale=sa.numpy(), b_scale=sb.numpy(), C_bf16=_bf16_bits(C))

    ma = _load(os.path.join(k, "gemm-fused/fused_gemm_a8w8_blockscale_mul_add/test_parity.py"), "ref_bs_ma")
    a, b, sa, sb, c_a, c_b = ma.generate_test_data()
    ref = ma.reference_blockscale_gemm_mul_add(a, b, sa, sb, c_a, c_b, ma.GROUP_K)
    np.savez_compressed(os.path.join(HERE, "fused_blockscale_mul_add.npz"), ref=ref.astype(np.float32),
                        a_sum=np.float64(a.astype(np.float64).sum()), c_b_sum=np.float64(c_b.astype(np.float64).sum()))
    fa = _load(os.path.join(k, "gemm-fused/fused_gemm_afp4wfp4_mul_add/test_parity.py"), "ref_fp4_ma")
    a, b, sa, sb, c_a, c_b = fa.generate_test_data()
    ref = fa.reference_fp4_gemm_mul_add(a, b, sa, sb, c_a, c_b, fa.SCALE_GROUP)
    np.savez_compressed(os.path.join(HERE, "fused_afp4_mul_add.npz"), ref=ref.astype(np.float32),
                        a_sum=np.float64(a.astype(np.float64).sum()), c_b_sum=np.float64(c_b.astype(np.float64).sum()))

    fb = _load(os.path.join(k, "gemm-batched/batched_gemm_afp4wfp4/test_parity.py"), "ref_fp4b")
    A_dq, B_dq, C = fb.reference_torch()          # A [B,M,K] bf16, B [B,K,N] bf16, C [B,M,N] bf16
    lut = np.array([0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)

    def encode(x):                                 # x [.., R, K] fp32, exact fp4 * 2^s per 32 -> codes, bytes
        R, K = x.shape[-2:]
        g = x.reshape(*x.shape[:-1], K // 32, 32)
        codes = np.zeros(g.shape, dtype=np.uint8)
        sbytes = np.zeros(g.shape[:-1], dtype=np.uint8)
        done = np.zeros(g.shape[:-1], dtype=bool)
        for s in range(-8, 9):                     # smallest exponent that represents the block exactly
            q = np.abs(g) / np.float32(2.0 ** s)
            idx = np.abs(q[..., None] - lut).argmin(-1)
            ok = (lut[idx] == q).all(-1) & ~done
            codes[ok] = (idx | ((g < 0) << 3)).astype(np.uint8)[ok]
            sbytes[ok] = s + 127
            done |= ok
        assert done.all()
        nib = codes.reshape(*x.shape)
        return (nib[..., 0::2] | (nib[..., 1::2] << 4)).astype(np.uint8), sbytes

    Af = A_dq.float().numpy()
    Bf = B_dq.float().numpy().transpose(0, 2, 1).copy()     # -> [B, N, K], K-contiguous like the kernels take it
    a_codes, a_sc = encode(Af)
    b_codes, b_sc = encode(Bf)
    np.savez_compressed(os.path.join(HERE, "gemm_afp4_batched.npz"), A=a_codes, B=b_codes, a_scales=a_sc,
                        b_scales=b_sc, A_dq=Af.astype(np.float32), B_dq=Bf.astype(np.float32), C_bf16=_bf16_bits(C))

    sc = _load(os.path.join(k, "gemm-fused/fused_gemm_a8w8_blockscale_split_cat/test_parity.py"), "ref_bs_sc")
    rng = np.random.RandomState(7)
    a = rng.randint(-8, 9, (64, 256)).astype(np.float32)
    b = rng.randint(-8, 9, (sc.N, 256)).astype(np.float32)
    sa = (rng.rand(64, 2) * 0.1 + 0.01).astype(np.float32)
    sb = (rng.rand(2, sc.N) * 0.1 + 0.01).astype(np.float32)
    y = rng.randn(64, sc.D, sc.S3).astype(np.float32)
    c1, c2 = sc.reference_blockscale_gemm_split_cat(a, b, sa, sb, y, sc.GROUP_K, sc.D, sc.S1, sc.S2, sc.S3)
    np.savez_compressed(os.path.join(HERE, "fused_blockscale_split_cat.npz"), a=a, b=b, a_scale=sa, b_scale=sb, y=y, c1=c1, c2=c2,
                        D=sc.D, S1=sc.S1, S2=sc.S2, S3=sc.S3)

    mo = _load(os.path.join(k, "moe-gemm/moe_op_gemm_a8w8_blockscale/test_parity.py"), "ref_moe_bs")
    np.random.seed(42)
    tokens, E, top_k, Kd, Nd = 96, 4, 2, 256, 256
    X = np.random.randint(-16, 17, (tokens, Kd)).astype(np.int8)           # integers e4m3 holds exactly
    Wm = np.random.randint(-16, 17, (E, Kd, Nd)).astype(np.int8)          # the reference's [E, K, N] form
    xs = (np.random.rand(tokens, Kd // 128).astype(np.float32) * 0.01)
    wsc = (np.random.rand(E, Kd // 128, Nd // 128).astype(np.float32) * 0.01)
    hist, offs, gather, expt_data, grid_m = mo.generate_ogs_routing(tokens, E, top_k)
    Y = mo.reference_moe_a8w8_bs(X, Wm, xs, wsc, gather, hist, offs, expt_data, top_k, 128, 128)
    np.savez_compressed(os.path.join(HERE, "moe_gemm_blockscale.npz"), X=X, W_nk=Wm.transpose(0, 2, 1).copy(), x_scale=xs,
                        w_scale=wsc, hist=hist, offs=offs, gather=gather, expt_data=expt_data, top_k=top_k, Y=Y)

    mx = _load(os.path.join(k, "moe-gemm/moe_op_mxfp4/test_parity.py"), "ref_moe_mxfp4")
    np.random.seed(42)
    tokens, E, top_k, Kd, Nd = 80, 3, 2, 128, 64
    A = np.random.randint(0, 255, (tokens, Kd // 2)).astype(np.uint8)
    Bm = np.random.randint(0, 255, (E, Kd // 2, Nd)).astype(np.uint8)          # the reference's [E, K/2, N] form
    A_mx = np.random.randint(120, 134, (tokens, Kd // 32)).astype(np.uint8)
    B_mx = np.random.randint(120, 134, (E, Kd // 32, Nd)).astype(np.uint8)
    a_scale = np.float32(0.01)
    b_scale = (np.random.rand(E).astype(np.float32) * 0.01)
    ids, block_experts, weights, num_padded, num_valid = mx.generate_routing(tokens, E, top_k)
    Cm = mx.reference_moe_mxfp4(A, Bm, A_mx, B_mx, a_scale, b_scale, ids, block_experts, weights, num_valid, top_k, Kd, mul_weight=True)
    np.savez_compressed(os.path.join(HERE, "moe_gemm_mxfp4.npz"), A=A, B_nk=Bm.transpose(0, 2, 1).copy(), A_mx=A_mx,
                        B_mx_nk=B_mx.transpose(0, 2, 1).copy(), a_scale=a_scale, b_scale=b_scale, sorted_ids=ids,
                        expert_ids=block_experts, weights_sorted=weights, num_valid=num_valid, top_k=top_k, C_sorted=Cm)

    pq = _load(os.path.join(k, "gemm-batched/batched_gemm_a8w8_ptgq/test_parity.py"), "ref_ptgq")
    A, B_int8, b_scale, bias, C = pq.reference_torch()          # A [B,M,K] bf16, B [B,K,N] int8, bias [B,1,N] bf16
    np.savez_compressed(os.path.join(HERE, "gemm_ptgq.npz"), A_bf16=_bf16_bits(A),
                        B_nk=B_int8.numpy().transpose(0, 2, 1).copy(), b_scale=np.float32(b_scale.item()),
                        bias_bf16=_bf16_bits(bias), C_bf16=_bf16_bits(C))

    # tests/test_misc.py:522-536 (INT8 per-token), first 64 rows of the 1024x4096 input
    torch.manual_seed(42)
    x = torch.randn(1024, 4096, dtype=torch.bfloat16)[:64]
    xf = x.float()
    row_max = xf.abs().max(dim=1, keepdim=True).values
    ref_scales = (row_max / 127.0).clamp(min=1e-10)
    ref_q = (xf / ref_scales).round().clamp(-127, 127).to(torch.int8)
    np.savez_compressed(os.path.join(HERE, "quant_int8_per_token.npz"), x_bf16=_bf16_bits(x),
                        q=ref_q.numpy(), scales=ref_scales.numpy())

    # tests/test_moe.py:984-999 (static FP8 cast)
    torch.manual_seed(42)
    x = torch.randn(256, 128, dtype=torch.bfloat16)
    scaled = (x.float() / 0.5).clamp(-448, 448)
    ref_bytes = scaled.to(torch.float8_e4m3fn).view(torch.uint8)
    np.savez_compressed(os.path.join(HERE, "quant_static_fp8.npz"), x_bf16=_bf16_bits(x), bytes=ref_bytes.numpy())

    mx = _load(os.path.join(k, "moe-gemm/moe_op_mxfp4/test_parity.py"), "ref_mx")
    allb = np.arange(256, dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "e2m1_lut.npz"), lut=mx.FP4_LUT,
                        e8m0=mx.decode_mx_scale(allb)[1:255], lo=mx.unpack_fp4(allb, 0), hi=mx.unpack_fp4(allb, 1))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
