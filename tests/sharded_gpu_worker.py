"""Worker of tests/test_sharded_gpu.py: one process per GPU under torchrun (NCCL).  Every rank builds the
same seeded problem, runs the column-sharded block-scale GEMM in its three output forms and compares
with the single-GPU GEMM of the whole problem computed on its own device.  Writes rank<r>.json into
$HKB_TEST_OUT; exits non-zero on any mismatch."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "amd-kernels_b200"))

import hipkittens as hk  # noqa: E402
from hipkittens import sharded  # noqa: E402


def problem(M, N, K, dev):
    g = torch.Generator(device=dev).manual_seed(42)          # same bits on every rank
    A = torch.randn(M, K, generator=g, device=dev).bfloat16()
    W = (torch.randn(N, K, generator=g, device=dev) * 0.02).bfloat16()
    idx = torch.randperm(K, generator=torch.Generator().manual_seed(42))[:max(1, K // 100)].to(dev)
    A[:, idx] = (A[:, idx].float() * 20).bfloat16()
    aq = torch.empty(M, K, dtype=torch.uint8, device=dev); sa = torch.empty(M, K // 128, device=dev)
    wq = torch.empty(N, K, dtype=torch.uint8, device=dev); sw = torch.empty(K // 128, N // 128, device=dev)
    hk.fused_rmsnorm_fp8_quant_fwd(A, None, aq, sa, 1e-6)
    hk.weight_quant_128x128(W, wq, sw)
    full = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    hk.gemm.a8w8_blockscale.dispatch(aq, wq, full, sa, sw)
    return aq, sa, wq, sw, full


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    out = {"rank": rank, "world": world}
    ok = True

    # (1) a config-5-shaped shard: K = 8192, 7168 columns per rank
    M, K = 1024, 8192
    N = 7168 * world
    aq, sa, wq, sw, full = problem(M, N, K, dev)
    n0, n1 = sharded.shard_bounds(N, world, rank)
    wq_r, sw_r = sharded.shard_weight(wq, sw, world, rank)
    C_r = torch.empty(M, n1 - n0, dtype=torch.bfloat16, device=dev)
    got = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r)
    out["shard_equals_full_slice"] = bool(got is C_r and torch.equal(C_r, full[:, n0:n1]))
    blocked = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r, gather="blocked")
    out["blocked_gather_ok"] = bool(all(torch.equal(blocked[r], full[:, r * 7168:(r + 1) * 7168]) for r in range(world)))
    assembled = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r, gather=True)
    out["assembled_gather_ok"] = bool(torch.equal(assembled, full))
    # the all-gather fused into the GEMM's epilogue (peer stores into every rank's [M, N])
    peer = sharded.PeerMatrix(M, N, dev)
    peer.local.fill_(float("nan"))
    peer.barrier()
    torch.cuda.synchronize()
    res = sharded.gemm_a8w8_blockscale_gathered(aq, wq_r, sa, sw_r, peer, n0)
    torch.cuda.synchronize()
    out["fused_gather_ok"] = bool(torch.equal(res, full))
    out["fused_gather_kernel"] = hk.last_kernel()

    # (2) an uneven split: 3 column blocks of 128 over the ranks (no gather: shards differ in size)
    M2, N2, K2 = 256, 128 * (2 * world - 1), 512
    aq2, sa2, wq2, sw2, full2 = problem(M2, N2, K2, dev)
    m0, m1 = sharded.shard_bounds(N2, world, rank)
    wq2_r, sw2_r = sharded.shard_weight(wq2, sw2, world, rank)
    C2 = torch.empty(M2, m1 - m0, dtype=torch.bfloat16, device=dev)
    sharded.gemm_a8w8_blockscale(aq2, wq2_r, C2, sa2, sw2_r)
    out["uneven_split_ok"] = bool(torch.equal(C2, full2[:, m0:m1]))
    out["uneven_columns"] = [m0, m1]

    torch.cuda.synchronize()
    ok = all(v for k, v in out.items() if k.endswith("_ok") or k == "shard_equals_full_slice")
    # one file per rank: the ranks' stdout shares a pipe and lines can interleave
    with open(os.path.join(os.environ["HKB_TEST_OUT"], f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
