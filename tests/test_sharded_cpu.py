"""CPU tier: host logic of the N-sharded block-scale GEMM with two `gloo` ranks.  The CUDA GEMM
is replaced by the oracle (allowed here: this is the test-suite) so that partitioning, the
optional all-gather and the re-tiling of the gathered shards are exercised without a GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hipkittens import sharded
from oracle import gemm as ogemm, inputs, quant as oquant


def test_shard_bounds_cover_n_without_overlap():
    for N, g in [(57344, 8), (57344, 4), (14336, 8), (1024, 3), (128, 2), (384, 2)]:
        edges = [sharded.shard_bounds(N, g, r) for r in range(g)]
        assert edges[0][0] == 0 and edges[-1][1] == N
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0 and a0 % 128 == 0 and a1 % 128 == 0
        sizes = [b - a for a, b in edges]
        assert max(sizes) - min(sizes) <= 128
    assert sharded.shard_bounds(57344, 8, 3) == (21504, 28672)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1000, 2, 0)
    with pytest.raises(ValueError):
        sharded.shard_bounds(1024, 2, 2)


def test_c_abi_shard_bounds_agree_with_the_python_rule():
    import ctypes
    lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "amd-kernels_b200", "kernels", "libhkb200.so"))
    i64 = ctypes.c_int64
    for N, g in [(57344, 8), (57344, 3), (1024, 3), (128, 2), (384, 2)]:
        for r in range(g):
            a, b = i64(), i64()
            assert lib.hkb_shard_bounds(i64(N), i64(g), i64(r), ctypes.byref(a), ctypes.byref(b)) == 0
            assert (a.value, b.value) == sharded.shard_bounds(N, g, r)
    a, b = i64(), i64()
    assert lib.hkb_shard_bounds(i64(1000), i64(2), i64(0), ctypes.byref(a), ctypes.byref(b)) == -2
    assert lib.hkb_shard_bounds(i64(1024), i64(2), i64(2), ctypes.byref(a), ctypes.byref(b)) == -1


def test_shard_weight_slices_codes_and_scales_consistently():
    _, W = inputs.make_inputs(128, 512, 256)
    wq, sw = oquant.quant_fp8_128x128(W)
    wq, sw = torch.from_numpy(wq), torch.from_numpy(sw)
    parts = [sharded.shard_weight(wq, sw, 2, r) for r in range(2)]
    assert torch.equal(torch.cat([p[0] for p in parts], 0), wq)
    assert torch.equal(torch.cat([p[1] for p in parts], 1), sw)
    # gn = 1 layout: one scale per output column
    sw1 = sw.repeat_interleave(128, dim=1)
    p1 = sharded.shard_weight(wq, sw1, 2, 1)
    assert p1[1].shape == (2, 256) and torch.equal(p1[1], sw1[:, 256:])


def _oracle_gemm(A, B, C, sa, sb):
    C.copy_(torch.from_numpy(ogemm.gemm_fp8_blockscale(A, B, sa, sb)).bfloat16())


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A, W = inputs.make_inputs(128, 512, 256, outliers=True)      # identical on every rank (seeded)
        aq, sa = oquant.quant_fp8_1x128(A)
        wq, sw = oquant.quant_fp8_128x128(W)
        aq, sa, wq, sw = map(torch.from_numpy, (aq, sa, wq, sw))
        wq_r, sw_r = sharded.shard_weight(wq, sw, world, rank)
        n0, n1 = sharded.shard_bounds(512, world, rank)
        C_r = torch.empty(128, n1 - n0, dtype=torch.bfloat16)
        # without gather: the local shard only, no collective
        got = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r, gemm_fn=_oracle_gemm)
        assert got is C_r
        full = torch.from_numpy(ogemm.gemm_fp8_blockscale(aq, wq, sa, sw)).bfloat16()
        assert torch.equal(C_r, full[:, n0:n1])
        # with gather: every rank ends up with the assembled [M, N]
        out = torch.empty(128, 512, dtype=torch.bfloat16)
        got = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r, gather=True, out=out, gemm_fn=_oracle_gemm)
        assert got is out and torch.equal(out, full)
        got2 = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r, gather=True, gemm_fn=_oracle_gemm)
        assert torch.equal(got2, full) and got2.is_contiguous()
        # blocked form: what the collective produces, block r = rank r's columns, no re-tiling copy
        blocked = sharded.gemm_a8w8_blockscale(aq, wq_r, C_r, sa, sw_r, gather="blocked", gemm_fn=_oracle_gemm)
        assert blocked.shape == (world, 128, 512 // world)
        assert all(torch.equal(blocked[r], full[:, r * (512 // world):(r + 1) * (512 // world)]) for r in range(world))
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_gather(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")


def test_gather_layout_is_column_blocks_in_rank_order():
    # [g, M, N/g] -> [M, N]: what the gather path does after the collective
    g, M, n = 4, 3, 2
    blocked = torch.arange(g * M * n).reshape(g, M, n)
    full = blocked.permute(1, 0, 2).reshape(M, g * n)
    for r in range(g):
        assert torch.equal(full[:, r * n:(r + 1) * n], blocked[r])
    assert np.array_equal(full[0].numpy(), [0, 1, 6, 7, 12, 13, 18, 19])


def test_bind_host_to_gpu_leaves_affinity_alone_without_a_gpu():
    before = os.sched_getaffinity(0)
    got = sharded.bind_host_to_gpu(torch.device("cuda", 0))
    if not torch.cuda.is_available():
        assert got is None and os.sched_getaffinity(0) == before
    else:
        assert got is None or set(got) <= before
    os.sched_setaffinity(0, before)
