"""N-sharded (column-parallel) block-scale FP8 GEMM across the GPUs of one node.

One process per GPU (torch.distributed, NCCL over NVLink).  The weight ``W[N, K]`` and its
``b_scale[K/128, N/gn]`` are split along N: rank r owns output columns
``[r*N/g, (r+1)*N/g)``; activations and ``a_scale`` are replicated.  The GEMM itself needs no
communication -- each rank writes its own ``C_r[M, N/g]``.  Only when the caller asks for the
assembled ``C[M, N]`` is there a collective: one all-gather of the bf16 shards.

The reference project has no multi-GPU code; this module is the multi-GPU form of
``hk.gemm.a8w8_blockscale.dispatch`` (kernels/gemm-basic/gemm_a8w8_blockscale/kernel.cpp:51-180).
"""
import torch
import torch.distributed as dist


def bind_host_to_gpu(device):
    """Restrict the calling process to the CPU cores NVML reports as nearest to ``device`` (same socket /
    NUMA node), so that pinned host buffers allocated afterwards are local to the GPU's PCIe root: with one
    process per GPU, uploads and downloads then do not cross the inter-socket link.  Only the process's
    own CPU affinity changes (``os.sched_setaffinity``); NVML is read, nothing on the GPU is set.
    Returns the sorted core list, or ``None`` when NVML has no answer or the cores are not available to
    this process (the affinity is then left as it was)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device).uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        near = {64 * w + b for w, bits in enumerate(words) for b in range(64) if (int(bits) >> b) & 1}
        cores = sorted(near & os.sched_getaffinity(0))
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None


def shard_bounds(N, world_size, rank, align=128):
    """Column range [n0, n1) of ``rank``: N is cut into ``align``-wide blocks which are dealt out
    as evenly as possible (the first ``blocks % world_size`` ranks get one more)."""
    if N % align:
        raise ValueError(f"N={N} must be a multiple of {align}")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    blocks = N // align
    base, extra = divmod(blocks, world_size)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return b0 * align, b1 * align


def shard_weight(Wq, b_scale, world_size, rank):
    """Slice a quantized weight [N, K] and its b_scale [K/128, N/gn] for ``rank``.
    Returns contiguous (Wq_r, b_scale_r)."""
    N = Wq.shape[0]
    gn = N // b_scale.shape[1]
    if gn not in (1, 128):
        raise ValueError(f"b_scale group size along N must be 1 or 128, got {gn}")
    n0, n1 = shard_bounds(N, world_size, rank)
    return Wq[n0:n1].contiguous(), b_scale[:, n0 // gn:n1 // gn].contiguous()


def _default_gemm(A, B, C, a_scale, b_scale):
    from . import gemm
    gemm.a8w8_blockscale.dispatch(A, B, C, a_scale, b_scale)


def gemm_a8w8_blockscale(A, Wq_r, C_r, a_scale, b_scale_r, gather=False, group=None, out=None,
                         gemm_fn=None):
    """Local shard GEMM ``C_r = blockscale(A, Wq_r)``.

    ``gather=False`` (default): no collective, returns ``C_r``.
    ``gather="blocked"``: one all-gather of the bf16 shards; returns the ``[g, M, N/g]`` tensor the
    collective produces (block r = columns of rank r), with no further copy.
    ``gather=True``: the assembled ``[M, N]`` (``out`` if given): the blocked form re-tiled by one
    full-size copy.  On GPUs prefer :func:`gemm_a8w8_blockscale_gathered`, which writes the assembled
    matrix from the GEMM's epilogue and needs neither the collective nor the copy.

    All ranks must hold equally sized shards when gathering (N/128 divisible by the world size).
    ``gemm_fn`` replaces the CUDA GEMM in host-logic tests.
    """
    (gemm_fn or _default_gemm)(A, Wq_r, C_r, a_scale, b_scale_r)
    if not gather:
        return C_r
    world = dist.get_world_size(group)
    M, n_local = C_r.shape
    blocked = torch.empty((world, M, n_local), dtype=C_r.dtype, device=C_r.device)
    dist.all_gather_into_tensor(blocked.view(world * M, n_local), C_r.contiguous(), group=group)
    if gather == "blocked":
        return blocked
    # [g, M, N/g] (what the collective produces) -> [M, N]
    full = blocked.permute(1, 0, 2).reshape(M, world * n_local)
    if out is not None:
        out.copy_(full)
        return out
    return full.contiguous()


class PeerMatrix:
    """A bf16 ``[M, N]`` matrix per rank whose storage every rank of the group can write: the target
    of the GEMM with the all-gather fused into its epilogue.

    Allocated from torch's symmetric memory (one CUDA virtual-memory allocation per rank, mapped into
    every peer of the node over NVLink; multicast binding is not requested -- only plain peer stores
    are used).  ``ptrs(col0)`` lists, own rank first, the device addresses of element ``[0, col0]`` in
    every rank's copy; ``barrier()`` orders all ranks' readers behind all ranks' writers on the
    current stream.
    """

    def __init__(self, M, N, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.M, self.N = M, N
        self.local = symm_mem.empty((M, N), dtype=torch.bfloat16, device=device)
        self._hdl = symm_mem.rendezvous(self.local, self.group)
        self.rank, self.world = self._hdl.rank, self._hdl.world_size
        self._ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)

    def ptrs(self, col0):
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self._ptrs[r] + col0 * 2 for r in order]

    def barrier(self):
        # A one-element all-reduce: it starts on a rank after that rank's GEMM (stream order) and ends
        # only once every rank has joined, i.e. once every rank's stores have been issued and its
        # kernel has completed.
        dist.all_reduce(self._flag, group=self.group)


def gemm_a8w8_blockscale_gathered(A, Wq_r, a_scale, b_scale_r, peer_out, n0):
    """Column-sharded block-scale GEMM whose epilogue writes this rank's ``[M, N/g]`` result into columns
    ``[n0, n0 + N/g)`` of EVERY rank's assembled matrix (``peer_out``, a :class:`PeerMatrix`): the
    all-gather rides on the GEMM's own stores over NVLink and overlaps its main loop.  Returns
    ``peer_out.local`` (complete after the barrier this call ends with)."""
    from . import gemm
    gemm.a8w8_blockscale.dispatch_scatter(A, Wq_r, peer_out.ptrs(n0), peer_out.N, a_scale, b_scale_r)
    peer_out.barrier()
    return peer_out.local
