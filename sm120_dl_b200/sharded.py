"""Multi-GPU partitioning of the two hot paths: one process per GPU, no exchange needed to
compute, an optional all-gather of the output when the caller wants it whole.

  GEMM       by N-column blocks: rank r owns columns [n0, n1) of C; it needs all of A and
             rows [n0, n1) of B ([N,K] row-major, so a contiguous slab) and produces
             C[:, n0:n1].
  attention  by heads: rank r owns heads [h0, h1) of every batch; the sequence stays whole.

Two ways to leave the whole output on every rank: all-gather after the kernel
(`gather=True`), or `gemm_column_shard_fused`, where the GEMM epilogue itself stores each
finished tile into every rank's C over NVLink (peer-mapped symmetric memory).

The reference has no multi-GPU code (both of its launchers even query device 0 for the SM
count, gemm/gemm_cute.hpp:343-346, flashattention/v3_mMnNkN/flashatten_v3.hpp:565-567);
this module is new.  Collectives go through torch.distributed (NCCL over NVLink on GPUs;
gloo in the CPU tests of the host logic).  The compute callables default to the sm_100a
kernels and can be replaced only so the partition / gather logic can be tested without a
GPU.
"""

import torch
import torch.distributed as dist


def shard_bounds(total, world, rank, granule=1):
    """[begin, end) of `rank`'s share of `total` items split into `world` contiguous
    shards whose sizes are multiples of `granule` (except that nothing is lost: total must
    be a multiple of granule).  Earlier ranks take the larger shards."""
    if total % granule != 0:
        raise ValueError(f"{total} is not a multiple of the granule {granule}")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    units = total // granule
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * granule, end * granule


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def gemm_column_shard(a, b, group=None, gather=False, granule=256, compute=None, config=None, out=None,
                      root=None, panels=1):
    """C = A @ B^T with the N dimension split across the ranks of `group`.

    a [M,K] is replicated; b is the FULL [N,K] matrix on every rank (each rank reads only
    its own row slab of it).  Returns (c, (n0, n1)): with gather=False c is this rank's
    contiguous [M, n1-n0] slab; with gather=True c is the full [M,N] on every rank.

    The gather takes the fast path when the caller supplies the output as
    out=(c_full, handle) from symmetric_empty(): the GEMM's epilogue then stores every
    finished tile straight into the ranks' copies of c_full over NVLink (see
    gemm_column_shard_fused; `root` limits the destinations to one rank).  Without such a
    buffer it falls back to an NCCL all-gather of the slabs plus a strided copy into place
    (column slabs of a row-major matrix are not contiguous).  With panels > 1 that fallback is
    pipelined over row panels of A: the slab of panel p is gathered (asynchronously, on the
    collective's own stream) while the GEMM of panel p+1 runs, so the collective hides the
    compute instead of following it.  (Equal shards only; M must divide into the panels.)
    """
    if gather and out is not None and compute is None:
        c_full, handle = out
        return gemm_column_shard_fused(a, b, c_full, handle, granule=granule, config=config, root=root)
    if compute is None:
        from . import ops
        compute = lambda x, y, out: ops.gemm_bf16_tn(x, y, out=out, config=config)  # noqa: E731
    world, rank = _world(group)
    M, _ = a.shape
    N = b.shape[0]
    n0, n1 = shard_bounds(N, world, rank, granule)
    slab = torch.empty((M, n1 - n0), dtype=a.dtype, device=a.device)
    sizes = [shard_bounds(N, world, r, granule) for r in range(world)]
    widths = [e - s for s, e in sizes]
    if gather and world > 1 and panels > 1 and len(set(widths)) == 1 and widths[0] > 0 and M % panels == 0:
        rows = M // panels
        full = torch.empty((M, N), dtype=a.dtype, device=a.device)
        staging = torch.empty((panels, world, rows, widths[0]), dtype=a.dtype, device=a.device)
        pending = []
        for p in range(panels):
            part = slab[p * rows:(p + 1) * rows]                     # contiguous: whole rows of the slab
            compute(a[p * rows:(p + 1) * rows], b[n0:n1], part)
            pending.append(dist.all_gather_into_tensor(staging[p].view(world * rows, widths[0]), part, group=group,
                                                       async_op=True))
        for p, work in enumerate(pending):
            work.wait()
            full[p * rows:(p + 1) * rows].view(rows, world, widths[0]).copy_(staging[p].permute(1, 0, 2))
        return full, (n0, n1)
    if n1 > n0:
        compute(a, b[n0:n1], slab)
    if not gather or world == 1:
        return slab, (n0, n1)
    full = torch.empty((M, N), dtype=a.dtype, device=a.device)
    if len(set(widths)) == 1:
        staging = torch.empty((world, M, widths[0]), dtype=a.dtype, device=a.device)
        dist.all_gather_into_tensor(staging.view(world * M, widths[0]), slab, group=group)
        full.view(M, world, widths[0]).copy_(staging.permute(1, 0, 2))
    else:
        # Uneven shards: every rank contributes a slab padded to the widest shard.
        wmax = max(widths)
        padded = torch.zeros((M, wmax), dtype=a.dtype, device=a.device)
        padded[:, :n1 - n0].copy_(slab)
        staging = torch.empty((world, M, wmax), dtype=a.dtype, device=a.device)
        dist.all_gather_into_tensor(staging.view(world * M, wmax), padded, group=group)
        for r, (s, e) in enumerate(sizes):
            full[:, s:e].copy_(staging[r, :, :e - s])
    return full, (n0, n1)


def symmetric_empty(shape, dtype, device, group=None):
    """A tensor every rank of `group` can address on every other rank (torch symmetric
    memory: peer-mapped over NVLink).  Collective.  Returns (local tensor, handle)."""
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(*shape, dtype=dtype, device=device)
    handle = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
    return t, handle


def gemm_column_shard_fused(a, b, c_full, handle, granule=256, config=None, sync=True, root=None):
    """C = A @ B^T split by N-column blocks, with the gather fused into the GEMM's epilogue.

    `c_full` [M,N] and `handle` come from symmetric_empty(); each rank's kernel stores every
    finished tile of its column slab into ALL ranks' copies of c_full (TMA stores to peer
    memory), so when the ranks have synchronised every copy holds the full C -- no
    all-gather, no staging buffer, no un-permute copy.  With `root` set, only rank `root`'s
    copy is written ("the full output on one rank"): every other rank then sends its slab once
    instead of world-1 times.  With sync=True the call ends with a barrier over the group on
    the current stream; a caller that reuses c_full must also keep readers of the previous
    contents ahead of the next call (same barrier).
    """
    from . import ops
    world, rank = handle.world_size, handle.rank
    M, N = c_full.shape
    n0, n1 = shard_bounds(N, world, rank, granule)
    if n1 > n0:
        targets = range(world) if root is None else [root]
        outs = [handle.get_buffer(r, (M, N), c_full.dtype)[:, n0:n1] for r in targets]
        if root is None:
            # own copy first: local stores start draining while the peer maps are touched
            outs = outs[rank:] + outs[:rank]
        ops.gemm_bf16_tn_scatter(a, b[n0:n1], outs, config=config)
    if sync:
        handle.barrier()
    return c_full, (n0, n1)


def attention_head_shard(q, k, v, causal=False, group=None, gather=False, compute=None, config=None, out=None,
                         root=None):
    """Attention forward with the heads split across the ranks of `group`.

    q, k, v are the FULL [B,S,H,D] tensors on every rank; each rank computes heads
    [h0, h1) through strided views.  Returns (o, (h0, h1)): with gather=False o is
    [B,S,h1-h0,D]; with gather=True the full [B,S,H,D] on every rank -- through the fused
    path when out=(o_full, handle) from symmetric_empty() is supplied, else through an NCCL
    all-gather and a strided copy.
    """
    if gather and out is not None and compute is None:
        o_full, handle = out
        return attention_head_shard_fused(q, k, v, o_full, handle, causal=causal, config=config, root=root)
    if compute is None:
        from . import ops
        compute = lambda x, y, z, c: ops.flash_attn_fwd(x, y, z, causal=c, config=config)  # noqa: E731
    world, rank = _world(group)
    B, S, H, D = q.shape
    h0, h1 = shard_bounds(H, world, rank)
    if h1 > h0:
        part = compute(q[:, :, h0:h1], k[:, :, h0:h1], v[:, :, h0:h1], causal)
    else:
        part = torch.empty((B, S, 0, D), dtype=q.dtype, device=q.device)
    if not gather or world == 1:
        return part, (h0, h1)
    sizes = [shard_bounds(H, world, r) for r in range(world)]
    counts = [e - s for s, e in sizes]
    full = torch.empty((B, S, H, D), dtype=q.dtype, device=q.device)
    if len(set(counts)) == 1:
        staging = torch.empty((world, B, S, counts[0], D), dtype=q.dtype, device=q.device)
        dist.all_gather_into_tensor(staging.view(world * B, S, counts[0], D), part.contiguous(), group=group)
        full.view(B, S, world, counts[0], D).copy_(staging.permute(1, 2, 0, 3, 4))
    else:
        cmax = max(counts)
        padded = torch.zeros((B, S, cmax, D), dtype=q.dtype, device=q.device)
        padded[:, :, :h1 - h0].copy_(part)
        staging = torch.empty((world, B, S, cmax, D), dtype=q.dtype, device=q.device)
        dist.all_gather_into_tensor(staging.view(world * B, S, cmax, D), padded, group=group)
        for r, (s, e) in enumerate(sizes):
            full[:, :, s:e].copy_(staging[r, :, :, :e - s])
    return full, (h0, h1)


def attention_head_shard_fused(q, k, v, o_full, handle, causal=False, config=None, sync=True, root=None):
    """Attention with the heads split across ranks and the gather fused into the kernel's
    epilogue: each rank stores its heads' output tiles into ALL ranks' copies of `o_full`
    ([B,S,H,D] from symmetric_empty()).  Same synchronisation rules as
    gemm_column_shard_fused."""
    from . import ops
    world, rank = handle.world_size, handle.rank
    B, S, H, D = o_full.shape
    h0, h1 = shard_bounds(H, world, rank)
    if h1 > h0:
        targets = range(world) if root is None else [root]
        outs = [handle.get_buffer(r, (B, S, H, D), o_full.dtype)[:, :, h0:h1] for r in targets]
        if root is None:
            outs = outs[rank:] + outs[:rank]
        ops.flash_attn_fwd_scatter(q[:, :, h0:h1], k[:, :, h0:h1], v[:, :, h0:h1], outs, causal=causal, config=config)
    if sync:
        handle.barrier()
    return o_full, (h0, h1)
