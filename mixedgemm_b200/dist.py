"""N-sharded multi-GPU use of the path (one process per GPU, torch.distributed for the plumbing).

The GEMM shards along N: rank r owns output columns [r*N/P, (r+1)*N/P), i.e. rows of the
quantised weight.  K is never split, so every output element is computed exactly as on one
GPU.  The one exchange step is the broadcast of the quantised activations (six buffers) from
the rank that quantised them; outputs stay sharded unless the caller gathers them.

The reference has no multi-GPU mode; these helpers are tensor-library agnostic on purpose
(they work on CPU tensors over gloo as well), the kernels never see another GPU's memory.
"""
import torch
import torch.distributed as dist


def shard_range(N, world, rank):
    """(first row, row count) of `rank`'s weight shard.  Shards are whole 128-row scale blocks."""
    if N % (128 * world) != 0:
        raise ValueError("N = %d cannot be split into %d shards of whole 128-row blocks" % (N, world))
    n = N // world
    return rank * n, n


def sf_shard(sf, N, kseg, world, rank):
    """The slice of a swizzled weight-scale buffer that belongs to `rank`'s rows: scale atoms of a
    128-row block are contiguous, so a row shard is a contiguous byte range."""
    r0, n = shard_range(N, world, rank)
    per_block = ((kseg + 127) // 128) * 512
    return sf[(r0 // 128) * per_block:((r0 + n) // 128) * per_block]


def shard_weights(B, N, KN, KS, KO, world, rank):
    """B = (BN, BS, BO, SFBN, SFBS, SFBO) of the full weight -> the same six for `rank`'s shard
    (views, no copy)."""
    r0, n = shard_range(N, world, rank)
    return (B[0][r0:r0 + n], B[1][r0:r0 + n], B[2][r0:r0 + n],
            sf_shard(B[3], N, KN, world, rank), sf_shard(B[4], N, KS, world, rank), sf_shard(B[5], N, KO, world, rank))


def broadcast_activations(A, src=0, group=None):
    """Broadcast the six quantised-activation buffers from `src` into every rank's own memory.
    Buffers carved from one allocation (alloc_quantized_x(one_buffer=True)) go as a single
    transfer; otherwise each buffer is sent on its own, row-pitched views with their padding."""
    live = [t for t in A if t.numel()]
    if not live:
        return
    storages = {t.untyped_storage().data_ptr() for t in live}
    if len(storages) == 1 and len(live) > 1:
        st = live[0].untyped_storage()
        flat = torch.empty(0, dtype=torch.uint8, device=live[0].device).set_(st, 0, (st.nbytes(),))
        dist.broadcast(flat, src=src, group=group)
        return
    for t in live:
        base = t
        if not t.is_contiguous():
            # a pitched view [rows, logical] of a [rows, pitch] buffer: send the whole buffer
            base = t.as_strided((t.size(0), t.stride(0)), (t.stride(0), 1), t.storage_offset())
        dist.broadcast(base, src=src, group=group)


def all_gather_output(Y_local, world, group=None):
    """[M, N/P] shards -> [M, N] (only for callers that need the full tensor)."""
    parts = [torch.empty_like(Y_local) for _ in range(world)]
    dist.all_gather(parts, Y_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)
