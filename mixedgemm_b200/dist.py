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


def _pitched_base(t):
    """[rows, pitch] buffer under a [rows, logical] row-pitched view (or the tensor itself)."""
    if t.is_contiguous():
        return t
    return t.as_strided((t.size(0), t.stride(0)), (t.stride(0), 1), t.storage_offset())


def activation_shard(A, M, split, world, rank):
    """Views of the six full-size activation buffers that hold rows [rank*M/P, (rank+1)*M/P):
    what this rank's quantiser writes when the quantisation itself is sharded along M.  M/P must
    be a multiple of 128 so that a shard is whole scale blocks."""
    if M % (128 * world) != 0:
        raise ValueError("M = %d cannot be split into %d shards of whole 128-row blocks" % (M, world))
    mp = M // world
    r0 = rank * mp
    out = [A[i][r0:r0 + mp] for i in range(3)]
    for i, k in enumerate(split):
        per_block = ((k + 127) // 128) * 512
        out.append(A[3 + i][(r0 // 128) * per_block:((r0 + mp) // 128) * per_block])
    return tuple(out)


def all_gather_activations(A, M, split, world, rank, group=None):
    """Every rank has quantised its own M/P rows in place (activation_shard); gather the other
    ranks' rows so that each GPU holds the whole quantised activation in its own memory."""
    mp = M // world
    for i in range(3):
        if A[i].numel() == 0:
            continue
        base = _pitched_base(A[i])
        dist.all_gather_into_tensor(base.view(-1), base[rank * mp:(rank + 1) * mp].reshape(-1), group=group)
    for i, k in enumerate(split):
        if k == 0:
            continue
        per_block = ((k + 127) // 128) * 512
        n = (M // 128) * per_block
        full = A[3 + i][:n]
        dist.all_gather_into_tensor(full, full[(rank * mp // 128) * per_block:((rank + 1) * mp // 128) * per_block],
                                    group=group)


def all_gather_output(Y_local, world, group=None):
    """[M, N/P] shards -> [M, N] (only for callers that need the full tensor)."""
    parts = [torch.empty_like(Y_local) for _ in range(world)]
    dist.all_gather(parts, Y_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def all_gather_rows(Y_local, world, group=None):
    """Token-sharded use (every rank multiplies its own M/P rows with all weights; nothing is
    exchanged on the way in): [M/P, N] shards -> [M, N], for callers that need the full tensor."""
    full = torch.empty((Y_local.size(0) * world,) + tuple(Y_local.shape[1:]), dtype=Y_local.dtype,
                       device=Y_local.device)
    dist.all_gather_into_tensor(full, Y_local.contiguous(), group=group)
    return full
