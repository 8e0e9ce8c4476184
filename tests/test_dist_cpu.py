"""world_size-2 CPU (gloo) test of the N-sharded path's host logic: shard ranges, slicing of the
swizzled scale buffers, the byte ranges the exchange moves (what mg_allgather_inplace and
mg_push_shard are told to copy), gather of output shards.  The compute on each rank is the CPU
oracle and the transfers are made by the test over gloo, so the check is on the bookkeeping:
shards recombine to exactly the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mx_oracle as orc
from tests import helpers as H

M, N, SPLIT = 48, 512, (256, 192, 64)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    from mixedgemm_b200 import dist as mgd
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        KN, KS, KO = SPLIT
        K = sum(SPLIT)
        X = H.make_x(M, K, seed=3)
        W = H.make_w(N, K, seed=4)
        idx = H.reorder_index(X).numpy()
        # every rank holds the full quantised weight here only to cut its shard out of it
        Bfull = [torch.from_numpy(np.ascontiguousarray(a)) for a in H.oracle_outputs(H.bits(W), idx, KN, KS, KO, True)]
        Bl = mgd.shard_weights(Bfull, N, KN, KS, KO, world, rank)
        A = [torch.from_numpy(np.ascontiguousarray(a)) for a in H.oracle_outputs(H.bits(X), idx, KN, KS, KO)]
        # quantisation sharded along M: each rank fills its rows of full-size buffers; the byte ranges
        # shard_byte_ranges names are what the exchange copies, here with gloo
        M2 = 256
        X2 = H.make_x(M2, K, seed=9)
        full = [np.ascontiguousarray(a) for a in H.oracle_outputs(H.bits(X2), idx, KN, KS, KO)]
        mine = [torch.zeros_like(torch.from_numpy(a)) for a in full]
        sh = mgd.activation_shard(mine, M2, SPLIT, world, rank)
        mp_ = M2 // world
        part = H.oracle_outputs(H.bits(X2[rank * mp_:(rank + 1) * mp_]), idx, KN, KS, KO)
        for dst, src in zip(sh, part):
            dst.copy_(torch.from_numpy(np.ascontiguousarray(src))[:dst.numel()].view(dst.shape))
        covered = True
        for i in range(6):
            ranges = [mgd.shard_byte_ranges(mine, M2, SPLIT, world, r)[i] for r in range(world)]
            # the ranks' ranges tile the buffer: consecutive, equal, no gap
            covered &= all(ranges[r][1] == r * ranges[0][2] and ranges[r][2] == ranges[0][2] for r in range(world))
            t, first, count = ranges[rank]
            flat = t.view(-1)
            parts = [torch.empty(count, dtype=torch.uint8) for _ in range(world)]
            dist.all_gather(parts, flat[first:first + count].clone())
            for r in range(world):
                flat[ranges[r][1]:ranges[r][1] + count].copy_(parts[r])
        ret["covered_%d" % rank] = bool(covered)
        ret["allgather_%d" % rank] = all(np.array_equal(m.numpy(), f) for m, f in zip(mine, full))
        # N-sharded product: every rank multiplies the whole activation with its weight rows
        r0, n = mgd.shard_range(N, world, rank)
        Yl = torch.from_numpy(orc.gemm_f64([t.numpy() for t in A], [t.numpy() for t in Bl], M, n, KN, KS, KO))
        parts = [torch.empty_like(Yl) for _ in range(world)]
        dist.all_gather(parts, Yl)
        Y = torch.cat(parts, dim=1)
        if rank == 0:
            Yref = orc.gemm_f64([t.numpy() for t in A], [t.numpy() for t in Bfull], M, N, KN, KS, KO)
            ret["equal"] = bool(np.array_equal(Y.numpy(), Yref))
            ret["shape"] = tuple(Y.shape)
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_recombines_exactly():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["shape"] == (M, N)
    assert ret["equal"]
    assert ret["covered_0"] and ret["covered_1"]
    assert ret["allgather_0"] and ret["allgather_1"]


def test_shard_helpers():
    from mixedgemm_b200 import dist as mgd
    assert mgd.shard_range(1024, 8, 3) == (384, 128)
    with pytest.raises(ValueError):
        mgd.shard_range(1024, 3, 0)
    with pytest.raises(ValueError):
        mgd.shard_range(512, 8, 0)  # 64-row shards would split scale atoms
    # scale slices: rows [256, 512) of a 512-row buffer, K segment of 448 (4 atoms per row block)
    sf = torch.arange(4 * 4 * 512, dtype=torch.int32)
    s = mgd.sf_shard(sf, 512, 448, 2, 1)
    assert s[0] == 2 * 4 * 512 and s.numel() == 2 * 4 * 512
    # and the slice holds exactly the scales of those rows
    full = np.arange(orc.sf_bytes(512, 448))
    r = np.arange(256, 512)[:, None]
    kb = np.arange(448 // 32)[None, :]
    want = full[orc.sf_offset(r, kb, 448)]
    got = mgd.sf_shard(torch.from_numpy(full), 512, 448, 2, 1).numpy()[orc.sf_offset(r - 256, kb, 448)]
    assert np.array_equal(got, want)


def test_sharded_activation_describes_equally_spaced_blocks():
    """api.ShardedActivation (the layout the overlapped exchange fills, one block per rank) works out
    the shard strides from the tensors it is given and refuses anything but equal, equally spaced,
    ascending shards of whole 128-row scale blocks.  Host logic only: CPU tensors."""
    from mixedgemm_b200.api import ShardedActivation
    mp_, block = 128, 40960
    flat = torch.zeros(4 * block, dtype=torch.uint8)

    def shard(r, rows=mp_):
        blk = flat[r * block:(r + 1) * block]
        return (blk[0:rows * 64].view(rows, 64), blk[8192:8192 + rows * 48].view(rows, 48),
                blk[16384:16384 + rows * 128].view(rows, 128)[:, :64], blk[32768:33280], blk[33792:34304], blk[34816:35328])

    sa = ShardedActivation([shard(r) for r in range(4)])
    assert sa.rows == 512 and sa.shard_rows == 128 and sa.stride == [block] * 6
    assert ShardedActivation([shard(0)]).rows == 128
    with pytest.raises(RuntimeError):
        ShardedActivation([shard(1), shard(0)])              # descending
    with pytest.raises(RuntimeError):
        ShardedActivation([shard(0), shard(1), shard(3)])    # not equally spaced
    with pytest.raises(RuntimeError):
        ShardedActivation([shard(0, 64), shard(1, 64)])      # not whole scale blocks
    with pytest.raises(RuntimeError):
        ShardedActivation([shard(0), shard(1)[:5]])          # not six tensors


def test_exchange_buffer_layout():
    """exchange_layout (host arithmetic of the overlapped exchange): parts do not overlap, start on
    1 KB boundaries, hold whole rows and whole scale atoms of a rank's M / P rows; the 70B step's block
    is the 17.25 MB per rank that the design quotes for 8 GPUs; bad shapes are refused."""
    from mixedgemm_b200 import dist as mgd
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    shapes = [(4096, (5120, 2816, 256))] * 3 + [(4096, (17920, 9856, 896))]
    for world in (1, 2, 4, 8):
        parts, block, flag_off, total = mgd.exchange_layout(shapes, world)
        assert flag_off == world * block and total >= flag_off + 4 * world and block % 1024 == 0
        spans = []
        for (M, split), (mp, logical, pitch, sizes, offs) in zip(shapes, parts):
            assert mp == M // world
            assert logical == (split[0] // 2, split[1] // 4 * 3, split[2])
            for i in range(3):
                assert pitch[i] >= logical[i] and pitch[i] % 16 == 0 and sizes[i] == mp * pitch[i]
                assert sizes[3 + i] == lib.mg_sf_bytes(mp, split[i]) == (mp // 128) * ((split[i] + 127) // 128) * 512
            for o, n in zip(offs, sizes):
                assert o % 1024 == 0
                spans.append((o, o + n))
        spans.sort()
        assert spans[0][0] == 0 and spans[-1][1] <= block
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    assert mgd.exchange_layout(shapes, 8)[1] == 17252352
    assert mgd.exchange_layout(shapes, 4)[1] == 34504704
    with pytest.raises(ValueError):
        mgd.exchange_layout([(4096, (5120, 2816, 256))], 3)
    with pytest.raises(ValueError):
        mgd.exchange_layout([(1024, (256, 128, 128))], 8)     # 128 rows per rank: not whole 256-row tile pairs


def _sets_are_safe(n_sets, world=3, steps=14):
    """Happens-before model of the pipelined exchange.  Per rank x and step k: P[x,k] = the push of batch
    k + 1 into set (k + 1) % n of every peer, issued in step k; R[x,k] = the GEMM reading set k % n.
    Orders that the streams and the ready flags enforce:
      R[x,k-1] -> P[x,k]      the push of step k is issued after the GEMM of step k - 1 (stream order)
      R[x,k-1] -> R[x,k]
      P[y,k-1] -> R[x,k]      the GEMM of batch k waits for every peer's push of batch k
    Safe means: every push into a set is ordered after the target's last GEMM on that set."""
    import itertools
    nodes = [(t, x, k) for t in "PR" for x in range(world) for k in range(steps)]
    succ = {v: set() for v in nodes}
    for x in range(world):
        for k in range(1, steps):
            succ[("R", x, k - 1)].add(("P", x, k))
            succ[("R", x, k - 1)].add(("R", x, k))
            for y in range(world):
                if y != x:
                    succ[("P", y, k - 1)].add(("R", x, k))

    def reaches(a, b):
        seen, todo = {a}, [a]
        while todo:
            v = todo.pop()
            if v == b:
                return True
            for w in succ[v]:
                if w not in seen:
                    seen.add(w)
                    todo.append(w)
        return False

    for x, y in itertools.permutations(range(world), 2):
        for k in range(steps):
            last_read = k + 1 - n_sets          # y's previous GEMM on the set that x's push of step k overwrites
            if last_read >= 0 and not reaches(("R", y, last_read), ("P", x, k)):
                return False
    return True


def test_four_buffer_sets_make_the_pipelined_exchange_safe():
    """The claim behind PushExchange's `n_sets`: when the push of batch i + 1 is issued before the GEMM
    of batch i, a rank can overwrite a peer's set only after the peer's last GEMM on it if FOUR sets
    rotate; with three it cannot be shown (a fast rank may run ahead of a slow one by that much)."""
    assert _sets_are_safe(4)
    assert _sets_are_safe(5)
    assert not _sets_are_safe(3)
    assert not _sets_are_safe(2)
