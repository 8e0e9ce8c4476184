"""Two GPUs: the N-sharded GEMM gives, shard by shard, the bytes of the single-GPU GEMM, with the
quantised activation travelling each of the three ways the C ABI offers - NCCL broadcast from the
rank that quantised it, NCCL all-gather of row shards, and the overlapped exchange (pushes by copy
engines, by a kernel's peer stores, or both, + ready flags that the GEMM waits for) in the three
orders a caller may use.  Skipped on a box with one GPU.  NVLS is switched off; the GEMM and the
quantiser are never given another GPU's memory; host plumbing (ids, IPC handles) goes over gloo.
The push kernel alone is also tested with every "rank's" buffer on one GPU."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

M, N, SPLIT = 512, 1024, (1280, 640, 128)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    # K is never cut across GPUs, but inside a GPU the library cuts it for problems with few tiles,
    # and a shard has fewer tiles than the whole: compare the uncut kernels
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", MG_GEMM_CSPLIT="0",
                      MG_GEMM_SPLITK="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import mixedgemm_b200 as mg
        from mixedgemm_b200 import dist as mgd
        from tests import helpers as H
        KN, KS, KO = SPLIT
        K = sum(SPLIT)
        dev = torch.device("cuda", rank)
        W = H.make_w(N, K, seed=2).cuda()
        Xs = [H.make_x(M, K, seed=10 + s).cuda() for s in range(4)]
        idx = H.reorder_index(Xs[0].cpu()).cuda()
        Bfull = mg.reorder_quantize_w(W, idx, KN, KS, KO, M, N)
        Bl = mgd.shard_weights(Bfull, N, KN, KS, KO, world, rank)
        n0, nl = mgd.shard_range(N, world, rank)

        def reference(X):
            Af = mg.reorder_quantize_x(X, idx, KN, KS, KO, M, N)
            return mg.matmul(Af[0], Bfull[0], Af[1], Bfull[1], Af[2], Bfull[2], Af[3], Bfull[3], Af[4], Bfull[4],
                             Af[5], Bfull[5])

        def ab(A, B):
            return (A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])

        ok = {}
        comm = mgd.Communicator(world, rank)
        # 1. quantise once on rank 0, broadcast, multiply the own weight shard, gather the output
        A = mg.alloc_quantized_x(M, KN, KS, KO, dev)
        for t in A:
            t.zero_()
        if rank == 0:
            mg.reorder_quantize_x(Xs[0], idx, KN, KS, KO, M, N, out=A)
        comm.broadcast_activations(A, src=0)
        Y = comm.all_gather_output(mg.matmul(*ab(A, Bl)))
        ok["bcast"] = bool(torch.equal(Y.view(torch.int16), reference(Xs[0]).view(torch.int16)))
        # 2. every rank quantises its rows, NCCL all-gathers complete the buffers
        A = mg.alloc_quantized_x(M, KN, KS, KO, dev)
        for t in A:
            t.zero_()
        mp_ = M // world
        mg.reorder_quantize_x(Xs[1][rank * mp_:(rank + 1) * mp_].contiguous(), idx, KN, KS, KO, mp_, N,
                              out=mgd.activation_shard(A, M, SPLIT, world, rank))
        comm.all_gather_activations(A, M, SPLIT)
        Yl = mg.matmul(*ab(A, Bl))
        ok["allgather"] = bool(torch.equal(Yl.view(torch.int16), reference(Xs[1])[:, n0:n0 + nl].contiguous().view(torch.int16)))
        comm.close()
        # 3. the overlapped exchange: two activations per step (different K splits) travel as one block
        # per peer.  First push, multiply and join one set per step; then the pipelined order, where
        # the push of step i + 1 is issued before the GEMM of step i (four sets).
        SPLIT2, N2 = (256, 128, 128), 512
        K2 = sum(SPLIT2)
        W2 = H.make_w(N2, K2, seed=3).cuda()
        X2s = [H.make_x(M, K2, seed=30 + s).cuda() for s in range(4)]
        idx2 = H.reorder_index(X2s[0].cpu()).cuda()
        B2full = mg.reorder_quantize_w(W2, idx2, *SPLIT2, M, N2)
        B2l = mgd.shard_weights(B2full, N2, *SPLIT2, world, rank)
        m0, ml = mgd.shard_range(N2, world, rank)

        def reference2(X):
            Af = mg.reorder_quantize_x(X, idx2, *SPLIT2, M, N2)
            return mg.matmul(*ab(Af, B2full))

        rows = slice(rank * mp_, (rank + 1) * mp_)
        good, piped = True, True
        for mode in ("sm", "ce", "hybrid"):   # a kernel's peer stores / copy-engine copies / both
            ex = mgd.PushExchange([(M, SPLIT), (M, SPLIT2)], world, rank, dev, n_sets=4, mode=mode)
            g_, p_ = _push_steps(mg, ex, Xs, X2s, idx, idx2, (KN, KS, KO), SPLIT2, rows, Bl, B2l, reference, reference2,
                                 (n0, nl), (m0, ml))
            good &= g_
            piped &= p_
            torch.cuda.synchronize()
            dist.barrier()
            ex.close()
            dist.barrier()
        ok["push"], ok["pipelined"] = good, piped
        ok["status"] = mg.device_status()
        ret[rank] = ok
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _push_steps(mg, ex, Xs, X2s, idx, idx2, split, SPLIT2, rows, Bl, B2l, reference, reference2, ncols, mcols):
    import torch.distributed as dist
    KN, KS, KO = split
    (n0, nl), (m0, ml) = ncols, mcols
    def fill(step, s):
        ex.begin_step(s)
        mg.reorder_quantize_x_multi([(Xs[step][rows].contiguous(), idx, KN, KS, KO, ex.shard(s, 0)),
                                     (X2s[step][rows].contiguous(), idx2, *SPLIT2, ex.shard(s, 1))])
        ex.push(s)

    def multiply(s):
        return mg.matmul_multi([(ex.buffers(s, 0), Bl, None), (ex.buffers(s, 1), B2l, None)],
                               flags=[ex.ready(s, 0), ex.ready(s, 1)])

    def check(step, outs):
        a = torch.equal(outs[0].view(torch.int16), reference(Xs[step])[:, n0:n0 + nl].contiguous().view(torch.int16))
        b = torch.equal(outs[1].view(torch.int16), reference2(X2s[step])[:, m0:m0 + ml].contiguous().view(torch.int16))
        return bool(a and b)

    good = True
    for step in range(4):
        s = step % 2
        fill(step, s)
        outs = multiply(s)
        ex.join()
        good &= check(step, outs)
    torch.cuda.synchronize()
    dist.barrier()
    piped = True
    fill(0, 0)
    for step in range(4):
        if step + 1 < 4:
            fill(step + 1, (step + 1) % 4)
        outs = multiply(step % 4)
        ex.join()
        piped &= check(step, outs)
    # two steps ahead: the pass that multiplies batch i pushes batch i + 1 first thing (quantised by
    # the pass before) and quantises batch i + 2
    torch.cuda.synchronize()
    dist.barrier()

    def quantise(step, s):
        ex.begin_step(s)
        mg.reorder_quantize_x_multi([(Xs[step][rows].contiguous(), idx, KN, KS, KO, ex.shard(s, 0)),
                                     (X2s[step][rows].contiguous(), idx2, *SPLIT2, ex.shard(s, 1))])

    quantise(0, 0)
    ex.push(0)
    ex.join()
    quantise(1, 1)
    for step in range(4):
        if step + 1 < 4:
            ex.push((step + 1) % 4)
        if step + 2 < 4:
            quantise(step + 2, (step + 2) % 4)
        outs = multiply(step % 4)
        piped &= check(step, outs)
    ex.join()
    return good, piped


def test_two_gpu_n_sharded_gemm_equals_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for rank in (0, 1):
        assert ret[rank]["bcast"] and ret[rank]["allgather"] and ret[rank]["push"] and ret[rank]["pipelined"], dict(ret[rank])
        assert ret[rank]["status"] == 0


def test_push_kernel_on_one_gpu():
    """mg_push_block with every "rank's" buffer on this GPU: each rank's block lands in every buffer,
    every flag word carries the epoch, the arrival counter is back at zero; block sizes that do not
    fill the last CTA, a capped grid, and the argument checks."""
    import ctypes
    from mixedgemm_b200 import _capi
    lib = _capi.load()
    dev = torch.device("cuda", 0)
    for world, block, ctas in ((4, 16 * 1237, 0), (8, 16 * 70001, 0), (2, 1 << 20, 3), (16, 4096, 1)):
        flag_off = world * block
        total = flag_off + 4 * world
        bufs = [torch.zeros(total, dtype=torch.uint8, device=dev) for _ in range(world)]
        want = [torch.randint(0, 256, (block,), dtype=torch.uint8, device=dev) for _ in range(world)]
        bases = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
        epoch = torch.full((1,), 5, dtype=torch.int32, device=dev)
        counter = torch.zeros(1, dtype=torch.int32, device=dev)
        for r in range(world):
            bufs[r][r * block:(r + 1) * block] = want[r]
        for r in range(world):
            st = lib.mg_push_block(world, r, bases, r * block, block, flag_off, epoch.data_ptr(), counter.data_ptr(), ctas, None)
            assert st == 0
        torch.cuda.synchronize()
        assert int(counter.item()) == 0
        for b in bufs:
            for r in range(world):
                assert torch.equal(b[r * block:(r + 1) * block], want[r]), (world, r)
            assert torch.all(b[flag_off:].view(torch.int32) == 5)
    # the two pushes sharing the peers: the kernel serves ring distances 1 and 2, a copy serves 3
    world, block = 4, 16 * 4099
    flag_off = world * block
    bufs = [torch.zeros(flag_off + 4 * world, dtype=torch.uint8, device=dev) for _ in range(world)]
    want = [torch.randint(0, 256, (block,), dtype=torch.uint8, device=dev) for _ in range(world)]
    bases = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    epoch.fill_(9)
    stream = torch.cuda.current_stream().cuda_stream
    streams = (ctypes.c_void_p * (world - 1))(*([stream] * (world - 1)))
    for r in range(world):
        bufs[r][r * block:(r + 1) * block] = want[r]
    for r in range(world):
        assert lib.mg_push_block_to(world, r, 0b011, bases, r * block, block, flag_off, epoch.data_ptr(),
                                    counter.data_ptr(), 2, stream) == 0
        off = (ctypes.c_size_t * 1)(r * block)
        nbytes = (ctypes.c_size_t * 1)(block)
        assert lib.mg_push_shard_to(world, r, 0b100, bases, off, nbytes, 1, flag_off, epoch.data_ptr(), streams) == 0
    torch.cuda.synchronize()
    for b in bufs:
        for r in range(world):
            assert torch.equal(b[r * block:(r + 1) * block], want[r]), r
        assert torch.all(b[flag_off:].view(torch.int32) == 9)
    bases = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    e, c = epoch.data_ptr(), counter.data_ptr()
    assert lib.mg_push_block(2, 0, bases, 0, 24, 4096, e, c, 0, None) == 3        # MG_ERR_ALIGN: not whole 16 bytes
    assert lib.mg_push_block(17, 0, bases, 0, 32, 4096, e, c, 0, None) == 1       # MG_ERR_SHAPE: more than 16 ranks
    assert lib.mg_push_block(2, 2, bases, 0, 32, 4096, e, c, 0, None) == 1
    assert lib.mg_push_block(2, 0, bases, 0, 32, 4096, None, c, 0, None) == 2     # MG_ERR_NULL
    assert lib.mg_push_block(2, 0, None, 0, 32, 4096, e, c, 0, None) == 2


def test_push_exchange_with_one_rank():
    """The exchange object on a single GPU (world = 1: buffers, layout, epochs, flags, the GEMM
    reading the block layout through its ready flags) in all three push modes, eagerly and
    replayed from a CUDA graph."""
    import mixedgemm_b200 as mg
    from mixedgemm_b200 import dist as mgd
    from tests import helpers as H
    dev = torch.device("cuda", 0)
    Mq, Nq = 512, 512
    KN, KS, KO = SPLIT
    K = sum(SPLIT)
    X = H.make_x(Mq, K, seed=41).cuda()
    W = H.make_w(Nq, K, seed=42).cuda()
    idx = H.reorder_index(X.cpu()).cuda()
    B = mg.reorder_quantize_w(W, idx, KN, KS, KO, Mq, Nq)
    A = mg.reorder_quantize_x(X, idx, KN, KS, KO, Mq, Nq)
    want = mg.matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    for mode in ("sm", "ce", "hybrid"):
        ex = mgd.PushExchange([(Mq, SPLIT)], 1, 0, dev, n_sets=2, mode=mode)
        out = torch.zeros((Mq, Nq), dtype=torch.bfloat16, device=dev)

        def step(s):
            ex.begin_step(s)
            mg.reorder_quantize_x_multi([(X, idx, KN, KS, KO, ex.shard(s, 0))])
            ex.push(s)
            mg.matmul_multi([(ex.buffers(s, 0), B, out)], flags=[ex.ready(s, 0)])
            ex.join()

        for s in (0, 1, 0):
            out.zero_()
            step(s)
            torch.cuda.synchronize()
            assert torch.equal(out.view(torch.int16), want.view(torch.int16)), (mode, s)
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            step(1)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                step(0)
                step(1)
            for _ in range(3):
                out.zero_()
                g.replay()
            torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), want.view(torch.int16)), mode
        assert mg.device_status() == 0
        assert int(ex.epoch[0]) >= 4 and torch.all(ex.sets[0]["flags"] == ex.epoch[0])
        ex.close()
