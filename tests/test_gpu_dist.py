"""Two GPUs: the N-sharded GEMM gives, shard by shard, the bytes of the single-GPU GEMM, with the
quantised activation travelling each of the three ways the C ABI offers - NCCL broadcast from the
rank that quantised it, NCCL all-gather of row shards, and the overlapped exchange (copy-engine
pushes + ready flags that the GEMM waits for).  Skipped on a box with one GPU.  NVLS is switched
off; no kernel is given another GPU's memory; host plumbing (ids, IPC handles) goes over gloo."""
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
        # 3. the overlapped exchange, four steps over two alternating buffer sets
        ex = mgd.PushExchange([(M, SPLIT)], world, rank, dev, n_sets=2)
        good = True
        for step in range(4):
            s = step % 2
            ex.begin_step()
            mg.reorder_quantize_x(Xs[step][rank * mp_:(rank + 1) * mp_].contiguous(), idx, KN, KS, KO, mp_, N,
                                  out=ex.shard(s, 0))
            ex.push(s, 0)
            out = mg.matmul_multi([(ex.buffers(s, 0), Bl, None)], flags=[ex.ready(s, 0)])[0]
            ex.join()
            good &= bool(torch.equal(out.view(torch.int16), reference(Xs[step])[:, n0:n0 + nl].contiguous().view(torch.int16)))
        torch.cuda.synchronize()
        ok["push"] = good
        ok["status"] = mg.device_status()
        dist.barrier()
        ex.close()
        ret[rank] = ok
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_n_sharded_gemm_equals_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for rank in (0, 1):
        assert ret[rank]["bcast"] and ret[rank]["allgather"] and ret[rank]["push"], dict(ret[rank])
        assert ret[rank]["status"] == 0
