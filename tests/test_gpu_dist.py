"""Two GPUs, NCCL: the N-sharded GEMM gives, shard by shard, the bytes of the single-GPU GEMM.
Skipped on a box with one GPU.  NVLS is switched off and nothing but NCCL touches peer memory."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

M, N, SPLIT = 384, 1024, (1280, 640, 128)


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
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import mixedgemm_b200 as mg
        from mixedgemm_b200 import dist as mgd
        from tests import helpers as H
        KN, KS, KO = SPLIT
        K = sum(SPLIT)
        X = H.make_x(M, K, seed=1).cuda()
        W = H.make_w(N, K, seed=2).cuda()
        idx = H.reorder_index(X.cpu()).cuda()
        Bfull = mg.reorder_quantize_w(W, idx, KN, KS, KO, M, N)
        Bl = mgd.shard_weights(Bfull, N, KN, KS, KO, world, rank)
        A = mg.alloc_quantized_x(M, KN, KS, KO, X.device)
        for t in A:
            t.zero_()
        if rank == 0:
            mg.reorder_quantize_x(X, idx, KN, KS, KO, M, N, out=A)
        mgd.broadcast_activations(A, src=0)
        Yl = mg.matmul(A[0], Bl[0], A[1], Bl[1], A[2], Bl[2], A[3], Bl[3], A[4], Bl[4], A[5], Bl[5])
        Y = mgd.all_gather_output(Yl, world)
        if rank == 0:
            Af = mg.reorder_quantize_x(X, idx, KN, KS, KO, M, N)
            Yref = mg.matmul(Af[0], Bfull[0], Af[1], Bfull[1], Af[2], Bfull[2], Af[3], Bfull[3], Af[4], Bfull[4],
                             Af[5], Bfull[5])
            torch.cuda.synchronize()
            ret["equal"] = bool(torch.equal(Y.view(torch.int16), Yref.view(torch.int16)))
            ret["status"] = mg.device_status()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_n_sharded_gemm_equals_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret["equal"] and ret["status"] == 0
