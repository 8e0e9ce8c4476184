"""The callers either side of the path: weight container round trip and the Linear-style module."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


def test_container_round_trip_and_module(tmp_path):
    import mixedgemm_b200 as mg
    from mixedgemm_b200.linear import MixedLinear, QuantizedWeights
    M, K = 300, 14336  # 64-tail segments: buffers are row-pitched on the device, dense in the file
    X = H.make_x(M, K, seed=1).cuda()
    Ws = [H.make_w(N, K, seed=2 + j).cuda() for j, N in enumerate((512, 256))]
    lin = MixedLinear.from_dense(Ws, X)
    # index = stable argsort of the per-channel absmax
    want_idx, _ = orc.np_reorder_index(H.bits(X.cpu()))
    assert np.array_equal(lin.reorder_index.cpu().numpy(), want_idx)
    y = lin(X)
    assert [tuple(t.shape) for t in y] == [(M, 512), (M, 256)]
    # save / load: same bytes, same product
    p = tmp_path / "w0.pt"
    lin.weights[0].save(str(p))
    w0 = QuantizedWeights.load(str(p), "cuda")
    for a, b in zip(w0.parts[:3], lin.weights[0].parts[:3]):
        assert torch.equal(a, b)
    y0 = MixedLinear(w0)(X)
    torch.cuda.synchronize()
    assert torch.equal(y0.view(torch.int16), y[0].view(torch.int16))
    # and the product tracks the unquantised one
    ref = X.float() @ Ws[0].float().T
    rel = (y[0].float() - ref).norm() / ref.norm()
    assert rel < 0.2, rel
    # batched input keeps its leading dimensions
    yb = MixedLinear(w0)(X[:256].reshape(2, 128, K))
    assert tuple(yb.shape) == (2, 128, 512)
    assert mg.device_status() == 0


def test_module_is_a_torch_op_with_bias_on_a_side_stream_and_in_a_graph():
    """MixedLinear runs as the torch operator mixedgemm_b200::mixed_linear: same bytes on a
    non-default stream and when replayed from a captured CUDA graph as on the default stream;
    an optional bias is added to the bf16 product; buffers allocated at construction serve any
    smaller token count."""
    import mixedgemm_b200 as mg
    from mixedgemm_b200.linear import MixedLinear, QuantizedWeights
    M, K = 384, 4096
    X = H.make_x(M, K, seed=5).cuda()
    Ws = [H.make_w(N, K, seed=6 + j).cuda() for j, N in enumerate((1024, 256))]
    idx = mg.reorder_index(X)
    qw = [QuantizedWeights.from_dense(W, idx) for W in Ws]
    bias = (torch.randn(1024, generator=torch.Generator().manual_seed(1)) * 0.1).to(torch.bfloat16).cuda()
    plain = MixedLinear(qw)
    lin = MixedLinear(qw, bias=[bias, None], max_tokens=512)
    y_ref = plain(X)
    y = lin(X)
    assert torch.equal(y[0], y_ref[0] + bias) and torch.equal(y[1].view(torch.int16), y_ref[1].view(torch.int16))
    assert lin._a[0].size(0) == 512  # the buffers of the constructor were used, not replaced
    # through the dispatcher by name, as any torch op
    outs = torch.ops.mixedgemm_b200.mixed_linear(X, idx, list(lin.split), lin._parts, lin._fused_parts,
                                                 lin._scratch(M, X.device))
    assert torch.equal(outs[1].view(torch.int16), y_ref[1].view(torch.int16))
    # a side stream
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        y_side = lin(X)
    side.synchronize()
    assert torch.equal(y_side[0], y[0]) and torch.equal(y_side[1], y[1])
    # captured and replayed with new input in the same buffer
    xin = X.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        lin(xin)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            y_g = lin(xin)
    X2 = H.make_x(M, K, seed=9).cuda()
    xin.copy_(X2)
    g.replay()
    torch.cuda.synchronize()
    want = plain(X2)
    assert torch.equal(y_g[0], want[0] + bias) and torch.equal(y_g[1].view(torch.int16), want[1].view(torch.int16))
    assert mg.device_status() == 0


def test_decode_tokens_take_one_launch_over_the_concatenated_weight(mgopt):
    """Up to 128 tokens q/k/v go out as one product with the row-concatenation of the three
    weights; the column ranges of its result are the bytes of one product per weight."""
    import mixedgemm_b200 as mg
    from mixedgemm_b200.linear import MixedLinear, QuantizedWeights
    mgopt.setenv("MG_GEMM_CSPLIT", "0")  # the kernel choice depends on the tile count; compare uncut kernels
    mgopt.setenv("MG_GEMM_SPLITK", "0")
    K = 4096
    Xc = H.make_x(256, K, seed=3).cuda()
    idx = mg.reorder_index(Xc)
    Ws = [H.make_w(N, K, seed=20 + j).cuda() for j, N in enumerate((4096, 1024, 1024))]
    lin = MixedLinear([QuantizedWeights.from_dense(W, idx) for W in Ws])
    assert lin.fused is not None and lin.fused.out_features == 6144
    for M in (1, 16, 128):
        X = Xc[:M].contiguous()
        ys = lin(X)
        A = mg.reorder_quantize_x(X, idx, *lin.split, M, 0)
        for y, w in zip(ys, lin.weights):
            B = w.parts
            ref = mg.matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
            assert y.shape == ref.shape and torch.equal(y.contiguous().view(torch.int16), ref.view(torch.int16))
    # and beyond 128 tokens the grouped launch still serves the same (re-pointed) weights
    ys = lin(Xc)
    A = mg.reorder_quantize_x(Xc, idx, *lin.split, 256, 0)
    B = lin.weights[1].parts
    ref = mg.matmul(A[0], B[0], A[1], B[1], A[2], B[2], A[3], B[3], A[4], B[4], A[5], B[5])
    assert torch.equal(ys[1].view(torch.int16), ref.view(torch.int16))
    assert mg.device_status() == 0
