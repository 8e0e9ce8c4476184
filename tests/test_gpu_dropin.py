"""The pybind11/torch module `mixedgemm` (the reference's module name and entry points) on a
GPU: the call sequence of the reference's smoke script (main.py:29-59) with its shapes."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import mx_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mixedgemm():
    from mixedgemm_b200 import build
    path = build.ext_path()
    if not os.path.exists(path):
        build.build_ext()
    sys.path.insert(0, os.path.dirname(path))  # what main.py does with 'build/'
    import mixedgemm as m
    return m


def test_entry_points_and_docstring(mixedgemm):
    assert mixedgemm.test_function() == "Hello from test_function!"
    for name in ("matmul", "reorder_quantize_x", "reorder_quantize_w"):
        assert hasattr(mixedgemm, name)
    assert "SFAN" in mixedgemm.matmul.__doc__ and "outfeatures" in mixedgemm.reorder_quantize_x.__doc__


def test_main_py_sequence(mixedgemm):
    M, N, K = 114, 3584, 3584
    KN, KS, KO = 2560, 3584 - 128 - 2560, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    signs = torch.randint(0, 2, (M, K), device="cuda", generator=g).to(torch.bfloat16) * 2 - 1
    X = torch.rand(M, K, dtype=torch.bfloat16, device="cuda", generator=g) * 3
    X[:, -KS:] = torch.rand(M, KS, dtype=torch.bfloat16, device="cuda", generator=g) * 14 + 14
    X[:, -KN:] = torch.rand(M, KN, dtype=torch.bfloat16, device="cuda", generator=g) * 256 + 256
    X = X * signs
    W = torch.rand(N, K, dtype=torch.bfloat16, device="cuda", generator=g) * 18 - 9
    reorder_index = torch.arange(K, dtype=torch.int16, device="cuda")
    AN, AS, AO, SFAN, SFAS, SFAO = mixedgemm.reorder_quantize_x(X, reorder_index, KN, KS, KO, M, N)
    BN, BS, BO, SFBN, SFBS, SFBO = mixedgemm.reorder_quantize_w(W, reorder_index, KN, KS, KO, M, N)
    # shapes and dtypes of the reference binding (src/bindings.cpp:88-93, :207-212)
    assert AN.shape == (M, KN // 2) and AS.shape == (M, KS // 4 * 3) and AO.shape == (M, KO)
    assert BN.shape == (N, KN // 2) and BS.shape == (N, KS // 2) and BO.shape == (N, KO // 2)
    assert SFAN.numel() >= (M // 128 + 1) * 128 * KN // 32 and SFBN.numel() >= N * KN // 32
    assert all(t.dtype == torch.uint8 for t in (AN, AS, AO, SFAN, SFAS, SFAO, BN, BS, BO, SFBN, SFBS, SFBO))
    C = mixedgemm.matmul(AN, BN, AS, BS, AO, BO, SFAN, SFBN, SFAS, SFBS, SFAO, SFBO)
    torch.cuda.synchronize()
    assert C.shape == (M, N) and C.dtype == torch.bfloat16
    # bytes: the module and the oracle agree
    a = H.oracle_outputs(H.bits(X.cpu()), reorder_index.cpu().numpy(), KN, KS, KO)
    b = H.oracle_outputs(H.bits(W.cpu()), reorder_index.cpu().numpy(), KN, KS, KO, weights=True)
    H.compare_quantised((AN, AS, AO, SFAN, SFAS, SFAO), a, M, (KN, KS, KO), "x")
    H.compare_quantised((BN, BS, BO, SFBN, SFBS, SFBO), b, N, (KN, KS, KO), "w")
    Yo = orc.gemm_f64(a, b, M, N, KN, KS, KO)
    y = C.float().cpu().numpy().astype(np.float64)
    yo16 = orc.bf16_round(Yo).astype(np.float64)
    assert np.linalg.norm(y - yo16) / np.linalg.norm(yo16) <= 1e-3
    # and, as main.py prints, the quantised product tracks the bf16 product of the raw operands
    Dref = (X.float() @ W.float().T).cpu().numpy()
    rel = np.linalg.norm(y - Dref) / np.linalg.norm(Dref)
    assert rel < 0.2, rel


def test_unknown_k_raises_runtime_error(mixedgemm):
    X = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
    idx = torch.arange(128, dtype=torch.int16, device="cuda")
    with pytest.raises(RuntimeError):
        mixedgemm.reorder_quantize_x(X, idx, 64, 32, 64, 4, 4)


def test_reference_smoke_script_runs_unmodified(mixedgemm, monkeypatch, capsys):
    """The acceptance smoke of a drop-in: the reference project's own main.py, executed as it is
    against this build of the `mixedgemm` module.  It needs a checkout of the reference, named by
    the environment variable MIXEDGEMM_REFERENCE; without one the test is skipped (the sequence of
    calls the script makes is covered by test_main_py_sequence either way)."""
    import runpy
    import time
    ref = os.environ.get("MIXEDGEMM_REFERENCE", "")
    script = os.path.join(ref, "main.py")
    if not ref or not os.path.exists(script):
        pytest.skip("MIXEDGEMM_REFERENCE does not name a checkout of the reference")
    monkeypatch.setattr(time, "sleep", lambda s: None)  # the script pauses a second between its ten rounds
    runpy.run_path(script, run_name="__main__")         # raises if any call into the module fails
    torch.cuda.synchronize()
    out = capsys.readouterr().out
    assert "Hello from test_function!" in out or len(out) > 0
    import mixedgemm_b200 as mg
    assert mg.device_status() == 0
