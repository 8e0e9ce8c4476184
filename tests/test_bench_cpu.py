"""Host-side logic of bench.py that needs no GPU: workload tables against the benchmark
definition, the byte and peak arithmetic behind the roofline figures, and the reference arm's
JSON line (the CPU restatement timed on a small sample)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_k_split_matches_the_benchmark_definition():
    assert bench.split_k(4096) == (2560, 1408, 128)
    assert bench.split_k(14336) == (8960, 4928, 448)
    assert bench.split_k(8192) == (5120, 2816, 256)
    assert bench.split_k(28672) == (17920, 9856, 896)
    assert bench.split_k(16384) == (10240, 5632, 512)


def test_workload_tables():
    w8 = bench.WORKLOADS["llama3-8b-m2048"]
    assert w8["M"] == 2048
    shapes = {(n, N, K) for (K, layers) in w8["groups"] for (n, N) in layers}
    assert shapes == {("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
                      ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)}
    w70 = bench.WORKLOADS["llama3-70b-m4096"]
    assert w70["M"] == 4096 and w70["dist"] == "student3" and w70["outlier"] == 30.0
    for K, layers in w70["groups"]:
        for _, N in layers:
            assert N % (128 * 8) == 0  # every 8-way shard is whole 128-row scale blocks


def test_roofline_arithmetic():
    # 2 bytes read + 0.6328125 bytes written per element for the standard split
    assert bench.reorder_bytes(8192, 16384) == int(8192 * 16384 * 2.6328125)
    # FP4 at 4x, FP6 / FP8 at 2x the bf16 rate, weighted by the K split: 1 / (0.625/4 + 0.375/2)
    assert abs(bench.blended_peak(1000.0, 4096) / 1000.0 - 1.0 / (0.625 / 4 + 0.375 / 2)) < 1e-9


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload",
                          "single-layer-m16", "--steps", "1", "--warmup", "1"], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    d = json.loads(out.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference" and d["metric"] == "mixed_mx_gemm_tflops" and d["unit"] == "TFLOP/s"
    assert d["value"] > 0 and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["config"]["workload"] == "single-layer-m16"
