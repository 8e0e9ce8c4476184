#!/usr/bin/env python
"""Benchmark of the hot path: activation reorder-and-quantise + mixed MXFP4/6/8 GEMM.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                  [--workload NAME] [--exchange push|push-ce|push-sm|push-hybrid|allgather|bcast|replicated]
                  [--no-pipeline] [--quantize each|multi] [--no-graph] [--no-fuse] [--no-extra]
  python bench.py --kernel gemm|reorder --shape M,N,K     one kernel, one shape
  python bench.py --sweep decode|square|all               the other benchmark configurations, a line per shape

One "step" is one pass over a projection set of a Llama-shaped layer stack: every distinct
activation is reorder-quantised once (all of them in one launch) and multiplied with each weight
that consumes it (q/k/v share one activation, gate/up another); all products of the step go out as
one GEMM launch.  Weights are quantised once, outside the timed region, as in deployment.

  N = 1 (default)   workload llama3-8b-m2048 (M = 2048 tokens on the Llama-3-8B projections)
  N > 1             workload llama3-70b-m4096: weights sharded along N over the ranks.  --exchange
                    push (default): every rank quantises its M / P rows of all activations with one
                    launch and sends them into every peer's buffer over NVLink - with one copy-engine
                    copy per peer, or with a small kernel that keeps a few SMs to itself - hidden
                    under the GEMM of the batch before (the exchange runs one step ahead;
                    --no-pipeline sends and multiplies the same batch in a step); the GEMM's
                    producer waits for the flags that follow the data;
                    push-ce / push-sm / push-hybrid: force copy-engine copies (one per peer; the
                    default up to four GPUs), the kernel (twelve SMs of its own), or the kernel for
                    all peers but two and copies for those (the default beyond four GPUs);
                    allgather: the same rows, completed by NCCL all-gathers before the GEMM;
                    bcast: rank 0 quantises, NCCL broadcast; replicated: every rank quantises
                    everything, nothing is exchanged

Prints ONE JSON line (rank 0).  `value` is the whole-job GEMM throughput with inputs resident
in HBM; `e2e` is the same metric with the activations starting in pinned host memory and the
outputs ending there (copies inside the timed region).  `--impl reference` times the CPU
restatement of the same path on the host cores (the reference has no CPU code and its GEMMs
do not run on sm_100).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: M, [(activation K, [(layer, N), ...]), ...], X distribution, outlier scale, W std
    "llama3-8b-m2048": dict(M=2048, dist="normal", outlier=20.0, wstd=0.02, groups=[
        (4096, [("q", 4096), ("k", 1024), ("v", 1024)]),
        (4096, [("o", 4096)]),
        (4096, [("gate", 14336), ("up", 14336)]),
        (14336, [("down", 4096)])]),
    "llama3-70b-m4096": dict(M=4096, dist="student3", outlier=30.0, wstd=0.015, groups=[
        (8192, [("q", 8192), ("k", 1024), ("v", 1024)]),
        (8192, [("o", 8192)]),
        (8192, [("gate", 28672), ("up", 28672)]),
        (28672, [("down", 8192)])]),
    # the CPU-runnable single layer
    "single-layer-m16": dict(M=16, dist="normal", outlier=20.0, wstd=0.02, groups=[(4096, [("proj", 4096)])]),
}


def split_k(K):
    KO = K // 32
    KN = K * 5 // 8
    return KN, K - KN - KO, KO


def reorder_bytes(M, K):
    KN, KS, KO = split_k(K)
    return M * K * 2 + M * (KN // 2 + KS // 4 * 3 + KO + K // 32)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def blended_peak(bf16_tflops, K):
    """Tensor peak of a K split 62.5/34.375/3.125 %: FP4 runs at 4x and FP6/FP8 at 2x the bf16 rate."""
    KN, KS, KO = split_k(K)
    return K / (KN / (4 * bf16_tflops) + (KS + KO) / (2 * bf16_tflops))


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append((time.time(), ln.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        for ln in rows:
            f = [x.strip() for x in ln.split(",")]
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
                for n, v in zip(names, f[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------- CPU arm
def cpu_arm(wl_name, rows, steps, warmup):
    """The CPU restatement of the path (oracle): reorder-quantise with the C/OpenMP oracle, then
    dequantise-then-matmul in fp32 on all host cores, bf16 output.  `rows` activation rows per
    step stand for the workload's M (rows are independent; throughput is reported per flop)."""
    import numpy as np
    from oracle import mx_oracle as orc
    wl = WORKLOADS[wl_name]
    rows = min(rows, wl["M"])
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    groups = []
    flops = 0
    qbytes = 0
    for K, layers in wl["groups"]:
        KN, KS, KO = split_k(K)
        X = torch.randn(rows, K, generator=g)
        ch = torch.randperm(K, generator=g)[:K // 32]
        X[:, ch] *= wl["outlier"]
        Xb = X.to(torch.bfloat16)
        idx = torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16).numpy()
        xbits = Xb.view(torch.int16).numpy().view(np.uint16)
        Ws = []
        for name, N in layers:
            Nc = min(N, 4096)  # bounded sample of output columns; flops counted for what is computed
            W = (torch.randn(Nc, K, generator=g) * wl["wstd"]).to(torch.bfloat16)
            wq = orc.c_reorder_quantize(W.view(torch.int16).numpy().view(np.uint16), idx, KN, KS, KO, weights=True)
            Wd = torch.from_numpy(np.concatenate(
                [orc.c_dequantize(wq[i], wq[3 + i], Nc, k, orc.FMT_E2M1) for i, k in enumerate((KN, KS, KO))], 1))
            Ws.append(Wd)
            flops += 2 * rows * Nc * K
        qbytes += reorder_bytes(rows, K)
        groups.append((xbits, idx, (KN, KS, KO), Ws))

    def step():
        tq = 0.0
        for xbits, idx, (KN, KS, KO), Ws in groups:
            t0 = time.perf_counter()
            a = orc.c_reorder_quantize(xbits, idx, KN, KS, KO)
            tq += time.perf_counter() - t0
            Ad = torch.from_numpy(np.concatenate(
                [orc.c_dequantize(a[i], a[3 + i], rows, k, f) for i, (k, f) in
                 enumerate(((KN, orc.FMT_E2M1), (KS, orc.FMT_E3M2), (KO, orc.FMT_E4M3)))], 1))
            for Wd in Ws:
                (Ad @ Wd.T).to(torch.bfloat16)
        return tq

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    tq = 0.0
    for _ in range(steps):
        tq += step()
    dt = time.perf_counter() - t0
    return dict(tflops=flops * steps / dt / 1e12, reorder_gbs=qbytes * steps / tq / 1e9, cores=cores,
                ms_per_step=dt / steps * 1e3,
                sample="%d of %d activation rows per step, output columns capped at 4096 per layer, %d steps" % (
                    rows, wl["M"], steps))


# ----------------------------------------------------------------------------- GPU arm
class Job:
    """Device-resident state of one rank: activations, reorder indices, quantised weight shards,
    output buffers, and - on several GPUs - the exchange that brings every rank the whole
    quantised activation."""

    def __init__(self, wl_name, rank, world, device, exchange, fused=True, pipeline=True, multi_q=None):
        import mixedgemm_b200 as mg
        self.mg = mg
        wl = WORKLOADS[wl_name]
        self.M = M = wl["M"]
        self.rank, self.world, self.device = rank, world, device
        # the push: copy engines up to four GPUs (their all-to-all rate is enough to hide under the GEMM
        # there and they cost no SM); beyond that a kernel on SMs of its own for all peers but the two
        # farthest down the ring, which the copy engines serve (measured best at 8 GPUs)
        self.push_mode = {"push-ce": "ce", "push-sm": "sm", "push-hybrid": "hybrid"}.get(exchange, "ce" if world <= 4 else "hybrid")
        # 12 SMs: a push SM sustains about 50 GB/s of peer stores and the fabric about 540 GB/s per rank
        # (measured with 4 GPUs), and at 8 GPUs 107 MB per rank and step must leave within the GEMM's 200 us
        self.push_ctas = 12
        if exchange in ("push-ce", "push-sm", "push-hybrid"):
            exchange = "push"
        self.exchange = exchange if world > 1 else "none"
        self.fused = fused
        self.sharded_q = self.exchange in ("push", "allgather")  # every rank quantises M / P rows
        g = torch.Generator(device=device).manual_seed(1234)  # same activations on every rank
        self.groups = []
        self.flops_local = 0
        self.flops_total = 0
        self.gemm_shapes = []
        for gi, (K, layers) in enumerate(wl["groups"]):
            KN, KS, KO = split_k(K)
            X = torch.randn(M, K, generator=g, device=device)
            if wl["dist"] == "student3":
                chi = torch.zeros(M, K, device=device)
                for _ in range(3):
                    chi += torch.randn(M, K, generator=g, device=device).pow_(2)
                X = X / (chi / 3).sqrt_() / (3 ** 0.5)
                del chi
            ch = torch.randperm(K, generator=g, device=device)[:K // 32]
            X[:, ch] *= wl["outlier"]
            Xb = X.to(torch.bfloat16)
            del X
            idx = torch.sort(Xb.float().abs().amax(0), stable=True).indices.to(torch.int16)
            if self.sharded_q:
                mp = M // world
                Xb = Xb[rank * mp:(rank + 1) * mp].contiguous()  # this rank's rows are all it ever reads
            Ls = []
            # Column shards that are not whole 256-column tiles (k and v of a grouped-query layer on 8
            # GPUs: 128 columns each) are multiplied as ONE weight per rank, its rows the rank's
            # rows of q, k and v one after the other - the fused QKV layout of a tensor-parallel layer.
            shard_n = [N // world for (_, N) in layers]
            merge = M > 128 and any(n % 256 for n in shard_n) and sum(shard_n) % 256 == 0
            parts = []
            for li, (name, N) in enumerate(layers):
                assert N % (128 * world) == 0, "every shard must be a multiple of 128 columns"
                Nl = N // world
                gw = torch.Generator(device=device).manual_seed(977 * gi + 31 * li + 7)
                W = (torch.randn(N, K, generator=gw, device=device) * wl["wstd"]).to(torch.bfloat16)
                Wl = W[rank * Nl:(rank + 1) * Nl].contiguous()
                del W
                self.flops_local += 2 * M * Nl * K
                self.flops_total += 2 * M * N * K
                if merge:
                    parts.append(Wl)
                    continue
                B = mg.reorder_quantize_w(Wl, idx, KN, KS, KO, M, Nl)
                del Wl
                Y = torch.empty((M, Nl), dtype=torch.bfloat16, device=device)
                Ls.append((name, Nl, B, Y))
                self.gemm_shapes.append((M, Nl, K))
            if merge:
                Wl = torch.cat(parts, 0)
                Nl = Wl.size(0)
                B = mg.reorder_quantize_w(Wl, idx, KN, KS, KO, M, Nl)
                del Wl, parts
                Ls.append(("+".join(n for (n, _) in layers), Nl, B, torch.empty((M, Nl), dtype=torch.bfloat16, device=device)))
                self.gemm_shapes.append((M, Nl, K))
            self.groups.append(dict(K=K, split=(KN, KS, KO), X=Xb, idx=idx, layers=Ls))
        # the fused launch and the exchange take the activations with the most work first
        self.order = sorted(range(len(self.groups)), key=lambda i: -sum(2 * M * Nl * self.groups[i]["K"]
                                                                         for (_, Nl, _, _) in self.groups[i]["layers"]))
        self.nsets = 1
        self.ex = self.comm = None
        # push: the quantise + push of step i + 1 is issued before the GEMM of step i, so that the
        # transfer runs under a GEMM that already has its data (steps are independent batches)
        self.pipeline = pipeline and self.exchange == "push"
        self.primed = False
        # The kernel push at 8 GPUs takes as long as the GEMM (214 against 203 us), so it gets the
        # whole step: the pass that multiplies batch i pushes batch i + 1 from its first instant (the
        # pass before quantised it) and quantises batch i + 2.
        self.lookahead = 2 if (self.pipeline and self.push_mode in ("sm", "hybrid")) else 1
        if self.exchange == "push":
            from mixedgemm_b200 import dist as mgd
            # buffer sets used in turn: a rank may push a later step while a peer still multiplies this one
            self.nsets = 4 if self.pipeline else 2
            self.ex = mgd.PushExchange([(M, gr["split"]) for gr in self.groups], world, rank, device, n_sets=self.nsets,
                                       mode=self.push_mode, push_ctas=self.push_ctas)
            if self.push_mode in ("sm", "hybrid"):
                # the GEMM and the quantiser leave the push kernel's SMs alone: a quantiser CTA fills an
                # SM's shared memory, so on the SMs where the push of the step before is still running
                # it would have to wait for it
                sms = torch.cuda.get_device_properties(device).multi_processor_count
                mg.set_option("GEMM_MAX_CLUSTERS", sms // 2 - self.push_ctas // 2)
                mg.set_option("REORDER_CTAS", sms - self.push_ctas)
            for gi, gr in enumerate(self.groups):
                gr["A"] = [self.ex.buffers(s, gi) for s in range(self.nsets)]
        else:
            if self.exchange in ("bcast", "allgather"):
                from mixedgemm_b200 import dist as mgd
                self.comm = mgd.Communicator(world, rank)
            for gr in self.groups:
                gr["A"] = [mg.alloc_quantized_x(M, *gr["split"], device)]
        nq = len(self.groups)
        can_fuse = M > 128 and all(Nl % 256 == 0 for gr in self.groups for (_, Nl, _, _) in gr["layers"]) and \
            sum(len(gr["layers"]) for gr in self.groups) <= 8
        self.fused = self.fused and can_fuse
        grouped = [M > 128 and len(gr["layers"]) <= 8 and all(Nl % 256 == 0 for (_, Nl, _, _) in gr["layers"])
                   for gr in self.groups]
        # one quantiser launch for all activations of a step: one wave of CTAs shared out by size instead
        # of a launch - and a partly filled last wave - per activation
        self.multi_q = (multi_q is None or multi_q) and self.exchange in ("none", "replicated", "push", "allgather") and nq <= 8
        if self.multi_q:
            nq = 1
        # kernels of this library per step: the quantisers + the GEMM launches (+ the epoch bump)
        self.n_kernels = nq + (1 if self.fused else sum(1 if g_ else len(gr["layers"]) for g_, gr in zip(grouped, self.groups)))
        self.n_kernels += (2 if self.push_mode in ("sm", "hybrid") else 1) if self.ex is not None else 0  # epoch bump (+ push kernel)
        self.reorder_bytes = sum(reorder_bytes(gr["X"].size(0), gr["K"]) for gr in self.groups)
        torch.cuda.synchronize()

    # -- pieces of a step
    def quantize(self, gi, s=0):
        """This rank's part of the quantisation of activation gi into buffer set s."""
        gr = self.groups[gi]
        KN, KS, KO = gr["split"]
        A = gr["A"][s]
        if self.sharded_q:
            from mixedgemm_b200 import dist as mgd
            out = self.ex.shard(s, gi) if self.ex is not None else mgd.activation_shard(A, self.M, gr["split"], self.world, self.rank)
            self.mg.reorder_quantize_x(gr["X"], gr["idx"], KN, KS, KO, gr["X"].size(0), 0, out=out)
        elif self.exchange == "bcast" and self.rank != 0:
            pass
        else:
            self.mg.reorder_quantize_x(gr["X"], gr["idx"], KN, KS, KO, self.M, 0, out=A)

    def quantize_all(self, s=0):
        """This rank's rows of every activation in one launch (sharded quantisation only)."""
        from mixedgemm_b200 import dist as mgd
        probs = []
        for gi in self.order:
            gr = self.groups[gi]
            if not self.sharded_q:
                out = gr["A"][s]
            elif self.ex is not None:
                out = self.ex.shard(s, gi)
            else:
                out = mgd.activation_shard(gr["A"][s], self.M, gr["split"], self.world, self.rank)
            probs.append((gr["X"], gr["idx"], *gr["split"], out))
        self.mg.reorder_quantize_x_multi(probs)

    def exchange_a(self, gi, s=0):
        gr = self.groups[gi]
        if self.exchange == "push":
            raise RuntimeError("the push exchange moves a whole step at once: fill()")
        elif self.exchange == "bcast":
            self.comm.broadcast_activations(gr["A"][s], src=0)
        elif self.exchange == "allgather":
            self.comm.all_gather_activations(gr["A"][s], self.M, gr["split"])

    def gemm_group(self, gi, s=0):
        gr = self.groups[gi]
        if self.ex is not None:  # the exchange's row-sharded buffers and its ready flags
            self.mg.matmul_multi([(gr["A"][s], B, Y) for (_, _, B, Y) in gr["layers"]],
                                 flags=[self.ex.ready(s, gi)] * len(gr["layers"]))
            return
        self.mg.matmul_group(gr["A"][s], [B for (_, _, B, _) in gr["layers"]], outs=[Y for (_, _, _, Y) in gr["layers"]])

    def gemm_fused(self, s=0):
        probs, flags = [], []
        for gi in self.order:
            gr = self.groups[gi]
            for (_, _, B, Y) in gr["layers"]:
                probs.append((gr["A"][s], B, Y))
                flags.append(self.ex.ready(s, gi) if self.ex is not None else None)
        self.mg.matmul_multi(probs, flags=flags if self.ex is not None else None)

    def fill(self, s):
        """Push exchange: quantise this rank's rows of every activation into set s and send them."""
        self.ex.begin_step(s)
        self.quantize_all(s)
        self.ex.push(s)

    def multiply(self, s):
        if self.fused:
            self.gemm_fused(s)
        else:
            for gi in range(len(self.groups)):
                self.gemm_group(gi, s)

    def step(self, s=0):
        """One pass: quantise (this rank's part of) every activation, exchange, multiply.  Pipelined
        push: the pass quantises and sends batch s + 1 and multiplies batch s, which the pass before
        sent (prime() sends the very first one)."""
        if self.ex is not None:
            n = self.nsets
            if self.pipeline and self.lookahead == 2:
                if not self.primed:
                    self.prime(s)
                self.ex.push((s + 1) % n)
                if s == 0:
                    self._pushed_first = []
                    for st in self.ex.used_streams():
                        e = torch.cuda.Event()
                        e.record(st)
                        self._pushed_first.append(e)
                if s == n - 1:
                    # this pass overwrites the block that the first push of the round read (earlier
                    # rounds' pushes were taken back by the join that ended them)
                    for e in self._pushed_first:
                        torch.cuda.current_stream().wait_event(e)
                self.ex.begin_step((s + 2) % n)
                self.quantize_all((s + 2) % n)
            elif self.pipeline:
                if not self.primed:
                    self.prime(s)
                self.fill((s + 1) % n)
            else:
                self.fill(s)
            self.multiply(s)
            # The copies read this rank's own block of a set that is not written again before the
            # set comes round, so in the pipelined order the main stream takes them back only at the
            # end of a round of sets (the unit that is captured and timed): a transfer may then run
            # on under the next step instead of holding it up.
            if not self.pipeline or s == self.nsets - 1:
                self.ex.join()
        elif self.multi_q:
            self.quantize_all(s)
            for gi in self.order:
                self.exchange_a(gi, s)
            self.multiply(s)
        elif self.fused:
            for gi in self.order:
                self.quantize(gi, s)
                self.exchange_a(gi, s)
            self.gemm_fused(s)
        else:
            for gi in range(len(self.groups)):
                self.quantize(gi, s)
                self.exchange_a(gi, s)
                self.gemm_group(gi, s)

    def prime(self, s=0):
        self.fill(s)
        self.ex.join()
        if self.lookahead == 2:
            self.ex.begin_step((s + 1) % self.nsets)
            self.quantize_all((s + 1) % self.nsets)
        self.primed = True

    def close(self):
        if self.ex is not None:
            self.ex.close()
        if self.comm is not None:
            self.comm.close()


def timed(fn, steps, sync, finish=None):
    """ms per call of fn by CUDA events on the current stream; `finish` (optional) makes that stream
    wait for work the calls put on other streams before the closing event is recorded."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for _ in range(steps):
        fn()
    if finish is not None:
        finish()
    e1.record()
    sync()
    return e0.elapsed_time(e1) / steps


def graph_time(fns, launches, warmup=3):
    """us per launch of fns[i % len(fns)] replayed as one CUDA graph of `launches` launches
    (rotating operand sets larger than L2 is the caller's business)."""
    nb = len(fns)
    for i in range(max(warmup, 1)):
        fns[i % nb]()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        fns[0]()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=st):
            for i in range(launches):
                fns[i % nb]()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / launches


def kernel_case(kernel, M, N, K, launches, buffers=0, warmup=3):
    """One kernel, one shape, rotating operand sets larger than L2 -> dict with us per launch and
    the roofline figures (what `--kernel` prints and what the `extra` entries of the default line hold)."""
    import mixedgemm_b200 as mg
    KN, KS, KO = split_k(K)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(5)
    pk = peaks()
    X = torch.randn(M, K, generator=g, device=dev)
    X[:, torch.randperm(K, generator=g, device=dev)[:K // 32]] *= 20
    X = X.to(torch.bfloat16)
    idx = torch.sort(X.float().abs().amax(0), stable=True).indices.to(torch.int16)
    L2 = 130 << 20
    if kernel == "reorder":
        per = reorder_bytes(M, K)
        nb = buffers or max(2, min(64, L2 // (M * K * 2) + 1))
        Xs = [X.clone() for _ in range(nb)]
        outs = [mg.alloc_quantized_x(M, KN, KS, KO, dev) for _ in range(nb)]
        fns = [lambda i=i: mg.reorder_quantize_x(Xs[i], idx, KN, KS, KO, M, 0, out=outs[i]) for i in range(nb)]
        work, unit, peak, bound = per / 1e9, "GB/s", pk["hbm"], "hbm"
    else:
        W = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        wbytes = N * K // 2 + N * K // 32
        nb = buffers or max(2, min(64, L2 // wbytes + 1))
        A = mg.reorder_quantize_x(X, idx, KN, KS, KO, M, N)
        Bs = [mg.reorder_quantize_w(W, idx, KN, KS, KO, M, N) for _ in range(nb)]
        del W
        Ys = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(nb)]
        fns = [lambda i=i: mg.matmul(A[0], Bs[i][0], A[1], Bs[i][1], A[2], Bs[i][2], A[3], Bs[i][3], A[4], Bs[i][4],
                                     A[5], Bs[i][5], out=Ys[i]) for i in range(nb)]
        work, unit, bound = 2.0 * M * N * K / 1e12, "TFLOP/s", "tensor"
        peak = blended_peak(pk["bf16"], K)
        if M <= 128:  # decode shapes are bound by reading the weights once
            work = (wbytes + M * (KN // 2 + KS // 4 * 3 + KO + K // 32) + 2 * M * N) / 1e9
            unit, bound, peak = "GB/s", "hbm", pk["hbm"]
    us = graph_time(fns, launches, warmup)
    assert mg.device_status() == 0
    return {"kernel": kernel, "M": M, "N": N, "K": K, "launches": launches, "operand_sets": nb,
            "us_per_launch": us, "achieved": work / (us * 1e-6), "unit": unit, "bound": bound,
            "peak": peak, "frac": work / (us * 1e-6) / peak,
            "peak_note": "%s burst figures (kernel timed alone)" % pk["source"]}


def single_kernel(a):
    """`--kernel`: one kernel, one shape; prints a short JSON line."""
    M, N, K = [int(v) for v in a.shape.split(",")]
    torch.cuda.set_device(0)
    print(json.dumps(kernel_case(a.kernel, M, N, K, a.steps, a.buffers, a.warmup)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=list(WORKLOADS))
    ap.add_argument("--exchange", default="push", choices=["push", "push-ce", "push-sm", "push-hybrid", "allgather", "bcast", "replicated"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--quantize", choices=["each", "multi"], default=None,
                    help="one quantiser launch per activation, or one for all of a step (default: multi)")
    ap.add_argument("--no-pipeline", action="store_true",
                    help="push exchange: send and multiply the same batch in a step instead of sending batch i + 1 under the GEMM of batch i")
    ap.add_argument("--no-fuse", action="store_true", help="one GEMM launch per activation instead of one over all layers")
    ap.add_argument("--no-extra", action="store_true", help="skip the `extra` kernels of the default line")
    ap.add_argument("--cpu-rows", type=int, default=128)
    ap.add_argument("--kernel", default=None, choices=["gemm", "reorder"],
                    help="run only this kernel on --shape (for profiling); prints a short JSON line")
    ap.add_argument("--shape", default="2048,4096,4096", help="M,N,K for --kernel")
    ap.add_argument("--sweep", default=None, choices=["decode", "square", "all"],
                    help="time every kernel of the decode-shape sweep (M = 1..128 on the Llama-3-8B layers) and/or the "
                         "large-square and standalone quantiser shapes; one JSON line each")
    ap.add_argument("--buffers", type=int, default=0,
                    help="--kernel: rotate this many operand sets (0 = enough to exceed L2)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl_name = a.workload or ("llama3-8b-m2048" if a.gpus == 1 else "llama3-70b-m4096")
    metric, unit = "mixed_mx_gemm_tflops", "TFLOP/s"

    if a.sweep:
        # the other benchmark configurations, one JSON line per kernel and shape (not the driver's line)
        shapes = []
        if a.sweep in ("decode", "all"):
            for M in (1, 8, 16, 32, 64, 128):
                shapes += [("reorder", M, 0, 4096), ("reorder", M, 0, 14336)]
                shapes += [("gemm", M, N, K) for (N, K) in ((4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336))]
        if a.sweep in ("square", "all"):
            shapes += [("reorder", 8192, 0, 16384), ("gemm", 8192, 8192, 8192), ("gemm", 16384, 16384, 16384)]
        for kernel, M, N, K in shapes:
            a.kernel, a.shape = kernel, "%d,%d,%d" % (M, N, K)
            single_kernel(a)
            torch.cuda.empty_cache()
        return
    if a.kernel:
        return single_kernel(a)

    if a.impl == "reference":
        if rank != 0:
            return
        steps = min(a.steps, 5)
        r = cpu_arm(wl_name, a.cpu_rows, steps, min(a.warmup, 1))
        cb = {"value": r["tflops"], "unit": unit, "cores": r["cores"], "kind": "port", "sample": r["sample"],
              "reorder_quant_gbs": r["reorder_gbs"]}
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": r["tflops"], "unit": unit, "n_gpus": a.gpus,
            "steps": steps, "warmup": min(a.warmup, 1), "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if a.gpus > 1 else "weak", "vs_baseline": None, "dtype": "mxfp4/mxfp6/mxfp8 x mxfp4, f32 accumulate",
            "data": "synthetic", "config": {"workload": wl_name, "note": "CPU restatement of the path on host cores; "
                                            "the reference ships no CPU code and its sm_120 GEMMs do not run on sm_100"},
            "cpu_baseline": cb,
            "e2e": {"value": r["tflops"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        import datetime
        # a short collective timeout: a rank that stalls must end the run, not hold the GPUs
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))

    def sync():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    job = Job(wl_name, rank, world, device, a.exchange, fused=not a.no_fuse, pipeline=not a.no_pipeline,
              multi_q=None if a.quantize is None else a.quantize == "multi")
    pk = peaks()
    nsets = job.nsets

    # ---- whole-step timing, inputs resident in HBM.  One "run" is `nsets` steps (the overlapped
    # exchange alternates between two buffer sets, so its replay unit is two steps).
    def run_eager():
        for s_ in range(nsets):
            job.step(s_)

    use_graph = not a.no_graph
    stream = torch.cuda.Stream()
    runs = (a.steps + nsets - 1) // nsets
    steps = runs * nsets
    with torch.cuda.stream(stream):
        for _ in range((a.warmup + nsets - 1) // nsets):
            run_eager()
        torch.cuda.synchronize()
        run = run_eager
        if use_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    run_eager()
                graph.replay()
                torch.cuda.synchronize()
                run = graph.replay
            except Exception as e:  # capture of NCCL or of a driver call may be refused
                use_graph = False
                sys.stderr.write("CUDA graph capture failed (%r); timing eager launches\n" % (e,))
                torch.cuda.synchronize()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")
        smi_index = vis[local_rank] if local_rank < len(vis) and vis[local_rank].strip().isdigit() else local_rank
        sampler = ClockSampler(smi_index)
        if rank == 0:
            sampler.start()
            time.sleep(0.25)
        t0 = time.time()
        ms = timed(run, runs, sync) / nsets
        t1 = time.time()
        # nvidia-smi samples every 100 ms: when the K timed steps are shorter than that, the clocks are
        # read over an identical window of back-to-back steps that follows them immediately
        clock_window = "the timed steps"
        # every rank must run the same number of steps (they may contain collectives): decide on rank 0's clock
        plan = torch.tensor([t1 - t0, ms], device=device, dtype=torch.float64)
        if world > 1:
            import torch.distributed as dist
            dist.broadcast(plan, src=0)
        span, ms_ref = plan.tolist()
        if span < 0.6:
            n_extra = int(0.6 / max(ms_ref * nsets / 1e3, 1e-6)) + 1
            t0 = time.time()
            timed(run, n_extra, sync)
            t1 = time.time()
            clock_window = "%d further identical steps right after the timed ones" % (n_extra * nsets)
        clocks = sampler.stop(t0, t1) if rank == 0 else None
        if clocks is not None:
            clocks["window"] = clock_window

        # ---- per-kernel durations: an instrumented pass of whole steps in launch order, so every kernel
        # sees the cache state it has inside a step.  A spin kernel keeps the GPU busy while the CPU
        # enqueues, so the event pairs bracket pure GPU execution rather than Python launch overhead.
        # The GEMMs are timed both ways: one launch per activation (so that every layer group has its
        # own figure) and the single launch over all layers that the step uses.
        ev = lambda: torch.cuda.Event(enable_timing=True)
        q_ms, g_ms, q_each, g_each, fused_ms, q_all_ms = 0.0, 0.0, [], [], None, None
        if world == 1:
            reps = max(3, min(a.steps, 10))
            marks = []
            torch.cuda.synchronize()
            torch.cuda._sleep(int(1.0e7) * reps)
            for _ in range(reps):
                for gi in range(len(job.groups)):
                    e0, e1 = ev(), ev()
                    e0.record()
                    job.quantize(gi)
                    e1.record()
                    marks.append((("q", gi), e0, e1))
                    e0, e1 = ev(), ev()
                    e0.record()
                    job.gemm_group(gi)
                    e1.record()
                    marks.append((("g", gi), e0, e1))
                if job.fused:
                    e0, e1 = ev(), ev()
                    e0.record()
                    job.gemm_fused()
                    e1.record()
                    marks.append((("f", 0), e0, e1))
                if job.multi_q:
                    e0, e1 = ev(), ev()
                    e0.record()
                    job.quantize_all()
                    e1.record()
                    marks.append((("qa", 0), e0, e1))
            torch.cuda.synchronize()
            acc = {}
            for key, e0, e1 in marks:
                acc[key] = acc.get(key, 0.0) + e0.elapsed_time(e1) / reps
            for gi, gr in enumerate(job.groups):
                q_each.append((gr["K"], acc[("q", gi)]))
                q_ms += acc[("q", gi)]
                names = "+".join(n for (n, _, _, _) in gr["layers"])
                Nsum = sum(Nl for (_, Nl, _, _) in gr["layers"])
                g_each.append((names, job.M, Nsum, gr["K"], acc[("g", gi)]))
                g_ms += acc[("g", gi)]
            fused_ms = acc.get(("f", 0))
            q_all_ms = acc.get(("qa", 0))

        # ---- end to end: activations from pinned host memory, results back to pinned host memory.
        # Every rank uploads the rows it quantises (all of them on one GPU; M / P with a sharded
        # quantiser) and downloads its output shards.
        hX = [gr["X"].cpu().pin_memory() for gr in job.groups]
        hY = [[torch.empty(Y.shape, dtype=Y.dtype).pin_memory() for (_, _, _, Y) in gr["layers"]] for gr in job.groups]
        h2d = sum(t.numel() * 2 for t in hX)
        d2h = sum(t.numel() * 2 for ys in hY for t in ys)

        # Three streams, as a caller with host buffers would run it: uploads, compute and downloads
        # overlap (PCIe is full duplex), ordered by events.  Every step uploads all its activations
        # and downloads all its outputs; the closing event waits for the last download.
        main_s = torch.cuda.current_stream()
        in_s, out_s = torch.cuda.Stream(), torch.cuda.Stream()
        ng = len(job.groups)
        ev_in = [torch.cuda.Event() for _ in range(ng)]      # activation g is on the device
        ev_xfree = [torch.cuda.Event() for _ in range(ng)]   # activation g has been quantised
        ev_done = [torch.cuda.Event() for _ in range(ng)]    # outputs of group g are complete
        ev_yfree = [torch.cuda.Event() for _ in range(ng)]   # outputs of group g are on the host
        for g in range(ng):
            ev_xfree[g].record(main_s)
            ev_yfree[g].record(main_s)
        e2e_count = [0]
        # On one GPU the GEMMs go out per activation here, so that a group's outputs travel to the
        # host while the next group multiplies (the link, not the GPU, bounds this leg); with the
        # overlapped exchange the single launch stays, because it is what waits for the flags.
        e2e_fused = job.fused and job.ex is not None

        def e2e_step():
            s_ = e2e_count[0] % nsets
            e2e_count[0] += 1
            order = job.order if e2e_fused else list(range(ng))
            for g in order:
                in_s.wait_event(ev_xfree[g])
                with torch.cuda.stream(in_s):
                    job.groups[g]["X"].copy_(hX[g], non_blocking=True)
                    ev_in[g].record(in_s)
            if job.ex is not None:
                # the push exchange moves a step's activations at once: all uploads, one quantiser
                # launch, one push, then the GEMMs (not pipelined across steps here)
                for g in order:
                    main_s.wait_event(ev_in[g])
                job.ex.begin_step(s_)
                job.quantize_all(s_)
                for g in order:
                    ev_xfree[g].record(main_s)
                job.ex.push(s_)
                for g in order:
                    main_s.wait_event(ev_yfree[g])
                job.multiply(s_)
                job.ex.join()
                for g in order:
                    ev_done[g].record(main_s)
            else:
                for g in order:
                    main_s.wait_event(ev_in[g])
                    job.quantize(g, s_)
                    ev_xfree[g].record(main_s)
                    job.exchange_a(g, s_)
                    main_s.wait_event(ev_yfree[g])
                    job.gemm_group(g, s_)
                    ev_done[g].record(main_s)
            for g in order:
                out_s.wait_event(ev_done[g])
                with torch.cuda.stream(out_s):
                    for (_, _, _, Y), hy in zip(job.groups[g]["layers"], hY[g]):
                        hy.copy_(Y, non_blocking=True)
                    ev_yfree[g].record(out_s)

        def e2e_finish():
            main_s.wait_stream(in_s)
            main_s.wait_stream(out_s)

        for _ in range(2 * nsets):
            e2e_step()
        e2e_ms = timed(e2e_step, max(4, min(a.steps, 10)) // nsets * nsets, sync, finish=e2e_finish)

    # max over ranks
    solo = None
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms, e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
        # The single-GPU figure of the SAME workload, so that the ratio of this line to one GPU does
        # not have to be taken against the (smaller) default workload of `--gpus 1`: rank 0 alone,
        # all weights, same graph-replay timing, while the other ranks wait.
        if rank == 0:
            job.mg.set_option("GEMM_MAX_CLUSTERS", 0)  # the single-GPU figure uses every SM
            job.mg.set_option("REORDER_CTAS", 0)
            job1 = Job(wl_name, 0, 1, device, "none", fused=not a.no_fuse)
            with torch.cuda.stream(stream):
                for _ in range(a.warmup):
                    job1.step()
                torch.cuda.synchronize()
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1, stream=stream):
                    job1.step()
                g1.replay()
                ms1 = timed(g1.replay, a.steps, torch.cuda.synchronize)
            solo = {"n_gpus": 1, "workload": wl_name, "value": job1.flops_total / (ms1 * 1e-3) / 1e12, "unit": unit,
                    "ms_per_step": ms1, "note": "rank 0 alone with all weights, same run, same timing"}
            del job1, g1
        dist.barrier()
    status = job.mg.device_status()
    if status != 0:
        raise SystemExit("a kernel reported device status %d" % status)
    def leave():
        # Every rank is between steps with nothing in flight (synchronised, then a barrier).  The
        # process then ends without tearing the communicators down: their destructors are
        # collective and gain nothing here.
        import torch.distributed as dist
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    if rank != 0:
        if world > 1:
            leave()
        return

    value = job.flops_total / (ms * 1e-3) / 1e12
    out = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": a.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "mxfp4/mxfp6/mxfp8 x mxfp4, f32 accumulate, bf16 out", "data": "synthetic",
        "config": {"workload": wl_name, "M": job.M,
                   "layers": [[gr["K"], [[n, N * world] for (n, N, _, _) in gr["layers"]]] for gr in job.groups],
                   "k_split": "62.5% fp4 / 34.375% fp6 / 3.125% fp8", "parallelism": "n-shard x%d" % world,
                   "exchange": (job.exchange + ("/" + job.push_mode if job.ex is not None else "")), "cuda_graph": use_graph,
                   "pipeline": (("every step sends batch i + 1 (one kernel on %d SMs of its own), quantises batch i + 2 (one "
                                 "launch) and multiplies batch i; %d buffer sets in turn" % (job.push_ctas, job.nsets))
                                if job.lookahead == 2 else
                                ("every step quantises and sends batch i + 1 (one quantiser launch, one copy per peer) and "
                                 "multiplies batch i, which the step before sent; %d buffer sets in turn" % job.nsets))
                   if job.pipeline else None,
                   "gemm_launch": "one launch over all layers" if job.fused else "one launch per activation",
                   "l2": "inputs larger than L2: one step touches ~%d MB of weights, activations and outputs" % (
                       (sum(t.numel() * t.element_size() for gr in job.groups for (_, _, B, Y) in gr["layers"]
                            for t in list(B) + [Y]) + h2d) >> 20)},
        "clocks": clocks,
        "gpu_launches": job.n_kernels * steps,
        "e2e": {"value": job.flops_total / (e2e_ms * 1e-3) / 1e12, "unit": unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world},
    }
    if solo is not None:
        out["same_workload_1gpu"] = solo
    if world == 1:
        gemm_flops = job.flops_local
        peak_s = blended_peak(pk["bf16_sustained"], 4096)  # same split for every K
        peak_b = blended_peak(pk["bf16"], 4096)
        g_best = fused_ms if (fused_ms is not None and job.fused) else g_ms
        achieved_t, unit_t, bound_t, kern_t = gemm_flops / (g_best * 1e-3) / 1e12, "TFLOP/s", "tensor", "mixed_gemm_pair_kernel"
        if job.M <= 128:  # decode shapes are bound by reading the weights once
            gbytes = sum(N * K // 2 + N * K // 32 + reorder_bytes(M, K) - 2 * M * K + 2 * M * N for (M, N, K) in job.gemm_shapes)
            achieved_t, unit_t, bound_t, kern_t = gbytes / (g_best * 1e-3) / 1e9, "GB/s", "hbm", "mixed_gemm_kernel"
            peak_s = peak_b = pk["hbm"]
        out["roofline"] = {
            "kernel": kern_t, "bound": bound_t, "achieved": achieved_t,
            "peak": peak_s, "unit": unit_t, "frac": achieved_t / peak_s,
            "frac_sustained": achieved_t / peak_s, "peak_burst": peak_b, "frac_burst": achieved_t / peak_b,
            "what": ("the step's single GEMM launch over all layers, %.1f us" % (g_best * 1e3)) if job.fused and fused_ms
            else "the step's GEMM launches, %.1f us together" % (g_best * 1e3),
            # dram__bytes_read.sum + dram__bytes_write.sum of the step's launch over all layers under ncu
            "traffic": 290.1e6 if (wl_name == "llama3-8b-m2048" and job.fused) else None,
            "traffic_source": "ncu capture of the step's launch, summarised in profiles/mixed_gemm_pair_kernel_llama3-8b-m2048_step.md",
            "peak_note": ("%s copy bandwidth" % pk["source"]) if job.M <= 128 else
            "K-blended tensor peak: fp4 segment at 4x and fp6/fp8 at 2x the %s bf16 rate (sustained %.1f, burst %.1f TF/s)" % (
                pk["source"], pk["bf16_sustained"], pk["bf16"]),
            "launches_per_activation": [{"layer": n, "M": M, "N": N, "K": K, "us": t * 1e3,
                                         "tflops": 2 * M * N * K / (t * 1e-3) / 1e12} for (n, M, N, K, t) in g_each],
            "launches_per_activation_us": g_ms * 1e3,
            "launch_all_layers_us": fused_ms * 1e3 if fused_ms is not None else None}
        rbytes = sum(reorder_bytes(job.M, K) for (K, _) in q_each)
        q_best = q_all_ms if (q_all_ms is not None and job.multi_q) else q_ms
        out["roofline_reorder"] = {
            "kernel": "reorder_quantize_multi_kernel" if q_best is q_all_ms else "reorder_quantize_kernel",
            "bound": "hbm", "achieved": rbytes / (q_best * 1e-3) / 1e9,
            "peak": pk["hbm"], "unit": "GB/s", "frac": rbytes / (q_best * 1e-3) / 1e9 / pk["hbm"],
            "what": ("the step's single quantiser launch over all activations, %.1f us" % (q_best * 1e3)) if q_best is q_all_ms
            else "the step's quantiser launches, %.1f us together" % (q_best * 1e3),
            "launches_per_activation_us": q_ms * 1e3,
            "launch_all_activations_us": q_all_ms * 1e3 if q_all_ms is not None else None,
            # the step's launch over the four activations under ncu: 109.3 MB read, 14.5 of the 34.5 MB
            # written have left L2 when the kernel ends
            "traffic": 123.8e6 if (wl_name == "llama3-8b-m2048" and q_best is q_all_ms) else None,
            "traffic_source": "ncu capture of the step's launch, summarised in profiles/reorder_quantize_multi_kernel_llama3-8b-m2048_step.md",
            "peak_note": "%s copy bandwidth" % pk["source"],
            "launches": [{"M": job.M, "K": K, "us": t * 1e3, "gbs": reorder_bytes(job.M, K) / (t * 1e-3) / 1e9}
                         for (K, t) in q_each]}
        out["reorder_quant_gbs"] = out["roofline_reorder"]["achieved"]
        if not a.no_extra:
            # the other benchmark configurations, each kernel alone over operand sets larger than L2:
            # the standalone quantiser, the 8192-cube GEMM and two points of the decode sweep
            job.close()
            del job
            torch.cuda.empty_cache()
            extra = {"standalone_reorder_8192x16384": kernel_case("reorder", 8192, 0, 16384, 10),
                     "gemm_8192_cube": kernel_case("gemm", 8192, 8192, 8192, 6)}
            torch.cuda.empty_cache()
            for M_ in (16, 128):
                # the four layers, then q+k+v and gate+up as one product over the concatenated weights
                cases = [kernel_case("gemm", M_, N_, K_, 20) for (N_, K_) in ((4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336),
                                                                                (6144, 4096), (28672, 4096))]
                cases.append(kernel_case("reorder", M_, 0, 4096, 20))
                cases.append(kernel_case("reorder", M_, 0, 14336, 20))
                extra["decode_m%d" % M_] = [{k: c[k] for k in ("kernel", "M", "N", "K", "us_per_launch", "achieved", "unit", "frac")}
                                           for c in cases]
                torch.cuda.empty_cache()
            out["extra"] = extra
            job = None
        r = cpu_arm(wl_name, a.cpu_rows, 2, 1)
        out["cpu_baseline"] = {"value": r["tflops"], "unit": unit, "cores": r["cores"], "kind": "port",
                               "sample": r["sample"], "reorder_quant_gbs": r["reorder_gbs"]}
    print(json.dumps(out))
    if world > 1:
        leave()


if __name__ == "__main__":
    main()
