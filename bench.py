"""Benchmark of the NVFP4 fused-MoE decode layer on B200 (the reference's headline: layer us/call and achieved HBM GB/s on
touched-expert bytes at M = 1..16, Qwen3-30B-A3B shape, random and fixed-8 routing).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--layers L] [--shape qwen|gemma]

One step = one pass over the ten (M, routing) cases; each case runs a chain of L layer calls over L DISTINCT weight sets
(L x 340 MB, larger than L2), so every call streams its experts from HBM as it would inside a model. Synthetic seeded
inputs stand in for the public checkpoint the reference measured on. Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

MS = (1, 2, 4, 8, 16)
ROUTINGS = ("random", "fixed8")


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def cases(cfg, only=None):
    from sm120fp4_b200 import synth
    out = []
    for routing in ROUTINGS:
        for m in MS:
            if only and f"{m}:{routing}" not in only:
                continue
            x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 1000 + m if routing == "random" else 7, routing)
            out.append(dict(m=m, routing=routing, x=x, ids=ids, wts=wts, touched=int(torch.unique(ids).numel())))
    return out


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled during the timed region (read-only queries)."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def build_layers(cfg, n_layers, device, shard=None):
    """n_layers independently seeded layers; weights drawn on the GPU as bf16 N(0, 0.02) and quantised by the library's
    own (bit-exact) quantizer with one global scale per expert, scales kept in the 128x4 swizzle."""
    import sm120fp4_b200 as pkg
    from sm120fp4_b200.vllm_backend import Weights
    e, h, i, k = cfg["experts"], cfg["hidden"], cfg["inter"], cfg["top_k"]
    layers = []
    for li in range(n_layers):
        g = torch.Generator(device=device).manual_seed(li)
        parts = {}
        for name, rows, cols in (("1", 2 * i, h), ("2", h, i)):
            w = (torch.randn(e, rows, cols, generator=g, device=device) * 0.02).to(torch.bfloat16)
            if shard is not None:   # expert-parallel: this rank keeps experts [lo, hi) of the same seeded layer
                w = w[shard[0]:shard[1]].contiguous()
            q, sw, gs = pkg.quantize_nvfp4_experts(w, swizzle=True)
            parts[name] = (q, sw, 1.0 / gs)
            del w
        layers.append(Weights(parts["1"][0], parts["1"][1], parts["1"][2], parts["2"][0], parts["2"][1], parts["2"][2], k,
                              scale_layout="128x4"))
    return layers


def time_region(fn, sync):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    s.record()
    fn()
    e.record()
    sync()
    return s.elapsed_time(e)


def run_ours(a):
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    from sm120fp4_b200 import synth
    cfg = dict(synth.QWEN if a.shape == "qwen" else synth.GEMMA)
    from sm120fp4_b200.ep import shard_range
    layers = build_layers(cfg, a.layers, dev)
    cs = cases(cfg, set(a.cases.split(",")) if a.cases else None)
    for c in cs:
        c["xd"], c["idd"], c["wd"] = c["x"].to(dev), c["ids"].to(dev), c["wts"].to(dev)
        c["out"] = torch.empty_like(c["xd"])
        c["hx"], c["hid"], c["hw"] = c["x"].pin_memory(), c["ids"].pin_memory(), c["wts"].pin_memory()
        c["hout"] = torch.empty_like(c["x"]).pin_memory()
    ebytes = layers[0].expert_bytes()

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- one CUDA graph per case: the chain of L layer calls (device-resident inputs)
    def chain(c):
        for w in layers:
            w.forward(c["xd"], c["idd"], c["wd"], out=c["out"])

    graphs, use_graph = {}, not a.no_graph
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for c in cs:
            chain(c)   # first call outside capture (function attributes, lazy init)
        torch.cuda.synchronize()
        if use_graph:
            try:
                for idx, c in enumerate(cs):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        chain(c)
                    graphs[idx] = g
            except Exception as ex:  # noqa: BLE001
                print(f"graph capture unavailable ({type(ex).__name__}: {ex}); timing direct launches", file=sys.stderr)
                graphs, use_graph = {}, False
                torch.cuda.synchronize()
    for w in layers:
        w.status()

    def run_case(idx):
        if use_graph:
            graphs[idx].replay()
        else:
            chain(cs[idx])

    def step():
        for idx in range(len(cs)):
            run_case(idx)

    def e2e_step():   # the C-ABI call with host buffers: copies in, layer, copy out, all inside the timed region
        for c in cs:
            for w in layers:
                w.forward_host(c["hx"], c["hid"], c["hw"], c["hout"])

    with torch.cuda.stream(stream):
        for _ in range(a.warmup):
            step()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        per_case_ms = np.zeros(len(cs))
        sync()
        t_total = 0.0
        for _ in range(a.steps):
            for idx in range(len(cs)):
                ms = time_region(lambda: run_case(idx), torch.cuda.synchronize)
                per_case_ms[idx] += ms
                t_total += ms
        sync()
        # the whole-step time, all cases back to back in one timed region (this is the reported step time)
        step_ms = time_region(lambda: [step() for _ in range(a.steps)], sync) / a.steps
        for _ in range(max(1, a.warmup // 2)):
            e2e_step()
        e2e_ms = time_region(lambda: [e2e_step() for _ in range(a.steps)], sync) / a.steps
        clocks = sampler.stop() if rank == 0 else None
    for w in layers:
        w.status()
    if dist is not None:
        t = torch.tensor([step_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms, e2e_ms = float(t[0]), float(t[1])
    extras = {}
    if not a.no_extras:
        with torch.cuda.stream(stream):
            if world == 1:
                extras["prefill"] = prefill_numbers(cfg, layers[:2], dev)
                extras["ep"] = ep_stack(cfg, layers, None, 1, 0, dev, stack=a.ep_layers)
            else:
                del graphs
                layers.clear()
                torch.cuda.empty_cache()
                sharded = build_layers(cfg, a.layers, dev, shard=shard_range(cfg["experts"], rank, world))
                extras["ep"] = ep_stack(cfg, sharded, dist, world, rank, dev, stack=a.ep_layers)
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak, peak_src = peaks()
    step_bytes = sum(c["touched"] for c in cs) * ebytes * a.layers
    value = world * step_bytes / (step_ms * 1e-3) / 1e9
    detail = []
    for idx, c in enumerate(cs):
        us = per_case_ms[idx] / a.steps / a.layers * 1e3
        gbs = c["touched"] * ebytes / (us * 1e-6) / 1e9
        detail.append({"m": c["m"], "routing": c["routing"], "touched_experts": c["touched"], "us_per_layer": round(us, 2),
                       "hbm_gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3)})
    launches = a.steps * len(cs) * a.layers
    kernel_ms = float(per_case_ms.sum()) / a.steps
    achieved = step_bytes / (kernel_ms * 1e-3) / 1e9
    traffic = None
    tp = ROOT / "profiles" / "decode_traffic.json"
    if tp.exists():
        traffic = json.loads(tp.read_text()).get("dram_bytes_per_launch")
    cpu = cpu_baseline(cfg, a) if not a.no_cpu else None
    line = {
        "metric": "moe_decode_layer_hbm_gbs_on_touched_expert_bytes", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 weights x f16 activations, fp32 accumulate (W4A16)", "data": "synthetic",
        "config": {"workload": f"{a.shape}-shaped MoE layer decode sweep M in {list(MS)} x routing {list(ROUTINGS)}; E={cfg['experts']} H={cfg['hidden']} I={cfg['inter']} top-{cfg['top_k']}",
                   "layers_in_chain": a.layers, "l2": f"inputs larger than L2: each call reads one of {a.layers} distinct {ebytes * cfg['experts'] / 1e6:.0f} MB weight sets",
                   "graph_replay": use_graph, "parallelism": "replicas" if world > 1 else "single"},
        "cases": detail,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": traffic, "peak_source": peak_src, "kernel": "k_moe_decode_tc",
                     "bytes_per_launch": round(step_bytes / (len(cs) * a.layers))},
        "e2e": {"value": round(world * step_bytes / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(e2e_ms, 3),
                "h2d_bytes_per_step": int(sum(c["x"].numel() * 2 + c["ids"].numel() * 4 + c["wts"].numel() * 4 for c in cs) * a.layers),
                "d2h_bytes_per_step": int(sum(c["x"].numel() * 2 for c in cs) * a.layers)},
        "gpu_launches": launches, "clocks": clocks, "cpu_baseline": cpu,
    }
    line.update(extras)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def prefill_numbers(cfg, layers, dev, reps=5):
    """W4A4 prefill (own tcgen05 grouped GEMM): us per layer call and TFLOP/s on 6*M*k*I*H flop at M = 256 .. 8192."""
    from sm120fp4_b200 import synth
    ws = None
    for w in layers:
        w.enable_prefill(max_tokens=8192, workspace=ws)
        ws = w.prefill.workspace
    rows = []
    for m in (256, 1024, 4096, 8192):
        x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 9000 + m)
        xd, idd, wd = x.to(dev), ids.to(dev), wts.to(dev)
        out = torch.empty_like(xd)
        for _ in range(2):
            for w in layers:
                w.forward(xd, idd, wd, out=out)
        ts = []
        for _ in range(reps):
            ts.append(time_region(lambda: [w.forward(xd, idd, wd, out=out) for w in layers], torch.cuda.synchronize) / len(layers))
        ts.sort()
        t = ts[len(ts) // 2]
        flop = 6.0 * m * cfg["top_k"] * cfg["inter"] * cfg["hidden"]
        rows.append({"m": m, "us_per_layer": round(t * 1e3, 1), "tflops": round(flop / t / 1e9, 1),
                     "frac_of_dense_fp4_nominal": round(flop / t / 1e9 / 9000.0, 4)})
    layers[0].prefill_status()
    for w in layers:
        w.prefill = None
    return rows


def ep_stack(cfg, layers, dist, world, rank, dev, stack=48, decode_tokens=16, prefill_tokens=4096, reps=3):
    """The expert-parallel stack of BASELINE configs[4]: `stack` layer calls (cycling over the resident layer objects, each
    holding E / world experts), decode with 16 tokens per GPU (fixed-capacity dispatch, no host sync) and prefill with 4096
    tokens per GPU (variable-size dispatch, W4A4 path). Device-timed, max over ranks. Returns tokens/s and per-layer us."""
    from sm120fp4_b200 import synth
    from sm120fp4_b200.ep import ExpertParallelMoE
    e, k = cfg["experts"], cfg["top_k"]
    res = {}
    for name, m, cap in (("decode", decode_tokens, decode_tokens), ("prefill", prefill_tokens, None)):
        ws = None
        if name == "prefill":
            for w in layers:
                w.enable_prefill(max_tokens=prefill_tokens * world, workspace=ws)
                ws = w.prefill.workspace
        if name == "decode" and world > 1:   # a rank receives 16 rows from every peer: one W4A16 call instead of `world` slices
            for w in layers:
                w.enable_mid(max_tokens=world * decode_tokens, workspace=ws)
                ws = w.mid.workspace
            ws = None
        eps = [ExpertParallelMoE(w.forward, e, k, capacity=cap) for w in layers]
        x, ids, wts = synth.decode_inputs(m, e, cfg["hidden"], k, 7000 + 13 * rank + m)
        xd, idd, wd = x.to(dev), ids.to(dev), wts.to(dev)

        def run():
            for li in range(stack):
                eps[li % len(eps)].forward(xd, idd, wd)

        def sync():
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
                torch.cuda.synchronize()
        run()
        run()
        launch, graphed = run, False
        if name == "decode":   # fixed-capacity dispatch: no host synchronisation inside, so the whole stack replays as one CUDA graph
            try:
                sync()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    run()
                launch, graphed = g.replay, True
                launch()
            except Exception as ex:  # noqa: BLE001 - e.g. a collective that cannot be captured on this build
                print(f"expert-parallel decode stack: graph capture unavailable ({type(ex).__name__}: {ex}); direct launches", file=sys.stderr)
                launch = run
        ts = [time_region(launch, sync) for _ in range(reps)]
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        res[name] = {"tokens_per_gpu": m, "tokens_per_s": round(world * m / (ms * 1e-3), 1), "us_per_layer": round(ms * 1e3 / stack, 1),
                     "rows_dispatched_per_layer_per_gpu": eps[0].last_sent_rows, "row_bytes": cfg["hidden"] * 2, "graph_replay": graphed}
        for w in layers:
            w.prefill = None
            w.mid = None
            w.status()
    res["stack_layers"] = stack
    return res


def host_layer(cfg, seed=0):
    """One layer's weights on the host for the CPU arm: drawn and quantised by the oracle itself (a few experts only:
    the ones the sampled batch touches are generated lazily)."""
    from oracle import nvfp4_oracle as O
    e, h, i = cfg["experts"], cfg["hidden"], cfg["inter"]

    class Lazy(O.ExpertWeights):
        def __init__(self):
            self.E, self.I, self.H = e, i, h
            self._cache = {}

        def dequant(self, ex):
            if ex not in self._cache:
                g = torch.Generator().manual_seed(seed * 1000 + ex)
                w13 = (torch.randn(2 * i, h, generator=g) * 0.02).to(torch.bfloat16).float().numpy()
                w2 = (torch.randn(h, i, generator=g) * 0.02).to(torch.bfloat16).float().numpy()
                q1, s1, g1 = O.quantize_nvfp4(w13)
                q2, s2, g2 = O.quantize_nvfp4(w2)
                self._packed = getattr(self, "_packed", {})
                self._packed[ex] = (q1, s1, g1, q2, s2, g2)
                self._cache[ex] = None
            return self._packed[ex]
    return Lazy()


def cpu_forward_timed(cfg, m, routing, repeats):
    """The oracle's dequantise-then-fp32-GEMM MoE forward, timed on the host cores. Weight generation and quantisation are
    outside the timed region; dequantisation is inside, as in the reference's CPU path."""
    from oracle import nvfp4_oracle as O
    from sm120fp4_b200 import synth
    x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 1000 + m if routing == "random" else 7, routing)
    lazy = host_layer(cfg)
    touched = sorted(set(ids.reshape(-1).tolist()))
    packed = {ex: lazy.dequant(ex) for ex in touched}
    e, h, i = cfg["experts"], cfg["hidden"], cfg["inter"]
    q1 = np.zeros((e, 2 * i, h // 2), np.uint8); s1 = np.zeros((e, 2 * i, h // 16), np.uint8); a1 = np.ones(e, np.float32)
    q2 = np.zeros((e, h, i // 2), np.uint8); s2 = np.zeros((e, h, i // 16), np.uint8); a2 = np.ones(e, np.float32)
    for ex, (p1, f1, g1, p2, f2, g2) in packed.items():
        q1[ex], s1[ex], a1[ex], q2[ex], s2[ex], a2[ex] = p1, f1, 1.0 / g1[0], p2, f2, 1.0 / g2[0]
    xs, idn, wn = x.float().numpy(), ids.numpy(), wts.numpy()
    times = []
    for _ in range(repeats):
        w = O.ExpertWeights(q1, s1, a1, q2, s2, a2)
        t0 = time.perf_counter()
        O.moe_reference(xs, w, idn, wn)
        times.append(time.perf_counter() - t0)
    return float(np.median(times)), len(touched) * O.expert_bytes(h, i)


def cpu_baseline(cfg, a):
    sec, nbytes = cpu_forward_timed(cfg, 4, "random", 3)
    return {"value": round(nbytes / sec / 1e9, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"oracle (numpy restatement of the reference's CPU path) on one layer call, M=4 random routing, median of 3 ({sec:.2f} s per call)"}


def run_reference(a):
    """The reference arm: the reference's CPU algorithm for this path (the oracle port; the reference itself is a PyTorch
    package that cannot travel to the GPU box) on the host cores, on a bounded sample of the same workload."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from sm120fp4_b200 import synth
    cfg = dict(synth.QWEN if a.shape == "qwen" else synth.GEMMA)
    for _ in range(min(a.warmup, 1)):
        cpu_forward_timed(cfg, 1, "random", 1)
    tot_s, tot_b = 0.0, 0
    for _ in range(a.steps):
        for m, routing in ((1, "random"), (4, "random"), (4, "fixed8")):
            s, b = cpu_forward_timed(cfg, m, routing, 1)
            tot_s += s
            tot_b += b
    val = tot_b / tot_s / 1e9
    sample = "per step: one layer call each at (M=1 random), (M=4 random), (M=4 fixed8) of the decode sweep; numpy/BLAS threads"
    line = {"impl": "reference", "metric": "moe_decode_layer_hbm_gbs_on_touched_expert_bytes", "value": round(val, 4), "unit": "GB/s",
            "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(tot_s / a.steps * 1e3, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 on dequantised NVFP4", "data": "synthetic",
            "config": {"workload": f"{a.shape}-shaped MoE layer decode sweep (bounded sample)"},
            "cpu_baseline": {"value": round(val, 4), "unit": "GB/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
            "e2e": {"value": round(val, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--layers", type=int, default=16, help="distinct weight sets in the chain (16 x 340 MB = 5.4 GB)")
    ap.add_argument("--shape", default="qwen", choices=("qwen", "gemma"))
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--cases", default="", help="subset of the sweep for profiling, e.g. 16:random,1:fixed8 (default: all ten)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill and expert-parallel stack measurements")
    ap.add_argument("--ep-layers", type=int, default=48, help="layer calls in the expert-parallel stack")
    a = ap.parse_args()
    if a.impl == "reference":
        return run_reference(a)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    run_ours(a)


if __name__ == "__main__":
    main()
