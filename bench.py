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
# "peer" (default): rows stored straight into the peers' memory over NVLink as flagged words; "peer_fence": plain rows, a
# system-scope fence and arrival counters; "nccl": one packed all-to-all each way
EP_TRANSPORT = os.environ.get("B200MOE_EP_TRANSPORT", "peer")


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def flush_l2(buf):
    buf.add_(1)   # a read-modify-write over a buffer larger than L2


def decode_sweep(cfg, layers, dev, steps, warmup, use_graph, rank, world, dist, eps=None, only=None, e2e=True, cold=True):
    """The ten-case decode sweep over a chain of layer calls. world == 1: `Weights.forward` per call. world > 1: every call
    goes through `ExpertParallelMoE` over sharded experts (dispatch and combine exchanges inside the timed region); every
    rank brings its own batch of M tokens per case. Returns per-case microseconds, the step time (max over ranks), the
    end-to-end step time and the bytes of a step."""
    from sm120fp4_b200 import synth
    e, h, k = cfg["experts"], cfg["hidden"], cfg["top_k"]
    cs = []
    for routing in ROUTINGS:
        for m in MS:
            if only and f"{m}:{routing}" not in only:
                continue
            seed = (1000 + m if routing == "random" else 7) + 7919 * rank
            x, ids, wts = synth.decode_inputs(m, e, h, k, seed, routing)
            c = dict(m=m, routing=routing, x=x, ids=ids, wts=wts, touched=int(torch.unique(ids).numel()))
            c["xd"], c["idd"], c["wd"] = x.to(dev), ids.to(dev), wts.to(dev)
            c["out"] = torch.empty_like(c["xd"])
            c["hx"], c["hid"], c["hw"] = x.pin_memory(), ids.pin_memory(), wts.pin_memory()
            c["hout"] = torch.empty_like(x).pin_memory()
            cs.append(c)
    n_layers = len(layers)

    def call(li, c, xd, idd, wd, out):
        if eps is None:
            layers[li].forward(xd, idd, wd, out=out)
        else:   # every rank brings c["m"] tokens: the exchange blocks hold exactly that many rows
            eps[li].forward(xd, idd, wd, out=out, rows=c["m"])

    def chain(c):
        for li in range(n_layers):
            call(li, c, c["xd"], c["idd"], c["wd"], c["out"])

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    graphs = {}
    stream = torch.cuda.current_stream()
    for c in cs:
        chain(c)   # first call outside capture (function attributes, lazy init, buffer allocation)
    sync()
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
            sync()

    def run_case(idx):
        if use_graph:
            graphs[idx].replay()
        else:
            chain(cs[idx])

    def step():
        for idx in range(len(cs)):
            run_case(idx)

    def e2e_step():   # host buffers in, host buffers out, every call, inside the timed region
        for c in cs:
            if eps is None:
                for w in layers:
                    w.forward_host(c["hx"], c["hid"], c["hw"], c["hout"])
            else:
                for li in range(n_layers):
                    xd = c["hx"].to(dev, non_blocking=True)
                    idd, wd = c["hid"].to(dev, non_blocking=True), c["hw"].to(dev, non_blocking=True)
                    call(li, c, xd, idd, wd, c["out"])
                    c["hout"].copy_(c["out"], non_blocking=True)

    for _ in range(warmup):
        step()
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    per_case_ms = np.zeros(len(cs))
    sync()
    for _ in range(steps):
        for idx in range(len(cs)):
            per_case_ms[idx] += time_region(lambda: run_case(idx), sync if dist is not None else torch.cuda.synchronize)
    sync()
    step_ms = time_region(lambda: [step() for _ in range(steps)], sync) / steps   # all cases back to back: the reported step time
    e2e_ms, e2e_direct_ms = None, None
    if e2e:
        for _ in range(max(1, warmup // 2)):
            e2e_step()
        e2e_ms = e2e_direct_ms = time_region(lambda: [e2e_step() for _ in range(steps)], sync) / steps
        if use_graph and eps is None:
            # the same host-buffer calls captured once per case and replayed, as a serving engine runs its decode steps: the
            # copies of x, ids and weights from the page-locked host tensors and the kernel's writes of the output into host
            # memory still happen on every replay; what goes away is the per-call launch work on the host
            try:
                hg = []
                for c in cs:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        for w in layers:
                            w.forward_host(c["hx"], c["hid"], c["hw"], c["hout"])
                    hg.append(g)
                for g in hg:
                    g.replay()
                sync()
                e2e_ms = min(e2e_direct_ms, time_region(lambda: [g.replay() for _ in range(steps) for g in hg], sync) / steps)
            except Exception as ex:  # noqa: BLE001
                print(f"host-buffer calls: graph capture unavailable ({type(ex).__name__}: {ex}); direct launches only", file=sys.stderr)
                sync()
    clocks = sampler.stop() if rank == 0 else None
    cold_us = None
    if cold and eps is None:
        # one layer call alone with L2 flushed before it (the reference's method, sm120fp4/kernels/micro_floor.py:189-222):
        # nothing of the call overlaps a predecessor, and its weights come from HBM
        flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
        cold_us = []
        for c in cs:
            ts = []
            for r in range(7):
                w = layers[r % n_layers]
                flush_l2(flush)
                ts.append(time_region(lambda: w.forward(c["xd"], c["idd"], c["wd"], out=c["out"]), torch.cuda.synchronize) * 1e3)
            cold_us.append(sorted(ts)[len(ts) // 2])
        del flush
    for w in layers:
        w.status()
    if dist is not None:
        t = torch.tensor([step_ms, e2e_ms or 0.0] + list(per_case_ms), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms, e2e_ms, per_case_ms = float(t[0]), (float(t[1]) if e2e else None), t[2:].cpu().numpy()
        e2e_direct_ms = e2e_ms   # expert-parallel calls have no captured host-buffer form
        tt = torch.tensor([c["touched"] for c in cs], device=dev, dtype=torch.float64)
        dist.all_reduce(tt)                       # sum over ranks of the experts each rank's own batch touches
        touched = tt.cpu().numpy()
    else:
        touched = np.array([c["touched"] for c in cs], dtype=np.float64)
    ebytes = 3 * cfg["inter"] * cfg["hidden"] // 2 + 3 * cfg["inter"] * cfg["hidden"] // 16
    detail = []
    for idx, c in enumerate(cs):
        us = per_case_ms[idx] / steps / n_layers * 1e3
        gbs = touched[idx] * ebytes / (us * 1e-6) / 1e9
        d = {"m": c["m"], "routing": c["routing"], "touched_experts": int(touched[idx]), "us_per_layer": round(us, 2), "hbm_gbs": round(gbs, 1)}
        if cold_us is not None:
            d["us_single_layer_cold"] = round(cold_us[idx], 2)
        detail.append(d)
    io = dict(h2d=int(sum(c["x"].numel() * 2 + c["ids"].numel() * 4 + c["wts"].numel() * 4 for c in cs) * n_layers),
              d2h=int(sum(c["x"].numel() * 2 for c in cs) * n_layers))
    return dict(detail=detail, step_ms=step_ms, e2e_ms=e2e_ms, e2e_direct_ms=e2e_direct_ms, step_bytes=float(touched.sum()) * ebytes * n_layers, per_case_ms=per_case_ms,
                clocks=clocks, graph=use_graph, cases=len(cs), io=io, ebytes=ebytes)


def run_ours(a):
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev, timeout=__import__("datetime").timedelta(seconds=240))   # a lost rank ends the run, it does not hang it
    from sm120fp4_b200 import synth
    from sm120fp4_b200.ep import ExpertParallelMoE, shard_range
    cfg = dict(synth.QWEN if a.shape == "qwen" else synth.GEMMA)
    only = set(a.cases.split(",")) if a.cases else None
    stream = torch.cuda.Stream()
    extras = {}
    if a.prefill_only:   # profiling helper: only the W4A4 prefill chain of two layers at the given sizes, one JSON line of its rows
        with torch.cuda.stream(stream):
            rows = prefill_numbers(cfg, build_layers(cfg, 2, dev), dev, reps=max(1, a.steps), sizes=[int(v) for v in a.prefill_only.split(",")],
                                   graph=not a.no_graph)
        print(json.dumps({"prefill": rows}))
        return
    with torch.cuda.stream(stream):
        if world == 1:
            layers = build_layers(cfg, a.layers, dev)
            eps = None
        else:   # experts sharded over the ranks: every layer call is dispatch -> local layer -> combine
            layers = build_layers(cfg, a.layers, dev, shard=shard_range(cfg["experts"], rank, world))
            ws = None
            for w in layers:   # a rank receives up to 16 rows from every peer: one W4A16 call for all of them
                w.enable_mid(max_tokens=world * MS[-1], workspace=ws, min_tokens=17)
                ws = w.mid.workspace
            eps = [ExpertParallelMoE(w.forward, cfg["experts"], cfg["top_k"], capacity=MS[-1], transport=EP_TRANSPORT) for w in layers]
        r = decode_sweep(cfg, layers, dev, a.steps, a.warmup, not a.no_graph, rank, world, dist, eps=eps, only=only)
        if world > 1:
            extras["ep_parity"] = ep_parity(cfg, eps[0], dist, world, rank, dev)
        if not a.no_extras:
            if world == 1:
                other = dict(synth.GEMMA if a.shape == "qwen" else synth.QWEN)
                extras["prefill"] = prefill_numbers(cfg, layers[:2], dev)
                extras["ep"] = ep_stack(cfg, layers, None, 1, 0, dev, stack=a.ep_layers)
                del layers[4:]
                torch.cuda.empty_cache()
                ol = build_layers(other, 8, dev)   # the second BASELINE shape: 8 distinct weight sets (larger than L2)
                ro = decode_sweep(other, ol, dev, max(2, a.steps // 4), a.warmup, not a.no_graph, 0, 1, None, e2e=False, cold=False)
                extras["cases_" + ("gemma" if a.shape == "qwen" else "qwen")] = {
                    "shape": other, "layers_in_chain": 8, "hbm_gbs": round(ro["step_bytes"] / (ro["step_ms"] * 1e-3) / 1e9, 1), "cases": ro["detail"]}
                del ol
            else:
                for w in layers:
                    w.mid = None
                extras["ep"] = ep_stack(cfg, layers, dist, world, rank, dev, stack=a.ep_layers)
    if rank != 0:
        finish(dist)
        return
    peak, peak_src = peaks()
    value = r["step_bytes"] / (r["step_ms"] * 1e-3) / 1e9
    for d in r["detail"]:
        d["frac_of_peak"] = round(d["hbm_gbs"] / world / peak, 3)
    launches = a.steps * r["cases"] * a.layers
    kernel_ms = float(r["per_case_ms"].sum()) / a.steps
    achieved = r["step_bytes"] / world / (kernel_ms * 1e-3) / 1e9
    traffic = None
    tp = ROOT / "profiles" / "decode_traffic.json"
    if tp.exists():
        traffic = json.loads(tp.read_text()).get("dram_bytes_per_launch")
    cpu = cpu_baseline(cfg, a) if (not a.no_cpu and world == 1) else None
    par = "single" if world == 1 else "expert"
    line = {
        "metric": "moe_decode_layer_hbm_gbs_on_touched_expert_bytes", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(r["step_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 weights x bf16 activations written as four nvfp4 terms (tcgen05 mxf4nvf4), fp32 accumulate (W4A16)", "data": "synthetic",
        "config": {"workload": workload_name(a.shape, cfg),
                   "layers_in_chain": a.layers, "l2": f"inputs larger than L2: each call reads one of {a.layers} distinct {r['ebytes'] * cfg['experts'] / 1e6:.0f} MB weight sets",
                   "graph_replay": r["graph"], "parallelism": par,
                   "bytes": "per case, the experts each GPU's own batch of M tokens touches x packed FP4 + scale bytes of an expert, summed over the GPUs"
                            + ("" if world == 1 else " (experts are sharded: one touched by several GPUs' batches is streamed once, by its owner; the exchanges are inside the timed region)")},
        "cases": r["detail"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": traffic if world == 1 else None, "peak_source": peak_src, "kernel": "k_moe_decode_tc" if world == 1 else "k_prefill_gemm_r<3>",
                     "bytes_per_launch": round(r["step_bytes"] / world / (r["cases"] * a.layers)), "per_gpu": world > 1},
        "e2e": {"value": round(r["step_bytes"] / (r["e2e_ms"] * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(r["e2e_ms"], 3),
                "h2d_bytes_per_step": r["io"]["h2d"] * world, "d2h_bytes_per_step": r["io"]["d2h"] * world,
                "graph_replay": bool(r["e2e_direct_ms"] and r["e2e_ms"] != r["e2e_direct_ms"]),
                "direct_launch_value": round(r["step_bytes"] / (r["e2e_direct_ms"] * 1e-3) / 1e9, 1) if r["e2e_direct_ms"] else None},
        "gpu_launches": launches * (2 if world == 1 else 12), "clocks": r["clocks"], "cpu_baseline": cpu,
    }
    line.update(extras)
    print(json.dumps(line), flush=True)
    finish(dist)


def finish(dist):
    """Leave the process group. With the peer-store transport the ranks hold mappings of one another's memory; they are
    dropped first, and all ranks leave together."""
    if dist is None:
        return
    import gc
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    if EP_TRANSPORT != "nccl":
        sys.stdout.flush()
        os._exit(0)        # the mappings are released with the process; a collective teardown after that has been seen to wait forever
    dist.destroy_process_group()


def ep_parity(cfg, ep, dist, world, rank, dev):
    """Expert-parallel output against the un-sharded layer: rank 0 also holds the full layer 0 (the same seeded weights the
    shards were cut from) and runs its own batch through it; reported as max-abs / RMS and as bit-identity from call to call."""
    from sm120fp4_b200 import synth
    res = {}
    full = build_layers(cfg, 1, dev)[0] if rank == 0 else None
    for m in (16, 1):
        x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 1000 + m + 7919 * rank)
        xd, idd, wd = x.to(dev), ids.to(dev), wts.to(dev)
        out = ep.forward(xd, idd, wd).clone()
        again = ep.forward(xd, idd, wd)
        if rank == 0:
            want = full.forward(xd, idd, wd).float()
            rms = float(want.pow(2).mean().sqrt())
            res[f"m{m}"] = {"max_abs_over_rms": round(float((out.float() - want).abs().max()) / rms, 5),
                            "bit_identical_call_to_call": bool(torch.equal(out, again))}
    if rank == 0:
        full.status()
        res["against"] = "the un-sharded layer on rank 0 (the shards' seeded weights), rank 0's batch; partial rows cross the exchange in bf16"
    return res


def prefill_numbers(cfg, layers, dev, reps=5, sizes=(256, 1024, 4096, 8192), graph=True):
    """W4A4 prefill (own tcgen05 grouped GEMM): us per layer call and TFLOP/s on 6*M*k*I*H flop at M = 256 .. 8192, CUDA-graph
    replay of the two-layer chain; with the fraction of the nominal dense FP4 peak and of the layer's HBM floor (all experts'
    packed weights once + x in + out: the bound at these sizes, see the roofline note)."""
    from sm120fp4_b200 import synth
    ws = None
    for w in layers:
        w.enable_prefill(max_tokens=8192, workspace=ws)
        ws = w.prefill.workspace
    peak_hbm, _ = peaks()
    rows = []
    ebytes = layers[0].expert_bytes()
    for m in sizes:
        x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 9000 + m)
        xd, idd, wd = x.to(dev), ids.to(dev), wts.to(dev)
        out = torch.empty_like(xd)

        def chain():
            for w in layers:
                w.forward(xd, idd, wd, out=out)
        for _ in range(2):
            chain()
        torch.cuda.synchronize()
        run, graphed = chain, False
        try:
            if graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=torch.cuda.current_stream()):
                    chain()
                run, graphed = g.replay, True
                run()
        except Exception as ex:  # noqa: BLE001
            print(f"prefill: graph capture unavailable ({type(ex).__name__}: {ex})", file=sys.stderr)
        ts = sorted(time_region(run, torch.cuda.synchronize) / len(layers) for _ in range(reps))
        t = ts[len(ts) // 2]
        flop = 6.0 * m * cfg["top_k"] * cfg["inter"] * cfg["hidden"]
        touched = int(torch.unique(ids).numel())
        floor_bytes = touched * ebytes + 2 * m * cfg["hidden"] * 2
        rows.append({"m": m, "us_per_layer": round(t * 1e3, 1), "tflops": round(flop / t / 1e9, 1), "graph_replay": graphed,
                     "roofline": {"bound": "tensor", "flop": flop, "achieved": round(flop / t / 1e9, 1), "peak": 9000.0, "unit": "TFLOP/s",
                                  "frac": round(flop / t / 1e9 / 9000.0, 4), "peak_source": "nominal dense FP4 (no measured FP4 peak on this pool)",
                                  "hbm_floor_us": round(floor_bytes / peak_hbm / 1e3, 1), "frac_of_hbm_floor": round(floor_bytes / peak_hbm / 1e3 / (t * 1e3), 4)}})
    layers[0].prefill_status()
    for w in layers:
        w.prefill = None
    return rows


def ep_stack(cfg, layers, dist, world, rank, dev, stack=48, decode_tokens=16, prefill_tokens=4096, reps=3):
    """The expert-parallel stack of 48 Qwen3-30B-A3B-shaped layers: `stack` layer calls (cycling over the resident layer
    objects, each holding E / world experts), decode with 16 tokens per GPU (fixed-capacity dispatch, no host sync) and
    prefill with 4096 tokens per GPU (variable-size dispatch, W4A4 path). Device-timed, max over ranks. Returns tokens/s and
    per-layer us."""
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
                w.enable_mid(max_tokens=world * decode_tokens, workspace=ws, min_tokens=17)
                ws = w.mid.workspace
            ws = None
        eps = [ExpertParallelMoE(w.forward, e, k, capacity=cap, transport=EP_TRANSPORT) for w in layers]
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


_HOST_EXPERTS = {}   # (shape, seed, expert) -> packed weights of that expert: drawn and quantised once per process


def host_expert(cfg, ex, seed=0):
    """One expert's weights on the host for the CPU arm: drawn like the GPU arm's (bf16 N(0, 0.02)) and quantised by the
    oracle's own quantiser. Generated lazily and kept: the sweep touches most experts, each costs a fraction of a second."""
    from oracle import nvfp4_oracle as O
    h, i = cfg["hidden"], cfg["inter"]
    key = (h, i, seed, ex)
    if key not in _HOST_EXPERTS:
        g = torch.Generator().manual_seed(seed * 1000 + ex)
        w13 = (torch.randn(2 * i, h, generator=g) * 0.02).to(torch.bfloat16).float().numpy()
        w2 = (torch.randn(h, i, generator=g) * 0.02).to(torch.bfloat16).float().numpy()
        _HOST_EXPERTS[key] = O.quantize_nvfp4(w13) + O.quantize_nvfp4(w2)
    return _HOST_EXPERTS[key]


def cpu_forward_timed(cfg, m, routing, repeats):
    """The oracle's dequantise-then-fp32-GEMM MoE forward, timed on the host cores. Weight generation and quantisation are
    outside the timed region; dequantisation is inside, as in the reference's CPU path."""
    from oracle import nvfp4_oracle as O
    from sm120fp4_b200 import synth
    x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 1000 + m if routing == "random" else 7, routing)
    touched = sorted(set(ids.reshape(-1).tolist()))
    e, h, i = cfg["experts"], cfg["hidden"], cfg["inter"]
    q1 = np.zeros((e, 2 * i, h // 2), np.uint8); s1 = np.zeros((e, 2 * i, h // 16), np.uint8); a1 = np.ones(e, np.float32)
    q2 = np.zeros((e, h, i // 2), np.uint8); s2 = np.zeros((e, h, i // 16), np.uint8); a2 = np.ones(e, np.float32)
    for ex in touched:
        p1, f1, g1, p2, f2, g2 = host_expert(cfg, ex)
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


def workload_name(shape, cfg):
    return (f"{shape}-shaped MoE layer decode sweep M in {list(MS)} x routing {list(ROUTINGS)}; E={cfg['experts']} H={cfg['hidden']} "
            f"I={cfg['inter']} top-{cfg['top_k']}")


REFERENCE_BUDGET_S = float(os.environ.get("B200MOE_REFERENCE_BUDGET_S", "120"))   # timed CPU work of the whole reference run


def run_reference(a):
    """The reference arm: the reference's CPU algorithm for this path (the oracle port; the reference itself is a PyTorch
    package that cannot travel to the GPU box) on the host cores, with all the threads numpy's BLAS takes. One step = one
    layer call for each of the ten cases of the sweep (same seeds as the GPU arm) when `steps` such steps fit the time budget
    of the run; otherwise every step takes the next few cases of the ten in turn (a bounded sample, evenly spread over the
    sweep). Dequantisation of the touched experts is inside the timed region, as in the reference's CPU path
    (sm120fp4/kernels/bench_moe_baseline.py:53-74); drawing and quantising the synthetic weights is not."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    from sm120fp4_b200 import synth
    cfg = dict(synth.QWEN if a.shape == "qwen" else synth.GEMMA)
    sweep = [(m, routing) for routing in ROUTINGS for m in MS]
    # warm-up: the smallest case once (BLAS threads, page faults); it also gives the time of one touched expert
    per_expert = None
    for _ in range(max(1, min(a.warmup, 2))):
        s, b = cpu_forward_timed(cfg, 1, "fixed8", 1)
        per_expert = s / 8
    touched_per_step = sum(8 if r == "fixed8" else min(cfg["experts"], round(cfg["experts"] * (1 - (1 - 1 / cfg["experts"]) ** (m * cfg["top_k"]))))
                           for m, r in sweep)
    full_step_s = per_expert * touched_per_step
    per_step = len(sweep)
    if full_step_s * a.steps > REFERENCE_BUDGET_S:
        per_step = max(1, min(len(sweep), int(len(sweep) * REFERENCE_BUDGET_S / (full_step_s * a.steps))))
    tot_s, tot_b, pos, ran = 0.0, 0, 0, 0
    for _ in range(a.steps):
        for _ in range(per_step):
            m, routing = sweep[pos % len(sweep)]
            pos += 1
            s, b = cpu_forward_timed(cfg, m, routing, 1)
            tot_s += s
            tot_b += b
            ran += 1
    val = tot_b / tot_s / 1e9
    what = ("one layer call for each of the ten cases of the sweep" if per_step == len(sweep)
            else f"{per_step} of the ten cases of the sweep, taken in turn ({ran} layer calls in all, {ran / len(sweep):.1f} passes over the sweep)")
    sample = f"per step: {what}; numpy/BLAS threads; dequantisation inside the timed region; {tot_s:.0f} s of timed CPU work"
    line = {"impl": "reference", "metric": "moe_decode_layer_hbm_gbs_on_touched_expert_bytes", "value": round(val, 4), "unit": "GB/s",
            "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(tot_s / a.steps * 1e3, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 on dequantised NVFP4", "data": "synthetic",
            "config": {"workload": workload_name(a.shape, cfg)},
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
    ap.add_argument("--prefill-only", default="", help="profiling helper: only the W4A4 prefill chain at these token counts, e.g. 4096")
    a = ap.parse_args()
    if a.impl == "reference":
        return run_reference(a)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    run_ours(a)


if __name__ == "__main__":
    main()
