"""Per-phase timeline of the decode layer kernel from its own cycle counters (diagnostic build only).

    python sm120-fp4_b200/build.py --diag          # libb200moe_diag.so: the product kernels + per-worker counters
    python sm120-fp4_b200/decode_timeline.py       # 8-layer chain under CUDA-graph replay, three cases of the sweep

Every worker (CTA) of `k_moe_decode_tc` records globaltimer at block start, at the end of its prologue and at exit, and
clock64 offsets of its phases; `b200moe_layer_debug_counters` copies them out after the run. Printed: when the blocks of
each layer of the chain start, begin their body and exit (first and last CTA), and for one layer in the middle of the chain
the median / extremes over the CTAs of each phase. The reference has the same kind of probe for its kernels
(sm120fp4/kernels/micro_floor.py: per-phase cycle counters of the FC2 kernel).
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
os.environ.setdefault("B200MOE_LIB", str(PKG / "libb200moe_diag.so"))
sys.path.insert(0, str(PKG.parent))

import numpy as np  # noqa: E402
import torch  # noqa: E402

PHASES = {0: "epilogue: waiting for accumulators (sum)", 1: "epilogue: FC1 SiLU*mul + expansion (sum)", 2: "epilogue: FC1 done @",
          3: "epilogue: first accumulator @", 6: "last MMA retired @", 7: "epilogue done @", 9: "producer 0: last record issued @"}


def main(layers_in_chain: int = 8) -> int:
    import bench
    from sm120fp4_b200 import _lib, synth
    if not hasattr(_lib.lib(), "b200moe_layer_debug_counters"):
        raise SystemExit("this needs the diagnostic build: python sm120-fp4_b200/build.py --diag")
    cfg = dict(synth.QWEN)
    layers = bench.build_layers(cfg, layers_in_chain, torch.device("cuda"))
    # clock64 ticks per microsecond = SM clock in MHz; these kernels run at the part's maximum SM clock (the bench samples it)
    mhz = getattr(torch.cuda.get_device_properties(0), "clock_rate", 1965000) / 1e3
    for m, routing in [(1, "fixed8"), (16, "fixed8"), (16, "random")]:
        x, ids, wts = synth.decode_inputs(m, cfg["experts"], cfg["hidden"], cfg["top_k"], 1000 + m if routing == "random" else 7, routing)
        xd, idd, wd = x.cuda(), ids.cuda(), wts.cuda()
        outs = [torch.empty_like(xd) for _ in layers]
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            for _ in range(3):
                for w, o in zip(layers, outs):
                    w.forward(xd, idd, wd, out=o)
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for w, o in zip(layers, outs):
                    w.forward(xd, idd, wd, out=o)
            for _ in range(5):
                g.replay()
            st.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(st)
            for _ in range(10):
                g.replay()
            e.record(st)
            st.synchronize()
            print(f"M={m} {routing}: {s.elapsed_time(e) * 1e3 / 10 / layers_in_chain:.1f} us per layer under graph replay")
            rows = []
            for w in layers:
                buf = (C.c_longlong * (16 * 512))()
                n = _lib.lib().b200moe_layer_debug_counters(w._h, _lib.ptr(w.workspace), buf, 256, st.cuda_stream)
                rows.append(np.array(buf[: n * 16], dtype=np.int64).reshape(n, 16)[:148])
        t0 = rows[0][:, 13].min()
        print("   layer: block start (first, last CTA) | body begin (first, last) | exit (first, last)   [us from the chain's first block start]")
        for a in rows:
            print("   " + "  ".join(f"{(v - t0) / 1e3:8.2f}" for v in (a[:, 13].min(), a[:, 13].max(), a[:, 15].min(), a[:, 15].max(),
                                                                       a[:, 14].min(), a[:, 14].max())))
        a = rows[-2]
        for i, name in PHASES.items():
            v = a[:, i] / mhz
            print(f"   {name:44s} median {np.median(v):7.2f}  max {v.max():7.2f}  min {v.min():7.2f} us after body begin")
        pro = (a[:, 15] - a[:, 13]) / 1e3
        print(f"   prologue (block start -> body begin): median {np.median(pro):.2f} max {pro.max():.2f} us; "
              f"period of the chain {(rows[-1][:, 13].min() - rows[-2][:, 13].min()) / 1e3:.2f} us")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
