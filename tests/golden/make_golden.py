"""Generate the golden vectors under tests/golden/ by importing the reference's own CPU code.

Run once where the reference checkout is available:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path to the sm120-fp4 checkout>

It calls `sm120fp4.reference` (quantize_nvfp4 / dequantize_nvfp4), `sm120fp4.layouts` (to_128x4 / from_128x4 /
linear_to_128x4_index), the torch router of `sm120fp4/kernels/fc1_w4a16.py` and the layer oracle `reference()` of
`sm120fp4/kernels/bench_moe_baseline.py`, and stores small inputs/outputs plus SHA-256 digests of the full-size ones.
The tests never import the reference; they read these files.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def sha(t) -> str:
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return hashlib.sha256(a.tobytes()).hexdigest()


def load_synth():
    spec = importlib.util.spec_from_file_location("synth", ROOT / "sm120-fp4_b200" / "synth.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True)
    ap.add_argument("--skip-full", action="store_true", help="skip the full-size configuration-0 digests (about a minute)")
    a = ap.parse_args()
    sys.path.insert(0, str(a.reference))
    sys.dont_write_bytecode = True
    import sm120fp4
    from sm120fp4 import dequantize_nvfp4, from_128x4, linear_to_128x4_index, quantize_nvfp4, to_128x4
    from sm120fp4.reference import e2m1_decode, e2m1_encode, global_scale_for

    kdir = a.reference / "sm120fp4" / "kernels"
    mods = {}
    for name in ("bench_moe_baseline", "micro_floor", "fc1_w4a16"):
        spec = importlib.util.spec_from_file_location(name, kdir / f"{name}.py")
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        mods[name] = m
    bench, fc1 = mods["bench_moe_baseline"], mods["fc1_w4a16"]
    synth = load_synth()
    meta = {"torch": torch.__version__, "reference_version": getattr(sm120fp4, "__version__", "unknown")}

    # ---------------------------------------------------------------- E2M1 / quantizer
    out = {}
    probe = torch.tensor([0.0, -0.0, 0.25, -0.25, 0.2500001, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.0000005, 6.0, 7.0, -100.0,
                          0.24999999, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, -1e-9, 1e-30, 0.7499999, 1.7500001, 2.4999998, 3.4999998],
                         dtype=torch.float32)
    out["e2m1_probe_in"] = probe.numpy()
    out["e2m1_probe_codes"] = e2m1_encode(probe).numpy()
    out["e2m1_all_decode"] = e2m1_decode(torch.arange(16, dtype=torch.uint8)).numpy()

    def qcase(name, x, gs=None):
        q, sf, g = quantize_nvfp4(x, None if gs is None else torch.tensor([gs], dtype=torch.float32))
        out[f"q_{name}_x"] = x.float().numpy()
        out[f"q_{name}_gs_in"] = np.array([0.0 if gs is None else gs], dtype=np.float32)
        out[f"q_{name}_packed"] = q.numpy()
        out[f"q_{name}_sf"] = sf.numpy()
        out[f"q_{name}_gs"] = g.numpy()
        out[f"q_{name}_deq"] = dequantize_nvfp4(q, sf, g).numpy()

    torch.manual_seed(0)
    qcase("randn3", torch.randn(64, 256) * 3)                                    # the reference's own round-trip test input
    g = torch.Generator().manual_seed(5)
    qcase("act_gs1", torch.randn(24, 512, generator=g).to(torch.bfloat16), 1.0)   # activation quantisation, global scale 1
    qcase("act_auto", torch.randn(24, 512, generator=g).to(torch.bfloat16))
    qcase("w_small", (torch.randn(48, 256, generator=g) * 0.02).to(torch.bfloat16))
    edge = torch.zeros(8, 64)
    edge[1, :16] = -1e-9                                   # sign kept on zero, scale byte 0
    edge[2, :16] = 2.265625                                # with gs = 307.2 the scale is an exact E4M3 midpoint
    edge[3, :] = torch.linspace(-7, 7, 64)
    edge[4, 0] = 1e4                                       # saturating scale
    edge[5, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    edge[6, :] = 1e-6
    edge[7, 16:32] = 3e-3
    qcase("edge_gs307", edge, 307.2)
    qcase("edge_gs1", edge, 1.0)
    qcase("edge_auto", edge)
    big = (torch.randn(256, 2048, generator=g)).to(torch.bfloat16)
    qb, sb, gb = quantize_nvfp4(big, torch.ones(1))
    meta["q_big_gs1"] = {"recipe": "Generator(5) after the four draws above: randn(256,2048).bf16, gs=1",
                         "packed_sha256": sha(qb), "sf_sha256": sha(sb), "sf128x4_sha256": sha(to_128x4(sb))}
    out["q_big_head_packed"] = qb[:2, :64].numpy()
    out["q_big_head_sf"] = sb[:2, :8].numpy()
    np.savez_compressed(HERE / "quantize.npz", **out)

    # ---------------------------------------------------------------- layouts
    out = {}
    for rows, cols in [(128, 4), (256, 32), (100, 5), (1, 1), (129, 9), (1024, 256), (1536, 128), (2048, 48), (1408, 176), (2816, 44)]:
        gg = torch.Generator().manual_seed(rows * 1000 + cols)
        sf = torch.randint(0, 256, (rows, cols), dtype=torch.uint8, generator=gg)
        sw = to_128x4(sf)
        assert torch.equal(from_128x4(sw, rows, cols), sf)
        key = f"{rows}x{cols}"
        if rows * cols <= 4096:
            out[f"lin_{key}"] = sf.numpy()
            out[f"swz_{key}"] = sw.numpy()
            out[f"idx_{key}"] = linear_to_128x4_index(rows, cols).numpy()
        meta[f"layout_{key}"] = {"seed": rows * 1000 + cols, "lin_sha256": sha(sf), "swz_sha256": sha(sw), "shape": list(sw.shape)}
    np.savez_compressed(HERE / "layouts.npz", **out)

    # ---------------------------------------------------------------- router
    out = {}
    cases = []
    for m in (1, 2, 4, 8, 16):
        _, ids, _ = synth.decode_inputs(m, 128, 64, 8, 1000 + m, "random")
        cases.append((f"random_m{m}", ids))
        _, ids, _ = synth.decode_inputs(m, 128, 64, 8, 7, "fixed8")
        cases.append((f"fixed8_m{m}", ids))
    gg = torch.Generator().manual_seed(77)
    cases.append(("prefill_m512", torch.topk(torch.randn(512, 128, generator=gg), 8, dim=-1).indices.to(torch.int32)))
    cases.append(("skewed_m64", torch.randint(0, 3, (64, 8), generator=gg, dtype=torch.int32) * 50))
    cases.append(("e256_m33", torch.topk(torch.randn(33, 256, generator=gg), 6, dim=-1).indices.to(torch.int32)))
    for name, ids in cases:
        ex, off, pairs = fc1.route(ids)
        out[f"{name}_ids"] = ids.numpy()
        out[f"{name}_experts"] = ex.numpy()
        out[f"{name}_offsets"] = off.numpy()
        out[f"{name}_pairs"] = pairs.numpy()
    np.savez_compressed(HERE / "route.npz", **out)

    # ---------------------------------------------------------------- the layer, CPU-sized
    out = {}
    cfg = synth.TINY
    e, h, i, k = cfg["experts"], cfg["hidden"], cfg["inter"], cfg["top_k"]

    def quant_layer(w13, w2):
        q1, s1, a1, q2, s2, a2, w1d, w2d = [], [], [], [], [], [], [], []
        for ex in range(w13.shape[0]):
            q, s, gs = quantize_nvfp4(w13[ex].float())
            q1.append(q); s1.append(s); a1.append(1.0 / gs); w1d.append(dequantize_nvfp4(q, s, gs))
            q, s, gs = quantize_nvfp4(w2[ex].float())
            q2.append(q); s2.append(s); a2.append(1.0 / gs); w2d.append(dequantize_nvfp4(q, s, gs))
        return (torch.stack(q1), torch.stack(s1), torch.cat(a1), torch.stack(q2), torch.stack(s2), torch.cat(a2),
                torch.stack(w1d), torch.stack(w2d))

    w13, w2 = synth.layer_weights_bf16(e, h, i, seed=3)
    q1, s1, a1, q2, s2, a2, w1d, w2d = quant_layer(w13, w2)
    meta["tiny_layer"] = {"cfg": cfg, "seed": 3, "q1_sha256": sha(q1), "s1_sha256": sha(s1), "q2_sha256": sha(q2),
                          "s2_sha256": sha(s2), "alpha1_sha256": sha(a1), "alpha2_sha256": sha(a2)}
    out["tiny_alpha1"], out["tiny_alpha2"] = a1.numpy(), a2.numpy()
    wd = {"w1d": w1d, "w2d": w2d}
    for m, routing, seed in [(1, "random", 11), (6, "random", 12), (16, "random", 13), (5, "fixed8", 14), (40, "random", 15)]:
        x, ids, wts = synth.decode_inputs(m, e, h, k, seed, routing)
        for aq in (False, True):
            ref = bench.reference(x, wd, ids, wts, i, act_quant=aq)
            out[f"tiny_m{m}_{routing}_{'w4a4' if aq else 'w4a16'}"] = ref.numpy()
    np.savez_compressed(HERE / "layer_tiny.npz", **out)

    # ---------------------------------------------------------------- configuration 0 at full size (digests + output)
    if not a.skip_full:
        cfg = synth.QWEN
        e, h, i, k = cfg["experts"], cfg["hidden"], cfg["inter"], cfg["top_k"]
        w13, w2 = synth.layer_weights_bf16(e, h, i, seed=0)
        q1, s1, a1, q2, s2, a2, w1d, w2d = quant_layer(w13, w2)
        s1_sw = torch.stack([to_128x4(s1[x]) for x in range(e)])
        s2_sw = torch.stack([to_128x4(s2[x]) for x in range(e)])
        meta["cfg0"] = {"cfg": cfg, "seed": 0, "q1_sha256": sha(q1), "s1_sha256": sha(s1), "s1_128x4_sha256": sha(s1_sw),
                        "q2_sha256": sha(q2), "s2_sha256": sha(s2), "s2_128x4_sha256": sha(s2_sw),
                        "alpha1_sha256": sha(a1), "alpha2_sha256": sha(a2)}
        x, ids, wts = synth.decode_inputs(4, e, h, k, 100, "random")
        ref = bench.reference(x, {"w1d": w1d, "w2d": w2d}, ids, wts, i, act_quant=False)
        np.savez_compressed(HERE / "layer_cfg0.npz", out_m4=ref.numpy(), ids=ids.numpy(), wts=wts.numpy(),
                            alpha1=a1.numpy(), alpha2=a2.numpy())
        meta["cfg0"]["out_rms"] = float(ref.pow(2).mean().sqrt())

    (HERE / "golden_meta.json").write_text(json.dumps(meta, indent=1) + "\n", encoding="utf-8")
    print("golden vectors written to", HERE)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
