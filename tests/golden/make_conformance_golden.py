"""Generate tests/golden/conformance.npz by importing the reference's exact oracle (sm120fp4/oracle.py).

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_conformance_golden.py --reference <path to the sm120-fp4 checkout>

Stores NVFP4 operands of a few small GEMMs together with the reference's exact values and bounds (exact_gemm_nvfp4,
exact_gemm_bf16_nvfp4, exact_grouped_gemm_nvfp4) and its quantizer-conformance verdicts on the scale-tie example of its
selftest. tests/test_conformance_cpu.py holds oracle/conformance.py to them; the tests never import the reference.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True)
    a = ap.parse_args()
    sys.path.insert(0, str(a.reference))
    sys.dont_write_bytecode = True
    from sm120fp4 import oracle as R
    from sm120fp4.reference import e2m1_encode, pack_e2m1, quantize_nvfp4

    out = {}
    g = torch.Generator().manual_seed(20261125)
    for i, (m, n, k) in enumerate(((4, 8, 64), (16, 32, 1024), (3, 5, 4096))):
        av, bv = torch.randn(m, k, generator=g) * 3.0, torch.randn(n, k, generator=g)
        ap_, asf, ags = quantize_nvfp4(av)
        bp, bsf, bgs = quantize_nvfp4(bv)
        exact, bound = R.exact_gemm_nvfp4(ap_, asf, ags, bp, bsf, bgs, out_dtype=torch.bfloat16)
        abf = av.to(torch.bfloat16)
        e16, b16 = R.exact_gemm_bf16_nvfp4(abf, bp, bsf, bgs, out_dtype=torch.bfloat16)
        for name, t in (("ap", ap_), ("asf", asf), ("ags", ags), ("bp", bp), ("bsf", bsf), ("bgs", bgs), ("exact", exact), ("bound", bound),
                        ("a_bf16", abf.float()), ("exact16", e16), ("bound16", b16), ("a", av)):
            out[f"g{i}_{name}"] = t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()
        q = R.quantizer_conformance(av, ap_, asf, ags)
        out[f"g{i}_qconf"] = np.array([q["codes_differ"], q["scales_differ"], int(q["conformant"])])
    # grouped
    e_n, n, k = 3, 8, 256
    av = torch.randn(10, k, generator=g)
    ap_, asf, ags = quantize_nvfp4(av)
    bs = [quantize_nvfp4(torch.randn(n, k, generator=g)) for _ in range(e_n)]
    bp, bsf, bgs = torch.stack([b[0] for b in bs]), torch.stack([b[1] for b in bs]), torch.cat([b[2] for b in bs])
    indptr = torch.tensor([0, 4, 4, 10])
    ge, gb = R.exact_grouped_gemm_nvfp4(ap_, asf, ags, bp, bsf, bgs, indptr)
    for name, t in (("ap", ap_), ("asf", asf), ("ags", ags), ("bp", bp), ("bsf", bsf), ("bgs", bgs), ("indptr", indptr), ("exact", ge), ("bound", gb)):
        out[f"grp_{name}"] = t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()
    # the scale-tie example of the reference's selftest (sm120fp4/oracle.py:302-314)
    tie_x, tie_gs = torch.full((1, 16), 2.265625), torch.tensor([307.2])
    tp, tsf, _ = quantize_nvfp4(tie_x, tie_gs)
    up = tsf.clone()
    up[0, 0] = torch.tensor(120.0).to(torch.float8_e4m3fn).view(torch.uint8)
    codes_up = e2m1_encode(tie_x * (tie_gs / 120.0)).view(1, 16)
    qt = R.quantizer_conformance(tie_x, pack_e2m1(codes_up), up, tie_gs)
    off = tsf.clone()
    off[0, 0] = torch.tensor(128.0).to(torch.float8_e4m3fn).view(torch.uint8)
    qo = R.quantizer_conformance(tie_x, tp, off, tie_gs)
    out["tie_ref_sf"] = tsf.view(torch.uint8).numpy()
    out["tie_ref_packed"] = tp.numpy()
    out["tie_up_packed"] = pack_e2m1(codes_up).numpy()
    out["tie_up_verdict"] = np.array([qt["scales_differ_at_tie"], qt["scales_differ_not_at_tie"], int(qt["conformant"])])
    out["tie_off_verdict"] = np.array([qo["scales_differ_at_tie"], qo["scales_differ_not_at_tie"], int(qo["conformant"])])
    np.savez_compressed(HERE / "conformance.npz", **out)
    print("wrote", HERE / "conformance.npz", sum(v.nbytes for v in out.values()), "bytes raw")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
