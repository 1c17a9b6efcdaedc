"""HBM streaming floor of the kernels' access patterns: the B200 counterpart of the reference's read-only streaming probe
(sm120fp4/kernels/micro_floor.py:59-95, k_stream). No math: every CTA pulls its share of a buffer through a shared-memory
ring with TMA, so the numbers are the ceiling any weight-streaming kernel with that pattern and ring depth can reach.

    python sm120-fp4_b200/micro_floor.py          # streaming out of HBM
    python sm120-fp4_b200/micro_floor.py --l2     # the same patterns on buffers that stay in L2
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

PATTERNS = [
    ("2-D box 128 B x 64 rows, pitch 1024 B, 8 stages, 1 producer", (0, 1024, 64, 0, 8, 1)),
    ("2-D box 128 B x 64 rows, pitch 1024 B, 8 stages, 4 producers", (0, 1024, 64, 0, 8, 4)),
    ("2-D box 128 B x 128 rows, pitch 1024 B, 8 stages, 2 producers", (0, 1024, 128, 0, 8, 2)),
    ("2-D box 128 B x 256 rows, pitch 1024 B, 6 stages, 2 producers", (0, 1024, 256, 0, 6, 2)),
    ("1-D bulk 16 KB, 8 stages, 1 producer", (1, 0, 0, 16384, 8, 1)),
    ("1-D bulk 8 KB, 16 stages, 4 producers", (1, 0, 0, 8192, 16, 4)),
    ("1-D bulk 64 KB, 3 stages, 1 producer", (1, 0, 0, 65536, 3, 1)),
]


def median_ms(h, L, buf, status, nbytes, args, reps=6):
    ts, off = [], 0
    for _ in range(reps):
        b = buf[off:off + nbytes]
        off = (off + nbytes) % (buf.numel() - nbytes + 1)
        off -= off % 4096
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        L.check(h.b200moe_stream_probe(L.ptr(b), nbytes, *args, L.ptr(status), L.stream_ptr()), "stream_probe")
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts = sorted(ts[1:])
    return ts[len(ts) // 2]


L2_PATTERNS = [
    ("1-D bulk 16 KB, 8 stages, 1 producer", (1, 0, 0, 16384, 8, 1)),
    ("1-D bulk 16 KB, 8 stages, 2 producers", (1, 0, 0, 16384, 8, 2)),
    ("1-D bulk 18 KB, 4 stages, 2 producers", (1, 0, 0, 18432, 4, 2)),
    ("1-D bulk 18 KB, 7 stages, 2 producers", (1, 0, 0, 18432, 7, 2)),
    ("1-D bulk 10 KB, 7 stages, 2 producers", (1, 0, 0, 10240, 7, 2)),
    ("1-D bulk 10 KB, 12 stages, 4 producers", (1, 0, 0, 10240, 12, 4)),
    ("1-D bulk 32 KB, 4 stages, 1 producer", (1, 0, 0, 32768, 4, 1)),
    ("1-D bulk 64 KB, 3 stages, 1 producer", (1, 0, 0, 65536, 3, 1)),
]


def graph_us(h, L, buf, status, nbytes, args, launches):
    """Median time of one probe launch over `nbytes` of `buf`, from CUDA-graph replays of `launches` back-to-back launches on
    the same bytes (so a buffer smaller than L2 is read out of L2 from the second launch on)."""
    b = buf[:nbytes]
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            L.check(h.b200moe_stream_probe(L.ptr(b), nbytes, *args, L.ptr(status), st.cuda_stream), "stream_probe")
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(launches):
                L.check(h.b200moe_stream_probe(L.ptr(b), nbytes, *args, L.ptr(status), st.cuda_stream), "stream_probe")
        g.replay()
        st.synchronize()
        ts = []
        for _ in range(5):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(st)
            g.replay()
            e.record(st)
            st.synchronize()
            ts.append(s.elapsed_time(e) / launches * 1e3)
    return sorted(ts)[2]


def l2_table(h, L, status) -> None:
    """The same probe on buffers that stay in L2 (18 and 36 MiB, 20 launches per graph): what the SMs can pull out of L2 with
    each copy size, ring depth and number of issuing threads - the ceiling for operands that several CTAs re-read."""
    buf = torch.empty(512 << 20, dtype=torch.uint8, device="cuda").random_(0, 255)
    print("pattern | 18 MiB us | 36 MiB us | marginal GB/s out of L2 | marginal GB/s out of HBM (216 vs 432 MiB)")
    for name, a in L2_PATTERNS:
        unit = a[3] * 148
        s1, s2 = (18 << 20) // unit * unit, (36 << 20) // unit * unit
        t1, t2 = graph_us(h, L, buf, status, s1, a, 20), graph_us(h, L, buf, status, s2, a, 20)
        b1, b2 = (216 << 20) // unit * unit, (432 << 20) // unit * unit
        u1, u2 = graph_us(h, L, buf, status, b1, a, 4), graph_us(h, L, buf, status, b2, a, 4)
        print(f"{name} | {t1:.2f} | {t2:.2f} | {(s2 - s1) / (t2 - t1) / 1e3:.0f} | {(b2 - b1) / (u2 - u1) / 1e3:.0f}")


def main() -> int:
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import sm120fp4_b200._lib as L
    h = L.lib()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if "--l2" in sys.argv[1:]:
        l2_table(h, L, status)
        return int(status.item())
    buf = torch.empty(4 << 30, dtype=torch.uint8, device="cuda").random_(0, 255)
    small, large = 216 << 20, 864 << 20
    print("pattern | 216 MiB us | 864 MiB us | marginal GB/s")
    for name, a in PATTERNS:
        unit = a[1] * a[2] if a[0] == 0 else a[3]
        t0 = median_ms(h, L, buf, status, small - small % unit, a)
        t1 = median_ms(h, L, buf, status, large - large % unit, a)
        print(f"{name} | {t0 * 1e3:.1f} | {t1 * 1e3:.1f} | {(large - small) / (t1 - t0) / 1e6:.0f}")
    return int(status.item())


if __name__ == "__main__":
    raise SystemExit(main())
