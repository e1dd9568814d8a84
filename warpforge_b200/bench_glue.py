"""Times the fp32 operations between the projections on prefill-sized tensors and reports each against
the HBM roofline (algorithmic bytes = one read of every input + one write of the output).

    python -m warpforge_b200.bench_glue [--rows 8192] [--n 4096] [--iters 20]

Inputs are larger than L2 (8192 x 4096 fp32 = 134 MB per tensor), device-resident, timed with events
on the launching stream after three warm-up calls.  One JSON line per operation.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import _native as N
from .backend import CudaContext

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="")
    ap.add_argument("--exact-exp", action="store_true", help="silu / swiglu / softmax with the host's (float) exp((double) x)")
    a = ap.parse_args()
    ctx = CudaContext(0)
    lib, h = ctx._lib, ctx.handle
    ctx.set_exact_exp(a.exact_exp)
    rows, n, total = a.rows, a.n, a.rows * a.n
    rng = np.random.default_rng(1)
    x = rng.standard_normal((rows, n), dtype=np.float32)
    vocab = 32000
    d_a, d_b, d_y = (ctx.allocate(total * 4) for _ in range(3))
    d_g, d_idx, d_tab = ctx.allocate(n * 4), ctx.allocate(rows * 8), ctx.allocate(vocab * n * 4)
    ctx.copy_to_device(d_a, x)
    ctx.copy_to_device(d_b, x[::-1].copy())
    ctx.copy_to_device(d_g, np.ones(n, np.float32))
    ctx.copy_to_device(d_idx, rng.integers(0, vocab, rows).astype(np.int64))
    ctx.copy_to_device(d_tab, rng.standard_normal((vocab, n), dtype=np.float32))
    t4 = total * 4
    ops = {
        "rms_norm": (lambda: lib.wf_rms_norm(h, d_a, d_g, d_y, rows, n, 1e-5, 0), 2 * t4),
        "layer_norm": (lambda: lib.wf_layer_norm(h, d_a, d_g, d_g, d_y, rows, n, 1e-5, 0), 2 * t4),
        "softmax": (lambda: lib.wf_softmax(h, d_a, d_y, rows, n, 0), 2 * t4),
        "silu": (lambda: lib.wf_silu(h, d_a, d_y, total, 0), 2 * t4),
        "swiglu": (lambda: lib.wf_swiglu(h, d_a, d_b, d_y, total, 0), 3 * t4),
        "add": (lambda: lib.wf_add(h, d_a, d_b, d_y, total, 0), 3 * t4),
        "embedding": (lambda: lib.wf_embedding(h, d_idx, d_tab, d_y, rows, vocab, n, 0), 2 * t4 + rows * 8),
    }
    peak, src = hbm_peak()
    e0, e1 = ctx.create_event(), ctx.create_event()
    for name, (call, nbytes) in ops.items():
        if a.only and name != a.only:
            continue
        for _ in range(3):
            N.check(name, call(), h)
        ctx.synchronize()
        ctx.record_event(e0)
        for _ in range(a.iters):
            N.check(name, call(), h)
        ctx.record_event(e1)
        ctx.synchronize()
        us = ctx.elapsed_ms(e0, e1) * 1e3 / a.iters
        gbs = nbytes / us / 1e3
        print(json.dumps({"op": name, "shape": [rows, n], "us": round(us, 2), "algorithmic_bytes": nbytes,
                          "achieved_gbs": round(gbs, 1), "peak_gbs": peak, "peak": src, "frac": round(gbs / peak, 3), "exact_exp": bool(a.exact_exp)}), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
