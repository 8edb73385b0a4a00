"""Writes tests/golden/bench_cnn_b2048_losses.json: the losses of the first 30 training steps of
the benchmark workload (widened CNN, global batch 2048, Adam lr 1e-3, seeded pool and weights of
mantle_b200.models) computed by the CPU oracle, i.e. by the restatement of the reference's own
loop forward / zero_grad / backward / step.  bench.py compares the global-mean loss of its own
first 30 steps with these at 1e-3 relative, at every GPU count.

    python tests/golden/make_bench_losses.py          # about a quarter of an hour on 8 host cores
"""
import json
import os
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from mantle_b200.models import build_cnn, cnn_batch_pool, cnn_weights  # noqa: E402

GLOBAL_BATCH, POOL, STEPS = 2048, 4096, 30


def main():
    oracle.build()
    threads = oracle.set_threads(os.cpu_count() or 1)
    g = oracle.Graph()
    build_cnn(oracle, g, GLOBAL_BATCH, 64, 128)
    m = oracle.Model(g)
    tr = [s for s in g.params() if s.trainable]
    for s, w in zip(tr, cnn_weights([s.shape for s in tr], seed=43)):
        m.set_tensor(s, w)
    opt = oracle.Adam(m, lr=1e-3)
    x, _, y = cnn_batch_pool(POOL, seed=42)
    losses = []
    t0 = time.time()
    for i in range(STEPS):
        lo = (i % (POOL // GLOBAL_BATCH)) * GLOBAL_BATCH
        losses.append(float(m.forward(x[lo:lo + GLOBAL_BATCH], y[lo:lo + GLOBAL_BATCH])))
        opt.zero_grad(); m.backward(); opt.step()
        print("step %d loss %.7f (%.0f s)" % (i, losses[-1], time.time() - t0), flush=True)
    out = {"workload": "cnn_c64_c128_fc6272_b2048", "global_batch": GLOBAL_BATCH, "pool": POOL, "lr": 1e-3,
           "pool_seed": 42, "weight_seed": 43, "steps": STEPS, "threads": threads,
           "made_by": "tests/golden/make_bench_losses.py (CPU oracle)", "losses": losses}
    (Path(__file__).resolve().parent / "bench_cnn_b2048_losses.json").write_text(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
