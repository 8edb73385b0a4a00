"""Writes tests/golden/cnn_wide_b96_drift.json: how far two correct implementations of the SAME
training run drift apart on the widened CNN (Conv 1->64, Conv 64->128, Linear 6272->10, Adam lr 1e-3,
batch 96, four seeded batches used in turn, 100 steps).  PyTorch on the CPU runs it three times:
in float64, in float32 with four threads and in float32 with one thread (only the order of the
sums differs between the last two).  The file holds the float64 losses and the two relative
deviation curves; tests/test_parity_full_size_gpu.py uses them as the yardstick for the
free-running comparison of the CUDA path with the CPU oracle.

    python tests/golden/make_drift_fixture.py
"""
import json
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from mantle_b200.models import cnn_batch_pool, cnn_weights  # noqa: E402

B, STEPS = 96, 100
SHAPES = [(64, 1, 5, 5), (64,), (128, 64, 5, 5), (128,), (6272, 10), (10,)]


def run(dtype, threads):
    torch.set_num_threads(threads)
    x, _, y = cnn_batch_pool(4 * B, seed=7)
    ws = [torch.tensor(w, dtype=dtype, requires_grad=True) for w in cnn_weights(SHAPES, 43)]
    opt = torch.optim.Adam(ws, lr=1e-3, eps=1e-8)
    losses = []
    for i in range(STEPS):
        lo = (i % 4) * B
        tx, ty = torch.tensor(x[lo:lo + B], dtype=dtype), torch.tensor(y[lo:lo + B], dtype=dtype)
        h = F.max_pool2d(F.relu(F.conv2d(tx, ws[0], ws[1], padding=2)), 2)
        h = F.max_pool2d(F.relu(F.conv2d(h, ws[2], ws[3], padding=2)), 2)
        loss = -(ty * F.log_softmax(h.reshape(B, -1) @ ws[4] + ws[5], dim=1)).sum() / B
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return np.array(losses)


def main():
    f64, f32a, f32b = run(torch.float64, 4), run(torch.float32, 4), run(torch.float32, 1)
    out = {"batch": B, "steps": STEPS, "lr": 1e-3, "pool_seed": 7, "weight_seed": 43, "torch": torch.__version__,
           "losses_f64": f64.tolist(),
           "drift_f32_vs_f64": (np.abs(f32a - f64) / np.abs(f64)).tolist(),
           "drift_f32_4_threads_vs_1_thread": (np.abs(f32a - f32b) / np.abs(f32b)).tolist()}
    (Path(__file__).resolve().parent / "cnn_wide_b96_drift.json").write_text(json.dumps(out, indent=1))
    for k in (9, 19, 29, 49, 74, 99):
        print("step %3d  f32 vs f64 %.2e   f32 4 threads vs 1 thread %.2e" % (k, max(out["drift_f32_vs_f64"][:k + 1]),
                                                                            max(out["drift_f32_4_threads_vs_1_thread"][:k + 1])))


if __name__ == "__main__":
    main()
