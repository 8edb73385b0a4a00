"""Tiles of a partial last wave of the implicit-GEMM convolution kernel split along the reduction over two
CTAs (MANTLE_CONV_TAIL_SPLIT, read when the library is first used, hence child processes): forward, input
gradient and the fused CONV2D + RELU + MAXPOOL2D forward at shapes whose plans split, in both tensor-core
modes, against the same calls with the split switched off (the two differ by one fp32 re-association per
output, so 5e-6 of the largest value; pooling indices identical except where two window elements are that
close); two runs of the split path give identical bits.  The unsplit kernels are held to float64 elsewhere."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r'''
import sys, ctypes as C
import numpy as np
sys.path.insert(0, %r)
import mantle_b200 as mb
from mantle_b200 import OP
out_path = sys.argv[1]
ctx = mb.Context(0)
rng = np.random.default_rng(11)
res = {}
# (N, Cin, H, Kout, k, pad): the CNN's second layer at the batches of 8-, 16- and 4-way data parallelism,
# a 3x3 layer, and a layer with more than 64 input channels
CASES = ((256, 64, 14, 128, 5, 2), (128, 64, 14, 128, 5, 2), (500, 64, 14, 128, 5, 2), (40, 96, 28, 64, 3, 1))
for ci, (n, c, hw, k, r, pad) in enumerate(CASES):
    x = rng.normal(0, 1, (n, c, hw, hw)).astype(np.float32)
    w = (rng.normal(0, 1, (k, c, r, r)) * 0.05).astype(np.float32)
    b = rng.normal(0, 1, (k,)).astype(np.float32)
    ug = rng.normal(0, 1, (n, k, hw, hw)).astype(np.float32)
    dx_, dw_, db_, dug = ctx.array(x), ctx.array(w), ctx.array(b), ctx.array(ug)
    for mode, name in ((mb.MATH_TF32, "tf32"), (mb.MATH_TF32X3, "x3")):
        ctx.set_math_mode(mode)
        for rep in range(2):
            y, gx = ctx.empty((n, k, hw, hw)), ctx.empty((n, c, hw, hw))
            ctx.forward_op(OP.CONV2D, y, dx_, dw_, db_, padding=(pad, pad))
            ctx.backward_op(0, OP.CONV2D, dug, dx_, dw_, db_, grad=gx, accumulate=False, padding=(pad, pad))
            pv, pi = ctx.empty((n, k, hw // 2, hw // 2)), ctx.empty((n, k, hw // 2, hw // 2), np.int32)
            d = mb.conv_desc(n, c, hw, hw, k, r, r, (pad, pad), (1, 1), (1, 1))
            pd = mb.conv_desc(n, k, hw, hw, 1, 2, 2, (0, 0), (2, 2), (1, 1))
            ctx._check(ctx.lib.mtl_conv2d_fwd_act_pool_cl(ctx.handle, pv.ptr, pi.ptr, None, dx_.ptr, None, dw_.ptr, db_.ptr,
                                                          C.byref(d), int(OP.RELU), C.byref(pd)))
            res["%%d_%%s_y_%%d" %% (ci, name, rep)] = y.numpy()
            res["%%d_%%s_gx_%%d" %% (ci, name, rep)] = gx.numpy()
            res["%%d_%%s_pv_%%d" %% (ci, name, rep)] = pv.numpy()
            res["%%d_%%s_pi_%%d" %% (ci, name, rep)] = pi.numpy()
assert ctx.device_status() == 0
res["split_tiles"] = np.array([ctx.conv_split_tiles()])
np.savez(out_path, **res)
print("CHILD_OK")
'''


def run_child(tmp_path, split):
    out = tmp_path / ("split%d.npz" % split)
    env = dict(os.environ, MANTLE_CONV_TAIL_SPLIT=str(split))
    r = subprocess.run([sys.executable, "-c", CHILD % str(ROOT), str(out)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "CHILD_OK" in r.stdout, (r.stdout + r.stderr)[-3000:]
    return np.load(out)


def test_split_tiles_match_whole_tiles(tmp_path):
    on, off = run_child(tmp_path, 1), run_child(tmp_path, 0)
    assert int(on["split_tiles"][0]) > 0, "no plan of this test split a tile"
    assert int(off["split_tiles"][0]) == 0
    for key in off.files:
        if key == "split_tiles" or key.endswith("_1"):
            continue
        a, b = on[key], off[key]
        if "_pi_" in key:
            differ = a != b
            if differ.any():
                # a different argmax is legitimate only where the two candidates are within rounding of each other
                pv_on, pv_off = on[key.replace("_pi_", "_pv_")], off[key.replace("_pi_", "_pv_")]
                assert differ.mean() < 1e-4, (key, differ.mean())
                assert np.allclose(pv_on[differ], pv_off[differ], rtol=0, atol=4e-6 * np.abs(pv_off).max()), key
            continue
        scale = np.abs(b).max()
        assert np.max(np.abs(a - b)) <= 5e-6 * scale, (key, float(np.max(np.abs(a - b)) / scale))
        # the split path does not depend on which half arrives second
        assert np.array_equal(a, on[key[:-1] + "1"]), key
