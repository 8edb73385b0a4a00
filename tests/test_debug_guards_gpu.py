"""The guard-zone mode of the allocator (MANTLE_CUDA_DEBUG=1), in a child process because the switch
is read when the library is first used.  A whole training step runs clean under it; a fill that is
told four elements too many -- it lands inside the block's own rear guard zone, memory this library
owns, so nothing faults -- is reported with the block and the distance named."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r'''
import sys
import numpy as np
sys.path.insert(0, %r)
import mantle_b200 as mb
from mantle_b200 import host_api, OP
from mantle_b200.models import GpuNs, build_cnn, cnn_weights
ctx = mb.Context(0)
g = host_api.Graph(); build_cnn(GpuNs, g, 8, 64, 128)
m = host_api.Model(ctx, g)
tr = [s for s in g.params() if s.trainable]
for s, w in zip(tr, cnn_weights([s.shape for s in tr])): m.set_tensor(s, w)
opt = host_api.Adam(m, lr=1e-3)
t = host_api.Trainer(m, opt, use_graph=True)
rng = np.random.default_rng(0)
x = rng.uniform(0, 1, (8, 1, 28, 28)).astype(np.float32); y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 8)]
for _ in range(3): t.step(x, y)
ctx.sync()                                   # verifies every guard zone
assert ctx.lib.mtl_debug_check(ctx.handle) == 0
a = ctx.zeros((100,))
ctx._check(ctx.lib.mtl_fill_f32(ctx.handle, a.ptr, 104, 1.0))   # 16 bytes into the rear guard zone
rc = ctx.lib.mtl_debug_check(ctx.handle)
msg = ctx.lib.mtl_last_error(ctx.handle).decode()
print("RC", rc, msg)
assert rc == 1 and "after" in msg and "400 bytes" in msg, msg
print("CHILD_OK")
'''


def test_guard_zones_catch_a_write_past_the_end():
    env = dict(os.environ, MANTLE_CUDA_DEBUG="1")
    r = subprocess.run([sys.executable, "-c", CHILD % str(ROOT)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "CHILD_OK" in r.stdout, (r.stdout + r.stderr)[-3000:]
