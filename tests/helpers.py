"""Helpers shared by the CPU and GPU tests."""
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"

# assert_tensors_equal["almost"]: rtol = atol = 1e-5 per element, tests/testing_utils.mojo:16-27
RTOL = 1e-5
ATOL = 1e-5


def golden(name):
    return np.load(GOLDEN / (name + ".npz"))


def cases(npz, prefix):
    """Names `x` of entries `prefix_x__field`."""
    return sorted({k[len(prefix):].split("__")[0] for k in npz.files if k.startswith(prefix)})


def assert_close(a, b, rtol=RTOL, atol=ATOL, what=""):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, "%s shape %s vs %s" % (what, a.shape, b.shape)
    if not np.allclose(a, b, rtol=rtol, atol=atol, equal_nan=True):
        err = np.abs(a.astype(np.float64) - b.astype(np.float64))
        i = np.unravel_index(np.argmax(err), err.shape)
        raise AssertionError("%s mismatch: max abs err %.3e at %s (got %r, want %r), rtol %g atol %g" %
                             (what, err.max(), i, a[i], b[i], rtol, atol))
