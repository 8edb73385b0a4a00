"""CPU-only checks of the drop-in boundary: libmantle_cuda.so loads and exports every symbol that
include/mantle_cuda.h declares, host-only helpers answer, and the host mirror builds the
reference's graphs (node sequences, shapes, trainable propagation).  No kernel is launched."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "mantle_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"MTL_API\s+[\w\s\*]+?\b(mtl_\w+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for need in ("mtl_dot_fwd", "mtl_dot_bwd", "mtl_conv2d_fwd", "mtl_conv2d_bwd", "mtl_maxpool2d_fwd",
                 "mtl_maxpool2d_bwd", "mtl_binary_fwd", "mtl_unary_bwd", "mtl_reduce_fwd", "mtl_adam_step",
                 "mtl_dp_allreduce_async", "mtl_graph_launch"):
        assert need in names
    assert len(names) >= 50


def test_library_exports_every_declared_symbol(built):
    import mantle_b200 as mb
    lib = C.CDLL(str(mb._lib.CUDA_LIB_PATH))
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    # the typed binding covers the same set
    assert sorted(mb._lib.SIGNATURES) == declared_symbols()
    assert mb.cuda_lib().mtl_version().decode().startswith("mantle_cuda")


def test_no_cpu_fallback(built):
    """Without a CUDA device a context cannot be created; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import mantle_b200 as mb
    with pytest.raises(mb.MantleError) as e:
        mb.Context(0)
    assert e.value.code == 2  # MTL_ERR_CUDA


def test_conv_out_shape_kat(built):
    # get_result_shape cases of tests/python/test_conv.mojo:17-64 through the C ABI's host helper
    import mantle_b200 as mb
    assert mb.conv2d_out_shape((1, 4, 28, 28), (1, 4, 1, 16), (2, 2), (1, 1), (1, 1)) == (32, 17)
    assert mb.conv2d_out_shape((1, 4, 32, 17), (1, 4, 2, 2), (0, 0), (1, 1), (1, 1)) == (31, 16)
    assert mb.conv2d_out_shape((1, 4, 32, 17), (1, 4, 2, 2), (3, 1), (1, 1), (2, 2)) == (36, 17)
    assert mb.conv2d_out_shape((1, 4, 32, 17), (1, 4, 3, 2), (3, 2), (2, 1), (2, 3)) == (17, 18)
    with pytest.raises(mb.MantleError):
        mb.conv2d_out_shape((1, 1, 2, 2), (1, 1, 5, 5))  # kernel larger than the padded input


def test_null_context_is_rejected(built):
    import mantle_b200 as mb
    lib = mb.cuda_lib()
    assert lib.mtl_sync(None) == 1  # MTL_ERR_INVALID
    assert lib.mtl_dot_fwd(None, None, None, None, 1, 1, 1) == 1
    assert lib.mtl_dp_world_size(None) == 1


def _both():
    import oracle
    from mantle_b200 import host_api
    import mantle_b200 as mb

    class GpuNs:
        OP = mb.OP
        nn = host_api.nn
        Graph = host_api.Graph

    return oracle, GpuNs


def test_host_graph_matches_reference_node_sequences(built, oracle_mod):
    from test_oracle_kat import build_cnn, build_regression, build_sin
    oracle, gpu = _both()
    OP = gpu.OP
    want = {
        "reg": [OP.DOT, OP.ADD, OP.SUB, OP.POW, OP.MEAN],
        "sin": [OP.DOT, OP.ADD, OP.RELU, OP.DOT, OP.ADD, OP.RELU, OP.DOT, OP.ADD, OP.SUB, OP.POW, OP.MEAN],
        "cnn": [OP.CONV2D, OP.RELU, OP.MAXPOOL2D, OP.CONV2D, OP.RELU, OP.MAXPOOL2D, OP.RESHAPE, OP.DOT, OP.ADD,
                OP.MAX, OP.SUB, OP.EXP, OP.SUM, OP.LOG, OP.SUB, OP.MUL, OP.SUM, OP.MUL],
    }
    for name, builder in (("reg", build_regression), ("sin", build_sin), ("cnn", build_cnn)):
        g = gpu.Graph()
        builder(gpu, g)
        og = oracle.Graph()
        builder(oracle, og)
        assert g.counts() == og.counts(), name
        ops = [g.node(i)["op"] for i in range(g.counts()["nodes"])]
        assert ops == want[name], name
        for i, n in enumerate(og.nodes):  # same symbol ids, shapes and trainable flags on both sides
            hn = g.node(i)
            assert hn["inputs"] == [s.id for s in n.inputs]
            out = host_symbol(g, hn["output"])
            assert (out.shape, out.trainable) == (n.outputs[0].shape, n.outputs[0].trainable)
        assert [(p.shape, p.trainable) for p in g.params()] == [(p.shape, p.trainable) for p in og.params()]


def host_symbol(g, sid):
    from mantle_b200.host_api import Symbol
    return Symbol(g, sid)


def test_host_graph_shape_rules(built):
    _, gpu = _both()
    OP = gpu.OP
    g = gpu.Graph()
    x = g.input((2, 3, 4))
    assert g.op(OP.SUM, x).shape == (1,)
    assert g.op(OP.MAX, x, axis=1).shape == (2, 1, 4)
    assert g.op(OP.MEAN, x, axis=2).shape == (2, 3, 1)
    assert g.op(OP.FLATTEN, x).shape == (2, 12)
    assert g.op(OP.RESHAPE, x, shape=(6, 4)).shape == (6, 4)
    assert g.op(OP.ADD, x, g.input((3, 1))).shape == (2, 3, 4)
    assert g.op(OP.UNSQUEEZE, x, dims=(0,)).shape == (1, 2, 3, 4)
    assert g.op(OP.SQUEEZE, g.input((2, 1, 3))).shape == (2, 3)
    y = g.op(OP.MUL, x, 2.0)                      # literal operand becomes a [1] constant, not trainable
    assert y.shape == (2, 3, 4) and not y.trainable
    w = g.param((4, 5))
    assert g.op(OP.DOT, g.input((7, 4)), w).trainable
    c = gpu.nn.Conv2d(g, g.input((4, 3, 32, 17)), 2, (2, 2), padding=(3, 1), stride=(2, 3), dilation=(2, 3))
    assert c.shape[:2] == (4, 2)
    p = gpu.nn.MaxPool2d(g, g.input((4, 1, 28, 28)), (2, 2))  # stride defaults to the kernel size
    assert p.shape == (4, 1, 14, 14)
    import mantle_b200 as mb
    with pytest.raises(mb.MantleError):
        g.op(OP.ADD, x, g.input((5,)))            # not broadcastable
    with pytest.raises(mb.MantleError):
        g.op(OP.DOT, g.input((2, 3)), g.input((4, 5)))
    with pytest.raises(mb.MantleError):
        g.op(23, x)                               # CONCAT: a multi-output "dynamic" node, C ABI only
    assert g.op(OP.TRANSPOSE, x).shape == (4, 3, 2)
    assert g.op(OP.TRANSPOSE, x, axes=(1, 2, 0)).shape == (3, 4, 2)
    assert g.op(OP.SLICE, x, starts=(1,), ends=(3,), steps=(1,), axes=(2,)).shape == (2, 3, 2)
    assert g.op(OP.SLICE, x, starts=(0, 2, -1), ends=(2, 0, -5), steps=(1, -1, -2)).shape == (2, 2, 2)
    with pytest.raises(mb.MantleError):
        g.op(OP.SLICE, x, starts=(3,), ends=(1,), axes=(1,))   # empty
