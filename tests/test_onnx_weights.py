"""ONNX weight load (serialize/onnx_utils.mojo:139-198): initializer i -> parameter i, reversed shapes are
transposed, FLOAT / INT32 / INT64 only.  The files are assembled here byte by byte from the protobuf wire
format (onnx.proto3 field numbers), in the encodings exporters use: raw_data, packed float_data, one
fixed32 per float, packed and unpacked dims, int64_data."""
import struct
from pathlib import Path

import os

import numpy as np
import pytest

import oracle
from mantle_b200 import onnx_weights as ow
from test_oracle_kat import build_cnn


def _varint(v):
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _len(field, payload):
    return _varint((field << 3) | 2) + _varint(len(payload)) + payload


def _tensor(name, arr, how):
    arr = np.asarray(arr)
    dt = {np.dtype("float32"): ow.FLOAT, np.dtype("int32"): ow.INT32, np.dtype("int64"): ow.INT64}[arr.dtype]
    body = b""
    if how.get("packed_dims"):
        body += _len(1, b"".join(_varint(d) for d in arr.shape))
    else:
        body += b"".join(_varint((1 << 3) | 0) + _varint(d) for d in arr.shape)
    body += _varint((2 << 3) | 0) + _varint(dt)
    if how["data"] == "raw":
        body += _len(9, arr.astype(arr.dtype.newbyteorder("<")).tobytes())
    elif how["data"] == "packed":
        if dt == ow.FLOAT:
            body += _len(4, arr.astype("<f4").tobytes())
        else:
            body += _len(5 if dt == ow.INT32 else 7, b"".join(_varint(int(x)) for x in arr.ravel()))
    else:  # one field per element
        for x in arr.ravel():
            if dt == ow.FLOAT:
                body += _varint((4 << 3) | 5) + struct.pack("<f", float(x))
            else:
                body += _varint(((5 if dt == ow.INT32 else 7) << 3) | 0) + _varint(int(x))
    body += _len(8, name.encode())
    return body


def write_onnx(path, tensors):
    graph = _len(1, b"node-bytes-to-skip") + b"".join(_len(5, _tensor(*t)) for t in tensors) + _len(2, b"g")
    model = _varint((1 << 3) | 0) + _varint(8) + _len(2, b"test") + _len(7, graph)
    Path(path).write_bytes(model)


def test_reader_handles_every_encoding(tmp_path):
    rng = np.random.default_rng(3)
    a = rng.normal(0, 1, (3, 4)).astype(np.float32)
    b = rng.normal(0, 1, (5,)).astype(np.float32)
    c = rng.normal(0, 1, (2, 1, 2)).astype(np.float32)
    i64 = np.array([[-3, 7], [1 << 40, 0]], np.int64)
    i32 = np.array([4, -5, 6], np.int32)
    p = tmp_path / "m.onnx"
    write_onnx(p, [("a", a, dict(data="raw", packed_dims=True)), ("b", b, dict(data="packed")),
                   ("c", c, dict(data="each")), ("i64", i64, dict(data="packed", packed_dims=True)),
                   ("i32", i32, dict(data="each"))])
    got = ow.read_initializers(p)
    assert [n for n, _ in got] == ["a", "b", "c", "i64", "i32"]
    for (_, g), w in zip(got, (a, b, c, i64, i32)):
        assert g.shape == w.shape and g.dtype == w.dtype and np.array_equal(g, w)


def test_load_in_order_with_transposition(tmp_path):
    g = oracle.Graph()
    x = g.input((2, 6))
    h = oracle.nn.Linear(g, x, 4)          # W [6, 4], b [4]
    g.out(h)
    m = oracle.Model(g)
    params = g.params()
    rng = np.random.default_rng(5)
    w_torch = rng.normal(0, 1, (4, 6)).astype(np.float32)   # torch keeps [out, in]
    bias = rng.normal(0, 1, (4,)).astype(np.float32)
    p = tmp_path / "lin.onnx"
    write_onnx(p, [("w", w_torch, dict(data="raw")), ("b", bias, dict(data="packed"))])
    notes = ow.load_onnx_weights(p, m, params)
    assert notes == ["Transposing tensor before copying 0"]
    assert np.array_equal(m.tensors[params[0].id], w_torch.T) and np.array_equal(m.tensors[params[1].id], bias)
    write_onnx(p, [("w", rng.normal(0, 1, (4, 5)).astype(np.float32), dict(data="raw"))])
    with pytest.raises(ValueError, match="Shape mismatch for tensor 0"):
        ow.load_onnx_weights(p, m, params)
    bad = _len(7, _len(5, _len(1, _varint(2)) + _varint((2 << 3) | 0) + _varint(11) + _len(9, b"\0" * 16)))  # DOUBLE
    p.write_bytes(bad)
    with pytest.raises(ValueError, match="Unsupported data type"):
        ow.read_initializers(p)


# The reference ships an exported torch CNN as examples/data/mnist_torch.onnx.  Point
# MANTLE_REFERENCE_DIR at a checkout of the reference to run the test below; without it the test is
# skipped (the byte-assembled files above cover the reader).
REF_FILE = Path(os.environ.get("MANTLE_REFERENCE_DIR", "")) / "examples" / "data" / "mnist_torch.onnx"


@pytest.mark.skipif(not REF_FILE.exists(), reason="the reference's example file is not on this machine")
def test_reference_example_file_loads_into_the_mnist_graph():
    """examples/mnist_load_model.mojo: the exported torch CNN (conv 1->16, 16->32, Linear 1568->10) fills the six
    parameters of the same graph; the Linear weight arrives [10, 1568] and is transposed."""
    inits = ow.read_initializers(REF_FILE)
    assert [a.shape for _, a in inits] == [(16, 1, 5, 5), (16,), (32, 16, 5, 5), (32,), (10, 1568), (10,)]
    g = oracle.Graph()
    build_cnn(oracle, g, 2)
    m = oracle.Model(g)
    params = g.params()
    notes = ow.load_onnx_weights(REF_FILE, m, params)
    assert notes == ["Transposing tensor before copying 4"]
    for i, (_, a) in enumerate(inits):
        assert np.array_equal(m.tensors[params[i].id], a.T if i == 4 else a)
    x = np.random.default_rng(1).uniform(0, 1, (2, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[[3, 7]]
    assert np.isfinite(m.forward(x, y))


@pytest.mark.gpu
def test_load_into_device_model(tmp_path):
    import mantle_b200 as mb
    from mantle_b200 import host_api
    ctx = mb.Context(0, mb.MATH_TF32X3)
    try:
        g = host_api.Graph()
        x = g.input((2, 6))
        g.out(host_api.nn.Linear(g, x, 4))
        m = host_api.Model(ctx, g)
        params = g.params()
        rng = np.random.default_rng(6)
        w_torch = rng.normal(0, 1, (4, 6)).astype(np.float32)
        bias = rng.normal(0, 1, (4,)).astype(np.float32)
        p = tmp_path / "lin.onnx"
        write_onnx(p, [("w", w_torch, dict(data="raw")), ("b", bias, dict(data="each"))])
        assert ow.load_onnx_weights(p, m, params) == ["Transposing tensor before copying 0"]
        assert np.array_equal(m.tensor(params[0]), w_torch.T) and np.array_equal(m.tensor(params[1]), bias)
    finally:
        ctx.close()
