"""ONNX weight load against the device arenas (serialize/onnx_utils.mojo:139-198 of the reference).

The reference walks `onnx_model.graph.initializer` IN ORDER and copies initializer i into parameter
symbol i of the graph (names are not used), transposing an initializer whose shape is the model
tensor's shape reversed (torch stores Gemm weights [out, in], Mantle's Linear keeps [in, out]).  It
goes through the Python `onnx` package; this module reads the protobuf wire format itself, so it has
no dependency beyond numpy.  Only FLOAT, INT32 and INT64 initializers are accepted, as there.

Wire format read here (onnx.proto3): ModelProto.graph = 7; GraphProto.initializer = 5 (repeated);
TensorProto.dims = 1, data_type = 2, float_data = 4, int32_data = 5, int64_data = 7, name = 8,
raw_data = 9 (little-endian, the form torch.onnx.export writes)."""
from __future__ import annotations

import struct
from typing import Iterator, List, Sequence, Tuple

import numpy as np

FLOAT, INT32, INT64 = 1, 6, 7
_DTYPES = {FLOAT: np.dtype("<f4"), INT32: np.dtype("<i4"), INT64: np.dtype("<i8")}


def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    result = shift = 0
    while True:
        if pos >= len(buf):
            raise ValueError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise ValueError("varint too long")


def _fields(buf: bytes) -> Iterator[Tuple[int, int, object]]:
    """Yields (field number, wire type, value); value is an int for varint / fixed fields and a
    bytes slice for length-delimited ones."""
    pos = 0
    while pos < len(buf):
        key, pos = _varint(buf, pos)
        field, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            val = struct.unpack_from("<Q", buf, pos)[0]
            pos += 8
        elif wt == 2:
            n, pos = _varint(buf, pos)
            if pos + n > len(buf):
                raise ValueError("truncated length-delimited field")
            val = buf[pos:pos + n]
            pos += n
        elif wt == 5:
            val = struct.unpack_from("<I", buf, pos)[0]
            pos += 4
        else:
            raise ValueError("unsupported protobuf wire type %d" % wt)
        yield field, wt, val


def _signed64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(val, wt) -> List[int]:
    if wt == 0:
        return [_signed64(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_signed64(v))
    return out


def _tensor(buf: bytes) -> Tuple[str, np.ndarray]:
    dims: List[int] = []
    dtype = None
    name = ""
    raw = None
    floats: List[float] = []
    ints: List[int] = []
    for field, wt, val in _fields(buf):
        if field == 1:
            dims.extend(_packed_varints(val, wt))
        elif field == 2:
            dtype = int(val)
        elif field == 4:   # float_data: packed (wire type 2) or one fixed32 per element
            if wt == 2:
                floats.extend(np.frombuffer(val, "<f4").tolist())
            else:
                floats.append(struct.unpack("<f", struct.pack("<I", val))[0])
        elif field in (5, 7):   # int32_data / int64_data as varints
            ints.extend(_packed_varints(val, wt))
        elif field == 8:
            name = bytes(val).decode("utf-8", "replace")
        elif field == 9:
            raw = bytes(val)
    if dtype not in _DTYPES:
        raise ValueError("Unsupported data type %r of initializer %r" % (dtype, name))
    n = int(np.prod(dims)) if dims else 1
    if raw is not None:
        arr = np.frombuffer(raw, _DTYPES[dtype])
    elif dtype == FLOAT:
        arr = np.asarray(floats, np.float32)
    else:
        arr = np.asarray(ints, _DTYPES[dtype])
    if arr.size != n:
        raise ValueError("initializer %r holds %d elements, its dims %s ask for %d" % (name, arr.size, dims, n))
    return name, arr.reshape(dims).copy()


def read_initializers(path) -> List[Tuple[str, np.ndarray]]:
    """(name, array) of every graph initializer of an ONNX file, in file order."""
    buf = open(path, "rb").read()
    out: List[Tuple[str, np.ndarray]] = []
    for field, wt, val in _fields(buf):
        if field == 7 and wt == 2:                      # ModelProto.graph
            for gf, gwt, gval in _fields(val):
                if gf == 5 and gwt == 2:                # GraphProto.initializer
                    out.append(_tensor(gval))
    return out


def load_onnx_weights(path, model, param_symbols: Sequence) -> List[str]:
    """Copies initializer i into parameter symbol i (`param_symbols[i]`, anything with a `.shape`) through
    `model.set_tensor(symbol, array)`; an initializer whose shape is the symbol's shape reversed is transposed
    first.  Returns a note per transposed tensor.  Raises on a shape mismatch, like the reference."""
    notes = []
    inits = read_initializers(path)
    if len(inits) > len(param_symbols):
        raise ValueError("the file holds %d initializers, the graph %d parameters" % (len(inits), len(param_symbols)))
    for i, (name, arr) in enumerate(inits):
        want = tuple(int(d) for d in param_symbols[i].shape)
        if tuple(arr.shape) != want:
            if arr.ndim == len(want) and tuple(reversed(arr.shape)) == want:
                notes.append("Transposing tensor before copying %d" % i)
                arr = arr.transpose()
            else:
                raise ValueError("Shape mismatch for tensor %d. Expected shape: %s, got shape: %s"
                                 % (i, want, tuple(arr.shape)))
        model.set_tensor(param_symbols[i], np.ascontiguousarray(arr, dtype=np.float32))
    return notes
