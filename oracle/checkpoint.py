"""TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): CPU restatement of Mantle's native checkpoint
format, mantle/serialize/checkpoint.mojo.

    header  u32 magic 0x42534C54 ("BSLT"), u32 version 1, u32 iter, u32 n_tensors, u32 n_optim   (:222-226, :262-269)
    entry   u32 symbol id, u8 kind (0 tensor / 1 Adam momentum / 2 Adam rms), u32 rank, u32 dims[rank],
            fp32 data                                                                           (:86-116)

Tensors are written in Parameters.tensors order = allocation order (inputs, parameters, node
outputs; model.mojo:332-377), optimizer entries as all momentum tensors then all rms tensors in
get_trainable_parameters order (:281-292).  Loading matches by symbol id and skips unknown ids (:150-167).
"""
from __future__ import annotations

import struct

import numpy as np

MAGIC = 0x42534C54
VERSION = 1
KIND_NONE, KIND_MOMENTUM, KIND_RMS = 0, 1, 2


def _entry(symbol_id: int, kind: int, t: np.ndarray) -> bytes:
    t = np.ascontiguousarray(t, np.float32)
    out = struct.pack("<IBI", symbol_id, kind, t.ndim)
    out += b"".join(struct.pack("<I", d) for d in t.shape)
    return out + t.astype("<f4").tobytes()


def _allocation_order(model):
    g = model.g
    seen, order = set(), []
    for s in list(g.inputs) + list(g.param_syms) + [o for n in g.nodes for o in n.outputs]:
        if s.id not in seen:
            seen.add(s.id)
            order.append(s)
    return order


def save_checkpoint(path, model, adam=None, iter: int = 0):
    """save_checkpoint (adam None) / save_checkpoint_with_optim, checkpoint.mojo:197-300."""
    syms = _allocation_order(model)
    blob = struct.pack("<IIIII", MAGIC, VERSION, iter, len(syms), 0 if adam is None else 2 * len(adam.trainable))
    for s in syms:
        blob += _entry(s.id, KIND_NONE, model.tensors[s.id])
    if adam is not None:
        for s in adam.trainable:
            blob += _entry(s.id, KIND_MOMENTUM, adam.m[s.id])
        for s in adam.trainable:
            blob += _entry(s.id, KIND_RMS, adam.v[s.id])
    with open(path, "wb") as f:
        f.write(blob)


def parse(path):
    """All entries of a file: (iter, [(symbol id, kind, array)], n_tensors, n_optim)."""
    data = open(path, "rb").read()
    magic, version, it, n_t, n_o = struct.unpack_from("<IIIII", data, 0)
    if magic != MAGIC:
        raise ValueError("Not a mantle checkpoint file (bad magic): %s" % path)
    if version != VERSION:
        raise ValueError("Unsupported checkpoint version: %d" % version)
    off, entries = 20, []
    for _ in range(n_t + n_o):
        sid, kind, rank = struct.unpack_from("<IBI", data, off)
        off += 9
        dims = struct.unpack_from("<%dI" % rank, data, off)
        off += 4 * rank
        n = int(np.prod(dims)) if rank else 1
        entries.append((sid, kind, np.frombuffer(data, "<f4", n, off).reshape(dims).copy()))
        off += 4 * n
    return it, entries, n_t, n_o


def load_checkpoint(path, model, adam=None):
    """load_checkpoint (adam None) / load_checkpoint_with_optim, checkpoint.mojo:303-440.
    Returns (iter, has_optim_state)."""
    it, entries, n_t, n_o = parse(path)
    for sid, kind, arr in entries[:n_t]:
        if sid in model.tensors:
            model.tensors[sid] = arr.reshape(model.tensors[sid].shape).copy()
    if adam is not None:
        for sid, kind, arr in entries[n_t:]:
            dst = adam.m if kind == KIND_MOMENTUM else adam.v
            if sid in dst:
                dst[sid] = arr.reshape(dst[sid].shape).copy()
        if n_o > 0:
            adam.iter = it
    return it, n_o > 0
