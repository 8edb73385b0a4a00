"""TEST INFRASTRUCTURE ONLY (see oracle/__init__.py): CPU restatement of Mantle's layout operators.

TRANSPOSE  mantle/autograd/ops/basics.mojo:618-703   (axes None = reversed axes; backward = inverse permutation)
SLICE      mantle/autograd/ops/mlops.mojo:376-656     (adjust_boundary :378-382, result_shape :420-450, reorder_positions
           :456-478; element i of the result along an axis is start + i * step; backward stores ug at those positions
           of a zero tensor)
CONCAT     mantle/autograd/ops/dynamics.mojo:25-108   (chunks of prod(shape[:dim]) rows copied side by side)
SPLIT      mantle/autograd/ops/dynamics.mojo:111-199
Written with explicit index loops over the sliced / concatenated axis, not numpy's own slicing rules.
"""
from __future__ import annotations

import numpy as np


def transpose_fwd(t, axes=None):
    axes = tuple(range(t.ndim - 1, -1, -1)) if axes is None else tuple(axes)
    out = np.empty([t.shape[a] for a in axes], np.float32)
    for idx in np.ndindex(*out.shape):
        src = [0] * t.ndim
        for d, a in enumerate(axes):
            src[a] = idx[d]
        out[idx] = t[tuple(src)]
    return out


def transpose_bwd(ug, t_shape, axes=None):
    rank = len(t_shape)
    axes = tuple(range(rank - 1, -1, -1)) if axes is None else tuple(axes)
    inv = [0] * rank
    for i, a in enumerate(axes):
        inv[a] = i                      # create_inverse_axes, basics.mojo:676-685
    return transpose_fwd(np.asarray(ug, np.float32), inv)


def adjust_boundary(s, dim):
    v = s if s >= 0 else dim + s
    return max(min(v, dim), 0)


def slice_plan(shape, starts, ends, steps=None, axes=None):
    rank = len(shape)
    steps = [1] * len(starts) if steps is None else list(steps)
    axes = list(range(len(starts))) if axes is None else list(axes)
    start, step, out = [0] * rank, [1] * rank, list(shape)
    for i, a in enumerate(axes):
        s, e = adjust_boundary(starts[i], shape[a]), adjust_boundary(ends[i], shape[a])
        start[a], step[a], out[a] = s, steps[i], len(range(s, e, steps[i]))
    return start, step, out


def slice_fwd(t, starts, ends, steps=None, axes=None):
    start, step, out_shape = slice_plan(t.shape, starts, ends, steps, axes)
    out = np.empty(out_shape, np.float32)
    for idx in np.ndindex(*out_shape):
        out[idx] = t[tuple(start[d] + idx[d] * step[d] for d in range(t.ndim))]
    return out


def slice_bwd(ug, t_shape, starts, ends, steps=None, axes=None):
    start, step, out_shape = slice_plan(t_shape, starts, ends, steps, axes)
    res = np.zeros(t_shape, np.float32)
    ug = np.asarray(ug, np.float32).reshape(out_shape)
    for idx in np.ndindex(*out_shape):
        res[tuple(start[d] + idx[d] * step[d] for d in range(len(t_shape)))] = ug[idx]
    return res


def concat_fwd(ts, dim=0):
    n_chunks = int(np.prod(ts[0].shape[:dim], dtype=np.int64))          # calc_chunks, dynamics.mojo:42-49
    chunks = [t.size // n_chunks for t in ts]
    shape = list(ts[0].shape)
    shape[dim] = sum(t.shape[dim] for t in ts)
    out = np.empty(int(np.prod(shape)), np.float32)
    total = sum(chunks)
    for i in range(n_chunks):
        off = 0
        for t, c in zip(ts, chunks):
            out[i * total + off:i * total + off + c] = t.reshape(-1)[i * c:(i + 1) * c]
            off += c
    return out.reshape(shape)


def concat_bwd(ug, in_shapes, input_id, dim=0):
    n_chunks = int(np.prod(in_shapes[0][:dim], dtype=np.int64))
    chunks = [int(np.prod(s)) // n_chunks for s in in_shapes]
    total, off = sum(chunks), sum(chunks[:input_id])
    flat = np.asarray(ug, np.float32).reshape(-1)
    res = np.empty(int(np.prod(in_shapes[input_id])), np.float32)
    c = chunks[input_id]
    for i in range(n_chunks):
        res[i * c:(i + 1) * c] = flat[i * total + off:i * total + off + c]
    return res.reshape(in_shapes[input_id])


def split_fwd(t, sections, dim=0):
    shapes = [tuple(s if a == dim else t.shape[a] for a in range(t.ndim)) for s in sections]
    return [concat_bwd(t, shapes, j, dim) for j in range(len(sections))]


def split_bwd(ugs, in_shape, sections, dim=0):
    return concat_fwd([np.asarray(u, np.float32) for u in ugs], dim).reshape(in_shape)
