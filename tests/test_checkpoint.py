"""Native checkpoint format (mantle/serialize/checkpoint.mojo): the CPU restatement against a
hand-assembled known-answer file and the reference's own round-trip cases
(tests/mojo/test_checkpoint.mojo:25-94); the device-arena implementation against the restatement,
byte for byte, and a resumed run against an uninterrupted one."""
import struct

import numpy as np
import pytest

import oracle
from test_oracle_kat import build_regression, build_cnn


def _linreg(ns, g):
    # linear_regression(4, 3, 1) of tests/mojo/test_checkpoint.mojo:12-21
    x = g.input((4, 3))
    y = g.input((4, 1))
    pred = ns.nn.Linear(g, x, 1)
    g.out(pred)
    g.loss(ns.nn.MSELoss(g, pred, y))


def _xy():
    x = (np.arange(12, dtype=np.float32) * np.float32(0.1)).reshape(4, 3)
    y = np.arange(4, dtype=np.float32).reshape(4, 1)
    return x, y


def test_known_answer_bytes(tmp_path):
    """Header and entry layout, little endian, assembled by hand from checkpoint.mojo:86-116, 222-226."""
    g = oracle.Graph()
    _linreg(oracle, g)
    m = oracle.Model(g)
    w = [s for s in g.param_syms if s.trainable][0]
    m.set_tensor(w, np.array([[1.5], [-2.0], [0.25]], np.float32))
    p = tmp_path / "ka.bin"
    oracle.checkpoint.save_checkpoint(p, m, None, iter=7)
    blob = p.read_bytes()
    syms = list(g.inputs) + list(g.param_syms) + [o for n in g.nodes for o in n.outputs]
    assert blob[:20] == struct.pack("<IIIII", 0x42534C54, 1, 7, len(syms), 0)
    assert blob[:4] == b"TLSB"          # "BSLT" packed as a little-endian u32
    # first entry: input x, symbol id of g.inputs[0], kind 0, rank 2, dims 4 3, 12 zeros
    first = struct.pack("<IBIII", g.inputs[0].id, 0, 2, 4, 3) + np.zeros(12, "<f4").tobytes()
    assert blob[20:20 + len(first)] == first
    want_w = struct.pack("<IBIII", w.id, 0, 2, 3, 1) + np.array([1.5, -2.0, 0.25], "<f4").tobytes()
    assert want_w in blob
    total = 20 + sum(9 + 4 * len(s.shape) + 4 * int(np.prod(s.shape)) for s in syms)
    assert len(blob) == total


def test_reference_round_trips(tmp_path):
    """test_save_load_checkpoint_plain / _with_optim, tests/mojo/test_checkpoint.mojo:25-94."""
    x, y = _xy()
    g = oracle.Graph()
    _linreg(oracle, g)
    m = oracle.Model(g, seed=1)
    m.forward(x, y)
    w = [s for s in g.param_syms if s.trainable][0]
    oracle.checkpoint.save_checkpoint(tmp_path / "plain.bin", m)
    m2 = oracle.Model(g, seed=2)
    it, has = oracle.checkpoint.load_checkpoint(tmp_path / "plain.bin", m2)
    assert np.array_equal(m2.tensor(w), m.tensor(w)) and not has and it == 0

    opt = oracle.Adam(m, lr=0.01)
    m.forward(x, y); opt.zero_grad(); m.backward(); opt.step()
    oracle.checkpoint.save_checkpoint(tmp_path / "optim.bin", m, opt, iter=opt.iter)
    m3 = oracle.Model(g, seed=3)
    opt3 = oracle.Adam(m3, lr=0.01)
    it, has = oracle.checkpoint.load_checkpoint(tmp_path / "optim.bin", m3, opt3)
    assert np.array_equal(m3.tensor(w), m.tensor(w))
    assert np.array_equal(opt3.m[w.id], opt.m[w.id]) and np.array_equal(opt3.v[w.id], opt.v[w.id])
    assert it == 1 and has and opt3.iter == 1
    # a plain load of a file with optimizer state skips that state (checkpoint.mojo:345-349)
    m4 = oracle.Model(g, seed=4)
    it, has = oracle.checkpoint.load_checkpoint(tmp_path / "optim.bin", m4)
    assert has and np.array_equal(m4.tensor(w), m.tensor(w))


def test_bad_files_are_rejected(tmp_path):
    p = tmp_path / "bad.bin"
    p.write_bytes(struct.pack("<IIIII", 0x12345678, 1, 0, 0, 0))
    with pytest.raises(ValueError, match="bad magic"):
        oracle.checkpoint.parse(p)
    p.write_bytes(struct.pack("<IIIII", 0x42534C54, 2, 0, 0, 0))
    with pytest.raises(ValueError, match="Unsupported checkpoint version"):
        oracle.checkpoint.parse(p)


@pytest.mark.gpu
def test_device_checkpoint_matches_restatement_and_resumes(ctx, tmp_path):
    import mantle_b200 as mb
    from mantle_b200 import host_api
    from test_models_gpu import make_pair, GpuNs
    B = 8
    build = lambda ns, gg: build_cnn(ns, gg, B)
    rng = np.random.default_rng(50)
    x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    (g, m), (og, om) = make_pair(ctx, build, seed=51)
    adam, oadam = host_api.Adam(m, lr=1e-3), oracle.Adam(om, lr=1e-3)

    def step(mm, aa):
        loss = mm.forward(x, y); aa.zero_grad(); mm.backward(); aa.step()
        return loss

    for _ in range(3):
        step(m, adam)
    # device -> file: the restatement reads back exactly the device tensors and Adam state
    p = tmp_path / "gpu.bin"
    host_api.save_checkpoint(p, m, adam, iter=3)
    it, entries, n_t, n_o = oracle.checkpoint.parse(p)
    tr = [s for s in g.params() if s.trainable]
    assert it == 3 and n_t == len(og.inputs) + len(og.param_syms) + len(og.nodes) and n_o == 2 * len(tr)
    by_id = {(sid, kind): arr for sid, kind, arr in entries}
    for s in tr:
        assert np.array_equal(by_id[(s.id, 0)], m.tensor(s))
    assert [k for _, k, _ in entries[n_t:]] == [1] * len(tr) + [2] * len(tr)
    # the same bytes as the restatement writes for a model holding the same values
    for (sid, kind, arr) in entries[:n_t]:
        om.tensors[sid] = arr.copy()
    for (sid, kind, arr) in entries[n_t:]:
        (oadam.m if kind == 1 else oadam.v)[sid] = arr.copy()
    q = tmp_path / "cpu.bin"
    oracle.checkpoint.save_checkpoint(q, om, oadam, iter=3)
    assert p.read_bytes() == q.read_bytes()

    # resume: a fresh model + optimizer loaded from the file continues exactly like the original
    want = [step(m, adam) for _ in range(3)]
    (g2, m2), _ = make_pair(ctx, build, seed=99)
    adam2 = host_api.Adam(m2, lr=1e-3)
    it, has = host_api.load_checkpoint(p, m2, adam2)
    assert it == 3 and has
    got = [step(m2, adam2) for _ in range(3)]
    assert got == want
    # plain load ignores the optimizer state; an unknown file is refused
    (g3, m3), _ = make_pair(ctx, build, seed=98)
    it, has = host_api.load_checkpoint(p, m3)
    assert has and np.array_equal(m3.tensor(tr[0]), by_id[(tr[0].id, 0)])
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"nope" * 8)
    with pytest.raises(Exception, match="bad magic"):
        host_api.load_checkpoint(bad, m3)
    # a header whose dimensions multiply to more floats than the file holds (or wrap around 2^64)
    # is refused as a corrupt file, not answered with an allocation failure
    import struct
    for dims in ((0x80000000, 0x80000000, 4), (0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF), (1 << 30,)):
        blob = struct.pack("<IIIII", 0x42534C54, 1, 0, 1, 0) + struct.pack("<IBI", tr[0].id, 0, len(dims))
        blob += b"".join(struct.pack("<I", d) for d in dims) + b"\0" * 64
        bad.write_bytes(blob)
        with pytest.raises(Exception, match="more elements than the file holds|truncated"):
            host_api.load_checkpoint(bad, m3)
