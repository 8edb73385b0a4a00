"""Model-level parity: the host mirror of Mantle's executor (Model.forward / backward, Adam.step)
driving the CUDA kernels, against the CPU oracle's executor and the PyTorch fixtures, on the
graphs of the reference's three example networks with identical injected weights.  Loss trajectories are held to
1e-3 relative (1e-4 for the two regression networks, as tests/python/test_models_*.mojo do)."""
import numpy as np
import pytest

import mantle_b200 as mb
import oracle
from mantle_b200 import OP, host_api
from helpers import assert_close, golden
from test_oracle_kat import TRAJ, _train, build_cnn, load_weights

pytestmark = pytest.mark.gpu


class GpuNs:
    OP = OP
    nn = host_api.nn
    Graph = host_api.Graph


def make_pair(ctx, builder, weights=None, seed=0):
    """The same graph on the GPU mirror and on the oracle, with the same parameter values."""
    g, og = host_api.Graph(), oracle.Graph()
    builder(GpuNs, g)
    builder(oracle, og)
    m, om = host_api.Model(ctx, g), oracle.Model(og)
    tr, otr = [s for s in g.params() if s.trainable], [s for s in og.params() if s.trainable]
    if weights is None:
        rng = np.random.default_rng(seed)
        weights = []
        for s in otr:
            fan_in = s.shape[0] if len(s.shape) <= 2 else int(np.prod(s.shape[1:]))
            if len(s.shape) == 1:
                fan_in = 64
            weights.append(rng.uniform(-1, 1, s.shape).astype(np.float32) / np.float32(np.sqrt(fan_in)))
    for s, os_, w in zip(tr, otr, weights):
        m.set_tensor(s, w)
        om.set_tensor(os_, w)
    return (g, m), (og, om)


@pytest.mark.parametrize("name,builder,lr,rtol,steps", TRAJ)
def test_loss_trajectories(ctx, name, builder, lr, rtol, steps):
    z = golden("models")
    n_tr = {"reg": 2}.get(name, 6)
    (g, m), (og, om) = make_pair(ctx, builder, load_weights(z, name, n_tr))
    inputs = (z[name + "__x"], z[name + "__y"])
    got = _train(m, host_api.Adam(m, lr=lr), inputs, steps)
    want = _train(om, oracle.Adam(om, lr=lr), inputs, steps)
    assert_close(got, want, rtol, 1e-6, name + " vs oracle")
    assert_close(got, z[name + "__losses"][:steps], max(rtol, 1e-3) if name.startswith("cnn") else rtol, 1e-6,
                 name + " vs torch fixture")
    # final parameters agree as well
    # final parameters agree as well (Adam's per-element normalisation amplifies rounding on
    # elements with tiny gradients, so the comparison is per tensor, in the L2 norm)
    for s, os_ in zip([s for s in g.params() if s.trainable], [s for s in og.params() if s.trainable]):
        a, b = m.tensor(s).astype(np.float64), om.tensor(os_).astype(np.float64)
        assert np.linalg.norm(a - b) <= 2e-2 * np.linalg.norm(b) + 1e-6, name + " final parameters"


def test_single_step_gradients_match_oracle(ctx):
    """One forward/backward of the CNN: every parameter gradient and the activations' gradients."""
    (g, m), (og, om) = make_pair(ctx, lambda ns, gg: build_cnn(ns, gg, 8), seed=3)
    rng = np.random.default_rng(4)
    x = rng.uniform(0, 1, (8, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 8)]
    for strict in (True, False):
        m.set_overwrite_first(not strict)
        loss, oloss = m.forward(x, y), om.forward(x, y)
        assert abs(loss - oloss) <= 1e-5 * abs(oloss) + 1e-6
        m.zero_grads(); om.zero_grads()
        m.backward(); om.backward()
        for s, os_ in zip(g.params(), og.params()):
            if s.trainable:
                assert_close(m.grad(s), om.grad(os_), 1e-4, 1e-6, "grad of param %d (strict=%s)" % (s.id, strict))
        for i in range(g.counts()["nodes"]):  # activations: outputs and their gradients
            sid = g.node(i)["output"]
            s, os_ = host_api.Symbol(g, sid), og.nodes[i].outputs[0]
            assert_close(m.tensor(s), om.tensor(os_), 1e-4, 1e-5, "output of node %d" % i)
            if s.trainable:
                assert_close(m.grad(s), om.grad(os_), 1e-4, 1e-6, "grad of node %d output" % i)


def test_accumulation_across_backward_calls_in_strict_mode(ctx):
    """Without zero_grad a second backward() adds to the gradients (ops.mojo:405,463,498)."""
    from test_oracle_kat import build_sin
    (g, m), (og, om) = make_pair(ctx, build_sin, seed=5)
    m.set_overwrite_first(False)
    rng = np.random.default_rng(6)
    x = rng.uniform(-3, 3, (32, 1)).astype(np.float32)
    y = np.sin(x)
    m.forward(x, y); om.forward(x, y)
    m.zero_grads(); om.zero_grads()
    m.backward(); om.backward()
    first = [om.grad(s) for s in og.params() if s.trainable]
    m.backward(); om.backward()
    for s, os_, f in zip([s for s in g.params() if s.trainable], [s for s in og.params() if s.trainable], first):
        assert_close(m.grad(s), om.grad(os_), 1e-4, 1e-5, "accumulated grad")
        assert not np.allclose(om.grad(os_), f) or np.allclose(f, 0)


def test_inference_outputs(ctx):
    (g, m), (og, om) = make_pair(ctx, lambda ns, gg: build_cnn(ns, gg, 4), seed=7)
    rng = np.random.default_rng(8)
    x = rng.uniform(0, 1, (4, 1, 28, 28)).astype(np.float32)
    y = np.zeros((4, 10), np.float32)
    out_sym = host_api.Symbol(g, g.node(8)["output"])  # the logits (g.out)
    got = m.inference(x, y, outputs=[out_sym])[0]
    want = om.inference(x, y)[0]
    assert got.shape == (4, 10)
    assert_close(got, want, 1e-4, 1e-5, "logits")


def test_widened_cnn_uses_tensor_cores_and_matches(ctx):
    """The widened CNN (Conv 1->64, 64->128, Linear 6272->10) at a small batch: conv2's
    forward and input gradient run on the tcgen05 implicit-GEMM kernels."""
    B = 8
    build = lambda ns, gg: build_cnn(ns, gg, B, 64, 128)
    (g, m), (og, om) = make_pair(ctx, build, seed=9)
    rng = np.random.default_rng(10)
    x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    got = _train(m, host_api.Adam(m, lr=1e-3), (x, y), 20)
    want = _train(om, oracle.Adam(om, lr=1e-3), (x, y), 20)
    assert_close(got, want, 1e-3, 1e-6, "widened CNN, 3xTF32")
    assert ctx.device_status() == 0
    # plain TF32: same trajectory within the looser tolerance
    (g2, m2), _ = make_pair(ctx, build, seed=9)
    ctx.set_math_mode(mb.MATH_TF32)
    try:
        got2 = _train(m2, host_api.Adam(m2, lr=1e-3), (x, y), 20)
    finally:
        ctx.set_math_mode(mb.MATH_TF32X3)
    assert_close(got2, want, 5e-2, 1e-4, "widened CNN, TF32")


def test_trainer_graph_replay_equals_eager(ctx):
    """The captured-and-replayed step produces the same losses as step-by-step execution."""
    B = 8
    build = lambda ns, gg: build_cnn(ns, gg, B, 64, 128)
    rng = np.random.default_rng(11)
    xs = rng.uniform(0, 1, (6, B, 1, 28, 28)).astype(np.float32)
    ys = np.eye(10, dtype=np.float32)[rng.integers(0, 10, (6, B))]
    losses = {}
    for use_graph in (False, True):
        (g, m), _ = make_pair(ctx, build, seed=12)
        adam = host_api.Adam(m, lr=1e-3)
        tr = host_api.Trainer(m, adam, use_graph=use_graph)
        losses[use_graph] = [tr.step(xs[i], ys[i]) for i in range(6)]
        assert tr.graph_active() == use_graph
        assert adam.iter == 6
        tr.close()
    assert_close(np.array(losses[True]), np.array(losses[False]), 1e-6, 1e-7, "graph vs eager")
    # and the eager trainer equals the reference's loop order forward / zero_grad / backward / step
    (g, m), (og, om) = make_pair(ctx, build, seed=12)
    oad = oracle.Adam(om, lr=1e-3)
    want = []
    for i in range(6):
        want.append(om.forward(xs[i], ys[i])); oad.zero_grad(); om.backward(); oad.step()
    assert_close(np.array(losses[False]), np.array(want, np.float32), 1e-3, 1e-6, "trainer vs oracle loop")


@pytest.mark.parametrize("strict", (False, True))
def test_chain_fusion_matches_unfused(ctx, strict):
    """CONV2D+RELU forward, MAXPOOL2D+RELU backward and the Linear layer as single launches
    (Model.set_fusion): loss trajectory, every parameter gradient and the final parameters equal the
    unfused run up to the order of a few sums (conv bias gradients, the Linear layer's slices, the rows
    of the loss); only the CONV2D / DOT outputs and the gradients of the RELU outputs are left unwritten."""
    B = 8
    build = lambda ns, gg: build_cnn(ns, gg, B, 64, 128)
    rng = np.random.default_rng(21)
    x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    runs = []
    for fuse in (False, True):
        (g, m), _ = make_pair(ctx, build, seed=20)
        m.set_overwrite_first(not strict)
        m.set_fusion(fuse)
        adam = host_api.Adam(m, lr=1e-3)
        losses = _train(m, adam, (x, y), 6)
        m.forward(x, y); m.zero_grads(); m.backward()
        grads = [m.grad(s) for s in g.params() if s.trainable]
        params = [m.tensor(s) for s in g.params() if s.trainable]
        logits = m.tensor(host_api.Symbol(g, g.node(8)["output"]))
        runs.append((losses, grads, params, logits))
    a, b = runs
    # the first loss and the first backward see identical parameters: equal up to summation order (the
    # conv bias gradients inside mtl_conv2d_bwd_fused, the rows of the loss inside mtl_cross_entropy_fwd)
    assert abs(a[0][0] - b[0][0]) <= 2e-6 * abs(a[0][0])   # the fused loss sums the rows in another order
    assert_close(np.asarray(a[0]), np.asarray(b[0]), 1e-5, 1e-7, "losses")
    # The fused Linear layer folds its k / batch slices in another order than the separate kernels: last-bit
    # differences in its gradients, which six Adam steps (a step is lr * sign for an element whose gradient
    # is tiny) turn into parameter differences of a fraction of lr = 1e-3.  The absolute part of the
    # tolerance therefore scales with the tensor's largest element.
    for u, v in zip(a[1] + a[2] + [a[3]], b[1] + b[2] + [b[3]]):
        assert_close(u, v, 2e-3, 1e-6 + 3e-3 * float(np.abs(v).max()), "fused vs unfused")
    assert ctx.device_status() == 0


def test_pipelined_steps_equal_synchronous_steps(ctx):
    """Trainer.step_async with a new batch every call (host copy of batch i + 1 staged while step i
    runs, one pinned loss word per step) gives the losses of one synchronous step() per batch."""
    import ctypes as C
    B, steps = 16, 7
    build = lambda ns, gg: build_cnn(ns, gg, B)
    rng = np.random.default_rng(31)
    xs = rng.uniform(0, 1, (steps, B, 1, 28, 28)).astype(np.float32)
    ys = np.eye(10, dtype=np.float32)[rng.integers(0, 10, (steps, B))]
    results = []
    for mode in ("sync", "async"):
        (g, m), _ = make_pair(ctx, build, seed=30)
        tr = host_api.Trainer(m, host_api.Adam(m, lr=1e-3), use_graph=True)
        if mode == "sync":
            losses = [tr.step(xs[i], ys[i]) for i in range(steps)]
        else:
            px, py, pl = C.c_void_p(), C.c_void_p(), C.c_void_p()
            ctx._check(ctx.lib.mtl_host_alloc(ctx.handle, xs.nbytes, C.byref(px)))
            ctx._check(ctx.lib.mtl_host_alloc(ctx.handle, ys.nbytes, C.byref(py)))
            ctx._check(ctx.lib.mtl_host_alloc(ctx.handle, 4 * steps, C.byref(pl)))
            C.memmove(px.value, xs.ctypes.data, xs.nbytes)
            C.memmove(py.value, ys.ctypes.data, ys.nbytes)
            for i in range(steps):
                tr.step_async_ptrs([px.value + i * xs[0].nbytes, py.value + i * ys[0].nbytes], pl.value + 4 * i)
            ctx.sync()
            losses = list(np.ctypeslib.as_array(C.cast(pl, C.POINTER(C.c_float)), (steps,)).copy())
            for p in (px, py, pl):
                ctx.lib.mtl_host_free(ctx.handle, p)
        tr.close()
        results.append(np.asarray(losses, np.float32))
    assert np.array_equal(results[0], results[1]), results
    assert results[0][0] != results[0][-1]


def test_workspace_growth_keeps_a_captured_step_valid(ctx):
    """A captured step holds the scratch pointers it was recorded with.  Asking the context for a larger
    workspace afterwards (another model, a large standalone operator) must not free that block while
    the graph is alive: the replayed step has to produce the same losses as an undisturbed run."""
    import ctypes as C
    B = 8
    build = lambda ns, gg: build_cnn(ns, gg, B, 64, 128)
    rng = np.random.default_rng(21)
    xs = rng.uniform(0, 1, (6, B, 1, 28, 28)).astype(np.float32)
    ys = np.eye(10, dtype=np.float32)[rng.integers(0, 10, (6, B))]

    def info():
        nbytes, block, live, retired = C.c_size_t(), C.c_void_p(), C.c_int32(), C.c_int32()
        ctx._check(ctx.lib.mtl_ctx_workspace_info(ctx.handle, C.byref(nbytes), C.byref(block), C.byref(live), C.byref(retired)))
        return nbytes.value, block.value, live.value, retired.value

    (g, m), _ = make_pair(ctx, build, seed=22)
    tr = host_api.Trainer(m, host_api.Adam(m, lr=1e-3), use_graph=True)
    want = [tr.step(xs[i], ys[i]) for i in range(6)]
    tr.close()

    (g, m), _ = make_pair(ctx, build, seed=22)
    tr = host_api.Trainer(m, host_api.Adam(m, lr=1e-3), use_graph=True)
    got = [tr.step(xs[i], ys[i]) for i in range(3)]
    assert tr.graph_active()
    size0, block0, live0, retired0 = info()
    assert live0 >= 1
    ctx.reserve_workspace(size0 + (64 << 20))           # forces a new, larger block
    size1, block1, live1, retired1 = info()
    assert size1 > size0 and live1 == live0 and retired1 == retired0 + 1, "the old block must be parked, not freed"
    # scribble over the NEW block through a standalone operator, then go on replaying
    a = ctx.array(rng.normal(0, 1, (512, 512)).astype(np.float32))
    c = ctx.empty((512, 512))
    ctx.forward_op(OP.DOT, c, a, a)
    got += [tr.step(xs[i], ys[i]) for i in range(3, 6)]
    assert got == want, "replay after workspace growth differs from the undisturbed run"
    tr.close()
    assert info()[3] == 0 or info()[2] > 0, "parked blocks are released with the last graph"
    assert ctx.device_status() == 0


def test_eager_and_trainer_steps_share_one_adam_counter(ctx):
    """Two eager Adam.step() calls followed by two Trainer steps (the second one replayed from the
    captured graph) must equal four steps of the reference's loop: the bias corrections 1 - beta^t
    continue at t = 3, 4 instead of starting over."""
    B = 8
    build = lambda ns, gg: build_cnn(ns, gg, B)
    rng = np.random.default_rng(31)
    x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    (g, m), (og, om) = make_pair(ctx, build, seed=32)
    adam, oadam = host_api.Adam(m, lr=1e-2), oracle.Adam(om, lr=1e-2)
    want = []
    for _ in range(5):
        want.append(om.forward(x, y)); oadam.zero_grad(); om.backward(); oadam.step()
    got = []
    for _ in range(2):
        got.append(m.forward(x, y)); adam.zero_grad(); m.backward(); adam.step()
    assert adam.iter == 2
    tr = host_api.Trainer(m, adam, use_graph=True, fuse=False)
    got += [tr.step(x, y) for _ in range(3)]
    assert adam.iter == 5
    tr.close()
    assert_close(np.array(got, np.float32), np.array(want, np.float32), 1e-4, 1e-6, "mixed eager / Trainer steps")


def test_trainer_builds_one_hot_targets_on_the_device(ctx):
    """A Trainer fed fp32 class labels (what the reference's DataLoader yields) writes the one-hot rows
    on the device; losses are bit-identical to feeding the one-hot rows examples/mnist.mojo:92-97
    builds on the host, and the step copies B floats instead of B * 10 for that input."""
    B = 16
    build = lambda ns, gg: build_cnn(ns, gg, B)
    rng = np.random.default_rng(41)
    xs = rng.uniform(0, 1, (5, B, 1, 28, 28)).astype(np.float32)
    labels = rng.integers(0, 10, (5, B)).astype(np.float32)
    losses = {}
    for on_device in (False, True):
        (g, m), _ = make_pair(ctx, build, seed=42)
        tr = host_api.Trainer(m, host_api.Adam(m, lr=1e-3), use_graph=True)
        if on_device:
            tr.set_label_input(1, 10)
            assert tr.input_bytes_per_step() == (B * 784 + B) * 4
            losses[on_device] = [tr.step(xs[i], labels[i]) for i in range(5)]
        else:
            assert tr.input_bytes_per_step() == (B * 784 + B * 10) * 4
            losses[on_device] = [tr.step(xs[i], oracle.one_hot(labels[i], 10)) for i in range(5)]
        tr.close()
    assert losses[True] == losses[False]
    (g, m), _ = make_pair(ctx, build, seed=42)
    tr = host_api.Trainer(m, host_api.Adam(m, lr=1e-3), use_graph=False)
    with pytest.raises(mb.MantleError):
        tr.set_label_input(0, 10)      # the image input is not [B, 10]
    tr.close()


def test_per_node_profile_table(ctx, tmp_path):
    """PerfMetrics (perf_utils.mojo:60-236) on device time: every node that launches kernels gets a forward
    and a backward time, the shares add up to 100 %, fused-away nodes show zero, and the report has the
    reference's columns."""
    B = 8
    (g, m), _ = make_pair(ctx, lambda ns, gg: build_cnn(ns, gg, B, 64, 128), seed=61)
    rng = np.random.default_rng(62)
    x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    n_nodes = g.counts()["nodes"]
    m.forward(x, y); m.zero_grads(); m.backward()          # unprofiled warm-up (workspace growth)
    m.set_profiling(True)
    for _ in range(3):
        m.forward(x, y); m.zero_grads(); m.backward()
    per_node, fp, bp = m.perf_metrics()
    assert fp == 3 and bp == 3 and per_node.shape == (n_nodes, 4)
    assert np.all(per_node[:, 0] > 0), "every node of the unfused graph does some forward work on the device"
    assert (per_node[:, 2] >= 3).sum() >= n_nodes - 2     # a copy node may be a plain memory copy, not a kernel
    with_bwd = [i for i in range(n_nodes) if per_node[i, 3] > 0]
    assert len(with_bwd) >= n_nodes // 2 and np.all(per_node[with_bwd, 1] > 0)
    rep = m.perf_report(True, "ms", True)
    assert "Forward pass performance metrics" in rep and "CONV2D" in rep and "Percentage [%]" in rep
    assert rep.count("\n") >= n_nodes + 4 and "Total average Forward time" in rep
    shares = [float(line.split("|")[3].replace("%", "")) for line in rep.splitlines() if line[:1].isdigit()]
    assert len(shares) == n_nodes and abs(sum(shares) - 100.0) < 0.1
    assert "Backward pass performance metrics" in m.perf_report(False, "ns", False)
    dump = tmp_path / "prof.csv"
    ctx._check(ctx.lib.mtl_prof_dump(ctx.handle, str(dump).encode()))
    lines = dump.read_text().splitlines()
    assert lines[0].startswith("tag,ranges,kernel_launches") and len(lines) >= 2 * n_nodes - 1
    # with chain fusion the nodes a fused call computes show zero and the head of the chain carries the time
    m.set_fusion(True)
    m.set_profiling(True)
    m.forward(x, y); m.zero_grads(); m.backward()
    fused, _, _ = m.perf_metrics()
    assert (fused[:, 2] == 0).sum() >= 4 and fused[0, 0] > 0
    m.set_profiling(False)
    m.close()
