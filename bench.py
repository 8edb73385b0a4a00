"""Benchmark of the hot path: data-parallel training of the widened MNIST-shaped CNN
(Conv 1->64 5x5 p2, ReLU, MaxPool 2x2, Conv 64->128 5x5 p2, ReLU, MaxPool 2x2, Linear 6272->10,
softmax cross-entropy, Adam lr 1e-3) at global batch 2048 on N B200s of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...   # the CPU restatement of the reference on the host cores

One "step" is one pass of the reference's training loop (examples/mnist.mojo:92-104: forward,
zero_grad, backward, Adam.step) over one global batch of seeded synthetic 28x28 images.  Rank 0
prints ONE JSON line.

What is timed.  A ROUND is exactly K (= --steps) steps bracketed by a barrier and a device
synchronisation on both sides and timed with CUDA events on the launching stream; the maximum over
ranks is the round's time.  Rounds are repeated until at least --min-seconds (2 s) of device time
have been measured, so that the GPU reaches its power-limited steady state, and the MEDIAN round is
reported (`ms_per_step` = that round's time / K).  `value` is samples/s with the batch already
resident in HBM; `e2e` is the same loop through the host mirror's public call with the batch in
pinned HOST memory: images and fp32 class labels are copied to the device every step (the one-hot
targets are built on the device) and the loss is read back every step.

Before anything is timed, the first 30 steps are checked: the mean of the ranks' losses must agree
with the losses the CPU oracle produced for the same 30 global batches
(tests/golden/bench_cnn_b2048_losses.json) at 1e-3 relative in 3xTF32 mode (measured as a second,
device-resident line) and at 5e-3 in plain TF32 mode; a run that fails a check exits non-zero.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GLOBAL_BATCH = 2048
POOL = 4096                       # synthetic samples; two global batches, alternated
FLOP_PER_SAMPLE = 246.2e6         # forward + backward of the widened CNN (algorithmic)
CONV2_FLOP_PER_SAMPLE = 80.28e6   # one of conv2's three GEMMs: 2 * 128 * 64 * 14 * 14 * 25
WORKLOAD = "cnn_c64_c128_fc6272_b2048"
LOSS_FIXTURE = ROOT / "tests" / "golden" / "bench_cnn_b2048_losses.json"
CHECK_STEPS = 30
# relative tolerance on the losses of the first 30 steps against the CPU oracle: 1e-3 in the
# fp32-faithful 3xTF32 mode; plain TF32 products are 5e-3 accurate by specification and the measured
# deviation of its loss over these steps is 1.1e-3, so that mode is held to 5e-3
LOSS_RTOL = {"tf32x3": 1e-3, "fp32": 1e-3, "tf32": 5e-3}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# ------------------------------------------------------------------ clocks -------------------

class ClockSampler:
    """nvidia-smi sampled every 50 ms while the timed rounds run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin=None, t_end=None) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, pw, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for t, ln in self.lines:
            if t_begin is not None and not (t_begin <= t <= t_end):
                continue
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w_median": statistics.median(pw) if pw else None,
                "samples": len(sm), "period_ms": 50, "reasons": sorted(reasons)}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------ CPU reference arm --------

def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def oracle_step_fn(batch):
    """The CPU restatement of the reference's training step on the same network and data, on every
    host core (the launcher's OMP_NUM_THREADS=1 for multi-process jobs is overridden)."""
    import oracle
    from mantle_b200.models import build_cnn, cnn_batch_pool, cnn_weights
    threads = oracle.set_threads(host_cores())
    g = oracle.Graph()
    build_cnn(oracle, g, batch, 64, 128)
    m = oracle.Model(g)
    tr = [s for s in g.params() if s.trainable]
    for s, w in zip(tr, cnn_weights([s.shape for s in tr])):
        m.set_tensor(s, w)
    opt = oracle.Adam(m, lr=1e-3)
    x, _, y = cnn_batch_pool(POOL)

    def step(i):
        lo = (i * batch) % (POOL - batch + 1)
        loss = m.forward(x[lo:lo + batch], y[lo:lo + batch])
        opt.zero_grad(); m.backward(); opt.step()
        return loss
    return step, threads


def sample_batch(cores):
    """The reference parallelises its convolutions over the images of a batch (conv.mojo:171,224,338):
    a sample with at least two images per core keeps every core busy."""
    return max(32, ((2 * cores + 15) // 16) * 16)


def cpu_baseline(target_seconds=15.0):
    """Bounded sample of the same workload on the host cores: samples/s of the oracle."""
    cores = host_cores()
    batch = sample_batch(cores)
    step, threads = oracle_step_fn(batch)
    t0 = time.perf_counter(); step(0); first = time.perf_counter() - t0
    n = max(2, min(20, int(target_seconds / max(first, 1e-3))))
    t0 = time.perf_counter()
    for i in range(n):
        step(i + 1)
    dt = time.perf_counter() - t0
    return {"value": n * batch / dt, "unit": "samples/s", "cores": threads, "kind": "port",
            "sample": "%d steps at batch %d of the same network (oracle/, OpenMP over %d host threads)" % (n, batch, threads)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_cores()
    batch = sample_batch(cores)
    step, threads = oracle_step_fn(batch)
    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i)
    dt = time.perf_counter() - t0
    v = args.steps * batch / dt
    sample = "%d steps at batch %d per step (bounded sample of the 2048-sample step), %d OpenMP threads" % (args.steps, batch, threads)
    print(json.dumps({
        "impl": "reference", "metric": "cnn_train_samples_per_s", "value": v, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "sample_batch": batch, "threads": threads,
                   "note": "CPU restatement of Mantle's Mojo kernels (the Mojo toolchain is not installable here)"},
        "cpu_baseline": {"value": v, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ standalone operators -----

def op_sweep(ctx, pk, iters=5):
    """OP.DOT (square), OP.CONV2D on [256, 64, 56, 56] with a 3x3 kernel and MAXPOOL2D 2x2 on
    [256, 64, 112, 112], forward and backward, in plain TF32 and 3xTF32, each call timed alone with
    CUDA events after a 256 MB device fill (larger than the 126 MB L2), median of `iters` calls.
    Rates are ALGORITHMIC (2 M N K flop; tensor bytes read + written once); fractions are of the
    measured burst peaks (a kernel timed alone): TF32 = bf16 burst / 2, HBM copy."""
    import mantle_b200 as mb
    from mantle_b200 import OP
    rng = np.random.default_rng(0)
    flush = ctx.empty((64 * 1024 * 1024,))
    tf32_peak, hbm_peak = pk["bf16_burst"] / 2.0, pk["hbm_gbs"]
    out = {"peak_tf32_tflops": tf32_peak, "peak_hbm_gbs": hbm_peak, "peak_source": pk["source"] + " burst", "rows": []}

    def timed(fn):
        fn(); fn()
        ctx.sync()
        ms = []
        for _ in range(iters):
            flush.zero()
            ctx.timer_start(2)
            fn()
            ctx.timer_stop(2)
            ms.append(ctx.timer_ms(2))
        return statistics.median(ms)

    def tensor_row(name, mode, flop, fn):
        ms = timed(fn)
        tf = flop / ms / 1e9
        out["rows"].append({"op": name, "math": mode, "ms": round(ms, 4), "tflops": round(tf, 1), "frac": round(tf / tf32_peak, 3)})

    def hbm_row(name, mode, nbytes, fn):
        ms = timed(fn)
        gbs = nbytes / ms / 1e6
        out["rows"].append({"op": name, "math": mode, "ms": round(ms, 4), "gbs": round(gbs, 0), "frac": round(gbs / hbm_peak, 3)})

    modes = (("tf32", mb.MATH_TF32), ("tf32x3", mb.MATH_TF32X3))
    for s in (1024, 2048, 4096, 8192):
        a = ctx.array(rng.normal(0, 1, (s, s)).astype(np.float32))
        b = ctx.array(rng.normal(0, 1, (s, s)).astype(np.float32))
        ug = ctx.array(rng.normal(0, 1, (s, s)).astype(np.float32))
        c = ctx.empty((s, s))
        for mname, mode in modes:
            ctx.set_math_mode(mode)
            tensor_row("DOT %d fwd" % s, mname, 2.0 * s ** 3, lambda: ctx.forward_op(OP.DOT, c, a, b))
            tensor_row("DOT %d bwd A" % s, mname, 2.0 * s ** 3, lambda: ctx.backward_op(0, OP.DOT, ug, a, b, grad=c, accumulate=False))
            tensor_row("DOT %d bwd B" % s, mname, 2.0 * s ** 3, lambda: ctx.backward_op(1, OP.DOT, ug, a, b, grad=c, accumulate=False))
        for t in (a, b, c, ug):
            t.free()

    N, Cc, K, H, R = 256, 64, 64, 56, 3
    kw = dict(padding=(1, 1))
    x = ctx.array(rng.normal(0, 1, (N, Cc, H, H)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, Cc, R, R)) / 24.0).astype(np.float32))
    bias = ctx.array(np.zeros(K, np.float32))
    ug = ctx.array(rng.normal(0, 1, (N, K, H, H)).astype(np.float32))
    y, dx, dw, db = ctx.empty((N, K, H, H)), ctx.empty((N, Cc, H, H)), ctx.empty((K, Cc, R, R)), ctx.empty((K,))
    fl = 2.0 * N * K * Cc * H * H * R * R
    for mname, mode in modes:
        ctx.set_math_mode(mode)
        tensor_row("CONV2D 256x64x56x56 k3 fwd", mname, fl, lambda: ctx.forward_op(OP.CONV2D, y, x, w, bias, **kw))
        tensor_row("CONV2D bwd input", mname, fl, lambda: ctx.backward_op(0, OP.CONV2D, ug, x, w, bias, grad=dx, accumulate=False, **kw))
        tensor_row("CONV2D bwd kernel", mname, fl, lambda: ctx.backward_op(1, OP.CONV2D, ug, x, w, bias, grad=dw, accumulate=False, **kw))
    hbm_row("CONV2D bwd bias", "f32", N * K * H * H * 4,
            lambda: ctx.backward_op(2, OP.CONV2D, ug, x, w, bias, grad=db, accumulate=False, **kw))
    for t in (x, w, bias, ug, y, dx, dw, db):
        t.free()

    N, Cc, H = 256, 64, 112
    pkw = dict(kernel_size=(2, 2))
    x = ctx.array(rng.normal(0, 1, (N, Cc, H, H)).astype(np.float32))
    y, idx = ctx.empty((N, Cc, H // 2, H // 2)), ctx.empty((N, Cc, H // 2, H // 2), np.int32)
    ug, dx = ctx.array(rng.normal(0, 1, (N, Cc, H // 2, H // 2)).astype(np.float32)), ctx.empty((N, Cc, H, H))
    n_in, n_out = N * Cc * H * H, N * Cc * H * H // 4
    hbm_row("MAXPOOL2D 256x64x112x112 fwd (+indices)", "f32", (n_in + 2 * n_out) * 4,
            lambda: ctx.forward_op(OP.MAXPOOL2D, y, x, indices=idx, **pkw))
    hbm_row("MAXPOOL2D bwd (from indices)", "f32", (n_in + 2 * n_out) * 4,
            lambda: ctx.backward_op(0, OP.MAXPOOL2D, ug, x, grad=dx, accumulate=False, indices=idx, **pkw))
    hbm_row("MAXPOOL2D bwd (reference form, re-scans X)", "f32", (2 * n_in + n_out) * 4,
            lambda: ctx.backward_op(0, OP.MAXPOOL2D, ug, x, grad=dx, accumulate=False, **pkw))
    for t in (x, y, idx, ug, dx, flush):
        t.free()
    ctx.set_math_mode(mb.MATH_TF32)
    return out


# ------------------------------------------------------------------ GPU arm ------------------

def run_ours(args):
    import mantle_b200 as mb
    from mantle_b200 import host_api
    from mantle_b200.models import GpuNs, build_cnn, cnn_batch_pool, cnn_weights

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    dist = None
    if world > 1:
        # the collective library's banner and debug lines must not reach stdout: rank 0 prints
        # exactly one JSON line there
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)  # control plane only

    mode = {"tf32": mb.MATH_TF32, "tf32x3": mb.MATH_TF32X3, "fp32": mb.MATH_FP32}[args.math]
    ctx = mb.Context(local, mode)
    lib = ctx.lib
    if world > 1:
        import torch
        idbuf = torch.zeros(mb._lib.MTL_DP_ID_BYTES, dtype=torch.uint8)
        if rank == 0:
            raw = (C.c_uint8 * mb._lib.MTL_DP_ID_BYTES)()
            assert lib.mtl_dp_get_unique_id(raw) == 0, "NCCL is not loadable"
            idbuf = torch.tensor(list(raw), dtype=torch.uint8)
        dist.broadcast(idbuf, 0)
        raw = (C.c_uint8 * mb._lib.MTL_DP_ID_BYTES)(*idbuf.tolist())
        # NCCL prints its version banner on file descriptor 1 while the communicator is created
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            ctx._check(lib.mtl_dp_init(ctx.handle, raw, rank, world))
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    B = GLOBAL_BATCH // world
    K = args.steps

    g = host_api.Graph()
    build_cnn(GpuNs, g, B, 64, 128)
    model = host_api.Model(ctx, g)
    tr = [s for s in g.params() if s.trainable]
    for s, w in zip(tr, cnn_weights([s.shape for s in tr])):
        model.set_tensor(s, w)
    adam = host_api.Adam(model, lr=1e-3)
    trainer = host_api.Trainer(model, adam, use_graph=not args.no_graph, bucket_bytes=args.bucket_kb * 1024)
    trainer.set_label_input(1, 10)      # targets travel as B fp32 labels; one-hot rows are built on the device

    # synthetic pool in pinned host memory: images and fp32 class labels
    x, labels, _ = cnn_batch_pool(POOL, one_hot=False)
    px, py = C.c_void_p(), C.c_void_p()
    ctx._check(lib.mtl_host_alloc(ctx.handle, x.nbytes, C.byref(px)))
    ctx._check(lib.mtl_host_alloc(ctx.handle, labels.nbytes, C.byref(py)))
    C.memmove(px.value, x.ctypes.data, x.nbytes)
    C.memmove(py.value, labels.ctypes.data, labels.nbytes)
    ploss = C.c_void_p()
    ctx._check(lib.mtl_host_alloc(ctx.handle, 4096, C.byref(ploss)))
    loss_view = np.ctypeslib.as_array(C.cast(ploss, C.POINTER(C.c_float)), (1024,))

    def batch_ptrs(step):
        row = (step % (POOL // GLOBAL_BATCH)) * GLOBAL_BATCH + rank * B
        return [px.value + row * 784 * 4, py.value + row * 4]

    h2d_bytes = trainer.input_bytes_per_step()
    assert h2d_bytes == B * (784 + 1) * 4

    def barrier():
        ctx.sync()
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.synchronize()
        except Exception:
            pass
        if dist is not None:
            dist.barrier()

    def reduce_ranks(values, op):
        if dist is None:
            return list(values)
        import torch
        t = torch.tensor(list(values), dtype=torch.float64)
        dist.all_reduce(t, op={"max": dist.ReduceOp.MAX, "sum": dist.ReduceOp.SUM}[op])
        return t.tolist()

    # ---- the first 30 steps against the CPU oracle's losses (also the warm-up) -------------------
    for i in range(CHECK_STEPS):
        trainer.step_async_ptrs(batch_ptrs(i), ploss.value + 4 * i)
    ctx.sync()
    mean_losses = [v / world for v in reduce_ranks([float(v) for v in loss_view[:CHECK_STEPS]], "sum")]
    rtol = LOSS_RTOL[args.math]
    loss_check = {"steps": CHECK_STEPS, "rtol": rtol, "reference": "CPU oracle, " + LOSS_FIXTURE.name}
    if GLOBAL_BATCH == 2048 and LOSS_FIXTURE.exists():
        want = json.loads(LOSS_FIXTURE.read_text())["losses"][:CHECK_STEPS]
        dev = [abs(a - b) / abs(b) for a, b in zip(mean_losses, want)]
        loss_check.update({"max_rel_dev": max(dev), "ok": max(dev) <= rtol, "loss_step_29": mean_losses[-1],
                           "oracle_step_29": want[-1]})
        if not loss_check["ok"] and not args.no_loss_check:
            raise SystemExit("loss check failed: global-mean loss deviates from the CPU oracle's by %.3e (> %.0e) within "
                             "the first %d steps: %r vs %r" % (max(dev), rtol, CHECK_STEPS, mean_losses, want))
    else:
        loss_check.update({"ok": None, "note": "no oracle losses for this configuration"})
    for i in range(args.warmup):
        trainer.step_async_ptrs(batch_ptrs(CHECK_STEPS + i), ploss.value)
    step_no = CHECK_STEPS + args.warmup

    def timed_rounds(fn_step, slot):
        """Rounds of exactly K steps until --min-seconds of device time; returns per-round ms (max over ranks)."""
        rounds, total, n_max = [], 0.0, 100000
        while True:
            barrier()
            ctx.timer_start(slot)
            for i in range(K):
                fn_step(i)
            ctx.timer_stop(slot)
            ms = ctx.timer_ms(slot)
            barrier()
            ms = reduce_ranks([ms], "max")[0]     # every rank sees the same number, so all stop together
            rounds.append(ms)
            total += ms
            if (total >= args.min_seconds * 1e3 and len(rounds) >= 3) or len(rounds) >= n_max:
                return rounds

    # ---- end to end: pinned host batch -> device every step, loss -> host every step ----------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    time.sleep(0.1)
    launches0 = ctx.launch_count()
    t_begin = time.perf_counter()

    # Trainer.step_async: every step copies its batch from pinned host memory (copy stream, two
    # staging buffers) and writes its loss to its own pinned word; the host only waits at the end
    # of a round, so the copy of batch i + 1 overlaps the kernels of step i
    def e2e_step(i):
        nonlocal step_no
        trainer.step_async_ptrs(batch_ptrs(step_no), ploss.value + 4 * (i % 1024))
        step_no += 1
    e2e_rounds = timed_rounds(e2e_step, 0)
    launches_per_round = (ctx.launch_count() - launches0) // len(e2e_rounds)

    # ---- device resident: the same captured step, batch already in HBM -------------------------
    def dev_step(i):
        trainer.step_async_ptrs([], ploss.value)
    dev_rounds = timed_rounds(dev_step, 1)
    t_end = time.perf_counter()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    final_loss = reduce_ranks([float(loss_view[0])], "sum")[0] / world
    e2e_ms, dev_ms = statistics.median(e2e_rounds), statistics.median(dev_rounds)

    # ---- data parallel: the same step without the gradient exchange (a timing diagnostic, not training):
    # the difference to the full step is the part of the communication that the backward pass does not hide
    compute_only_ms = None
    trainer.close()
    if world > 1:
        trainer_c = host_api.Trainer(model, adam, use_graph=not args.no_graph, bucket_bytes=args.bucket_kb * 1024)
        trainer_c.set_label_input(1, 10)
        trainer_c.set_exchange(False)
        for i in range(3):
            trainer_c.step_async_ptrs(batch_ptrs(i), ploss.value)
        saved = args.min_seconds
        args.min_seconds = min(saved, 0.5)
        compute_only_ms = statistics.median(timed_rounds(lambda i: trainer_c.step_async_ptrs([], ploss.value), 4)) / K
        args.min_seconds = saved
        trainer_c.close()

    # ---- per-kernel durations of the dominant kernels, live, while the GPU is still hot: eager
    # steps with CUDA-event brackets on the launching stream around each tensor-core launch
    prof_trainer = host_api.Trainer(model, adam, use_graph=False)
    prof_trainer.set_label_input(1, 10)
    ctx._check(lib.mtl_prof_reset(ctx.handle))
    ctx._check(lib.mtl_prof_enable(ctx.handle, 1))
    prof_steps = 40
    for i in range(prof_steps):
        prof_trainer.step_async_ptrs(batch_ptrs(i), ploss.value)
    ctx.sync()
    ctx._check(lib.mtl_prof_enable(ctx.handle, 0))
    kern = {}
    for name, kid in (("dot_tc", 0), ("conv_igemm", 1), ("conv_wgrad", 2), ("conv_first", 3)):
        ms, n = C.c_float(), C.c_int32()
        ctx._check(lib.mtl_prof_get(ctx.handle, kid, C.byref(ms), C.byref(n)))
        kern[name] = {"launches": n.value, "avg_ms": (ms.value / n.value) if n.value else None}
    prof_trainer.close()

    # ---- the same step in 3xTF32 (the fp32-faithful mode), device resident, for the second line ----
    other = None
    if args.math == "tf32" and not args.no_x3:
        ctx.set_math_mode(mb.MATH_TF32X3)
        model3 = host_api.Model(ctx, g)
        for s_, w in zip(tr, cnn_weights([s_.shape for s_ in tr])):
            model3.set_tensor(s_, w)
        adam3 = host_api.Adam(model3, lr=1e-3)
        trainer3 = host_api.Trainer(model3, adam3, use_graph=not args.no_graph)
        trainer3.set_label_input(1, 10)
        for i in range(CHECK_STEPS):
            trainer3.step_async_ptrs(batch_ptrs(i), ploss.value + 4 * i)
        ctx.sync()
        x3_losses = [v / world for v in reduce_ranks([float(v) for v in loss_view[:CHECK_STEPS]], "sum")]
        saved_min = args.min_seconds
        args.min_seconds = min(args.min_seconds, 1.0)
        x3_rounds = timed_rounds(lambda i: trainer3.step_async_ptrs([], ploss.value), 3)
        args.min_seconds = saved_min
        x3_ms = statistics.median(x3_rounds)
        other = {"dtype": "tf32x3", "value": K * GLOBAL_BATCH / (x3_ms * 1e-3), "unit": "samples/s", "ms_per_step": x3_ms / K,
                 "rounds": len(x3_rounds)}
        if loss_check.get("ok") is not None:
            want = json.loads(LOSS_FIXTURE.read_text())["losses"][:CHECK_STEPS]
            other["loss_check"] = {"rtol": LOSS_RTOL["tf32x3"], "max_rel_dev": max(abs(a - b) / abs(b) for a, b in zip(x3_losses, want))}
            other["loss_check"]["ok"] = other["loss_check"]["max_rel_dev"] <= LOSS_RTOL["tf32x3"]
            if not other["loss_check"]["ok"] and not args.no_loss_check:
                raise SystemExit("loss check failed in 3xTF32 mode: %r vs %r" % (x3_losses, want))
        trainer3.close(); adam3.close(); model3.close()
        ctx.set_math_mode(mode)
    status = ctx.device_status()

    if rank == 0:
        pk = peaks()
        region_s = (sum(e2e_rounds) + sum(dev_rounds)) / 1e3
        # a kernel timed inside seconds of back-to-back steps is held against the sustained peak
        tf32_peak = pk["bf16_sustained"] / 2.0   # TF32 tensor rate is half the bf16 rate
        flops_per_launch = CONV2_FLOP_PER_SAMPLE * B
        ig = kern["conv_igemm"]
        achieved = flops_per_launch / (ig["avg_ms"] * 1e-3) / 1e12 if ig["avg_ms"] else None
        out = {
            "metric": "cnn_train_samples_per_s", "value": K * GLOBAL_BATCH / (dev_ms * 1e-3),
            "unit": "samples/s", "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"tf32": "tf32", "tf32x3": "tf32x3", "fp32": "f32"}[args.math], "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_gpu_batch": B, "parallelism": "dp%d" % world,
                       "math_mode": args.math, "cuda_graph": not args.no_graph,
                       "timing": "median of %d (device-resident) / %d (e2e) rounds of %d steps, %.2f s of device time in all; "
                                 "%d checked + %d more warm-up steps before" % (len(dev_rounds), len(e2e_rounds), K, region_s,
                                                                               CHECK_STEPS, args.warmup),
                       "l2": "per-step working set (>= 0.4 GB of activations per GPU at N<=4) exceeds the 126 MB L2; "
                             "a fresh batch every step in the e2e rounds"},
            "rounds": {"device_ms": {"n": len(dev_rounds), "min": min(dev_rounds), "median": dev_ms, "max": max(dev_rounds)},
                       "e2e_ms": {"n": len(e2e_rounds), "min": min(e2e_rounds), "median": e2e_ms, "max": max(e2e_rounds)}},
            "e2e": {"value": K * GLOBAL_BATCH / (e2e_ms * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / K,
                    "inputs": "images + fp32 class labels from pinned host memory; one-hot targets built on the device"},
            "gpu_launches": int(launches_per_round),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "k_conv_igemm_t (conv2 forward / input gradient)",
                         "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": (achieved / tf32_peak) if achieved else None,
                         "frac_of_burst": (achieved / (pk["bf16_burst"] / 2.0)) if achieved else None,
                         # dram read + write per launch: the average of the step's two launches of this kernel
                         # (157.7 MB pooled forward, 278.1 MB input gradient at batch 2048; both scale with the
                         # batch) from the ncu capture summarised in the file named below
                         "traffic": 217.9e6 * B / 2048, "traffic_unit": "bytes",
                         "traffic_source": "profiles/ncu_conv_chains_b2048_tf32.md (ncu dram__bytes_read.sum + dram__bytes_write.sum)",
                         "peak_source": "%s bf16 sustained %.1f TF/s / 2 (TF32 runs at half the bf16 tensor rate); kernel "
                                        "timed inside %.1f s of back-to-back steps; burst peak %.1f TF/s / 2 for frac_of_burst"
                                        % (pk["source"], pk["bf16_sustained"], region_s, pk["bf16_burst"]),
                         "flops_per_launch": flops_per_launch, "avg_launch_ms": ig["avg_ms"], "launches_timed": ig["launches"]},
            "kernels": kern,
            "step_tflops": K * GLOBAL_BATCH * FLOP_PER_SAMPLE / (dev_ms * 1e-3) / 1e12,
            "data_parallel": None if world == 1 else {
                "compute_only_ms_per_step": compute_only_ms, "exposed_exchange_ms_per_step": dev_ms / K - compute_only_ms,
                "note": "compute_only = the same captured step with the gradient all-reduce left out (timing diagnostic)"},
            "loss_check": loss_check, "loss_last": final_loss,
            "loss": "mean over ranks; loss_last is the loss after the device-resident rounds, which repeat one batch",
            "device_status": status,
        }
        if other is not None:
            out["tf32x3"] = other
        if world == 1 and not args.no_ops:
            try:
                out["ops"] = op_sweep(ctx, pk)
            except Exception as e:
                out["ops"] = {"failed": repr(e)}
        if world == 1 and not args.no_cpu_baseline:
            try:
                out["cpu_baseline"] = cpu_baseline()
            except Exception as e:  # the checker is optional for the GPU number
                out["cpu_baseline"] = {"value": None, "unit": "samples/s", "cores": host_cores(), "kind": "port",
                                       "sample": "failed: %r" % (e,)}
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()


def main():
    global GLOBAL_BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--math", choices=("tf32", "tf32x3", "fp32"), default="tf32")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="device time each of the two timed arms accumulates before it stops (rounds of --steps)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--bucket-kb", type=int, default=256,
                    help="data parallel: gradient spans are exchanged once this many KB of them are final")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="diagnostic only: the headline number is quoted at the default")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-x3", action="store_true", help="skip the additional 3xTF32 measurement")
    ap.add_argument("--no-ops", action="store_true", help="skip the standalone operator sweep (N = 1 only)")
    ap.add_argument("--no-loss-check", action="store_true", help="report a failed loss check instead of exiting")
    args = ap.parse_args()
    GLOBAL_BATCH = args.global_batch
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
