"""Benchmark of the hot path: data-parallel training of the widened CNN of BASELINE config 4
(Conv 1->64 5x5 p2, ReLU, MaxPool 2x2, Conv 64->128 5x5 p2, ReLU, MaxPool 2x2, Linear 6272->10,
softmax cross-entropy, Adam lr 1e-3) at global batch 2048 on N B200s of one node.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...   # the CPU restatement of the reference on the host cores

One "step" is one pass of the reference's training loop (examples/mnist.mojo:92-104: forward,
zero_grad, backward, Adam.step) over one global batch of seeded synthetic 28x28 images.  Rank 0
prints ONE JSON line.  `value` is samples/s with the batch already resident in HBM; `e2e` is the
same loop through the host mirror's public call with the batch in pinned HOST memory, copied to
the device every step, and the loss read back every step.
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
sys.path.insert(0, str(ROOT / "tests"))

GLOBAL_BATCH = 2048
POOL = 4096                       # synthetic samples; two global batches, alternated
FLOP_PER_SAMPLE = 246.2e6         # forward + backward of the widened CNN (algorithmic)
CONV2_FLOP_PER_SAMPLE = 80.28e6   # one of conv2's three GEMMs: 2 * 128 * 64 * 14 * 14 * 25
WORKLOAD = "cnn_c64_c128_fc6272_b2048"


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# ------------------------------------------------------------------ clocks -------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ workload -----------------

def synthetic_pool(seed=42):
    """Pixels ~ U(0,1), labels uniform over 0..9 as one-hot rows (BASELINE config 2/4)."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(0.0, 1.0, (POOL, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, POOL)]
    return x, y


def init_weights(shapes, seed=43):
    """U(+-1/sqrt(fan_in)), fan_in = C*R*S for conv, rows for Linear (nn/layers/*.mojo)."""
    rng = np.random.default_rng(seed)
    fans = {0: 25, 1: 25, 2: 1600, 3: 1600, 4: 6272, 5: 6272}
    return [rng.uniform(-1, 1, s).astype(np.float32) / np.float32(np.sqrt(fans[i])) for i, s in enumerate(shapes)]


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------ CPU reference arm --------

def oracle_step_fn(batch):
    """The CPU restatement of the reference's training step on the same network and data."""
    import oracle
    from test_oracle_kat import build_cnn
    g = oracle.Graph()
    build_cnn(oracle, g, batch, 64, 128)
    m = oracle.Model(g)
    tr = [s for s in g.params() if s.trainable]
    for s, w in zip(tr, init_weights([s.shape for s in tr])):
        m.set_tensor(s, w)
    opt = oracle.Adam(m, lr=1e-3)
    x, y = synthetic_pool()

    def step(i):
        lo = (i * batch) % (POOL - batch + 1)
        loss = m.forward(x[lo:lo + batch], y[lo:lo + batch])
        opt.zero_grad(); m.backward(); opt.step()
        return loss
    return step


def cpu_baseline(target_seconds=15.0):
    """Bounded sample of the same workload on the host cores: samples/s of the oracle."""
    cores = os.cpu_count() or 1
    batch = 16
    step = oracle_step_fn(batch)
    t0 = time.perf_counter(); step(0); first = time.perf_counter() - t0
    n = max(1, min(20, int(target_seconds / max(first, 1e-3))))
    t0 = time.perf_counter()
    for i in range(n):
        step(i + 1)
    dt = time.perf_counter() - t0
    return {"value": n * batch / dt, "unit": "samples/s", "cores": cores, "kind": "port",
            "sample": "%d steps at batch %d of the same network (oracle/, OpenMP over %d host threads)" % (n, batch, cores)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = 16
    step = oracle_step_fn(batch)
    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i)
    dt = time.perf_counter() - t0
    v = args.steps * batch / dt
    cores = os.cpu_count() or 1
    sample = "%d steps at batch %d per step (bounded sample of the 2048-sample step)" % (args.steps, batch)
    print(json.dumps({
        "impl": "reference", "metric": "cnn_train_samples_per_s", "value": v, "unit": "samples/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "sample_batch": batch,
                   "note": "CPU restatement of Mantle's Mojo kernels (the Mojo toolchain is not installable here)"},
        "cpu_baseline": {"value": v, "unit": "samples/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------ GPU arm ------------------

def run_ours(args):
    import mantle_b200 as mb
    from mantle_b200 import host_api
    from test_oracle_kat import build_cnn

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

    class Ns:
        OP, nn, Graph = mb.OP, host_api.nn, host_api.Graph
    g = host_api.Graph()
    build_cnn(Ns, g, B, 64, 128)
    model = host_api.Model(ctx, g)
    tr = [s for s in g.params() if s.trainable]
    for s, w in zip(tr, init_weights([s.shape for s in tr])):
        model.set_tensor(s, w)
    adam = host_api.Adam(model, lr=1e-3)
    trainer = host_api.Trainer(model, adam, use_graph=not args.no_graph)

    # synthetic pool in pinned host memory
    x, y = synthetic_pool()
    px, py = C.c_void_p(), C.c_void_p()
    ctx._check(lib.mtl_host_alloc(ctx.handle, x.nbytes, C.byref(px)))
    ctx._check(lib.mtl_host_alloc(ctx.handle, y.nbytes, C.byref(py)))
    C.memmove(px.value, x.ctypes.data, x.nbytes)
    C.memmove(py.value, y.ctypes.data, y.nbytes)
    ploss = C.c_void_p()
    ctx._check(lib.mtl_host_alloc(ctx.handle, 4096, C.byref(ploss)))
    loss_view = np.ctypeslib.as_array(C.cast(ploss, C.POINTER(C.c_float)), (1024,))

    def batch_ptrs(step):
        row = (step % (POOL // GLOBAL_BATCH)) * GLOBAL_BATCH + rank * B
        return [px.value + row * 784 * 4, py.value + row * 10 * 4]

    h2d_bytes = B * (784 + 10) * 4

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

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    losses = []
    for i in range(args.warmup):
        losses.append(trainer.step_ptrs(batch_ptrs(i)))

    # ---- end to end: pinned host batch -> device every step, loss -> host every step ----------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = ctx.launch_count()
    ctx.timer_start(0)
    w0 = time.perf_counter()
    # Trainer.step_async: every step copies its batch from pinned host memory (copy stream, two
    # staging buffers) and writes its loss to its own pinned word; the host only waits at the end,
    # so the copy of batch i + 1 overlaps the kernels of step i
    for i in range(args.steps):
        trainer.step_async_ptrs(batch_ptrs(args.warmup + i), ploss.value + 4 * (i % 1024))
    ctx.timer_stop(0)
    e2e_ms = ctx.timer_ms(0)
    e2e_wall_ms = (time.perf_counter() - w0) * 1e3
    losses.extend(float(v) for v in loss_view[:min(args.steps, 1024)])
    launches = ctx.launch_count() - launches0
    barrier()
    e2e_ms = max_over_ranks(max(e2e_ms, 0.0))

    # ---- device resident: the same captured step, batch already in HBM -------------------------
    trainer.step_async_ptrs([], ploss.value)  # untimed: re-captures the step for this loss slot
    barrier()
    ctx.timer_start(1)
    for i in range(args.steps):
        trainer.step_async_ptrs([], ploss.value)
    ctx.timer_stop(1)
    dev_ms = ctx.timer_ms(1)
    barrier()
    dev_ms = max_over_ranks(dev_ms)
    clocks = sampler.stop() if rank == 0 else None
    final_loss = float(loss_view[0])

    # ---- per-kernel durations of the dominant kernels, live, eager steps with event brackets ---
    trainer.close()
    prof_trainer = host_api.Trainer(model, adam, use_graph=False)
    ctx._check(lib.mtl_prof_reset(ctx.handle))
    ctx._check(lib.mtl_prof_enable(ctx.handle, 1))
    prof_steps = 4
    for i in range(prof_steps):
        prof_trainer.step_ptrs(batch_ptrs(i))
    ctx._check(lib.mtl_prof_enable(ctx.handle, 0))
    kern = {}
    for name, kid in (("dot_tc", 0), ("conv_igemm", 1), ("conv_wgrad", 2)):
        ms, n = C.c_float(), C.c_int32()
        ctx._check(lib.mtl_prof_get(ctx.handle, kid, C.byref(ms), C.byref(n)))
        kern[name] = {"launches": n.value, "avg_ms": (ms.value / n.value) if n.value else None}
    prof_trainer.close()
    status = ctx.device_status()

    if rank == 0:
        pk = peaks()
        tf32_peak = pk["bf16_sustained"] / 2.0   # TF32 tensor rate is half the bf16 rate
        flops_per_launch = CONV2_FLOP_PER_SAMPLE * B
        ig = kern["conv_igemm"]
        achieved = flops_per_launch / (ig["avg_ms"] * 1e-3) / 1e12 if ig["avg_ms"] else None
        out = {
            "metric": "cnn_train_samples_per_s", "value": args.steps * GLOBAL_BATCH / (dev_ms * 1e-3),
            "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"tf32": "tf32", "tf32x3": "tf32x3", "fp32": "f32"}[args.math], "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_gpu_batch": B, "parallelism": "dp%d" % world,
                       "math_mode": args.math, "cuda_graph": not args.no_graph,
                       "l2": "per-step working set (>= 0.4 GB of activations per GPU at N<=4) exceeds the 126 MB L2; "
                             "a fresh batch every step"},
            "e2e": {"value": args.steps * GLOBAL_BATCH / (e2e_ms * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": e2e_wall_ms / args.steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "k_conv_igemm_t (conv2 forward / input gradient)",
                         "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": (achieved / tf32_peak) if achieved else None,
                         # dram read + write per launch from the ncu capture summarised under profiles/
                         # (157.7 MB forward with the pooling in the epilogue, 278.1 MB input gradient at batch
                         # 2048: the average of the two launches of a step; both scale with the batch)
                         "traffic": 217.9e6 * B / 2048, "traffic_unit": "bytes",
                         "peak_source": "%s bf16 sustained %.1f TF/s / 2 (TF32 runs at half the bf16 tensor rate)"
                                        % (pk["source"], pk["bf16_sustained"]),
                         "flops_per_launch": flops_per_launch, "avg_launch_ms": ig["avg_ms"], "launches_timed": ig["launches"]},
            "kernels": kern,
            "step_tflops": args.steps * GLOBAL_BATCH * FLOP_PER_SAMPLE / (dev_ms * 1e-3) / 1e12,
            "loss_first": losses[0], "loss_last": final_loss, "device_status": status,
        }
        if world == 1 and not args.no_cpu_baseline:
            try:
                out["cpu_baseline"] = cpu_baseline()
            except Exception as e:  # the checker is optional for the GPU number
                out["cpu_baseline"] = {"value": None, "unit": "samples/s", "cores": os.cpu_count(), "kind": "port",
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
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="diagnostic only: the headline number is quoted at the default")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
