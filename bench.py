"""Benchmark of the fused map-reduce hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Default workload: the sharded data-parallel sinsum_add of 2^30 Float32 pairs
(f(x,y) = sum(sin.(x) .+ y)), sharded over a 1-D mesh of N GPUs -- the
configuration the metric "fused map-reduce HBM GB/s at 1/2/4/8 B200" is quoted
on.  At N = 1 it is the whole 2^30 problem on one GPU; at N > 1 (one process per
GPU under torch.distributed.run) the total problem is fixed (strong scaling):
each rank reduces its contiguous chunk and the partial sums are all-reduced.

One JSON line is printed by rank 0.  `value` is HBM GB/s over the whole job with
inputs resident in device memory; `e2e` is the same metric through the public
API with host buffers (pinned H2D of every step's inputs and D2H of the result
inside the timed region); `roofline` describes the dominant kernel; and
`cpu_baseline` is the CPU oracle timed on this host (N = 1 only).

Other workloads (single GPU): c1_sinsum_2p24, c2_logsumexp_32768x8192,
c3_jacobi2d_8192_100, c4_mlp_grad_bf16.  Inputs are seeded synthetic data with
the shapes and distributions of the benchmark configurations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

GiB = 1 << 30


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            t0 = time.time()
            while not self.rows and time.time() - t0 < 3.0:  # short regions: wait for the first sample
                time.sleep(0.05)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def pinned(n, dtype=np.float32):
    import torch
    tdt = {np.float32: torch.float32, np.uint16: torch.uint16}[dtype]
    t = torch.empty(n, dtype=tdt, pin_memory=torch.cuda.is_available())
    return t, t.numpy()


def fill_uniform(dst, seed, lo, hi):
    """Seeded U[lo,hi) Float32 fill, generated in chunks (keeps host memory bounded)."""
    rng = np.random.default_rng(seed)
    step = 1 << 24
    for i in range(0, dst.size, step):
        j = min(dst.size, i + step)
        dst[i:j] = rng.random(j - i, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)


# ----------------------------------------------------------------------------------------------
# workloads: each returns dict(thunk, make_args(), read(result), bytes/flops per step, ...)
# ----------------------------------------------------------------------------------------------
def setup_sinsum(rx, client, n_total, rank, world, seeds=(11, 12)):
    n_local = n_total // world
    _, hx = pinned(n_local)
    _, hy = pinned(n_local)
    # every rank draws its own chunk from a per-chunk stream so that the global input is fixed for a given world size
    fill_uniform(hx, seeds[0] * 1000 + rank, -np.pi, np.pi)
    fill_uniform(hy, seeds[1] * 1000 + rank, -np.pi, np.pi)
    text = rx.programs.sinsum_add(n_total, num_partitions=world)
    thunk = rx.compile(text, client)
    if world > 1:
        mesh = rx.Mesh(client.devices, ("x",))
        sh = rx.NamedSharding(mesh, ("x",))

        def upload():
            return rx.from_local_shards([hx], (n_total,), sh, client), rx.from_local_shards([hy], (n_total,), sh, client)
    else:
        def upload():
            return rx.to_rarray(hx, client), rx.to_rarray(hy, client)
    return dict(thunk=thunk, upload=upload, host=(hx, hy), read=lambda r: float(r),
                bytes_per_step=8 * n_total, h2d=8 * n_local, d2h=4, unit="GB/s", kind="reduce_full", dtype="f32",
                bound="hbm", kernel="k_reduce_full_sinadd")


def setup_logsumexp(rx, client, rows=32768, cols=8192):
    _, hx = pinned(rows * cols)
    rng = np.random.default_rng(3)
    step = 1 << 24
    for i in range(0, hx.size, step):
        hx[i:i + step] = rng.standard_normal(min(step, hx.size - i), dtype=np.float32)
    x = hx.reshape(cols, rows)  # boundary layout
    thunk = rx.compile(rx.programs.logsumexp_dims1(rows, cols), client)
    return dict(thunk=thunk, upload=lambda: (rx.to_rarray(x.T, client),), host=(x,), read=lambda r: np.asarray(r),
                bytes_per_step=4 * rows * cols + 4 * cols, h2d=4 * rows * cols, d2h=4 * cols, unit="GB/s", kind="logsumexp", dtype="f32",
                bound="hbm", kernel="k_logsumexp")


def setup_jacobi(rx, client, n=8192, steps=100):
    _, ha = pinned(n * n)
    _, hb = pinned(n * n)
    fill_uniform(ha, 4, 0.0, 1.0)
    fill_uniform(hb, 5, 0.0, 1.0)
    a, b = ha.reshape(n, n), hb.reshape(n, n)
    thunk = rx.compile(rx.programs.jacobi2d(n, steps), client)
    per_sweep = 4 * n * n + 4 * (n - 2) * (n - 2)
    return dict(thunk=thunk, upload=lambda: (rx.to_rarray(a.T, client), rx.to_rarray(b.T, client)), host=(a, b),
                read=lambda r: (np.asarray(r[0]), np.asarray(r[1])), bytes_per_step=per_sweep * steps, h2d=8 * n * n, d2h=8 * n * n,
                unit="GB/s", kind="stencil_tma", dtype="f32", bound="hbm", kernel="k_stencil", launches_per_step=steps, donates=True)


def setup_mlp(rx, client, rank=0, world=1, F=1024, H=4096, O=1024, B=4096):
    """MLP forward + gradients.  With N > 1 ranks the batch is sharded (weak scaling: B rows per GPU, global batch
    B * N), the weights are replicated, and every gradient is all-reduced (NCCL over NVLink) -- data-parallel training."""
    import ml_dtypes
    rng = np.random.default_rng(6)
    bf = lambda a: a.astype(np.float32).astype(ml_dtypes.bfloat16)
    W1 = bf(rng.standard_normal((F, H)) / np.sqrt(F))
    W2 = bf(rng.standard_normal((H, O)) / np.sqrt(H))
    b1 = (0.01 * rng.standard_normal(H)).astype(np.float32)
    b2 = (0.01 * rng.standard_normal(O)).astype(np.float32)
    rng = np.random.default_rng(600 + rank)  # this rank's rows of the global batch
    X = bf(rng.standard_normal((B, F)))
    Y = rng.standard_normal((B, O)).astype(np.float32)
    ins = [W1, b1, W2, b2, X, Y]

    def staged(a):
        """The array in pinned host memory, laid out as it crosses the boundary: a column-major (Julia) array, i.e. a
        transposed view of a C-contiguous buffer, which the upload hands to the library without another host copy."""
        t = np.ascontiguousarray(a)
        raw = np.uint16 if t.dtype == ml_dtypes.bfloat16 else np.float32
        _keep, buf = pinned(t.size, raw)
        host = buf.view(t.dtype).reshape(t.shape)
        host[...] = t
        host_keep.append(_keep)
        return host.T

    host_keep = []
    ins_t = [staged(a) for a in ins]
    thunk = rx.compile(rx.programs.mlp_grad(F, H, O, B * world, num_partitions=world), client)
    flops = (2 * B * H * F * 2 + 2 * B * O * H * 3) * world
    nbytes = sum(a.nbytes for a in ins)
    if world > 1:
        mesh = rx.Mesh(client.devices, ("x",))
        rep2, rep1, batch = rx.NamedSharding(mesh, (None, None)), rx.NamedSharding(mesh, (None,)), rx.NamedSharding(mesh, (None, "x"))
        spec = [(rep2, (H, F)), (rep1, (H,)), (rep2, (O, H)), (rep1, (O,)), (batch, (F, B * world)), (batch, (O, B * world))]

        def upload():
            return tuple(rx.from_local_shards([a], shape, sh, client) for a, (sh, shape) in zip(ins_t, spec))
    else:
        def upload():
            return tuple(rx.to_rarray(a, client) for a in ins_t)
    # the step's result that travels back is the loss; the gradients stay on the device for the optimiser
    return dict(thunk=thunk, upload=upload, host=(ins_t, host_keep), read=lambda r: float(r[4]),
                flops_per_step=flops, h2d=nbytes, d2h=4, unit="TFLOP/s", kind="gemm_tc", dtype="bf16",
                bound="tensor", kernel="k_gemm", launches_per_step=5)


WORKLOADS = {
    "c5_sharded_sinsum_2p30": lambda rx, c, r, w: setup_sinsum(rx, c, 1 << 30, r, w),
    "c1_sinsum_2p24": lambda rx, c, r, w: setup_sinsum(rx, c, 1 << 24, r, w, seeds=(1, 2)),
    "c2_logsumexp_32768x8192": lambda rx, c, r, w: setup_logsumexp(rx, c),
    "c3_jacobi2d_8192_100": lambda rx, c, r, w: setup_jacobi(rx, c),
    "c4_mlp_grad_bf16": lambda rx, c, r, w: setup_mlp(rx, c, r, w),
}
# reduced sizes of the same programs for profiler captures (a few hundred MB on the device, still larger than L2)
WORKLOADS.update({
    "prof_sinsum_2p27": lambda rx, c, r, w: setup_sinsum(rx, c, 1 << 27, r, w, seeds=(1, 2)),
    "prof_logsumexp_32768x2048": lambda rx, c, r, w: setup_logsumexp(rx, c, 32768, 2048),
    "prof_jacobi2d_8192_4": lambda rx, c, r, w: setup_jacobi(rx, c, 8192, 4),
})
SMALL_INPUT = {"c1_sinsum_2p24", "c4_mlp_grad_bf16"}  # working set near or below the 126 MB L2: rotate input copies


# DRAM traffic per algorithmic byte of the dominant kernel, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured launch; traffic grows in
# proportion to the units processed, so the ratio carries over to the full-size launch).
TRAFFIC_RATIO = {
    "reduce_full": (1.073795e9 + 3.84e6) / (8 * (1 << 27)),          # profiles/k_reduce_full_sinadd__sinsum_2p27.md
    "logsumexp": (268.457728e6 + 3.685e6) / (4 * 32768 * 2048 + 12 * 2048),  # profiles/k_logsumexp__32768x2048.md
    "stencil_tma": (269.39392e6 + 219.197184e6) / (4 * 8192 * 8192 + 4 * 8190 * 8190),  # profiles/k_stencil_tma__jacobi2d_8192*.md
    "stencil_tma_loop": (0.930697e9 + 1.023089e9) / 4 / (4 * 8192 * 8192 + 4 * 8190 * 8190),  # profiles/k_stencil_loop__jacobi2d_8192_x4.md
}


def work_per_step(wl):
    return wl.get("bytes_per_step", wl.get("flops_per_step"))


def to_metric(wl, work, ms):
    return work / (ms * 1e-3) / (1e9 if wl["unit"] == "GB/s" else 1e12)


def time_resident(rx, client, wl, steps, warmup, rotate, dist, spans=False):
    """K steps with inputs resident in HBM, timed with CUDA events on the engine's stream.
    Workloads whose inputs would fit in L2 rotate over several resident copies of the inputs so that
    the set touched between two uses of the same copy is larger than L2.
    spans=True additionally brackets every launch with its own pair of events (per-kernel durations); those
    events cost 2-5 us per launch on the GPU timeline, so the pass that produces `value` runs without them."""
    dev = client.addressable_devices[0]
    thunk = wl["thunk"]
    sets = [wl["upload"]() for _ in range(rotate)]
    for k in range(warmup):
        r = thunk(*sets[k % rotate])
    dev.synchronize()
    dev.profile()  # drop spans recorded so far
    launches0 = dev.kernel_launches()
    dist.barrier()
    dev.set_profiling(spans)
    e0 = dev.record_event()
    for k in range(steps):
        r = thunk(*sets[(warmup + k) % rotate])
    dev.join_streams()  # gradient all-reduces of the last step (communication stream) end inside the timed region
    e1 = dev.record_event()
    e1.synchronize()
    ms = e0.elapsed_ms(e1)
    dev.synchronize()
    dev.set_profiling(False)
    launches = dev.kernel_launches() - launches0
    prof = dev.profile()
    dist.barrier()
    return ms, launches, prof, wl["read"](r)


def time_e2e(rx, client, wl, steps, warmup, dist):
    """Same metric through the public API with host buffers: upload + execute + read back, every step."""
    dev = client.addressable_devices[0]
    thunk = wl["thunk"]
    for _ in range(min(warmup, 2)):
        wl["read"](thunk(*wl["upload"]()))
    dev.synchronize()
    dist.barrier()
    e0 = dev.record_event()
    for _ in range(steps):
        out = wl["read"](thunk(*wl["upload"]()))
    e1 = dev.record_event()
    e1.synchronize()
    ms = e0.elapsed_ms(e1)
    dist.barrier()
    return ms, out


def cpu_baseline(name, seconds_budget=20.0):
    """The C/OpenMP oracle timed on this host's cores on a bounded sample of the workload."""
    _, cpu = entry.load_oracle()
    threads = cpu.threads()
    rng = np.random.default_rng(99)
    if "sinsum" in name:
        n = 1 << 27
        x = rng.random(n, dtype=np.float32) * np.float32(2 * np.pi) - np.float32(np.pi)
        y = rng.random(n, dtype=np.float32) * np.float32(2 * np.pi) - np.float32(np.pi)
        fn, work, unit, sample = (lambda: cpu.sinsum_add(x, y)), 8 * n, "GB/s", f"sinsum_add on 2^27 element pairs (1 GiB read) per repetition"
    elif "logsumexp" in name:
        rows, cols = 32768, 1024
        x = rng.standard_normal((cols, rows), dtype=np.float32)
        fn, work, unit, sample = (lambda: cpu.logsumexp_dims1(x)), 4 * rows * cols + 4 * cols, "GB/s", f"{cols} of 8192 columns of 32768 rows per repetition"
    elif "jacobi" in name:
        n, steps = 8192, 2
        a, b = rng.random((n, n), dtype=np.float32), rng.random((n, n), dtype=np.float32)
        fn, work, unit, sample = (lambda: cpu.jacobi2d(a, b, steps)), (4 * n * n + 4 * (n - 2) ** 2) * steps, "GB/s", "2 of 100 sweeps of the 8192^2 grid per repetition"
    else:
        return None
    fn()
    t0, reps, best = time.perf_counter(), 0, float("inf")
    while True:
        t = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t)
        reps += 1
        if time.perf_counter() - t0 > seconds_budget or reps >= 10:
            break
    return {"value": work / best / 1e9, "unit": unit, "cores": threads, "kind": "port", "sample": sample + f"; best of {reps}"}


def run_reference(args):
    """Reference arm: the CPU implementation of the path (the oracle port; the reference's own XLA-CPU
    path cannot be installed here: it needs Julia and the Reactant_jll binary) on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _, cpu = entry.load_oracle()
    name = args.workload
    n = 1 << 27
    rng = np.random.default_rng(11)
    x = rng.random(n, dtype=np.float32) * np.float32(2 * np.pi) - np.float32(np.pi)
    y = rng.random(n, dtype=np.float32) * np.float32(2 * np.pi) - np.float32(np.pi)
    for _ in range(max(1, args.warmup)):
        cpu.sinsum_add(x, y)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.sinsum_add(x, y)
    dt = (time.perf_counter() - t0) / args.steps
    value = 8 * n / dt / 1e9
    sample = "each step reduces 2^27 of the 2^30 element pairs (1 GiB read)"
    line = {"impl": "reference", "metric": "fused map-reduce HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": name, "sample": sample},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cpu.threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5_sharded_sinsum_2p30", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} processes (WORLD_SIZE={world})")
    rx = entry.load_package()
    dist = rx.dist.Dist(world)
    client = rx.Client(node_id=dist.rank, num_nodes=world, allowed_devices=[dist.local_rank])
    allreduce = "none"
    if world > 1:
        if args.workload not in ("c5_sharded_sinsum_2p30", "c1_sinsum_2p24", "c4_mlp_grad_bf16"):
            raise SystemExit("the sinsum workloads and the data-parallel MLP step shard; the others run as single-GPU configurations")
        default_mode = "mailbox+nccl" if args.workload == "c4_mlp_grad_bf16" else "mailbox"
        allreduce = rx.dist.connect_collectives(rx, client, dist, os.environ.get("RX_ALLREDUCE", default_mode))
    wl = WORKLOADS[args.workload](rx, client, dist.rank, world)
    rotate = 4 if args.workload in SMALL_INPUT else 1
    peaks = measured_peaks()
    with ClockSampler(dist.local_rank) as clk:  # sampling covers warm-up and the timed region
        ms, launches, _, result = time_resident(rx, client, wl, args.steps, args.warmup, rotate, dist)
        # per-kernel spans from a repeat of the same K steps, each launch bracketed by its own events
        _, _, prof, _ = time_resident(rx, client, wl, args.steps, 1, rotate, dist, spans=True)
    ms = dist.reduce(ms, "max")
    launches = int(dist.reduce(launches, "sum"))
    work = work_per_step(wl)
    value = to_metric(wl, work * args.steps, ms)
    # dominant kernel: average span of its step kind, measured in the timed region on the launching stream
    kind = wl["kind"]
    launches_per_step, kernel = wl.get("launches_per_step", 1), wl["kernel"]
    if kind == "stencil_tma" and "stencil_tma_loop" in prof:
        # the whole counted loop ran as one cooperative launch: a launch processes every sweep of the step
        kind, launches_per_step, kernel = "stencil_tma_loop", 1, "k_stencil_loop"
    roof = None
    if kind in prof and prof[kind]["launches"]:
        if launches == args.steps * world:
            # one launch per step: the timed region itself is that kernel's launches back to back
            per_launch_ms, timed = ms / args.steps, "timed region / steps (one launch per step)"
        else:
            per_launch_ms, timed = prof[kind]["ms"] / prof[kind]["launches"], "per-launch event pairs, repeat of the timed region"
        per_launch_ms = dist.reduce(per_launch_ms, "max")
        per_launch_work = work / launches_per_step
        achieved = to_metric(wl, per_launch_work, per_launch_ms)
        peak = (peaks["hbm_gbs"] if wl["bound"] == "hbm" else peaks["bf16_tflops"]) * world
        traffic = None
        if kind in TRAFFIC_RATIO:
            traffic = TRAFFIC_RATIO[kind] * per_launch_work / world  # bytes per launch on one GPU
        roof = {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": wl["unit"], "frac": achieved / peak, "traffic": traffic,
                "kernel": kernel, "peak_source": f"of {peaks['source']}" + (f" x{world} GPUs" if world > 1 else ""),
                "ms_per_launch": per_launch_ms, "timed_by": timed}
    e2e = None
    if not args.no_e2e:
        e_steps = max(2, min(args.steps, 5))
        ems, _ = time_e2e(rx, client, wl, e_steps, args.warmup, dist)
        ems = dist.reduce(ems, "max")
        e2e = {"value": to_metric(wl, work * e_steps, ems), "unit": wl["unit"], "h2d_bytes_per_step": wl["h2d"] * world, "d2h_bytes_per_step": wl["d2h"] * world,
               "steps": e_steps, "ms_per_step": ems / e_steps}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(args.workload)
    if dist.rank == 0:
        line = {"metric": "fused map-reduce HBM GB/s" if wl["unit"] == "GB/s" else "dot_general TFLOP/s", "value": value, "unit": wl["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if "sinsum" in args.workload and (world > 1 or "c5" in args.workload) else "weak",
                "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
                "config": {"workload": args.workload, "l2": f"{rotate} rotating resident input sets, together larger than L2" if rotate > 1 else "inputs larger than L2", "all_reduce": allreduce,
                           "result": result if isinstance(result, float) else None},
                "clocks": clk.summary(), "e2e": e2e, "gpu_launches": launches, "roofline": roof, "cpu_baseline": cpu, "profile_ms": prof}
        print(json.dumps(line), flush=True)
    client.close()
    dist.close()


if __name__ == "__main__":
    main()
