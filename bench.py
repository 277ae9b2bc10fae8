"""Benchmark of the fused map-reduce / stencil / dot_general hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Default workload: the sharded data-parallel sinsum_add of 2^30 Float32 pairs
(f(x,y) = sum(sin.(x) .+ y)), sharded over a 1-D mesh of N GPUs -- the
configuration the metric "fused map-reduce HBM GB/s at 1/2/4/8 B200" is quoted
on.  At N = 1 it is the whole 2^30 problem on one GPU; at N > 1 (one process per
GPU under torch.distributed.run) the total problem is fixed (strong scaling):
each rank reduces its contiguous chunk and the partial sums are all-reduced.
The global input does not depend on N: it is drawn as 8 fixed chunks, each from
its own seeded stream, and rank r owns chunks r*8/N .. (r+1)*8/N - 1.

One JSON line is printed by rank 0.  `value` is the metric over the whole job with
inputs resident in device memory; `e2e` is the same metric through the public
API with host buffers (pinned H2D of every step's inputs and D2H of the result
inside the timed region); `roofline` describes the dominant kernel; `parity`
compares what the timed steps computed with the CPU oracle on the same inputs
(the process exits 1 when it does not hold); `cpu_baseline` is the CPU oracle
timed on this host (N = 1 only).  In the default single-GPU run the other
single-GPU configurations (c1_sinsum_2p24, c2_logsumexp_32768x8192,
c3_jacobi2d_8192_100 and its two-half-step spelling, c4_mlp_grad_bf16) are
measured and checked as well and reported under `configs`.

`--impl reference` times the CPU implementation of the chosen workload (the
C/OpenMP or numpy oracle port: the reference's own XLA-CPU path needs Julia and
its binary artefact, neither of which exists here) on all host cores.
Inputs are seeded synthetic data with the shapes and distributions of the
benchmark configurations.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
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

N_CHUNKS = 8  # the sharded vectors are drawn as this many independently seeded chunks, whatever the mesh size


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        return os.cpu_count() or 1


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
        # the median under load: samples taken while the GPU idled between regions sit at the idle clock
        busy = [v for v in sm if mx and v >= 0.5 * max(mx)] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


def pinned(rx, n, dtype=np.float32):
    """Page-locked host array from the library's own allocator (pageable numpy memory where no GPU is present)."""
    if getattr(rx, "PinnedArray", None) is not None:
        p = rx.PinnedArray(n, dtype)
        return p, p.array
    a = np.empty(n, dtype=dtype)
    return a, a


def fill_uniform(dst, seed, lo, hi):
    """Seeded U[lo,hi) Float32 fill, generated in pieces (keeps host memory bounded)."""
    rng = np.random.default_rng(seed)
    step = 1 << 24
    for i in range(0, dst.size, step):
        j = min(dst.size, i + step)
        dst[i:j] = rng.random(j - i, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)


def fill_chunks(dst, seed, first_chunk, n_chunks, chunk_len, lo=-np.pi, hi=np.pi):
    """Chunks first_chunk .. first_chunk + n_chunks - 1 of the global vector, each from its own stream."""
    for c in range(n_chunks):
        fill_uniform(dst[c * chunk_len:(c + 1) * chunk_len], seed * 1000 + first_chunk + c, lo, hi)


def parity_record(got, want, scale, tol, against, **extra):
    err = abs(got - want) / scale if scale else abs(got - want)
    rec = {"got": got, "want": want, "rel_err": err, "tol": tol, "ok": bool(err <= tol), "against": against}
    rec.update(extra)
    return rec


# ----------------------------------------------------------------------------------------------
# workloads: each returns dict(thunk, upload(), read(result), work per step, check(result), ...)
# ----------------------------------------------------------------------------------------------
def setup_sinsum(rx, client, dist, n_total, seeds=(11, 12)):
    rank, world = dist.rank, dist.world
    if N_CHUNKS % world or n_total % N_CHUNKS:
        raise SystemExit(f"the sharded vector is drawn as {N_CHUNKS} chunks: the mesh size must divide it")
    chunk_len, per_rank = n_total // N_CHUNKS, N_CHUNKS // world
    n_local = n_total // world
    kx, hx = pinned(rx, n_local)
    ky, hy = pinned(rx, n_local)
    fill_chunks(hx, seeds[0], rank * per_rank, per_rank, chunk_len)
    fill_chunks(hy, seeds[1], rank * per_rank, per_rank, chunk_len)
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

    def check(result):
        """float64 sum of this rank's chunks (C oracle, sin in double), summed over the ranks; every rank must
        hold the same Float32 bits."""
        ref, cpu = entry.load_oracle()
        cpu.set_threads(max(1, host_cores() // world))
        s, q = cpu.sinsum_add_f64(hx, hy)
        want = dist.reduce(s, "sum")
        norm = math.sqrt(dist.reduce(q, "sum"))
        got = float(result)
        same = dist.reduce(got, "max") == dist.reduce(got, "min")
        tol = ref.reduction_tolerance(n_total)
        rec = parity_record(got, want, max(abs(want), norm), tol, "float64 sum of sin(x)+y over the same seeded input (C oracle), error relative to the 2-norm of the terms; tol = 1e-5*sqrt(log2 n)",
                            same_bits_on_every_rank=bool(same))
        rec["ok"] = rec["ok"] and bool(same)
        return rec

    def cpu_run():
        _, cpu = entry.load_oracle()
        return cpu.sinsum_add(hx, hy)

    return dict(thunk=thunk, upload=upload, host=(kx, ky, hx, hy), read=lambda r: float(r), check=check, cpu_run=cpu_run,
                cpu_sample=f"the whole step: sinsum_add over 2^{int(math.log2(n_total))} element pairs ({8 * n_total / 2**30:g} GiB read)",
                bytes_per_step=8 * n_total, h2d=8 * n_local, d2h=4, unit="GB/s", kind="reduce_full", dtype="f32",
                bound="hbm", kernel="k_reduce_full_sinadd", shape={"elements": n_total, "chunks": N_CHUNKS, "seeds": list(seeds)})


def setup_logsumexp(rx, client, dist, rows=32768, cols=8192):
    keep, hx = pinned(rx, rows * cols)
    rng = np.random.default_rng(3)
    step = 1 << 24
    for i in range(0, hx.size, step):
        hx[i:i + step] = rng.standard_normal(min(step, hx.size - i), dtype=np.float32)
    x = hx.reshape(cols, rows)  # boundary layout
    thunk = rx.compile(rx.programs.logsumexp_dims1(rows, cols), client)

    def check(result):
        ref, cpu = entry.load_oracle()
        cpu.set_threads(host_cores())
        want = cpu.logsumexp_dims1(x).astype(np.float64)
        got = np.asarray(result, dtype=np.float64).reshape(-1)
        err = float(np.max(np.abs(got - want) / np.abs(want)))
        tol = ref.reduction_tolerance(rows)
        return {"got": float(got[0]), "want": float(want[0]), "rel_err": err, "tol": tol, "ok": bool(err <= tol and got.shape == want.shape),
                "against": f"C oracle on the same {rows}x{cols} input, max relative error over the {cols} results; tol = 1e-5*sqrt(log2 rows)"}

    def cpu_run():
        _, cpu = entry.load_oracle()
        return cpu.logsumexp_dims1(x)

    return dict(thunk=thunk, upload=lambda: (rx.to_rarray(x.T, client),), host=(keep, x), read=lambda r: np.asarray(r), check=check, cpu_run=cpu_run,
                cpu_sample=f"the whole step: logsumexp over dims=1 of the {rows}x{cols} matrix",
                bytes_per_step=4 * rows * cols + 4 * cols, h2d=4 * rows * cols, d2h=4 * cols, unit="GB/s", kind="logsumexp", dtype="f32",
                bound="hbm", kernel="k_logsumexp", shape={"rows": rows, "cols": cols, "seed": 3})


def setup_jacobi(rx, client, dist, n=8192, steps=100, form="dus"):
    """With N > 1 ranks both arrays are split into row blocks of the [n][n] tensors (Julia's second dimension) over the
    mesh: every sweep each rank updates the rows it owns and the boundary rows travel to the neighbours' halos."""
    rank, world = dist.rank, dist.world
    if n % world:
        raise SystemExit("the mesh size must divide the number of rows")
    L = n // world
    fa, fb = np.empty(n * n, np.float32), np.empty(n * n, np.float32)
    fill_uniform(fa, 4, 0.0, 1.0)
    fill_uniform(fb, 5, 0.0, 1.0)
    a, b = fa.reshape(n, n), fb.reshape(n, n)            # the global arrays (the same for every mesh size)
    ka, ha = pinned(rx, L * n)
    kb, hb = pinned(rx, L * n)
    la, lb = ha.reshape(L, n), hb.reshape(L, n)          # this rank's rows, in page-locked memory
    la[...] = a[rank * L:(rank + 1) * L]
    lb[...] = b[rank * L:(rank + 1) * L]
    sweeps = steps if form != "halfsteps" else 2 * steps
    order = "polybench" if form == "halfsteps" else "baseline"
    thunk = rx.compile(rx.programs.jacobi2d(n, steps, form=form, num_partitions=world), client)
    per_sweep = 4 * n * n + 4 * (n - 2) * (n - 2)
    if world > 1:
        sh = rx.NamedSharding(rx.Mesh(client.devices, ("x",)), (None, "x"))

        def upload():
            return rx.from_local_shards([la.T], (n, n), sh, client), rx.from_local_shards([lb.T], (n, n), sh, client)

        def local(r):
            return np.asarray(r.data[0].to_host())
    else:
        def upload():
            return rx.to_rarray(la.T, client), rx.to_rarray(lb.T, client)

        def local(r):
            return np.asarray(r).T

    def check(_result):
        """The timed steps keep sweeping the same donated arrays, so parity is taken on a run of its own: fresh
        upload, one execution (all the sweeps), every element of this rank's rows compared with the C oracle's."""
        _, cpu = entry.load_oracle()
        cpu.set_threads(max(1, host_cores() // world))
        ra, rb = thunk(*upload())
        ga, gb = local(ra), local(rb)
        wa, wb = cpu.jacobi2d(a, b, sweeps, order)
        wa, wb = wa[rank * L:(rank + 1) * L], wb[rank * L:(rank + 1) * L]
        bad = int(dist.reduce(float(np.count_nonzero(ga != wa) + np.count_nonzero(gb != wb)), "sum"))
        return {"got": float(ga[L // 2, n // 2]), "want": float(wa[L // 2, n // 2]), "rel_err": bad / (2.0 * n * n), "tol": 0.0, "ok": bad == 0,
                "against": f"C oracle, {sweeps} sweeps of the same {n}x{n} arrays, bit-exact on every rank's rows (rel_err = fraction of differing elements)"}

    def cpu_run():
        _, cpu = entry.load_oracle()
        return cpu.jacobi2d(a, b, 10, order)

    return dict(thunk=thunk, upload=upload, host=(ka, kb, a, b),
                read=lambda r: (local(r[0]), local(r[1])), check=check, cpu_run=cpu_run, cpu_work=per_sweep * 10,
                cpu_sample=f"10 of the {sweeps} sweeps of the {n}^2 grid per step",
                bytes_per_step=per_sweep * sweeps, h2d=8 * n * L, d2h=8 * n * L,
                unit="GB/s", kind="stencil_tma" if world == 1 else "stencil_rows", dtype="f32", bound="hbm", kernel="k_stencil", launches_per_step=sweeps, donates=True,
                shape={"n": n, "sweeps": sweeps, "form": form, "seeds": [4, 5]})


def setup_mlp(rx, client, dist, F=1024, H=4096, O=1024, B=4096):
    """MLP forward + gradients.  With N > 1 ranks the batch is sharded (weak scaling: B rows per GPU, global batch
    B * N), the weights are replicated, and every gradient is all-reduced (NCCL over NVLink) -- data-parallel training."""
    import ml_dtypes
    rank, world = dist.rank, dist.world
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
        _keep, buf = pinned(rx, t.size, raw)
        host = buf.view(t.dtype).reshape(t.shape)
        host[...] = t
        host_keep.append(_keep)
        return host.T

    host_keep = []
    ins_t = [staged(a) for a in ins]
    text = rx.programs.mlp_grad(F, H, O, B * world, num_partitions=world)
    thunk = rx.compile(text, client)
    flops = (2 * B * H * F * 2 + 2 * B * O * H * 3) * world
    nbytes = sum(a.nbytes for a in ins)
    out_bytes = 2 * F * H + 4 * H + 2 * H * O + 4 * O + 4
    if world > 1:
        mesh = rx.Mesh(client.devices, ("x",))
        rep2, rep1, batch = rx.NamedSharding(mesh, (None, None)), rx.NamedSharding(mesh, (None,)), rx.NamedSharding(mesh, (None, "x"))
        spec = [(rep2, (H, F)), (rep1, (H,)), (rep2, (O, H)), (rep1, (O,)), (batch, (F, B * world)), (batch, (O, B * world))]

        def upload():
            return tuple(rx.from_local_shards([a], shape, sh, client) for a, (sh, shape) in zip(ins_t, spec))
    else:
        def upload():
            return tuple(rx.to_rarray(a, client) for a in ins_t)

    def read(r):
        """The step's results: both weight gradients, both bias gradients and the loss, copied to the host."""
        return [np.asarray(o.data[0].to_host()) for o in r]

    def check(result):
        """Every gradient and the loss against the numpy oracle (float64 accumulation) of the same module on the same
        inputs; each output within 2e-2 of its largest magnitude (the bf16 dot_general bar)."""
        if world > 1:
            return check_data_parallel(result)
        ref, _ = entry.load_oracle()
        f32 = lambda a: np.asarray(a, dtype=np.float32)
        want = ref.run_module(text, [f32(W1), b1, f32(W2), b2, f32(X), Y])
        worst, names = 0.0, ("dW1", "db1", "dW2", "db2", "loss")
        detail = {}
        for name, g, w in zip(names, result, want):
            g, w = np.asarray(g, dtype=np.float64), np.asarray(w, dtype=np.float64)
            e = float(np.max(np.abs(g - w)) / max(float(np.max(np.abs(w))), 1e-30))
            detail[name] = e
            worst = max(worst, e)
        return {"got": float(np.asarray(result[4], dtype=np.float64)), "want": float(want[4]), "rel_err": worst, "tol": 2e-2, "ok": bool(worst <= 2e-2), "per_output": detail,
                "against": "numpy StableHLO oracle (float64 accumulation) on the same inputs; per output max|got - want| / max|want|"}

    def check_data_parallel(result):
        """N > 1: the global batch lives on several ranks, so the all-reduced gradients are checked by decomposition.
        Every rank runs the unsharded step on its own rows (the program whose results the N = 1 run checks against the
        oracle); the ranks' gradients and losses are gathered, and their mean -- what the data-parallel step must
        produce, every rank holding the same number of rows -- is compared with this rank's result.  Independent of the
        all-reduce path: the local programs contain no collective."""
        local = rx.compile(rx.programs.mlp_grad(F, H, O, B), client)
        lres = local(*[rx.to_rarray(a, client) for a in ins_t])
        mine = [np.asarray(o.data[0].to_host()).astype(np.float32) for o in lres]
        worst, names, detail = 0.0, ("dW1", "db1", "dW2", "db2", "loss"), {}
        for name, g, m in zip(names, result, mine):
            parts = dist.all_gather_bytes(np.ascontiguousarray(m).tobytes())
            mean = sum(np.frombuffer(p, dtype=np.float32).astype(np.float64) for p in parts) / world
            g = np.asarray(g).astype(np.float64).reshape(-1)
            e = float(np.max(np.abs(g - mean)) / max(float(np.max(np.abs(mean))), 1e-30))
            detail[name] = e
            worst = max(worst, e)
        worst = dist.reduce(worst, "max")
        loss = float(np.asarray(result[4], dtype=np.float64))
        same = dist.reduce(loss, "max") == dist.reduce(loss, "min")
        return {"got": loss, "want": None, "rel_err": worst, "tol": 2e-2, "ok": bool(worst <= 2e-2 and same), "per_output": detail, "same_bits_on_every_rank": bool(same),
                "against": "mean over the ranks of the unsharded step's results on each rank's own rows (that program is checked against the numpy oracle at N = 1); per output max|got - want| / max|want|"}

    def cpu_run():
        ref, _ = entry.load_oracle()
        f32 = lambda a: np.asarray(a, dtype=np.float32)
        return ref.run_module(text, [f32(W1), b1, f32(W2), b2, f32(X), Y])

    return dict(thunk=thunk, upload=upload, host=(ins_t, host_keep), read=read, check=check, cpu_run=cpu_run,
                cpu_sample="the whole step through the numpy StableHLO oracle (BLAS float64 contractions)",
                flops_per_step=flops, h2d=nbytes, d2h=out_bytes, unit="TFLOP/s", kind="gemm_tc", dtype="bf16",
                bound="tensor", kernel="k_gemm", launches_per_step=5,
                shape={"features": F, "hidden": H, "out": O, "batch_per_gpu": B, "seeds": [6, 600]})


WORKLOADS = {
    "c5_sharded_sinsum_2p30": lambda rx, c, d: setup_sinsum(rx, c, d, 1 << 30),
    "c1_sinsum_2p24": lambda rx, c, d: setup_sinsum(rx, c, d, 1 << 24, seeds=(1, 2)),
    "c2_logsumexp_32768x8192": lambda rx, c, d: setup_logsumexp(rx, c, d),
    "c3_jacobi2d_8192_100": lambda rx, c, d: setup_jacobi(rx, c, d),
    "c3_jacobi2d_8192_50_halfsteps": lambda rx, c, d: setup_jacobi(rx, c, d, 8192, 50, form="halfsteps"),
    "c4_mlp_grad_bf16": lambda rx, c, d: setup_mlp(rx, c, d),
}
# reduced sizes of the same programs for profiler captures (a few hundred MB on the device, still larger than L2)
WORKLOADS.update({
    "prof_sinsum_2p27": lambda rx, c, d: setup_sinsum(rx, c, d, 1 << 27, seeds=(1, 2)),
    "prof_logsumexp_32768x2048": lambda rx, c, d: setup_logsumexp(rx, c, d, 32768, 2048),
    "prof_jacobi2d_8192_4": lambda rx, c, d: setup_jacobi(rx, c, d, 8192, 4),
    "prof_jacobi2d_8192_12": lambda rx, c, d: setup_jacobi(rx, c, d, 8192, 12),
})
SMALL_INPUT = {"c1_sinsum_2p24", "c4_mlp_grad_bf16"}  # working set near or below the 126 MB L2: rotate input copies
EXTRA_CONFIGS = ["c1_sinsum_2p24", "c2_logsumexp_32768x8192", "c3_jacobi2d_8192_100", "c3_jacobi2d_8192_50_halfsteps", "c4_mlp_grad_bf16"]
SHARDED = ("c5_sharded_sinsum_2p30", "c1_sinsum_2p24", "c4_mlp_grad_bf16", "c3_jacobi2d_8192_100", "c3_jacobi2d_8192_50_halfsteps",
           "prof_jacobi2d_8192_4", "prof_jacobi2d_8192_12")


# DRAM traffic per algorithmic byte of the dominant kernel, from profiler captures of the reduced-size workloads
# above (dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured launch; traffic
# grows in proportion to the units processed, so the ratio carries over to the full-size launch).
TRAFFIC_RATIO = {
    "reduce_full": (1.073795e9 + 3.84e6) / (8 * (1 << 27)),
    "logsumexp": (268.457728e6 + 3.685e6) / (4 * 32768 * 2048 + 12 * 2048),
    "stencil_tma": (269.39392e6 + 219.197184e6) / (4 * 8192 * 8192 + 4 * 8190 * 8190),
}


def stencil_loop_traffic(n, sweeps):
    """DRAM bytes of one whole-loop launch over n x n arrays.  The loop kernel does two sweeps per pass over memory
    for all but its last two (three, for an odd count) sweeps.  Per pass, from profiler captures of 4 and 12 sweeps at
    n = 8192 (1476.3 MB and 3425.4 MB: 1 resp. 5 double passes + 2 single sweeps): 487.3 MB per double pass, 494.5 MB per
    single sweep (less than the arrays' 536.7 MB because a sweep starts on what the previous one left in L2); both grow
    with the number of points."""
    tail = min(sweeps, 2 + sweeps % 2) if sweeps >= 4 else sweeps
    double = (sweeps - tail) // 2
    return (double * 487.3e6 + tail * 494.5e6) * (n * n) / (8192.0 * 8192.0)


def work_per_step(wl):
    return wl.get("bytes_per_step", wl.get("flops_per_step"))


def to_metric(wl, work, ms):
    return work / (ms * 1e-3) / (1e9 if wl["unit"] == "GB/s" else 1e12)


def config_of(name, wl, world):
    """What both arms of the benchmark print as `config`: the workload, its shape and seeds, the L2 policy."""
    rotate = 4 if name in SMALL_INPUT else 1
    return {"workload": name, **wl["shape"], "n_gpus": world,
            "l2": f"{rotate} rotating resident input sets, together larger than L2" if rotate > 1 else "inputs larger than L2"}


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


def time_cpu(wl, steps, warmup, seconds_budget=None):
    """The CPU port of the workload's step on every host core; returns (seconds per step, steps timed)."""
    _, cpu = entry.load_oracle()
    cpu.set_threads(host_cores())
    for _ in range(warmup):
        wl["cpu_run"]()
    t0, done, best = time.perf_counter(), 0, float("inf")
    while done < steps:
        t = time.perf_counter()
        wl["cpu_run"]()
        best = min(best, time.perf_counter() - t)
        done += 1
        if seconds_budget is not None and time.perf_counter() - t0 > seconds_budget:
            break
    return (time.perf_counter() - t0) / done, best, done


def cpu_baseline(wl, seconds_budget=15.0):
    """The oracle port timed on this host's cores, bounded to `seconds_budget` of CPU work."""
    per_step, best, done = time_cpu(wl, 10, 1, seconds_budget)
    work = wl.get("cpu_work", work_per_step(wl))
    return {"value": to_metric(wl, work, best * 1e3), "unit": wl["unit"], "cores": host_cores(), "kind": "port", "sample": wl["cpu_sample"] + f"; best of {done}"}


class NoDist:
    """The reference arm runs on rank 0 alone: no process group."""
    world, rank, local_rank = 1, 0, 0

    def barrier(self): pass
    def reduce(self, v, op="max"): return v
    def close(self): pass


class HostOnly:
    """Stands in for the engine in the reference arm, which needs the workloads' host arrays and module text
    but never touches a GPU: no pinned memory, no compilation."""
    PinnedArray = None

    def __init__(self, rx):
        self.programs = rx.programs

    def compile(self, *a, **k):
        return None


def run_reference(args):
    """Reference arm: the CPU implementation of the path (the oracle port; the reference's own XLA-CPU
    path cannot be installed here: it needs Julia and the Reactant_jll binary) on all host threads, on the
    same workload, shape and seeds as the GPU arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rx = entry.load_package()
    host = HostOnly(rx)
    dist = NoDist()
    wl = WORKLOADS[args.workload](host, None, dist)
    per_step, best, done = time_cpu(wl, args.steps, args.warmup, seconds_budget=150.0)  # the whole run ends within a few minutes
    work = wl.get("cpu_work", work_per_step(wl))
    value = to_metric(wl, work, per_step * 1e3)
    cfg = config_of(args.workload, wl, args.gpus)
    line = {"impl": "reference", "metric": "fused map-reduce HBM GB/s" if wl["unit"] == "GB/s" else "dot_general TFLOP/s", "value": value, "unit": wl["unit"],
            "n_gpus": args.gpus, "steps": done, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": scaling_of(args.workload, args.gpus), "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": wl["unit"], "cores": host_cores(), "kind": "port", "sample": wl["cpu_sample"]},
            "e2e": {"value": value, "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def scaling_of(workload, world):
    return "strong" if ("sinsum" in workload or "jacobi" in workload) and (world > 1 or "c5" in workload) else "weak"


def roofline_of(wl, prof, ms, steps, launches, world, dist, peaks):
    """The dominant kernel: average span of its step kind, measured in the timed region on the launching stream."""
    kind = wl["kind"]
    launches_per_step, kernel = wl.get("launches_per_step", 1), wl["kernel"]
    work = work_per_step(wl)
    if kind == "stencil_tma" and "stencil_tma_loop" in prof:
        # the whole counted loop ran as one cooperative launch: a launch processes every sweep of the step
        kind, launches_per_step, kernel = "stencil_tma_loop", 1, "k_stencil_loop"
    if kind == "gemm_tc" and "gemm_tc_fused" in prof:
        # GEMMs with a fused epilogue are the same kernel compiled around a chain: one family for the roofline
        both = [prof[k] for k in ("gemm_tc", "gemm_tc_fused") if k in prof]
        prof = dict(prof, gemm_tc={"launches": sum(b["launches"] for b in both), "ms": sum(b["ms"] for b in both)})
    if kind not in prof or not prof[kind]["launches"]:
        return None
    if launches == steps * world:
        # one launch per step: the timed region itself is that kernel's launches back to back
        per_launch_ms, timed = ms / steps, "timed region / steps (one launch per step)"
    else:
        per_launch_ms, timed = prof[kind]["ms"] / prof[kind]["launches"], "per-launch event pairs, repeat of the timed region"
    per_launch_ms = dist.reduce(per_launch_ms, "max")
    per_launch_work = work / launches_per_step
    achieved = to_metric(wl, per_launch_work, per_launch_ms)
    if kind == "stencil_rows":
        per_launch_work = work / launches_per_step  # one launch per sweep on every rank, each over its own rows
    peak = (peaks["hbm_gbs"] if wl["bound"] == "hbm" else peaks["bf16_tflops"]) * world
    traffic = None
    if kind in TRAFFIC_RATIO:
        traffic = TRAFFIC_RATIO[kind] * per_launch_work / world  # bytes per launch on one GPU
    elif kind == "stencil_tma_loop" and world == 1:
        traffic = stencil_loop_traffic(wl["shape"]["n"], wl["shape"]["sweeps"])
    return {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": wl["unit"], "frac": achieved / peak, "traffic": traffic,
            "kernel": kernel, "peak_source": f"of {peaks['source']}" + (f" x{world} GPUs" if world > 1 else ""),
            "ms_per_launch": per_launch_ms, "timed_by": timed}


def measure(rx, client, dist, name, steps, warmup, peaks):
    """Device-resident timing, per-kernel spans, roofline and parity of one workload."""
    wl = WORKLOADS[name](rx, client, dist)
    rotate = 4 if name in SMALL_INPUT else 1
    ms, launches, _, result = time_resident(rx, client, wl, steps, warmup, rotate, dist)
    # per-kernel spans from a repeat of the same K steps, each launch bracketed by its own events
    _, _, prof, _ = time_resident(rx, client, wl, steps, 1, rotate, dist, spans=True)
    ms = dist.reduce(ms, "max")
    launches = int(dist.reduce(launches, "sum"))
    value = to_metric(wl, work_per_step(wl) * steps, ms)
    roof = roofline_of(wl, prof, ms, steps, launches, dist.world, dist, peaks)
    parity = wl["check"](result)
    return wl, dict(ms=ms, launches=launches, prof=prof, result=result, value=value, roofline=roof, parity=parity)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the other single-GPU configurations of the default run")
    args = ap.parse_args()
    default_run = args.workload is None
    args.workload = args.workload or "c5_sharded_sinsum_2p30"
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
        if args.workload not in SHARDED:
            raise SystemExit("the sinsum workloads, the Jacobi loops and the data-parallel MLP step shard; logsumexp runs as a single-GPU configuration")
        default_mode = "mailbox+nccl" if args.workload == "c4_mlp_grad_bf16" else "mailbox"
        allreduce = rx.dist.connect_collectives(rx, client, dist, os.environ.get("RX_ALLREDUCE", default_mode))
    peaks = measured_peaks()
    with ClockSampler(dist.local_rank) as clk:  # sampling covers warm-up and the timed region
        wl, m = measure(rx, client, dist, args.workload, args.steps, args.warmup, peaks)
    cfg, unit, dtype = config_of(args.workload, wl, world), wl["unit"], wl["dtype"]
    e2e = None
    if not args.no_e2e:
        e_steps = max(2, min(args.steps, 5))
        ems, _ = time_e2e(rx, client, wl, e_steps, args.warmup, dist)
        ems = dist.reduce(ems, "max")
        e2e = {"value": to_metric(wl, work_per_step(wl) * e_steps, ems), "unit": unit, "h2d_bytes_per_step": wl["h2d"] * world, "d2h_bytes_per_step": wl["d2h"] * world,
               "steps": e_steps, "ms_per_step": ems / e_steps}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(wl)
    ok = m["parity"] is None or m["parity"]["ok"]
    configs, configs_clocks = None, None
    if default_run and world == 1 and not args.no_configs:
        # the other single-GPU configurations, each with the same timing rules (3 warm-up steps, CUDA events on
        # the launching stream, inputs larger than L2 or rotated), its roofline and its parity check
        del wl  # frees the headline workload's host and device arrays
        gc.collect()
        configs = {}
        with ClockSampler(dist.local_rank) as cclk:
            for name in EXTRA_CONFIGS:
                k = min(args.steps, 20)
                w, r = measure(rx, client, dist, name, k, 3, peaks)
                roof = r["roofline"]
                configs[name] = {"value": r["value"], "unit": w["unit"], "ms_per_step": r["ms"] / k, "steps": k, "warmup": 3, "gpu_launches": r["launches"],
                                 "roofline": {q: roof[q] for q in ("bound", "achieved", "peak", "frac", "traffic", "kernel", "ms_per_launch", "peak_source")} if roof else None,
                                 "parity": r["parity"], "config": config_of(name, w, 1), "profile_ms": r["prof"]}
                ok = ok and (r["parity"] is None or r["parity"]["ok"])
                del w, r
                gc.collect()
        configs_clocks = cclk.summary()
    if dist.rank == 0:
        line = {"metric": "fused map-reduce HBM GB/s" if unit == "GB/s" else "dot_general TFLOP/s", "value": m["value"], "unit": unit, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": m["ms"] / args.steps, "higher_is_better": True, "scaling": scaling_of(args.workload, world),
                "vs_baseline": None, "dtype": dtype, "data": "synthetic",
                "config": cfg, "all_reduce": allreduce, "parity": m["parity"],
                "clocks": clk.summary(), "e2e": e2e, "gpu_launches": m["launches"], "roofline": m["roofline"], "cpu_baseline": cpu, "profile_ms": m["prof"]}
        if configs is not None:
            line["configs"] = configs
            line["configs_clocks"] = configs_clocks
        print(json.dumps(line), flush=True)
    client.close()
    dist.close()
    if not ok:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
