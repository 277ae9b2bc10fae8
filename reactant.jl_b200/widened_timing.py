"""Device-resident timings of the programs beyond the five benchmark configurations.

    python reactant.jl_b200/widened_timing.py [jacobi1d] [heat3d] [fdtd2d] [scan] [f64] [spellings] [--small]

For each program: milliseconds per call (CUDA events on the engine's stream around five calls, after three warm-up
calls), algorithmic GB/s, launches per call and the plan's step kinds.  Loop programs donate their arrays and keep
iterating on them from call to call, as a Reactant thunk does.  Parity of the same programs is covered by the tests
(tests/test_widened_gpu.py, tests/test_fdtd.py, tests/test_parity_gpu.py, tests/test_f64.py); this script only times.
`--small` runs every program at a fraction of the size, for profiler captures of the instruction mix.

Algorithmic bytes: one read and one write of every array a (half-)step updates -- jacobi_1d 8 B per point per
half-step, heat_3d 8 B per point per half-step, fdtd_2d ten array passes per time step (benchmark/polybench/
stencil.jl:42-72: EY and EX are read and written, HZ is read twice and then read and written with EX and EY read),
cumsum 8 B per element, the Float64 sinsum 16 B per pair, Jacobi-2D 4 n^2 + 4 (n - 2)^2 per sweep.
"""
from __future__ import annotations

import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import __graft_entry__ as entry  # noqa: E402


def timeit(dev, name, f, args, bytes_per_call, feed=True, reps=5, warmup=3):
    cur = list(args)

    def call():
        nonlocal cur
        out = f(*cur)
        if feed:  # results take the place of the donated arguments
            outs = out if isinstance(out, tuple) else (out,)
            cur = list(outs) + cur[len(outs):]

    for _ in range(warmup):
        call()
    dev.synchronize()
    l0 = dev.kernel_launches()
    e0 = dev.record_event()
    for _ in range(reps):
        call()
    e1 = dev.record_event()
    e1.synchronize()
    ms = e0.elapsed_ms(e1) / reps
    kinds = [s["kind"] for s in f.describe()["steps"]]
    print(f"{name}: {ms:.3f} ms per call, {bytes_per_call / ms / 1e6:.0f} GB/s algorithmic, {(dev.kernel_launches() - l0) // reps} launches per call, plan {kinds}", flush=True)


def main(argv):
    small = "--small" in argv
    which = [a for a in argv if not a.startswith("--")] or ["jacobi1d", "heat3d", "fdtd2d", "scan", "f64", "spellings"]
    rx = entry.load_package()
    client = rx.Client(allowed_devices=[0])
    dev = client.addressable_devices[0]
    P = rx.programs
    rng = np.random.default_rng(0)
    up = lambda x: rx.to_rarray(x, client)
    if "jacobi1d" in which:
        n, steps = (1 << 25) if small else (1 << 26), 10
        f = rx.compile(P.jacobi1d(n, steps), client)
        timeit(dev, f"jacobi_1d n={n} x{steps} iterations", f, [up(rng.random(n, dtype=np.float32)), up(rng.random(n, dtype=np.float32))], 2 * steps * 8.0 * n)
    if "heat3d" in which:
        n, steps = 320 if small else 512, 5
        f = rx.compile(P.heat3d(n, steps), client)
        timeit(dev, f"heat_3d n={n} x{steps} iterations", f, [up(rng.random((n, n, n), dtype=np.float32)), up(rng.random((n, n, n), dtype=np.float32))], 2 * steps * 8.0 * n ** 3)
    if "fdtd2d" in which:
        nx = ny = 2048 if small else 4096
        tmax = 10
        f = rx.compile(P.fdtd2d(nx, ny, tmax), client)
        args = [up(rng.random((nx, ny), dtype=np.float32)) for _ in range(3)] + [up(rng.random(tmax, dtype=np.float32))]
        timeit(dev, f"fdtd_2d {nx}x{ny} x{tmax} steps", f, args, tmax * 10 * 4.0 * nx * ny)
    if "scan" in which:
        n = (1 << 25) if small else (1 << 28)
        f = rx.compile(P.scan([n], 0), client)
        timeit(dev, f"cumsum n={n}", f, [up(rng.random(n, dtype=np.float32))], 8.0 * n, feed=False)
        r = c = 8192 if small else 16384
        x = rng.random((r, c), dtype=np.float32)
        for ax, what in ((0, "strided"), (1, "contiguous")):
            f = rx.compile(P.scan([r, c], ax), client)
            timeit(dev, f"cumsum {r}x{c} along the {what} dim", f, [up(x.T)], 8.0 * r * c, feed=False)
    if "f64" in which:
        n = (1 << 23) if small else (1 << 26)
        f = rx.compile(P.sinsum_add(n).replace("f32", "f64"), client)
        timeit(dev, f"sinsum Float64 n={n}", f, [up(rng.uniform(-3, 3, n)), up(rng.uniform(-3, 3, n))], 16.0 * n, feed=False)
    if "spellings" in which:
        n, steps = 4096 if small else 8192, 20
        a, b = rng.random((n, n), dtype=np.float32), rng.random((n, n), dtype=np.float32)
        for form in ("dus", "pad", "concat", "halfsteps"):
            f = rx.compile(P.jacobi2d(n, steps if form != "halfsteps" else steps // 2, form=form), client)
            timeit(dev, f"jacobi_2d {form} spelling n={n} x{steps} sweeps", f, [up(a), up(b)], steps * (4.0 * n * n + 4.0 * (n - 2) * (n - 2)))
    client.close()


if __name__ == "__main__":
    main(sys.argv[1:])
