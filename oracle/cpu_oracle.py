"""ctypes wrapper of the C oracle kernels (oracle/rx_oracle.c).

TEST INFRASTRUCTURE: only tests/, the smoke check and the CPU legs of bench.py
may import this.  Arrays are passed in the boundary layout (row-major over the
reversed Julia dims).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def _cpu_tag() -> str:
    """The library is built with -march=native, so it is keyed by the host's CPU flags."""
    import hashlib
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return "." + hashlib.sha1(flags.encode()).hexdigest()[:10]


_SO = os.path.join(HERE, f"librx_oracle{_cpu_tag()}.so")


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(os.path.join(HERE, "rx_oracle.c")):
            subprocess.run(["make", "-s", "-C", HERE, f"TAG={_cpu_tag()}"], check=True)
        _lib = C.CDLL(_SO)
        _lib.rx_oracle_sinsum_add.restype = C.c_float
        _lib.rx_oracle_sinsum_add.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        _lib.rx_oracle_logsumexp_dims1.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        _lib.rx_oracle_jacobi2d.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]
        _lib.rx_oracle_jacobi2d_order.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int]
        _lib.rx_oracle_threads.restype = C.c_int
        _lib.rx_oracle_set_threads.argtypes = [C.c_int]
        _lib.rx_oracle_sinsum_add_f64.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    return _lib


def threads() -> int:
    return int(lib().rx_oracle_threads())


def set_threads(n: int | None = None) -> int:
    """Use `n` OpenMP threads (default: every core this process may run on), whatever OMP_NUM_THREADS says."""
    if n is None:
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:  # pragma: no cover
            n = os.cpu_count() or 1
    lib().rx_oracle_set_threads(int(n))
    return threads()


def sinsum_add_f64(x, y):
    """(sum, sum of squares) of sin(x) + y in float64: the ground truth of the fp32 tolerance checks."""
    x, px = _f32(x)
    y, py = _f32(y)
    s, q = C.c_double(), C.c_double()
    lib().rx_oracle_sinsum_add_f64(px, py, x.size, C.byref(s), C.byref(q))
    return s.value, q.value


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.c_void_p)


def sinsum_add(x, y) -> float:
    x, px = _f32(x)
    y, py = _f32(y)
    return float(lib().rx_oracle_sinsum_add(px, py, x.size))


def logsumexp_dims1(x_xla) -> np.ndarray:
    """x_xla: [cols][rows]; returns [cols]."""
    x, px = _f32(x_xla)
    cols, rows = x.shape
    out = np.empty(cols, dtype=np.float32)
    lib().rx_oracle_logsumexp_dims1(px, rows, cols, out.ctypes.data_as(C.c_void_p))
    return out


def jacobi2d(a_xla, b_xla, steps: int, order: str = "baseline"):
    """`steps` sweeps with the roles of the arrays swapping after each.  order="baseline": terms added as centre,
    i-1, i+1, j-1, j+1 (Julia indices); order="polybench": centre, j-1, j+1, i+1, i-1, the order of
    benchmark/polybench/stencil.jl:267-287 (one of its iterations is two sweeps)."""
    a = np.array(a_xla, dtype=np.float32, order="C", copy=True)
    b = np.array(b_xla, dtype=np.float32, order="C", copy=True)
    lib().rx_oracle_jacobi2d_order(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), a.shape[0], steps, {"baseline": 0, "polybench": 1}[order])
    return a, b
