"""The bounds-checked build of the library (build.py --bounds, -DRX_BOUNDS=1): every element access of the chain
kernels, of the fused GEMM epilogues and of the stencil's stores is checked against the extent of the buffer behind
it; a miss is recorded, the access is skipped and the host reports it -- nothing traps.  It stands in for a memory
checker on machines where none can be run.

CPU: the variant builds, exports the whole ABI and compiles chains.  GPU (child processes, because a process can
hold only one build of the library): a sample of programs of every kernel family gives the same results as under the
normal build with no miss recorded, and with every extent understated by one element (RX_BOUNDS_SELFTEST=1, which
makes a correct program trip the check on a buffer's last element without any out-of-range access) the miss is
reported through the normal error path and the device stays usable."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOUNDS_LIB = os.path.join(ROOT, "reactant.jl_b200", "librx_b200_bounds.so")

CHILD = r"""
import json, os, sys
import numpy as np
sys.path.insert(0, os.environ["RX_ROOT"])
sys.path.insert(0, os.path.join(os.environ["RX_ROOT"], "tests"))
import __graft_entry__ as entry
rx = entry.load_package(); ref, _ = entry.load_oracle()
client = rx.Client(allowed_devices=[0])
out = {}
rng = np.random.default_rng(3)

def run(text, ins):
    args = [rx.to_rarray(np.ascontiguousarray(a.T), client) for a in ins]
    res = rx.compile(text, client)(*args)
    res = res if isinstance(res, (tuple, list)) else [res]
    return [np.asarray(r).T for r in res]

try:
    # full reduce over a generic chain (interpreter) and, above the threshold, the specialised kernel
    for n in (1000, (1 << 20) + 8):
        x = rng.uniform(-3, 3, n).astype(np.float32); y = rng.uniform(-3, 3, n).astype(np.float32)
        text = rx.programs.sinsum_add(n).replace("stablehlo.sine", "stablehlo.cosine")
        got = run(text, [x, y])[0]; want = ref.run_module(text, [x, y])[0]
        assert abs(float(got) - float(want)) <= 1e-4 * max(1.0, abs(float(want)) + np.sqrt(n)), (got, want)
    # strided maps and axis reductions
    a = rng.standard_normal((37, 53)).astype(np.float32)   # Julia layout: the module takes the reversed dims
    text = rx.programs.logsumexp_dims1(37, 53)
    got = np.asarray(rx.compile(text, client)(rx.to_rarray(a, client)))
    want = ref.run_module(text, [ref.julia_to_xla(a)])[0].T
    np.testing.assert_allclose(got, want, rtol=1e-5)
    # stencil: TMA path (row pitch a multiple of 16 bytes) and the strided map path
    for n, sweeps in ((36, 3), (33, 3), (516, 7)):   # the last one runs two sweeps per pass over memory
        A = rng.random((n, n), dtype=np.float32); B = rng.random((n, n), dtype=np.float32)
        text = rx.programs.jacobi2d(n, sweeps)
        ga, gb = run(text, [A, B]); wa, wb = ref.run_module(text, [A, B])
        assert np.array_equal(ga, wa) and np.array_equal(gb, wb)
    # GEMM with a fused epilogue (direct operand loads, staged and direct stores, column sums)
    from test_gemm_epilogue import bias_gelu_module
    M, N, K = 256, 256, 64
    P = ref.round_to_bf16(rng.standard_normal((M, K)).astype(np.float32)); Q = ref.round_to_bf16((rng.standard_normal((K, N)) / 8).astype(np.float32))
    bias = rng.standard_normal(N).astype(np.float32)
    text = bias_gelu_module(M, N, K, with_sum=True)
    f = rx.compile(text, client)
    h, s = f(rx.to_rarray(P.T.astype(rx.bfloat16), client), rx.to_rarray(Q.T.astype(rx.bfloat16), client), rx.to_rarray(bias, client))
    wh, ws = ref.run_module(text, [P, Q, bias])
    np.testing.assert_allclose(np.asarray(h).T.astype(np.float32), wh.astype(np.float32), atol=2e-2 * np.abs(wh).max())
    np.testing.assert_allclose(np.asarray(s), ws, atol=2e-2 * np.abs(ws).max())
    out["ok"] = True
except rx.ReactantError as e:
    out["error"] = str(e); out["code"] = e.code
    # the device is still usable after a reported miss
    if os.environ.get("RX_BOUNDS_SELFTEST"):
        os.environ.pop("RX_BOUNDS_SELFTEST")
    x = rx.to_rarray(np.zeros(16, np.float32), client)
    out["alive"] = float(np.asarray(x).sum()) == 0.0
print(json.dumps(out))
"""


def _child(env_extra):
    env = dict(os.environ, RX_ROOT=ROOT, RX_B200_LIB=BOUNDS_LIB, **env_extra)
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def test_bounds_variant_builds_and_exports_the_abi():
    if not os.path.exists(BOUNDS_LIB):
        pytest.skip("librx_b200_bounds.so has not been built (python reactant.jl_b200/build.py --bounds)")
    code = (
        "import os, sys; sys.path.insert(0, os.environ['RX_ROOT']); import __graft_entry__ as e; rx = e.load_package(); l = rx._lib.lib();"
        "assert rx._lib.LIB_PATH.endswith('_bounds.so');"
        "out = rx.specialise_check(rx.programs.sinsum_add(1 << 21)); assert out and all(o['cubin_bytes'] > 0 for o in out); print('ok')"
    )
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=dict(os.environ, RX_ROOT=ROOT, RX_B200_LIB=BOUNDS_LIB), cwd=ROOT)
    assert r.returncode == 0 and "ok" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])


@pytest.mark.gpu
def test_sample_of_every_kernel_family_runs_clean_under_the_bounds_build():
    if not os.path.exists(BOUNDS_LIB):
        pytest.skip("librx_b200_bounds.so has not been built")
    out = _child({})
    assert out.get("ok") is True, out


@pytest.mark.gpu
def test_an_understated_extent_is_reported_and_the_access_skipped():
    if not os.path.exists(BOUNDS_LIB):
        pytest.skip("librx_b200_bounds.so has not been built")
    out = _child({"RX_BOUNDS_SELFTEST": "1"})
    assert "bounds check" in out.get("error", "") and out.get("alive") is True, out
