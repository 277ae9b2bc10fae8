"""fdtd_2d_vectorized (benchmark/polybench/stencil.jl:42-72): a counted loop whose body reads a scalar at the traced
loop variable (`fict[t]`: stablehlo.dynamic_slice with a start index that is affine in the counter) and updates three
fields in place, each update reading its own target at the position it writes.

CPU: the oracle against a direct numpy restatement of the Julia loop; the plan (a dyn_slice step whose offset follows
the counter, four in-place maps, no copies); what is refused.  GPU: bit-exact against the oracle (every operation of
the body is a single correctly rounded add, subtract or multiply)."""
import numpy as np
import pytest


def direct(EX, EY, HZ, fict):
    ex, ey, hz = EX.copy(), EY.copy(), HZ.copy()
    h, s = np.float32(0.5), np.float32(0.7)
    for t in range(len(fict)):
        ey[0, :] = fict[t]
        ey[1:, :] = ey[1:, :] - h * (hz[1:, :] - hz[:-1, :])
        ex[:, 1:] = ex[:, 1:] - h * (hz[:, 1:] - hz[:, :-1])
        hz[:-1, :-1] = hz[:-1, :-1] - s * (((ex[:-1, 1:] - ex[:-1, :-1]) + ey[1:, :-1]) - ey[:-1, :-1])
    return ex, ey, hz


def fields(nx, ny, tmax, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.random((nx, ny), dtype=np.float32) for _ in range(3)] + [rng.random(tmax, dtype=np.float32)]


def test_oracle_matches_the_julia_loop(rx, ref):
    EX, EY, HZ, fict = fields(12, 10, 5)
    got = ref.run_module(rx.programs.fdtd2d(12, 10, 5), [EX.T.copy(), EY.T.copy(), HZ.T.copy(), fict])
    for g, w in zip(got, direct(EX, EY, HZ, fict)):
        assert np.array_equal(g.T, w)


def test_plan_follows_the_counter_and_updates_in_place(rx):
    p = rx.plan_describe(rx.programs.fdtd2d(1024, 2048, 256))
    assert [s["kind"] for s in p["steps"]] == ["loop"] and p["steps"][0]["trip"] == 256
    body = p["steps"][0]["body"]
    assert [s["kind"] for s in body] == ["dyn_slice", "map", "map", "map", "map"], body
    assert p["slots"] == 5   # three fields, fict, and the scalar read each iteration: no copy of any field
    # a start index that is not affine in the counter (here: the counter squared) is refused by name
    text = rx.programs.fdtd2d(12, 10, 5).replace("stablehlo.multiply %iterArg, %c_2", "stablehlo.multiply %iterArg, %iterArg")
    with pytest.raises(rx.ReactantError) as e:
        rx.plan_describe(text)
    assert e.value.code == 2 and "affine" in str(e.value)


def test_constant_start_indices_are_a_clamped_slice(rx, ref):
    t = "tensor<8x6xf32>"
    text = f"""module {{
  func.func @main(%arg0: {t}) -> tensor<3x6xf32> {{
    %c = stablehlo.constant dense<7> : tensor<i32>
    %z = stablehlo.constant dense<0> : tensor<i32>
    %0 = stablehlo.dynamic_slice %arg0, %c, %z, sizes = [3, 6] : ({t}, tensor<i32>, tensor<i32>) -> tensor<3x6xf32>
    return %0 : tensor<3x6xf32>
  }}
}}
"""
    x = np.arange(48, dtype=np.float32).reshape(8, 6)
    assert np.array_equal(ref.run_module(text, [x])[0], x[5:8])   # start 7 clamped to 5
    assert [s["kind"] for s in rx.plan_describe(text)["steps"]] in (["map"], ["copy"])


@pytest.mark.gpu
@pytest.mark.parametrize("nx,ny,tmax", [(12, 10, 5), (64, 96, 7), (260, 132, 9), (1024, 512, 4), (2308, 516, 3)])
def test_fdtd2d_bit_exact(rx, ref, client, nx, ny, tmax):
    EX, EY, HZ, fict = fields(nx, ny, tmax, seed=nx)
    text = rx.programs.fdtd2d(nx, ny, tmax)
    f = rx.compile(text, client)
    out = f(rx.to_rarray(EX, client), rx.to_rarray(EY, client), rx.to_rarray(HZ, client), rx.to_rarray(fict, client))
    want = ref.run_module(text, [EX.T.copy(), EY.T.copy(), HZ.T.copy(), fict])
    for g, w in zip(out, want):
        assert np.array_equal(np.asarray(g).T, w)


@pytest.mark.gpu
def test_constant_dynamic_slice_on_the_gpu(rx, ref, client):
    t = "tensor<8x6xf32>"
    text = f"""module {{
  func.func @main(%arg0: {t}) -> tensor<3x6xf32> {{
    %c = stablehlo.constant dense<7> : tensor<i32>
    %z = stablehlo.constant dense<0> : tensor<i32>
    %0 = stablehlo.dynamic_slice %arg0, %c, %z, sizes = [3, 6] : ({t}, tensor<i32>, tensor<i32>) -> tensor<3x6xf32>
    return %0 : tensor<3x6xf32>
  }}
}}
"""
    x = np.arange(48, dtype=np.float32).reshape(8, 6)
    got = np.asarray(rx.compile(text, client)(rx.to_rarray(np.ascontiguousarray(x.T), client))).T
    assert np.array_equal(got, x[5:8])
