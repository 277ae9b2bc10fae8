"""Programs either side of the hot path: the 1-D and 3-D slice-and-add loops of Reactant's polybench file, the gelu op
NNlib's activations trace to, and the executable / device queries Reactant's compile path makes besides execute."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,steps", [(8, 1), (2048, 5), ((1 << 20) + 6, 3)])
def test_jacobi_1d_bit_exact(rx, ref, client, n, steps):
    """benchmark/polybench/stencil.jl:201-221: both half-steps in place, as strided map launches."""
    rng = np.random.default_rng(n)
    a, b = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
    text = rx.programs.jacobi1d(n, steps)
    f = rx.compile(text, client)
    plan = f.describe()
    assert plan["slots"] == 2 and not any(s["kind"] == "copy" for s in plan["steps"][0]["body"])
    ra, rb = f(rx.to_rarray(a, client), rx.to_rarray(b, client))
    wa, wb = ref.run_module(text, [a, b])
    assert np.array_equal(np.asarray(ra), wa) and np.array_equal(np.asarray(rb), wb)


@pytest.mark.parametrize("n,steps", [(4, 1), (18, 3), (120, 2)])
def test_heat_3d_bit_exact(rx, ref, client, n, steps):
    """benchmark/polybench/stencil.jl:125-169: the 7-point update of the interior, A -> B then B -> A per iteration."""
    rng = np.random.default_rng(n)
    a, b = rng.random((n, n, n), dtype=np.float32), rng.random((n, n, n), dtype=np.float32)
    text = rx.programs.heat3d(n, steps)
    f = rx.compile(text, client)
    assert f.describe()["slots"] == 2
    ra, rb = f(rx.to_rarray(a.T, client), rx.to_rarray(b.T, client))
    wa, wb = ref.run_module(text, [a, b])
    assert np.array_equal(np.asarray(ra).T, wa) and np.array_equal(np.asarray(rb).T, wb)


@pytest.mark.parametrize("approx", ["TANH", "SIGMOID"])
def test_math_gelu_is_expanded_and_fused(rx, ref, client, approx):
    """enzymexla.math.gelu (ext/ReactantNNlibExt/Implementations.jl:12-25): accepted in MLIR's generic form, expanded into
    elementwise ops and fused with its neighbours; compared with the closed form in float64."""
    n = 1 << 16
    t = f"tensor<{n}xf32>"
    text = (f"module {{\n  func.func @main(%arg0: {t}) -> tensor<f32> {{\n    %cst = stablehlo.constant dense<0.000000e+00> : tensor<f32>\n"
            f'    %0 = "enzymexla.math.gelu"(%arg0) <{{gelu_approximation = #enzymexla<gelu_approximation {approx}>}}> : ({t}) -> {t}\n'
            f"    %1 = stablehlo.multiply %0, %0 : {t}\n"
            f"    %2 = stablehlo.reduce(%1 init: %cst) applies stablehlo.add across dimensions = [0] : ({t}, tensor<f32>) -> tensor<f32>\n"
            f"    return %2 : tensor<f32>\n  }}\n}}\n")
    assert [s["kind"] for s in rx.plan_describe(text)["steps"]] == ["reduce_full"]
    x = np.random.default_rng(1).standard_normal(n).astype(np.float32) * 2
    got = float(rx.compile(text, client)(rx.to_rarray(x, client)))
    want = float(ref.run_module(text, [x])[0])
    assert abs(got - want) <= 1e-5 * np.sqrt(16) * abs(want) + 1e-6 * abs(want)
    none = text.replace(approx, "NONE")
    with pytest.raises(rx.ReactantError) as e:
        rx.compile(none, client)
    assert e.value.code == 2 and "gelu" in str(e.value)


def test_dot_general_algorithm_presets(rx, ref, client):
    """src/Configuration.jl:216-238: BF16_BF16_F32 on bf16 operands is what the tensor-core kernel computes; the
    multi-pass presets and a bf16 accumulator are refused by name."""
    alg = lambda l, a, n: (f", algorithm = <lhs_precision_type = {l}, rhs_precision_type = {l}, accumulation_type = {a}, lhs_component_count = 1, "
                           f"rhs_component_count = 1, num_primitive_operations = {n}, allow_imprecise_accumulation = false>")
    base = rx.programs.matmul(256, 256, 256, et="bf16")
    ok = base.replace("precision = [DEFAULT, DEFAULT]", "precision = [DEFAULT, DEFAULT]" + alg("bf16", "f32", 1))
    rng = np.random.default_rng(0)
    a = ref.round_to_bf16(rng.standard_normal((256, 256)).astype(np.float32))
    b = ref.round_to_bf16(rng.standard_normal((256, 256)).astype(np.float32))
    up = lambda m: rx.to_rarray(m.T.astype(rx.bfloat16), client)
    got = np.asarray(rx.compile(ok, client)(up(a), up(b))).T.astype(np.float32)
    plain = np.asarray(rx.compile(base, client)(up(a), up(b))).T.astype(np.float32)
    assert np.array_equal(got, plain)
    for l, acc, n in [("bf16", "f32", 3), ("bf16", "bf16", 1), ("f32", "f32", 1)]:
        bad = base.replace("precision = [DEFAULT, DEFAULT]", "precision = [DEFAULT, DEFAULT]" + alg(l, acc, n))
        with pytest.raises(rx.ReactantError) as e:
            rx.compile(bad, client)
        assert e.value.code == 2 and "algorithm" in str(e.value)


def test_sharding_getters_and_handle_ownership(rx, client):
    """What Reactant asks of every loaded executable (src/xla/PJRT/LoadedExecutable.jl:34-60): parameter and result
    shardings as OpSharding objects, and the (absent) HLO modules."""
    lib = rx._lib.lib()
    f = rx.compile(rx.programs.logsumexp_dims1(64, 8), client)
    out = (C.c_void_p * 1)()
    lib.PjRtLoadedExecutableGetParameterShardings(f.handle, out, 1)
    rx._lib.check()
    assert lib.op_sharding_to_op_sharding_type(out[0]) == 0 and lib.op_sharding_has_tile_assignment_devices(out[0]) == 0
    lib.free_op_sharding(out[0])
    lib.PjRtLoadedExecutableGetOuputShardings(f.handle, out, 2)   # wrong count: reported, nothing written
    with pytest.raises(rx.ReactantError) as e:
        rx._lib.check()
    assert "Expected 2 shardings, got 1" in str(e.value)
    n = C.c_int32(7)
    lib.PjRtLoadedExecutableGetHloModules(f.handle, None, C.byref(n))
    assert n.value == 0
    x = rx.to_rarray(np.zeros((64, 8), np.float32), client)
    dev = client.addressable_devices[0]
    for h in (client.handle, dev.handle, f.handle, x.data[0].handle):
        assert lib.RxOwns(h) == 1
    junk = C.c_int(0)
    assert lib.RxOwns(C.addressof(junk)) == 0
    kind = rx._lib.take_string(lib.DeviceGetKind(dev.handle))
    assert "sm_" in kind and kind != "unknown"
    props = (C.c_ubyte * 128)()
    lib.ReactantCudaDeviceGetProperties(props, 0)
    rx._lib.check()
    assert int.from_bytes(bytes(props[0:8]), "little") > (1 << 30)  # totalGlobalMem
    assert lib.ReactantCudaDeviceGetWarpSizeInThreads() == 32 and lib.ReactantCudaDriverGetVersion() >= 12000


def test_sharded_executable_reports_tiled_op_shardings(rx):
    lib = rx._lib.lib()
    text = rx.programs.sinsum_add(1 << 12, num_partitions=4)
    # the getters only read the plan: no multi-GPU client is needed to compile a partitioned module
    client = rx.Client(allowed_devices=[0])
    try:
        f = rx.compile(text, client)
        out = (C.c_void_p * 2)()
        lib.PjRtLoadedExecutableGetParameterShardings(f.handle, out, 2)
        rx._lib.check()
        for k in range(2):
            assert lib.op_sharding_to_op_sharding_type(out[k]) == 3
            assert lib.op_sharding_tile_assignment_dimensions_size(out[k]) == 1 and lib.op_sharding_tile_assignment_devices_size(out[k]) == 4
            dims, devs = (C.c_int32 * 1)(), (C.c_int32 * 4)()
            lib.op_sharding_tile_assignment_dimensions(out[k], dims)
            lib.op_sharding_tile_assignment_devices(out[k], devs)
            assert list(dims) == [4] and list(devs) == [0, 1, 2, 3]
            lib.free_op_sharding(out[k])
        res = (C.c_void_p * 1)()
        lib.PjRtLoadedExecutableGetOuputShardings(f.handle, res, 1)
        assert lib.op_sharding_to_op_sharding_type(res[0]) == 0  # the all-reduced scalar is replicated
        lib.free_op_sharding(res[0])
    finally:
        client.close()
