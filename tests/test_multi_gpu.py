"""Sharded execution on several GPUs of one process (the shape a Julia session
has): XLAExecute with [device][arg] buffers, local reduce + all-reduce, every
device ends with the same bits.  Skipped when the box has fewer GPUs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ngpu():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.parametrize("ndev", [2, 4, 8])
@pytest.mark.parametrize("transport", ["mailbox", "nccl"])
def test_sharded_sinsum_matches_unsharded(rx, ref, ndev, transport, monkeypatch):
    if _ngpu() < ndev:
        pytest.skip(f"needs {ndev} GPUs")
    monkeypatch.setenv("RX_ALLREDUCE", transport)
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    client = rx.Client(allowed_devices=list(range(ndev)))
    try:
        n = ndev * ((1 << 18) + 4)
        rng = np.random.default_rng(ndev)
        x = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
        y = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
        mesh = rx.Mesh(client.devices, ("x",))
        sh = rx.NamedSharding(mesh, ("x",))
        X, Y = rx.to_rarray(x, client, sharding=sh), rx.to_rarray(y, client, sharding=sh)
        assert len(X.data) == ndev and X.data[1].dims == (n // ndev,)
        assert np.array_equal(np.asarray(X), x), "gathering the shards restores the array"
        f = rx.compile(rx.programs.sinsum_add(n, num_partitions=ndev), client)
        r = f(X, Y)
        assert len(r.data) == ndev, "the scalar result is replicated on every device"
        vals = [b.to_host().item() for b in r.data]
        assert len(set(np.float32(v).tobytes() for v in vals)) == 1, vals
        terms = np.sin(x.astype(np.float64)) + y
        assert abs(vals[0] - terms.sum()) <= ref.reduction_tolerance(n) * max(abs(terms.sum()), np.linalg.norm(terms))
        # a second call (next all-reduce epoch) gives the same bits
        r2 = f(X, Y)
        assert r2.data[0].to_host().tobytes() == r.data[0].to_host().tobytes()
    finally:
        client.close()


def test_sharded_executable_refuses_a_partial_mesh(rx):
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    client = rx.Client(allowed_devices=[0, 1])
    try:
        f = rx.compile(rx.programs.sinsum_add(1 << 12, num_partitions=4), client)
        mesh = rx.Mesh(client.devices, ("x",))
        sh = rx.NamedSharding(mesh, ("x",))
        x = np.zeros(1 << 11, np.float32)  # wrong on purpose: 2 devices for a 4-way program
        X = rx.to_rarray(x, client, sharding=sh)
        with pytest.raises(rx.ReactantError):
            f(X, X)
    finally:
        client.close()


def test_column_sharded_logsumexp_needs_no_collective(rx, ref):
    """logsumexp(x; dims=1) with the columns split over the mesh: every device reduces its own
    columns, the result stays sharded, and no all-reduce is planned."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    ndev = 2
    rows, cols = 4096, 64
    text = rx.programs.logsumexp_dims1(rows, cols)
    shard = ' {sdy.sharding = #sdy.sharding<@mesh, [{"x"}, {}]>}'
    text = text.replace("mhlo.num_partitions = 1", f"mhlo.num_partitions = {ndev}")
    text = text.replace("  func.func @main(%arg0: tensor<64x4096xf32>", f'  sdy.mesh @mesh = <["x"={ndev}]>\n  func.func @main(%arg0: tensor<64x4096xf32>{shard}')
    plan = rx.plan_describe(text)
    assert [s["kind"] for s in plan["steps"]] == ["logsumexp"], plan
    client = rx.Client(allowed_devices=list(range(ndev)))
    try:
        a = np.random.default_rng(5).standard_normal((rows, cols)).astype(np.float32)  # Julia rows x cols
        mesh = rx.Mesh(client.devices, ("x",))
        X = rx.to_rarray(a, client, sharding=rx.NamedSharding(mesh, (None, "x")))     # columns (Julia dim 2) sharded
        f = rx.compile(text, client)
        r = f(X)
        got = np.asarray(r)
        want = ref.run_module(rx.programs.logsumexp_dims1(rows, cols), [ref.julia_to_xla(a)])[0].T
        assert got.shape == want.shape == (1, cols)
        np.testing.assert_allclose(got, want, rtol=ref.reduction_tolerance(rows))
    finally:
        client.close()


@pytest.mark.parametrize("transport", ["mailbox", "nccl"])
def test_data_parallel_mlp_gradients(rx, ref, transport, monkeypatch):
    """Batch-sharded MLP forward + gradients: local GEMMs, then all-reduce of every gradient and of
    the loss (vector payloads go through NCCL, the scalar through the fused mailbox path unless
    NCCL is forced).  Must match the unsharded oracle."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    ndev = 2
    monkeypatch.setenv("RX_ALLREDUCE", transport)
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    F, H, O, B = 64, 128, 32, 512
    rng = np.random.default_rng(6)
    bf = lambda a: ref.round_to_bf16(a.astype(np.float32))
    X = bf(rng.standard_normal((B, F)))
    W1 = bf(rng.standard_normal((F, H)) / np.sqrt(F))
    W2 = bf(rng.standard_normal((H, O)) / np.sqrt(H))
    b1 = (0.01 * rng.standard_normal(H)).astype(np.float32)
    b2 = (0.01 * rng.standard_normal(O)).astype(np.float32)
    Y = rng.standard_normal((B, O)).astype(np.float32)
    want = ref.run_module(rx.programs.mlp_grad(F, H, O, B), [W1, b1, W2, b2, X, Y])
    client = rx.Client(allowed_devices=list(range(ndev)))
    try:
        mesh = rx.Mesh(client.devices, ("x",))
        rep2, rep1 = rx.NamedSharding(mesh, (None, None)), rx.NamedSharding(mesh, (None,))
        batch = rx.NamedSharding(mesh, (None, "x"))          # Julia (features, batch): batch is dim 2
        up = lambda a, sh, bf16=False: rx.to_rarray(a.T.astype(rx.bfloat16) if bf16 else a.T, client, sharding=sh)
        args = [up(W1, rep2, True), up(b1, rep1), up(W2, rep2, True), up(b2, rep1), up(X, batch, True), up(Y, batch)]
        f = rx.compile(rx.programs.mlp_grad(F, H, O, B, num_partitions=ndev), client)
        kinds = [s["kind"] for s in f.describe()["steps"]]
        assert kinds.count("all_reduce") == 5 and kinds.count("gemm") == 5
        outs = f(*args)
        for name, o, w in zip(("dW1", "db1", "dW2", "db2", "loss"), outs, want):
            assert len(o.data) == ndev
            per_dev = [np.asarray(b.to_host()).astype(np.float32) for b in o.data]
            assert all(np.array_equal(per_dev[0], p) for p in per_dev[1:]), f"{name} differs between devices"
            g = per_dev[0]
            scale = np.abs(w).max()
            assert np.abs(g - w).max() <= 2e-2 * scale, (name, np.abs(g - w).max(), scale)
    finally:
        client.close()


def test_sharded_reduce_with_a_nonzero_init_counts_it_once(rx, ref):
    """reduce(+, x; init = 5) over a sharded vector: the init value must enter the result once, not once per device."""
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    ndev, n = 2, 1 << 12
    client = rx.Client(allowed_devices=list(range(ndev)))
    try:
        text = rx.programs.sinsum_add(n, num_partitions=ndev).replace("dense<0.000000e+00> : tensor<f32>", "dense<5.000000e+00> : tensor<f32>")
        rng = np.random.default_rng(3)
        x = rng.uniform(-1, 1, n).astype(np.float32)
        y = rng.uniform(-1, 1, n).astype(np.float32)
        sh = rx.NamedSharding(rx.Mesh(client.devices, ("x",)), ("x",))
        r = rx.compile(text, client)(rx.to_rarray(x, client, sharding=sh), rx.to_rarray(y, client, sharding=sh))
        want = float(ref.run_module(text, [x, y])[0])
        for b in r.data:
            assert abs(float(b.to_host()) - want) <= 1e-4 * abs(want), (float(b.to_host()), want)
    finally:
        client.close()


def test_one_process_per_gpu_mesh_matches_the_float64_sum():
    """The deployment shape the scaling benchmark measures: two processes, one GPU each, mailboxes exchanged as
    IPC handles, local shards uploaded by their owners.  The benchmark itself compares the all-reduced result with
    the float64 sum of the same seeded input and exits non-zero when they disagree."""
    import json
    import os
    import subprocess
    import sys
    if _ngpu() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port", "29617",
           os.path.join(root, "bench.py"), "--gpus", "2", "--steps", "3", "--warmup", "3", "--workload", "c1_sinsum_2p24", "--no-e2e"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root, env=env)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    line = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")][-1]
    assert line["n_gpus"] == 2 and line["all_reduce"] == "nvlink-mailbox"
    assert line["parity"]["ok"] and line["parity"]["same_bits_on_every_rank"], line["parity"]


@pytest.mark.parametrize("whole_loop", [True, False])
@pytest.mark.parametrize("ndev", [2, 4])
@pytest.mark.parametrize("n,steps,form", [(64, 3, "dus"), (516, 5, "dus"), (1028, 12, "dus"), (64, 6, "dus"), (1028, 4, "halfsteps"), (260, 7, "halfsteps")])
def test_row_sharded_jacobi_with_halo_exchange_is_bit_exact(rx, ref, ndev, n, steps, form, whole_loop, monkeypatch):
    """Both arrays split into row blocks over the mesh (Julia's second dimension); every sweep each device updates the
    rows it owns and sends its boundary rows to its neighbours' halos.  Same bits as the unsharded program, whether
    the loop runs as one cooperative launch per device with the exchange between the sweeps inside the kernel, or
    (RX_STENCIL_LOOP=0) as one stencil launch and one exchange launch per sweep."""
    if _ngpu() < ndev:
        pytest.skip(f"needs {ndev} GPUs")
    if n % ndev:
        pytest.skip("rows do not divide")
    if whole_loop:
        monkeypatch.delenv("RX_STENCIL_LOOP", raising=False)
    else:
        monkeypatch.setenv("RX_STENCIL_LOOP", "0")
    client = rx.Client(allowed_devices=list(range(ndev)))
    try:
        rng = np.random.default_rng(n + steps)
        a = rng.random((n, n), dtype=np.float32)   # boundary layout [rows][cols]
        b = rng.random((n, n), dtype=np.float32)
        sh = rx.NamedSharding(rx.Mesh(client.devices, ("x",)), (None, "x"))
        A, B = rx.to_rarray(a.T, client, sharding=sh), rx.to_rarray(b.T, client, sharding=sh)
        assert A.data[0].dims == (n // ndev, n)
        f = rx.compile(rx.programs.jacobi2d(n, steps, form=form, num_partitions=ndev), client)
        kinds = [s["kind"] for s in f.describe()["steps"]]
        assert kinds == ["rows_in", "rows_in", "loop", "rows_out", "rows_out"], kinds
        before = [d.kernel_launches() for d in client.addressable_devices]
        ra, rb = f(A, B)
        launched = [d.kernel_launches() - b0 for d, b0 in zip(client.addressable_devices, before)]
        sweeps = steps * (2 if form == "halfsteps" else 1)
        # two exchange launches for the arrays' first halos, then one launch for the whole loop or two per sweep
        assert all(l == (3 if whole_loop else 2 + 2 * sweeps) for l in launched), launched
        wa, wb = ref.run_module(rx.programs.jacobi2d(n, steps, form=form), [a, b])
        assert np.array_equal(np.asarray(ra).T, wa) and np.array_equal(np.asarray(rb).T, wb)
        # a second execution (later sequence numbers of the exchange) continues from the results
        ra2, rb2 = f(ra, rb)
        wa2, wb2 = ref.run_module(rx.programs.jacobi2d(n, steps, form=form), [wa, wb])
        assert np.array_equal(np.asarray(ra2).T, wa2) and np.array_equal(np.asarray(rb2).T, wb2)
    finally:
        client.close()
