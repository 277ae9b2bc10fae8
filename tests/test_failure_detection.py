"""Failure detection without faulting a GPU.

Device side: every wait is bounded.  Here a two-rank mesh is declared but the
second rank never exists, so the word this rank waits for in its all-reduce
mailbox is never written; the kernel gives up after its poll limit, returns
normally, and the host reports RX_ERR_PEER_TIMEOUT at the next read -- the
context stays usable.  Host side: error codes for misuse of handles.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_all_reduce_wait_runs_out_and_is_reported(rx, ref):
    # rank 0 of a 2-process mesh; both mailbox slots point at this process's own mailbox,
    # so nothing ever writes rank 1's word
    client = rx.Client(node_id=0, num_nodes=2, allowed_devices=[0], peer_wait_ms=500)
    try:
        h = client.mailbox_handles()
        assert len(h) == 64
        client.open_mailboxes(h + h)
        n = 1 << 12
        f = rx.compile(rx.programs.sinsum_add(2 * n, num_partitions=2), client)
        mesh = rx.Mesh(client.devices, ("x",))
        sh = rx.NamedSharding(mesh, ("x",))
        x = np.ones(n, np.float32)
        X = rx.from_local_shards([x], (2 * n,), sh, client)
        Y = rx.from_local_shards([x], (2 * n,), sh, client)
        r = f(X, Y)                       # enqueues; the kernel polls for half a second (peer_wait_ms), then gives up
        with pytest.raises(rx.ReactantError) as e:
            float(r)
        assert e.value.code == 10 and "all-reduce" in str(e.value)
        # the device is still healthy: an unsharded program runs and is correct
        g = rx.compile(rx.programs.sinsum_add(n), client)
        got = float(g(rx.to_rarray(x, client), rx.to_rarray(x, client)))
        assert abs(got - n * (np.sin(1.0) + 1.0)) < 1e-2 * n ** 0.5
    finally:
        client.close()


def test_future_reports_the_same_failure(rx):
    import ctypes as C
    lib = rx._lib.lib()
    client = rx.Client(node_id=0, num_nodes=2, allowed_devices=[0], peer_wait_ms=500)
    try:
        h = client.mailbox_handles()
        client.open_mailboxes(h + h)
        n = 256
        f = rx.compile(rx.programs.sinsum_add(2 * n, num_partitions=2), client, sync=True)
        mesh = rx.Mesh(client.devices, ("x",))
        sh = rx.NamedSharding(mesh, ("x",))
        x = np.zeros(n, np.float32)
        X = rx.from_local_shards([x], (2 * n,), sh, client)
        with pytest.raises(rx.ReactantError) as e:
            f(X, X)                        # sync=True awaits the future inside the call
        assert e.value.code == 10
    finally:
        client.close()


def test_handle_misuse_is_an_error_not_a_crash(rx, client):
    lib = rx._lib.lib()
    f = rx.compile(rx.programs.sinsum_add(8), client)
    x = rx.to_rarray(np.zeros(8, np.float32), client)
    # a buffer from another client/device object of the same GPU is still accepted only if it is the same device handle
    other = rx.Client(allowed_devices=[0])
    try:
        y = rx.to_rarray(np.zeros(8, np.float32), other)
        with pytest.raises(rx.ReactantError) as e:
            f(x, y)
        assert e.value.code == 12
    finally:
        other.close()
    # results count mismatch is reported the way the reference words it (API.cpp:1610-1615)
    import ctypes as C
    args = (C.c_void_p * 2)(x.data[0].handle, x.data[0].handle)
    out = (C.c_void_p * 2)()
    mask = (C.c_uint8 * 2)(0, 0)
    hf = C.c_uint8(0)
    lib.XLAExecuteSharded(f.handle, 2, args, client.addressable_devices[0].handle, mask, 2, out, C.byref(hf), None)
    with pytest.raises(rx.ReactantError) as e:
        rx._lib.check()
    assert "num_results" in str(e.value)


def test_halo_exchange_wait_runs_out_and_is_reported(rx):
    """Rank 0 of a two-process mesh whose second process does not exist: the rows this rank waits for never arrive, the
    exchange kernel gives up after the client's peer wait and returns, and the next read reports the timeout."""
    client = rx.Client(node_id=0, num_nodes=2, allowed_devices=[0], peer_wait_ms=300)
    try:
        h = client.mailbox_handles()
        client.open_mailboxes(h + h)
        n = 64
        f = rx.compile(rx.programs.jacobi2d(n, 2, num_partitions=2), client)
        sh = rx.NamedSharding(rx.Mesh(client.devices, ("x",)), (None, "x"))
        z = np.zeros((n, n // 2), np.float32)      # this rank's half of the columns (Julia layout)
        A = rx.from_local_shards([z], (n, n), sh, client)
        B = rx.from_local_shards([z], (n, n), sh, client)
        ra, rb = f(A, B)
        with pytest.raises(rx.ReactantError) as e:
            ra.data[0].to_host()
        assert e.value.code == 10 and "halo exchange" in str(e.value)
        g = rx.compile(rx.programs.sinsum_add(16), client)   # the device is still usable
        x = rx.to_rarray(np.zeros(16, np.float32), client)
        assert float(g(x, x)) == 0.0
    finally:
        client.close()
