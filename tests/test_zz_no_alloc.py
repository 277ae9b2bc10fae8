"""The allocation-free entry point, RxSinSumAddNoAlloc.

It exists for hosts that cannot let the library allocate device memory (all of
it already belongs to the host's own arena, or a cudaMalloc stall is not
acceptable where the call is made): the caller passes device pointers for the
inputs and the output and the kernel's scratch is a fixed array inside the
library.  The test calls it through the C ABI on the caller's own buffers, twice
in a row with different data (the second call meets whatever the first one left
in the shared scratch array), and compares each result with the regular
compile-and-execute path on the same buffers.  A larger case gives every CTA several chunks
of the input, and the free device memory reported by the CUDA runtime is read
before and after a call to see that none was taken.  This file sorts last so that a
run that stops at the first failure has already run every other test; it also
passes on its own in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _existing_path(rx, client, n, X, Y):
    f = rx.compile(rx.programs.sinsum_add(n), client)
    return float(f(X, Y))


def _free_device_bytes():
    """Free memory on the current device as the CUDA runtime reports it (a stray cudaMalloc anywhere would move it,
    which the library's own pool counter would not see)."""
    rt = C.CDLL("libcudart.so.12")
    free, total = C.c_size_t(), C.c_size_t()
    assert rt.cudaMemGetInfo(C.byref(free), C.byref(total)) == 0
    return free.value


@pytest.mark.parametrize("n", [(1 << 20) + 3, 5, 1 << 16, (1 << 27) + 5])
def test_no_alloc_matches_existing_entry_point_twice_in_a_row(rx, ref, client, n):
    lib = rx._lib.lib()
    dev = client.addressable_devices[0]
    stream = lib.RxDeviceStream(dev.handle)
    rng = np.random.default_rng(n)
    out = rx.to_rarray(np.zeros((), np.float32), client)  # caller-owned output word
    out_ptr = lib.UnsafeBufferPointer(out.data[0].handle)
    for call in range(2):
        x = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
        y = rng.uniform(-np.pi, np.pi, n).astype(np.float32)
        X, Y = rx.to_rarray(x, client), rx.to_rarray(y, client)
        px = lib.UnsafeBufferPointer(X.data[0].handle)
        py = lib.UnsafeBufferPointer(Y.data[0].handle)
        if call == 0:  # the first call on a device resolves the scratch array's address (and may load the kernel)
            assert lib.RxSinSumAddNoAlloc(px, py, min(n, 4096), out_ptr, stream) == 0, lib.RxLastError().decode()
            dev.synchronize()
        before, free_before = dev.allocator_stats()["num_allocs"], _free_device_bytes()
        rc = lib.RxSinSumAddNoAlloc(px, py, n, out_ptr, stream)
        assert rc == 0, lib.RxLastError().decode()
        dev.synchronize()
        assert dev.allocator_stats()["num_allocs"] == before, "the entry point must not allocate from the library's pool"
        assert _free_device_bytes() == free_before, "the entry point must not take device memory from the driver either"
        got = float(out.data[0].to_host())  # synchronises the stream
        want = _existing_path(rx, client, n, X, Y)
        terms = np.sin(x.astype(np.float64)) + y.astype(np.float64)
        tol = ref.reduction_tolerance(n) * max(abs(terms.sum()), np.linalg.norm(terms))
        assert abs(got - want) <= tol, (call, got, want)
        assert abs(got - terms.sum()) <= tol, (call, got, terms.sum())


def test_no_alloc_rejects_sizes_beyond_its_fixed_scratch(rx, client):
    lib = rx._lib.lib()
    out = rx.to_rarray(np.zeros((), np.float32), client)
    x = rx.to_rarray(np.zeros(16, np.float32), client)
    px = lib.UnsafeBufferPointer(x.data[0].handle)
    rc = lib.RxSinSumAddNoAlloc(px, px, (1 << 30) + 1, lib.UnsafeBufferPointer(out.data[0].handle), None)
    assert rc == 13  # RX_ERR_TOO_LARGE: nothing was launched
    assert "2^30" in lib.RxLastError().decode()
    lib.RxClearError()
    assert lib.RxSinSumAddNoAlloc(px, px, -1, lib.UnsafeBufferPointer(out.data[0].handle), None) == 12
    lib.RxClearError()
