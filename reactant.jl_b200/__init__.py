"""Host-side mirror of the Reactant.jl surface that sits on top of the runtime
boundary, bound to librx_b200.so through its C ABI.

Julia (the reference's host language) is not available where this is built, so
this module plays the role of the Julia glue: it reproduces the calls that
Reactant's own types make into the runtime, with the same names and the same
argument meaning, so that tests read like Reactant's:

    x = to_rarray(host_x)                      # src/Tracing.jl:2160-2171
    f = compile(module_text)                   # @compile -> XLA.compile,
                                               #   src/compiler/Compiler.jl:1378-1512
    y = f(x)                                   # Thunk call, src/compiler/Thunk.jl:72-86
    np.asarray(y)                              # convert(Array, y), src/ConcreteRArray.jl:108-136

Arrays follow Julia's convention: a numpy array of shape (d1..dn) stands for
the Julia array of that size; it crosses the boundary column-major, i.e. as a
row-major tensor of dims (dn..d1) (src/xla/PJRT/Buffer.jl:9-17).

Tracing Julia code into StableHLO stays Reactant's job; `compile` therefore takes
the module text Reactant hands to its runtime.  `programs` holds that text for the
benchmark configurations.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import weakref

import numpy as np

from . import _lib, dist
from ._lib import ReactantError, lib, check, take_string

try:
    import ml_dtypes
    bfloat16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    ml_dtypes = None
    bfloat16 = None

# XLA primitive type codes (src/xla/Utils.jl:18-40)
_PTYPE = {np.dtype(np.bool_): 1, np.dtype(np.int8): 2, np.dtype(np.int16): 3, np.dtype(np.int32): 4, np.dtype(np.int64): 5,
          np.dtype(np.uint8): 6, np.dtype(np.uint16): 7, np.dtype(np.uint32): 8, np.dtype(np.uint64): 9,
          np.dtype(np.float16): 10, np.dtype(np.float32): 11, np.dtype(np.float64): 12}
if bfloat16 is not None:
    _PTYPE[np.dtype(bfloat16)] = 16
_NPTYPE = {v: k for k, v in _PTYPE.items()}


# ----------------------------------------------------------------------------
# client / devices  (src/xla/XLA.jl:126-185, src/accelerators/GPU.jl:7-37)
# ----------------------------------------------------------------------------
class Device:
    def __init__(self, client, handle):
        self.client, self.handle = client, handle

    @property
    def global_id(self):
        return lib().PjRtDeviceGetGlobalDeviceId(self.handle)

    @property
    def local_id(self):
        return lib().PjRtDeviceGetLocalDeviceId(self.handle)

    @property
    def addressable(self):
        return bool(lib().pjrt_device_is_addressable(self.handle))

    def synchronize(self):
        lib().RxDeviceSynchronize(self.handle)
        check()

    def join_streams(self):
        """Make the compute stream wait for the all-reduces queued on the communication stream so far."""
        lib().RxDeviceJoinStreams(self.handle)
        check()

    def kernel_launches(self) -> int:
        return int(lib().RxDeviceKernelLaunches(self.handle))

    def allocator_stats(self) -> dict:
        s = _lib.JLAllocatorStats()
        lib().PjRtDeviceGetAllocatorStats(self.handle, C.byref(s))
        return {n: getattr(s, n) for n, _ in s._fields_}

    def set_profiling(self, on: bool):
        lib().RxDeviceSetProfiling(self.handle, int(on))

    def profile(self) -> dict:
        return json.loads(take_string(lib().RxDeviceProfileJson(self.handle)) or "{}")

    def flush_l2(self):
        lib().RxDeviceFlushL2(self.handle)
        check()

    def record_event(self):
        e = lib().RxEventRecord(self.handle)
        check()
        return Event(e)


class Event:
    def __init__(self, handle):
        self.handle = handle
        self._fin = weakref.finalize(self, lib().RxEventFree, handle)

    def synchronize(self):
        lib().RxEventSynchronize(self.handle)
        check()

    def elapsed_ms(self, later: "Event") -> float:
        ms = lib().RxEventElapsedMs(self.handle, later.handle)
        check()
        return float(ms)


class Client:
    """MakeGPUClient wrapper (src/xla/PJRT/Client.jl, deps/ReactantExtra/API.cpp:528-582)."""

    def __init__(self, node_id=0, num_nodes=1, allowed_devices=None, memory_fraction=0.9, peer_wait_ms=None):
        err = C.c_char_p()
        if allowed_devices is None and os.environ.get("REACTANT_VISIBLE_GPU_DEVICES"):
            # the list Reactant reads at start-up and passes to MakeGPUClient as allowed_devices (src/xla/XLA.jl:230-233)
            allowed_devices = [int(v) for v in os.environ["REACTANT_VISIBLE_GPU_DEVICES"].split(",") if v.strip()]
        arr, n = None, 0
        if allowed_devices is not None:
            n = len(allowed_devices)
            arr = (C.c_int64 * n)(*allowed_devices)
        h = lib().MakeGPUClient(node_id, num_nodes, arr, n, memory_fraction, 0, b"cuda", C.byref(err), None)
        if not h:
            code = lib().RxLastErrorCode()
            msg = lib().RxLastError().decode()
            lib().RxClearError()
            raise ReactantError(code, msg)
        self.handle = h
        self.node_id, self.num_nodes = node_id, num_nodes
        self._fin = weakref.finalize(self, lib().FreeClient, h)
        n_addr = lib().ClientNumAddressableDevices(h)
        self.addressable_devices = [Device(self, lib().ClientGetAddressableDevice(h, i)) for i in range(n_addr)]
        self.devices = [Device(self, lib().ClientGetDevice(h, i)) for i in range(lib().ClientNumDevices(h))]
        if peer_wait_ms is not None:
            lib().RxClientSetPeerWaitMs(h, int(peer_wait_ms))
            check()

    @property
    def platform_name(self):
        return take_string(lib().ClientGetPlatformName(self.handle))

    def close(self):
        self._fin()

    # collectives bootstrap for multi-process meshes
    def init_collectives(self, unique_id: bytes | None):
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id) if unique_id is not None else None
        lib().RxClientInitCollectives(self.handle, buf)
        check()

    def mailbox_handles(self) -> bytes:
        out = b""
        for i in range(len(self.addressable_devices)):
            buf = (C.c_uint8 * 64)()
            lib().RxClientMailboxHandle(self.handle, i, buf)
            check()
            out += bytes(buf)
        return out

    def open_mailboxes(self, all_handles: bytes):
        n = len(all_handles) // 64
        buf = (C.c_uint8 * len(all_handles)).from_buffer_copy(all_handles)
        lib().RxClientOpenMailboxes(self.handle, buf, n)
        check()


def collectives_unique_id() -> bytes:
    buf = (C.c_uint8 * 128)()
    lib().RxCollectivesUniqueId(buf)
    check()
    return bytes(buf)


class PinnedArray:
    """A numpy array over page-locked host memory (RxHostAlloc): uploads from it and downloads into it run at
    the full PCIe rate.  Keep the object alive as long as `array` is in use; the memory is released with it."""

    def __init__(self, n: int, dtype=np.float32):
        dt = np.dtype(dtype)
        self.nbytes = max(1, int(n) * dt.itemsize)
        self.ptr = lib().RxHostAlloc(self.nbytes)
        check()
        self._fin = weakref.finalize(self, lib().RxHostFree, self.ptr)
        raw = (C.c_uint8 * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(raw, dtype=dt, count=int(n))


_default_client = None


def set_default_backend(name: str = "gpu", **kw):
    """Reactant.set_default_backend (src/Reactant.jl:401-404): only "gpu"/"cuda"
    exist here; there is no CPU backend to fall back to."""
    global _default_client
    if name not in ("gpu", "cuda"):
        raise ReactantError(12, f"backend {name!r} is not available in this engine (only \"gpu\")")
    if _default_client is None or kw:
        _default_client = Client(**kw)
    return _default_client


def default_client() -> Client:
    return set_default_backend("gpu")


# ----------------------------------------------------------------------------
# sharding  (src/Sharding.jl:30-105, 267-336; slices: src/xla/Sharding.jl:226-273)
# ----------------------------------------------------------------------------
class Mesh:
    def __init__(self, devices, axis_names=("x",)):
        self.devices = list(devices)
        self.axis_names = tuple(axis_names)
        if len(self.axis_names) != 1:
            raise ReactantError(2, "only 1-D meshes are supported")

    def __len__(self):
        return len(self.devices)


class NamedSharding:
    def __init__(self, mesh: Mesh, partition_spec):
        self.mesh = mesh
        self.partition_spec = tuple(partition_spec)

    def sharded_dim(self):
        dims = [i for i, a in enumerate(self.partition_spec) if a is not None]
        if len(dims) > 1:
            raise ReactantError(2, "only one sharded dimension is supported")
        return dims[0] if dims else None


# ----------------------------------------------------------------------------
# buffers and arrays  (src/Types.jl:155-263, src/ConcreteRArray.jl)
# ----------------------------------------------------------------------------
class _Buffer:
    def __init__(self, handle, device: Device):
        self.handle, self.device = handle, device
        self._fin = weakref.finalize(self, lib().PjRtBufferFree, handle)

    @property
    def dims(self):
        n = lib().BufferNDimensions(self.handle)
        p = lib().BufferShape(self.handle)
        return tuple(p[i] for i in range(n))

    @property
    def dtype(self):
        return _NPTYPE[lib().BufferPrimitiveType(self.handle)]

    def to_host(self) -> np.ndarray:
        out = np.empty(self.dims, dtype=self.dtype)
        lib().BufferToHost(self.handle, out.ctypes.data_as(C.c_void_p))
        check()
        return out


def _upload(client: Client, device: Device, a: np.ndarray) -> _Buffer:
    """Julia array -> device buffer with reversed dims and unchanged (column-major) bytes."""
    if a.dtype not in _PTYPE:
        raise ReactantError(3, f"unsupported element type {a.dtype}")
    rm = np.ascontiguousarray(a.T).reshape(a.T.shape)  # (ascontiguousarray promotes 0-d to 1-d)
    dims = (C.c_int64 * rm.ndim)(*rm.shape)
    h = lib().ArrayFromHostBuffer(client.handle, rm.ctypes.data_as(C.c_void_p), _PTYPE[a.dtype], rm.ndim, dims, device.handle)
    check()
    return _Buffer(h, device)


class ConcreteRArray:
    """ConcretePJRTArray{T,N,D}: D device buffers + logical (Julia) shape + sharding."""

    def __init__(self, buffers, shape, dtype, sharding=None, replicated=False):
        self.data = list(buffers)
        self.shape = tuple(shape)
        self.dtype = np.dtype(dtype)
        self.sharding = sharding
        self.replicated = replicated

    @property
    def ndim(self):
        return len(self.shape)

    def __array__(self, dtype=None, copy=None):
        a = self.to_host()
        return a.astype(dtype) if dtype is not None else a

    def to_host(self) -> np.ndarray:
        if self.sharding is None or self.replicated or len(self.data) == 1 and self.sharding.sharded_dim() is None:
            return self.data[0].to_host().T
        d = self.sharding.sharded_dim()
        parts = [b.to_host().T for b in self.data]
        return np.concatenate(parts, axis=d)

    def synchronize(self):
        for b in self.data:
            b.device.synchronize()


class ConcreteRNumber(ConcreteRArray):
    """ConcretePJRTNumber{T,D}: a rank-0 array (src/Types.jl:155-211)."""

    def __float__(self):
        return float(self.data[0].to_host())

    def __int__(self):
        return int(self.data[0].to_host())

    def item(self):
        return self.data[0].to_host().item()


def to_rarray(x, client: Client | None = None, device: Device | None = None, sharding: NamedSharding | None = None):
    """Reactant.to_rarray (src/Tracing.jl:2160-2171): upload a host array.

    With a NamedSharding the array is split into equal contiguous chunks along the
    partitioned dimension, chunk i going to mesh device i (src/Sharding.jl:406-430);
    in a multi-process mesh each process uploads only the chunks of its own devices.
    """
    client = client or default_client()
    a = np.asarray(x)
    if sharding is None:
        device = device or client.addressable_devices[0]
        buf = _upload(client, device, a)
        cls = ConcreteRNumber if a.ndim == 0 else ConcreteRArray
        return cls([buf], a.shape, a.dtype)
    d = sharding.sharded_dim()
    n = len(sharding.mesh)
    if d is not None and a.shape[d] % n:
        # a dimension the mesh does not divide is not split (nor padded): every device holds the whole array, which is
        # what the compiled module's parameter sharding says too (src/Sharding.jl:582-654 takes the sharding XLA reports)
        d = None
    bufs = []
    for i, dev in enumerate(sharding.mesh.devices):
        if not dev.addressable:
            continue
        if d is None:
            piece = a
        else:
            try:
                lo, hi = dist.shard_bounds(a.shape[d], n, i)
            except ValueError as e:
                raise ReactantError(2, str(e))
            sl = [slice(None)] * a.ndim
            sl[d] = slice(lo, hi)
            piece = a[tuple(sl)]
        bufs.append(_upload(client, dev, piece))
    return ConcreteRArray(bufs, a.shape, a.dtype, sharding=sharding, replicated=d is None)


def from_local_shards(pieces, global_shape, sharding: NamedSharding, client: Client | None = None):
    """Build a sharded array from the chunks this process owns (one per addressable
    mesh device, in mesh order).  The multi-process counterpart of the upload loop in
    src/Sharding.jl:406-430, where no process holds the whole array."""
    client = client or default_client()
    devs = [d for d in sharding.mesh.devices if d.addressable]
    if len(devs) != len(pieces):
        raise ReactantError(12, f"{len(pieces)} chunks for {len(devs)} addressable mesh devices")
    bufs = [_upload(client, d, np.asarray(p)) for d, p in zip(devs, pieces)]
    return ConcreteRArray(bufs, global_shape, np.asarray(pieces[0]).dtype, sharding=sharding)


# ----------------------------------------------------------------------------
# compile / Thunk  (src/compiler/Compiler.jl:1264-1512, src/compiler/Thunk.jl)
# ----------------------------------------------------------------------------
class Thunk:
    def __init__(self, client: Client, handle, sync: bool):
        self.client, self.handle, self.sync = client, handle, sync
        self._fin = weakref.finalize(self, lib().ExecutableFree, handle)
        l = lib()
        self.num_parameters = l.RxExecutableNumParameters(handle)
        self.num_results = l.RxExecutableNumResults(handle)
        self.num_partitions = l.PjRtLoadedExecutableNumPartitions(handle)
        self.param_sharded_dim = [l.RxExecutableParameterShardedDim(handle, i) for i in range(self.num_parameters)]
        self.result_sharded_dim = [l.RxExecutableResultShardedDim(handle, i) for i in range(self.num_results)]
        self.param_alias = [l.RxExecutableParameterAlias(handle, i) for i in range(self.num_parameters)]

    def describe(self) -> dict:
        return json.loads(take_string(lib().RxExecutableDescribe(self.handle)))

    def __call__(self, *args: ConcreteRArray, donate: bool = True):
        """Execute.  Arguments that carry `tf.aliasing_output` are donated (their
        storage becomes the aliased result's) and, as Reactant does for mutated
        arguments (src/compiler/Codegen.jl:1116-1170), the argument objects are
        re-pointed at the new buffers, so `A` stays usable after `f(A, B)`."""
        l = lib()
        if len(args) != self.num_parameters:
            raise ReactantError(12, f"thunk takes {self.num_parameters} arguments, got {len(args)}")
        sharded = self.num_partitions > 1
        ndev = len(self.client.addressable_devices) if sharded else 1
        for a in args:
            if len(a.data) != ndev:
                raise ReactantError(12, f"argument holds {len(a.data)} device buffers, executable runs on {ndev} local devices")
        flat = (C.c_void_p * (ndev * len(args)))()
        for k in range(ndev):
            for i, a in enumerate(args):
                flat[k * len(args) + i] = a.data[k].handle
        mask = (C.c_uint8 * max(1, len(args)))(*[1 if (donate and self.param_alias[i] >= 0) else 0 for i in range(len(args))])
        nres = self.num_results
        out = (C.c_void_p * max(1, ndev * nres))()
        futs = (C.c_void_p * max(1, ndev * nres))()
        has_fut = C.c_uint8(0)
        if sharded:
            l.XLAExecute(self.handle, ndev * len(args), flat, mask, nres, out, C.byref(has_fut), futs)
        else:
            dev = args[0].data[0].device if args else self.client.addressable_devices[0]
            l.XLAExecuteSharded(self.handle, len(args), flat, dev.handle, mask, nres, out, C.byref(has_fut), futs)
        check()
        devs = self.client.addressable_devices
        if has_fut.value:
            for q in range(ndev * nres):
                if self.sync and q % max(1, nres) == 0:
                    l.FutureAwait(futs[q])
                l.FreeFuture(futs[q])
            check()
        results = []
        for j in range(nres):
            bufs = []
            for k in range(ndev):
                dev = devs[k] if sharded else (args[0].data[0].device if args else devs[0])
                bufs.append(_Buffer(out[k * nres + j], dev))
            dims = bufs[0].dims
            jl_shape = tuple(reversed(dims))
            dt = bufs[0].dtype
            sd = self.result_sharded_dim[j]
            if sharded and sd >= 0:
                jd = len(dims) - 1 - sd
                shp = list(jl_shape)
                shp[jd] *= self.num_partitions
                mesh = None
                for a in args:
                    if a.sharding is not None:
                        mesh = a.sharding.mesh
                spec = [None] * len(dims)
                spec[jd] = "x"
                r = ConcreteRArray(bufs, shp, dt, sharding=NamedSharding(mesh, spec))
            else:
                cls = ConcreteRNumber if len(dims) == 0 else ConcreteRArray
                r = cls(bufs, jl_shape, dt, replicated=sharded)
                if sharded:
                    r.sharding = None
            results.append(r)
        # mutated (donated) arguments now live in the buffers of the result they alias
        for i, a in enumerate(args):
            k = self.param_alias[i]
            if donate and 0 <= k < nres:
                a.data = results[k].data
        return results[0] if nres == 1 else tuple(results)


def compile(module_text: str, client: Client | None = None, sync: bool = False) -> Thunk:
    """XLA.compile for this engine: parse the optimised StableHLO module, plan the
    fusion groups and bind kernels.  Raises ReactantError naming the op if the
    module needs anything outside the supported set (there is no fallback)."""
    client = client or default_client()
    t = module_text.encode()
    h = lib().ClientCompileText(client.handle, t, len(t), None, 0)
    check()
    return Thunk(client, h, sync)


def plan_describe(module_text: str) -> dict:
    """Parse and plan without a device (works on machines with no GPU)."""
    t = module_text.encode()
    p = lib().RxPlanDescribe(t, len(t))
    if not p:
        check()
    return json.loads(take_string(p))


def specialise_check(module_text: str) -> list:
    """Plan a module and compile each of its fused chains with NVRTC for every kernel family it could run in.
    Needs no device.  Raises with the compiler log if a chain does not compile."""
    t = module_text.encode()
    p = lib().RxPlanSpecialiseCheck(t, len(t))
    if not p:
        check()
    return json.loads(take_string(p))


def chain_specialiser(min_elems: int) -> None:
    """Launches covering at least `min_elems` elements run kernels compiled for their chain (default 2^20);
    a negative value switches specialisation off and everything runs the on-GPU interpreter."""
    lib().RxChainSpecialiser(int(min_elems))


def chain_specialiser_stats() -> dict:
    import ctypes
    out = (ctypes.c_int64 * 5)()
    lib().RxChainSpecialiserStats(out)
    return {"compiled": out[0], "cache_hits": out[1], "failed": out[2], "unavailable": bool(out[3]), "disk_hits": out[4]}


from . import programs  # noqa: E402,F401


def load_export(directory: str, function_name: str, index: int = 0, client: Client | None = None):
    """Open a bundle written by Reactant.Serialization.export_to_enzymejax (src/serialization/EnzymeJAX.jl:94-190):
    `{function_name}_{index}.mlir` holds the StableHLO module, `{function_name}_{index}_inputs.npz` the example
    inputs as `arr_1 .. arr_n`, already permuted to the row-major layout of the module's argument types
    (ext/ReactantNPZExt.jl:6-19).  Returns `(thunk, inputs)`: the compiled module and the inputs uploaded as
    ConcreteRArrays, so that `thunk(*inputs)` runs the exported function on the GPU."""
    import os
    client = client or default_client()
    base = os.path.join(directory, f"{function_name}_{index}")
    with open(base + ".mlir") as f:
        text = f.read()
    thunk = compile(text, client)
    inputs = []
    path = base + "_inputs.npz"
    if os.path.exists(path):
        with np.load(path) as data:
            keys = sorted((k for k in data.files if k.startswith("arr_")), key=lambda k: int(k.split("_")[1]))
            if len(keys) != thunk.num_parameters:
                raise ReactantError(12, f"{path} holds {len(keys)} arrays, the module takes {thunk.num_parameters} arguments")
            for k in keys:
                a = np.asarray(data[k])
                # the file holds the boundary (row-major, reversed dims) layout; host arrays here are column-major
                inputs.append(to_rarray(a.T if a.ndim else a, client))
    return thunk, inputs
