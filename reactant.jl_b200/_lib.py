"""ctypes binding of librx_b200.so: one prototype per symbol of include/rx_b200.h.

The library is required: importing this module raises if it has not been
built (python reactant.jl_b200/build.py).  There is no Python or CPU stand-in
for any entry point.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# RX_B200_LIB selects another build of the library (the bounds-checked one, say); the default is the in-tree build
LIB_PATH = os.environ.get("RX_B200_LIB") or os.path.join(HERE, "librx_b200.so")


class ReactantError(RuntimeError):
    """Raised where Reactant's ReactantThrowError callback would throw
    (src/xla/XLA.jl:203-204, src/xla/Utils.jl:3-15)."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


class JLAllocatorStats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "num_allocs", "bytes_in_use", "peak_bytes_in_use", "largest_alloc_size", "bytes_limit", "bytes_reserved",
        "peak_bytes_reserved", "bytes_reservable_limit", "largest_free_block_bytes", "pool_bytes", "peak_pool_bytes")]


P = C.c_void_p
PP = C.POINTER(C.c_void_p)
U8P = C.POINTER(C.c_uint8)

# name -> (restype, argtypes); every symbol include/rx_b200.h declares
PROTOTYPES = {
    "RxLastError": (C.c_char_p, []),
    "RxLastErrorCode": (C.c_int, []),
    "RxClearError": (None, []),
    "MakeGPUClient": (P, [C.c_int, C.c_int, C.POINTER(C.c_int64), C.c_int64, C.c_double, C.c_uint8, C.c_char_p, C.POINTER(C.c_char_p), P]),
    "FreeClient": (None, [P]),
    "ClientNumDevices": (C.c_int, [P]),
    "ClientNumAddressableDevices": (C.c_int, [P]),
    "ClientProcessIndex": (C.c_int, [P]),
    "ClientGetDevice": (P, [P, C.c_int]),
    "ClientGetAddressableDevice": (P, [P, C.c_int]),
    "ClientGetDevices": (None, [P, PP]),
    "ClientGetAddressableDevices": (None, [P, PP]),
    "ClientGetPlatformName": (P, [P]),
    "DeviceToClient": (P, [P]),
    "PjRtDeviceGetLocalDeviceId": (C.c_int64, [P]),
    "PjRtDeviceGetGlobalDeviceId": (C.c_int64, [P]),
    "PjRtDeviceGetLocalHardwareId": (C.c_int64, [P]),
    "DeviceGetKind": (P, [P]),
    "pjrt_device_is_addressable": (C.c_uint8, [P]),
    "PjRtDeviceGetAllocatorStats": (None, [P, C.POINTER(JLAllocatorStats)]),
    "ArrayFromHostBuffer": (P, [P, P, C.c_uint64, C.c_size_t, C.POINTER(C.c_int64), P]),
    "UninitPJRTBuffer": (P, [P, P, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64)]),
    "PjRtBufferFree": (None, [P]),
    "BufferShape": (C.POINTER(C.c_int64), [P]),
    "BufferNDimensions": (C.c_int64, [P]),
    "BufferPrimitiveType": (C.c_int, [P]),
    "BufferToDevice": (P, [P]),
    "BufferToClient": (P, [P]),
    "BufferOnCPU": (C.c_uint8, [P]),
    "BufferToHost": (None, [P, P]),
    "UnsafeBufferPointer": (P, [P]),
    "CopyBufferToDevice": (P, [P, P]),
    "CopyToBuffer": (None, [P, P, P, C.c_size_t, C.c_size_t, PP]),
    "CopyFromBuffer": (None, [P, P, P, C.c_size_t, C.c_size_t, PP]),
    "FreeFuture": (None, [P]),
    "FutureIsReady": (C.c_uint8, [P]),
    "FutureAwait": (None, [P]),
    "ClientCompileText": (P, [P, C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]),
    "ExecutableFree": (None, [P]),
    "PjRtLoadedExecutableGetClient": (P, [P]),
    "PjRtLoadedExecutableNumReplicas": (C.c_int, [P]),
    "PjRtLoadedExecutableNumPartitions": (C.c_int, [P]),
    "RxExecutableNumParameters": (C.c_int, [P]),
    "RxExecutableNumResults": (C.c_int, [P]),
    "RxExecutableParameterShardedDim": (C.c_int, [P, C.c_int]),
    "RxExecutableResultShardedDim": (C.c_int, [P, C.c_int]),
    "RxExecutableParameterAlias": (C.c_int, [P, C.c_int]),
    "RxExecutableDescribe": (P, [P]),
    "PjRtLoadedExecutableGetParameterShardings": (None, [P, PP, C.c_int32]),
    "PjRtLoadedExecutableGetOuputShardings": (None, [P, PP, C.c_int32]),
    "PjRtLoadedExecutableGetHloModules": (None, [P, PP, C.POINTER(C.c_int32)]),
    "free_op_sharding": (None, [P]),
    "op_sharding_to_op_sharding_type": (C.c_int32, [P]),
    "op_sharding_to_shard_group_type": (C.c_int32, [P]),
    "op_sharding_to_shard_group_id": (C.c_int32, [P]),
    "op_sharding_is_shard_group": (C.c_uint8, [P]),
    "op_sharding_replicate_on_last_tile_dim": (C.c_uint8, [P]),
    "op_sharding_has_last_tile_dims": (C.c_uint8, [P]),
    "op_sharding_last_tile_dims_size": (C.c_int32, [P]),
    "op_sharding_last_tile_dims": (None, [P, C.POINTER(C.c_int32)]),
    "op_sharding_has_iota_reshape_dims": (C.c_uint8, [P]),
    "op_sharding_iota_reshape_dims_size": (C.c_int32, [P]),
    "op_sharding_iota_reshape_dims": (None, [P, C.POINTER(C.c_int32)]),
    "op_sharding_has_iota_transpose_perm": (C.c_uint8, [P]),
    "op_sharding_iota_transpose_perm_size": (C.c_int32, [P]),
    "op_sharding_iota_transpose_perm": (None, [P, C.POINTER(C.c_int32)]),
    "op_sharding_has_tile_assignment_dimensions": (C.c_uint8, [P]),
    "op_sharding_tile_assignment_dimensions_size": (C.c_int32, [P]),
    "op_sharding_tile_assignment_dimensions": (None, [P, C.POINTER(C.c_int32)]),
    "op_sharding_has_tile_assignment_devices": (C.c_uint8, [P]),
    "op_sharding_tile_assignment_devices_size": (C.c_int32, [P]),
    "op_sharding_tile_assignment_devices": (None, [P, C.POINTER(C.c_int32)]),
    "ReactantCudaDeviceGetProperties": (None, [P, C.c_int32]),
    "ReactantCudaDriverGetVersion": (C.c_int32, []),
    "ReactantCudaDeviceGetComputeCapalilityMajor": (C.c_int32, []),
    "ReactantCudaDeviceGetComputeCapalilityMinor": (C.c_int32, []),
    "ReactantCudaDeviceGetWarpSizeInThreads": (C.c_int32, []),
    "RxPlanDescribe": (P, [C.c_char_p, C.c_size_t]),
    "RxPlanCacheHits": (C.c_int64, []),
    "RxChainSpecialiser": (None, [C.c_int64]),
    "RxChainSpecialiserStats": (None, [C.POINTER(C.c_int64)]),
    "RxPlanSpecialiseCheck": (P, [C.c_char_p, C.c_size_t]),
    "XLAExecuteSharded": (None, [P, C.c_int, PP, P, U8P, C.c_int, PP, U8P, PP]),
    "XLAExecute": (None, [P, C.c_int, PP, U8P, C.c_int, PP, U8P, PP]),
    "RxOwns": (C.c_uint8, [P]),
    "RxSetForeignExecute": (None, [P, P]),
    "RxSinSumAddNoAlloc": (C.c_int, [P, P, C.c_int64, P, P]),
    "RxCollectivesUniqueId": (C.c_int, [U8P]),
    "RxClientInitCollectives": (C.c_int, [P, U8P]),
    "RxClientMailboxHandle": (C.c_int, [P, C.c_int, U8P]),
    "RxClientSetPeerWaitMs": (C.c_int, [P, C.c_int64]),
    "RxClientOpenMailboxes": (C.c_int, [P, U8P, C.c_int]),
    "RxHostAlloc": (P, [C.c_size_t]),
    "RxHostFree": (None, [P]),
    "RxEventRecord": (P, [P]),
    "RxEventSynchronize": (None, [P]),
    "RxEventElapsedMs": (C.c_float, [P, P]),
    "RxEventFree": (None, [P]),
    "RxDeviceSynchronize": (None, [P]),
    "RxDeviceJoinStreams": (None, [P]),
    "RxDeviceKernelLaunches": (C.c_uint64, [P]),
    "RxDeviceSetProfiling": (None, [P, C.c_int]),
    "RxDeviceProfileJson": (P, [P]),
    "RxDeviceStream": (P, [P]),
    "RxDeviceFlushL2": (None, [P]),
}

_lib = None
_libc = C.CDLL(None)
_libc.free.argtypes = [C.c_void_p]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python reactant.jl_b200/build.py` (no fallback exists)")
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def check():
    """Raise if the last library call on this thread reported an error."""
    l = lib()
    code = l.RxLastErrorCode()
    if code:
        msg = l.RxLastError().decode()
        l.RxClearError()
        raise ReactantError(code, msg)


def take_string(ptr) -> str:
    """Copy and free a malloc'd C string returned by the library."""
    if not ptr:
        check()
        return ""
    s = C.string_at(ptr).decode()
    _libc.free(ptr)
    return s
