"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/rx_b200.h declares; factories fail loudly without a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "rx_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text))
    names -= {"ReactantThrowError", "void"}  # the callback slot is a variable, not a function
    return names


def test_every_declared_symbol_is_exported_and_bound(rx):
    lib = rx._lib.lib()
    decl = declared_symbols()
    assert len(decl) > 60
    for name in sorted(decl):
        assert hasattr(lib, name), f"{name} is declared in rx_b200.h but not exported"
    assert decl == set(rx._lib.PROTOTYPES), "ctypes prototypes and header are out of sync"
    assert ctypes.c_void_p.in_dll(lib, "ReactantThrowError").value is None


def test_error_callback_slot_is_called(rx):
    lib = rx._lib.lib()
    seen = []
    CB = ctypes.CFUNCTYPE(None, ctypes.c_char_p)
    cb = CB(lambda m: seen.append(m.decode()))
    slot = ctypes.c_void_p.in_dll(lib, "ReactantThrowError")
    slot.value = ctypes.cast(cb, ctypes.c_void_p).value
    try:
        assert not lib.RxPlanDescribe(b"module {", 8)
    finally:
        slot.value = None
    assert seen and "line" in seen[0]
    lib.RxClearError()


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.mark.skipif(_has_gpu(), reason="checks the no-device failure mode")
def test_client_creation_fails_loudly_without_a_device(rx):
    with pytest.raises(rx.ReactantError) as e:
        rx.Client()
    assert e.value.code == 9 and "CUDA" in str(e.value)


def test_only_gpu_backend_exists(rx):
    with pytest.raises(rx.ReactantError):
        rx.set_default_backend("cpu")
