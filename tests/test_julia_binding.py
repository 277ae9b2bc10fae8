"""The Julia binding cannot be executed where the engine is built (no Julia), so it is checked as text: every entry
point it binds must be declared in include/rx_b200.h with the same number of arguments and a compatible result
type, every symbol it looks up must exist in the built library, and the registration call must use the keywords
Reactant's `register_backend` really has."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
JL = os.path.join(ROOT, "reactant.jl_b200", "julia", "B200Backend.jl")


def header_prototypes():
    text = open(os.path.join(ROOT, "include", "rx_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b([A-Za-z_]\w*)\s*\(([^;{}]*)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if name in ("ReactantThrowError",) or "typedef" in ret:
            continue
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        protos[name] = (ret, n)
    return protos


def split_top(s):
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch in "({[":
            depth += 1
        elif ch in ")}]":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def table_rows():
    rows = []
    for line in open(JL):
        m = re.match(r"rx\(:(\w+),\s*(.+)\)\s*$", line.strip())
        if not m:
            continue
        parts = split_top(m.group(2))
        ret, args = parts[0], parts[1]
        assert args.startswith("(") and args.endswith(")")
        inner = args[1:-1].strip()
        arg_types = [a for a in split_top(inner) if a]
        handle = int(parts[2]) if len(parts) > 2 else 1
        rows.append((m.group(1), ret, arg_types, handle))
    return rows


RET_OK = {
    "Cvoid": ("void",), "Cint": ("int",), "Int64": ("int64_t",), "Int32": ("int32_t",), "UInt8": ("uint8_t",), "Bool": ("uint8_t",),
    "Cstring": ("const char*",), "P": ("*",), "Ptr{Int64}": ("const int64_t*",),
}


def test_every_bound_entry_point_matches_the_header(rx):
    protos = header_prototypes()
    rows = table_rows()
    assert len(rows) >= 60
    lib = rx._lib.lib()
    for name, ret, args, handle in rows:
        assert name in protos, f"{name} is bound in B200Backend.jl but not declared in rx_b200.h"
        c_ret, c_n = protos[name]
        assert len(args) == c_n, f"{name}: {len(args)} arguments in the binding, {c_n} in the header"
        assert 1 <= handle <= len(args)
        assert any(c_ret.replace(" ", "").endswith(ok.replace(" ", "")) for ok in RET_OK[ret]), f"{name}: Julia {ret} vs C {c_ret}"
        assert hasattr(lib, name)
    # the groups the PJRT wrappers call are all there
    bound = {r[0] for r in rows}
    for must in ("ClientNumDevices", "ArrayFromHostBuffer", "BufferToHost", "PjRtBufferFree", "FutureAwait", "XLAExecute", "XLAExecuteSharded",
                 "PjRtLoadedExecutableGetHloModules", "PjRtLoadedExecutableGetParameterShardings", "PjRtLoadedExecutableGetOuputShardings",
                 "op_sharding_tile_assignment_devices", "ExecutableFree", "FreeClient"):
        assert must in bound, must


def test_directly_looked_up_symbols_exist(rx):
    lib = rx._lib.lib()
    text = open(JL).read()
    names = set(re.findall(r"sym\)?\(:(\w+)\)", text))
    assert {"MakeGPUClient", "ClientCompileText", "RxOwns", "RxSetForeignExecute", "ReactantThrowError", "RxLastError"} <= names
    for n in names:
        assert hasattr(lib, n), n


def test_registration_uses_the_keywords_the_reference_has():
    text = open(JL).read()
    calls = re.findall(r"register_backend\(([^)]*)\)", text)
    calls = [c for c in calls if "priority" in c and "platform_name;" not in c]
    assert calls, "no register_backend call found"
    allowed = {"priority", "pjrt_initialize_function", "ifrt_initialize_function", "preinitialize_setup_function"}
    for c in calls:
        kws = set(re.findall(r"(\w+)\s*=", c))
        assert kws <= allowed, f"register_backend called with {kws - allowed}, which src/accelerators/Registration.jl:24-30 does not accept"


def test_integration_document_lists_the_committed_file():
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    m = re.search(r"```julia\n(.*?)```", doc, flags=re.S)
    assert m, "INTEGRATION.md holds no julia listing"
    assert m.group(1) == open(JL).read(), "the listing in INTEGRATION.md is not reactant.jl_b200/julia/B200Backend.jl"


def test_ownership_registry_distinguishes_foreign_handles(rx):
    lib = rx._lib.lib()
    junk = ctypes.c_int(0)
    assert lib.RxOwns(ctypes.addressof(junk)) == 0 and lib.RxOwns(None) == 0
