"""CPU oracle: a numpy interpreter for the StableHLO subset on the hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
module; it exists so that the parity tests, the smoke check and the CPU leg of
the benchmark have an independent statement of what a module must compute.

It restates the op semantics that Reactant's emitters promise for the ops the
engine accepts (paths are relative to the Reactant.jl source tree):

  * elementwise unary/binary ops          src/Ops.jl:398-460, 536-589
  * convert / compare / select            src/Ops.jl:1865-1961
  * broadcast_in_dim                      src/Ops.jl:1320-1357
  * transpose / pad / slice               src/Ops.jl:724-793
  * dot_general                           src/Ops.jl:1075-1200
  * while (counted loops)                 src/Ops.jl:2349-2447
  * reduce (monoid semantics)             src/Ops.jl:3491-3622
  * dynamic_update_slice                  src/Ops.jl:3624-3678
  * reduction identities                  src/TracedRArray.jl:128-140

The arithmetic itself lives in XLA, a third-party dependency that is not part
of the Reactant tree (it is fetched by deps/ReactantExtra/WORKSPACE:116-118 at
the revision pinned by Enzyme-JAX commit 51a4cd6c58b1950f28b650167d1e946eec8ec0d5;
binary artifact Reactant_jll 0.0.405).  The op semantics restated here are those
of the published StableHLO specification.  The restatement is pinned against
the closed-form fixtures of Reactant's own tests (tests/golden/).

Floating-point reductions and contractions accumulate in float64 and round
once at the end: this is the ground truth the fp32 tolerances are measured
against, not a bit-level model of any backend's summation order.

The parser here is deliberately independent of the engine's C++ parser (it is
line/regex based) so that a parsing mistake in one does not hide in the other.
"""
from __future__ import annotations

import re
import math
import numpy as np

try:  # bf16 storage type; the fallback rounds through uint32 arithmetic
    import ml_dtypes
    _BF16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    _BF16 = None


# ----------------------------------------------------------------------------
# dtypes
# ----------------------------------------------------------------------------
def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16, returned as f32 holding bf16 values."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if _BF16 is not None and x.size > 4096:  # same rounding, one C loop instead of five numpy passes
        with np.errstate(invalid="ignore"):  # signalling NaN inputs
            return x.astype(_BF16).astype(np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32).copy()
    out[nan] = np.nan
    return out.reshape(x.shape)


class T:
    """A tensor value: numpy data plus the MLIR element type name.

    bf16 tensors are stored as float32 arrays whose values are exactly
    representable in bf16, so that all arithmetic below can run in numpy.
    """
    __slots__ = ("a", "et")

    def __init__(self, a, et):
        self.a = a
        self.et = et

    @property
    def shape(self):
        return self.a.shape


_NP = {"f32": np.float32, "f64": np.float64, "bf16": np.float32, "f16": np.float16,
       "i1": np.bool_, "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64,
       "ui8": np.uint8, "ui16": np.uint16, "ui32": np.uint32, "ui64": np.uint64}


def make(a, et):
    a = np.asarray(a)
    if et == "bf16":
        return T(round_to_bf16(a.astype(np.float32)), et)
    return T(a.astype(_NP[et]), et)


def parse_type(s):
    s = s.strip()
    m = re.fullmatch(r"tensor<(.*)>", s)
    if not m:
        raise ValueError(f"unsupported type {s!r}")
    parts = m.group(1).split("x")
    et = parts[-1].strip()
    shape = tuple(int(p) for p in parts[:-1])
    return shape, et


# ----------------------------------------------------------------------------
# text -> nested op list
# ----------------------------------------------------------------------------
class Op:
    __slots__ = ("results", "name", "text", "regions", "result_count")

    def __init__(self, results, name, text):
        self.results = results
        self.name = name
        self.text = text
        self.regions = []


_RES = re.compile(r"^\s*((?:%[\w#.$-]+(?::\d+)?\s*,\s*)*%[\w#.$-]+(?::\d+)?)\s*=\s*(.*)$")


def _strip_loc(line):
    return re.sub(r"\s*loc\((?:[^()]|\([^()]*\))*\)", "", line)


def _split_top(s, sep=","):
    out, depth, cur = [], 0, []
    for ch in s:
        if ch in "<([{":
            depth += 1
        elif ch in ">)]}":
            depth -= 1
        if ch == sep and depth == 0:
            out.append("".join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    tail = "".join(cur).strip()
    if tail:
        out.append(tail)
    return out


class Func:
    def __init__(self, name, args, arg_attrs, body):
        self.name = name
        self.args = args            # [(name, (shape, et))]
        self.arg_attrs = arg_attrs  # [str]
        self.body = body            # [Op]


def _parse_block(lines, i):
    """Parse ops until the closing brace of the enclosing region."""
    ops = []
    while i < len(lines):
        line = lines[i].strip()
        if not line or line.startswith("//"):
            i += 1
            continue
        if line.startswith("}"):
            return ops, i
        if line.startswith("^"):  # block label of a generic-form region
            i += 1
            continue
        m = _RES.match(line)
        if m:
            results = []
            for r in _split_top(m.group(1)):
                if ":" in r:
                    base, n = r.split(":")
                    results += [f"{base}#{k}" for k in range(int(n))]
                else:
                    results.append(r)
            rest = m.group(2)
        else:
            results, rest = [], line
        name = re.match(r'"?([\w.]+)"?', rest).group(1)
        op = Op(results, name, rest)
        i += 1
        if name == "stablehlo.while":
            # "cond {" ... "} do {" ... "}"
            while "cond" not in lines[i - 1] and "cond" not in lines[i]:
                i += 1
            if "cond" in lines[i] and "{" in lines[i]:
                i += 1
            cond, i = _parse_block(lines, i)
            assert "do" in lines[i], lines[i]
            body, i = _parse_block(lines, i + 1)
            op.regions = [cond, body]
            i += 1
        elif name == "stablehlo.reduce_window":
            # generic form: '"stablehlo.reduce_window"(%x, %init) <{attrs}> ({', a block label, the body, '}) : (types) -> type'
            body, i = _parse_block(lines, i)
            op.regions = [body]
            op.text = rest + " " + lines[i].strip()
            i += 1
        elif name == "stablehlo.reduce" and "applies" not in rest:
            # long form: next line is "reducer(%a: t, %b: t) {"
            hdr = lines[i].strip()
            assert hdr.startswith("reducer"), hdr
            args = re.findall(r"(%[\w#.$-]+)\s*:", hdr)
            body, i = _parse_block(lines, i + 1)
            op.regions = [(args, body)]
            i += 1
        ops.append(op)
    return ops, i


def parse_module(text):
    lines = [_strip_loc(l) for l in text.splitlines()]
    mod = {"funcs": {}, "num_partitions": 1, "mesh": {}}
    m = re.search(r"mhlo\.num_partitions\s*=\s*(\d+)", text)
    if m:
        mod["num_partitions"] = int(m.group(1))
    for mm in re.finditer(r"sdy\.mesh\s+@(\w+)\s*=\s*<\[(.*?)\]", text):
        axes = dict((k, int(v)) for k, v in re.findall(r'"(\w+)"\s*=\s*(\d+)', mm.group(2)))
        mod["mesh"][mm.group(1)] = axes
    i = 0
    while i < len(lines):
        line = lines[i].strip()
        fm = re.match(r"func\.func\s+(?:public\s+|private\s+)?@([\w.$-]+)\s*\((.*)$", line)
        if not fm:
            i += 1
            continue
        name = fm.group(1)
        sig = fm.group(2)
        # arguments: up to the matching ')'
        depth, j = 1, 0
        while depth and j < len(sig):
            if sig[j] in "([{<":
                depth += 1
            elif sig[j] in ")]}>":
                depth -= 1
            j += 1
        argtxt = sig[: j - 1]
        args, attrs = [], []
        for a in _split_top(argtxt):
            am = re.match(r"(%[\w#.$-]+)\s*:\s*(tensor<[^>]*>)\s*(\{.*\})?", a)
            args.append((am.group(1), parse_type(am.group(2))))
            attrs.append(am.group(3) or "")
        body, i = _parse_block(lines, i + 1)
        mod["funcs"][name] = Func(name, args, attrs, body)
        i += 1
    return mod


# ----------------------------------------------------------------------------
# evaluation
# ----------------------------------------------------------------------------
def _float_from_attr(tok, et):
    tok = tok.strip()
    if tok.startswith("0x") or tok.startswith("0X"):
        bits = int(tok, 16)
        if et == "f32":
            return np.array([bits], dtype=np.uint32).view(np.float32)[0]
        if et == "f64":
            return np.array([bits], dtype=np.uint64).view(np.float64)[0]
        if et == "bf16":
            return np.array([bits << 16], dtype=np.uint32).view(np.float32)[0]
        return bits
    if tok in ("true", "false"):
        return tok == "true"
    return float(tok) if et.startswith(("f", "bf")) else int(tok)


def _parse_dense(body, shape, et):
    body = body.strip()
    if body.startswith('"0x') or body.startswith('"0X'):
        raw = bytes.fromhex(body.strip('"')[2:])
        if et == "bf16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32)
        else:
            arr = np.frombuffer(raw, dtype=_NP[et])
        return make(arr.reshape(shape), et)
    toks = re.findall(r"[-+]?(?:0x[0-9a-fA-F]+|inf|nan|true|false|\d+\.?\d*(?:[eE][-+]?\d+)?)", body)
    vals = [_float_from_attr(t, et) for t in toks]
    if len(vals) == 1:
        return make(np.full(shape, vals[0]), et)
    return make(np.array(vals).reshape(shape), et)


_UNARY = {
    "sine": np.sin, "cosine": np.cos, "exponential": np.exp, "log": np.log,
    "tanh": np.tanh, "sqrt": np.sqrt, "negate": np.negative, "abs": np.abs,
    "log_plus_one": np.log1p, "exponential_minus_one": np.expm1,
    "floor": np.floor, "ceil": np.ceil, "sign": np.sign,
    "rsqrt": lambda x: 1.0 / np.sqrt(x),
    "logistic": lambda x: 1.0 / (1.0 + np.exp(-x)),
    "not": lambda x: ~x,
    "tan": np.tan, "cbrt": np.cbrt, "round_nearest_even": np.rint,
    "round_nearest_afz": lambda x: np.sign(x) * np.floor(np.abs(x) + 0.5),
    "is_finite": np.isfinite,
}
_BINARY = {
    "add": np.add, "subtract": np.subtract, "multiply": np.multiply,
    "maximum": np.maximum, "minimum": np.minimum, "power": np.power,
    "and": np.bitwise_and, "or": np.bitwise_or, "xor": np.bitwise_xor,
    "atan2": np.arctan2, "remainder": np.fmod,
}
_CMP = {"LT": np.less, "LE": np.less_equal, "GT": np.greater, "GE": np.greater_equal,
        "EQ": np.equal, "NE": np.not_equal}


def _is_float(et):
    return et in ("f32", "f64", "bf16", "f16")


def _wide(t: T):
    """Operate in float64 for floats (then round once), native width for ints."""
    return t.a.astype(np.float64) if _is_float(t.et) else t.a


def _operands(text, env, start):
    """Leading %-operands of an op, up to the first ':' at depth 0 or keyword."""
    names = re.findall(r"%[\w#.$-]+", text[start:].split(" : ")[0])
    return [env[n] for n in names]


def _types_after_colon(text):
    sig = text.rsplit(" : ", 1)[1]
    if "->" in sig:
        ins, outs = sig.rsplit("->", 1)
        outs = outs.strip()
        if outs.startswith("("):
            outs = outs[1:-1]
        return [parse_type(t) for t in _split_top(outs)]
    return [parse_type(t) for t in _split_top(sig)]


class Interpreter:
    def __init__(self, module):
        self.mod = module if isinstance(module, dict) else parse_module(module)

    # -- public ----------------------------------------------------------
    def run(self, inputs, func="main"):
        f = self.mod["funcs"][func]
        assert len(inputs) == len(f.args), (len(inputs), len(f.args))
        env = {}
        for (name, (shape, et)), x in zip(f.args, inputs):
            x = np.asarray(x)
            assert tuple(x.shape) == shape, (name, x.shape, shape)
            env[name] = make(x, et)
        outs = self._run_block(f.body, env)
        return [o.a for o in outs]

    # -- internals -------------------------------------------------------
    def _run_block(self, ops, env):
        for op in ops:
            if op.name in ("return", "func.return", "stablehlo.return"):
                names = re.findall(r"%[\w#.$-]+", op.text.split(" : ")[0])
                return [env[n] for n in names]
            vals = self._eval(op, env)
            if not isinstance(vals, list):
                vals = [vals]
            for r, v in zip(op.results, vals):
                env[r] = v
            if len(op.results) == 1 and len(vals) == 1:
                env[op.results[0]] = vals[0]
        return []

    def _eval(self, op, env):
        name, text = op.name, op.text
        short = name.split(".", 1)[1] if "." in name else name
        if name == "stablehlo.constant":
            m = re.search(r"dense<(.*)>\s*:\s*(tensor<[^>]*>)\s*$", text)
            shape, et = parse_type(m.group(2))
            return _parse_dense(m.group(1), shape, et)
        if name == "stablehlo.iota":
            d = int(re.search(r"dim\s*=\s*(\d+)", text).group(1))
            (shape, et), = _types_after_colon(text)
            idx = np.arange(shape[d]).reshape([-1 if k == d else 1 for k in range(len(shape))])
            return make(np.broadcast_to(idx, shape), et)
        if name == "enzymexla.math.gelu":
            # ext/ReactantNNlibExt/Implementations.jl:12-25 -> src/Ops.jl:4153-4175; evaluated in float64 from the
            # closed forms (the engine expands it into elementwise ops, rounding after each)
            x = env[re.search(r"%[\w#.$-]+", text[len(name):]).group(0)]
            (shape, et) = _types_after_colon(text)[-1]
            v = _wide(x)
            if "TANH" in text:
                r = 0.5 * v * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3)))
            elif "SIGMOID" in text:
                r = v / (1.0 + np.exp(-1.702 * v))
            else:
                raise NotImplementedError("enzymexla.math.gelu NONE")
            return make(r, et)
        if short in _UNARY:
            (x,) = _operands(text, env, len(name))
            (shape, et), = _types_after_colon(text)
            if short == "not" and x.et != "i1":
                return make(~x.a, et)
            return make(_UNARY[short](_wide(x)), et)
        if short in _BINARY:
            a, b = _operands(text, env, len(name))
            (shape, et), = _types_after_colon(text)
            return make(_BINARY[short](_wide(a), _wide(b)), et)
        if short == "divide":
            a, b = _operands(text, env, len(name))
            (shape, et), = _types_after_colon(text)
            if _is_float(et):
                return make(_wide(a) / _wide(b), et)
            q = np.trunc(a.a.astype(np.float64) / b.a.astype(np.float64))
            return make(q, et)
        if short == "convert":
            (x,) = _operands(text, env, len(name))
            (shape, et), = _types_after_colon(text)
            if _is_float(x.et) and not _is_float(et):
                # float -> integer saturates and maps NaN to 0 (what XLA's CPU backend does for stablehlo.convert)
                t = np.nan_to_num(np.trunc(x.a.astype(np.float64)), nan=0.0, posinf=np.inf, neginf=-np.inf)
                if et != "i1":
                    info = np.iinfo(_NP[et])
                    t = np.clip(t, info.min, info.max)
                return make(t, et)
            return make(x.a, et)
        if short == "compare":
            m = re.search(r"compare\s+(\w+)\s*,", text)
            a, b = _operands(text, env, m.end())
            return T(_CMP[m.group(1)](a.a, b.a), "i1")
        if short == "select":
            p, a, b = _operands(text, env, len(name))
            return T(np.where(p.a, a.a, b.a), a.et)
        if short == "clamp":
            lo, x, hi = _operands(text, env, len(name))
            return T(np.minimum(np.maximum(x.a, lo.a), hi.a), x.et)
        if short == "broadcast_in_dim":
            (x,) = _operands(text, env, len(name))
            dims = [int(v) for v in re.search(r"dims\s*=\s*\[([^\]]*)\]", text).group(1).split(",") if v.strip()]
            (shape, et), = _types_after_colon(text)
            tmp = [1] * len(shape)
            for k, d in enumerate(dims):
                tmp[d] = x.shape[k]
            return T(np.broadcast_to(x.a.reshape(tmp), shape).copy(), et)
        if short == "transpose":
            (x,) = _operands(text, env, len(name))
            perm = [int(v) for v in re.search(r"dims\s*=\s*\[([^\]]*)\]", text).group(1).split(",") if v.strip()]
            return T(np.ascontiguousarray(np.transpose(x.a, perm)), x.et)
        if short == "reshape":
            (x,) = _operands(text, env, len(name))
            (shape, et), = _types_after_colon(text)
            return T(x.a.reshape(shape), et)
        if short == "slice":
            (x,) = _operands(text, env, len(name))
            spec = re.search(r"\[([^\]]*)\]\s*:", text).group(1)
            sl = []
            for part in spec.split(","):
                v = [int(p) for p in part.strip().split(":")]
                sl.append(slice(v[0], v[1], v[2] if len(v) > 2 else 1))
            return T(np.ascontiguousarray(x.a[tuple(sl)]), x.et)
        if short == "dynamic_slice":
            vals = _operands(text, env, len(name))
            x, starts = vals[0], vals[1:]
            sizes = [int(v) for v in re.search(r"sizes\s*=\s*\[([^\]]*)\]", text).group(1).split(",")]
            sl = []
            for d, (s, n) in enumerate(zip(starts, sizes)):
                st = int(np.clip(int(s.a), 0, x.shape[d] - n))
                sl.append(slice(st, st + n))
            return T(np.ascontiguousarray(x.a[tuple(sl)]), x.et)
        if short == "dynamic_slice":
            # %r = stablehlo.dynamic_slice %x, %i0, ..., sizes = [..]: start indices clamped so that the slice fits
            vals = _operands(text[:text.index("sizes")], env, len(name))
            x, starts = vals[0], vals[1:]
            sizes = [int(v) for v in re.search(r"sizes\s*=\s*\[([^\]]*)\]", text).group(1).split(",") if v.strip()]
            sl = []
            for d, st in enumerate(starts):
                b = int(np.clip(int(st.a), 0, x.shape[d] - sizes[d]))
                sl.append(slice(b, b + sizes[d]))
            return T(np.ascontiguousarray(x.a[tuple(sl)]), x.et)
        if short == "dynamic_update_slice":
            vals = _operands(text, env, len(name))
            x, u, starts = vals[0], vals[1], vals[2:]
            out = x.a.copy()
            sl = []
            for d, s in enumerate(starts):
                # start indices are clamped so that the update fits
                st = int(np.clip(int(s.a), 0, x.shape[d] - u.shape[d]))
                sl.append(slice(st, st + u.shape[d]))
            out[tuple(sl)] = u.a
            return T(out, x.et)
        if short == "pad":
            x, pv = _operands(text, env, len(name))
            get = lambda k: [int(v) for v in re.search(k + r"\s*=\s*\[([^\]]*)\]", text).group(1).split(",") if v.strip()]
            low, high, interior = get("low"), get("high"), get("interior")
            assert all(v == 0 for v in interior), "interior padding not on the path"
            assert all(v >= 0 for v in low + high), "negative padding not on the path"
            out = np.pad(x.a, list(zip(low, high)), constant_values=pv.a.item())
            return T(out, x.et)
        if short == "concatenate":
            vals = _operands(text, env, len(name))
            d = int(re.search(r"dim\s*=\s*(\d+)", text).group(1))
            return T(np.concatenate([v.a for v in vals], axis=d), vals[0].et)
        if short == "dot_general":
            a, b = _operands(text, env, len(name))
            cm = re.search(r"contracting_dims\s*=\s*\[([^\]]*)\]\s*x\s*\[([^\]]*)\]", text)
            bm = re.search(r"batching_dims\s*=\s*\[([^\]]*)\]\s*x\s*\[([^\]]*)\]", text)
            ints = lambda s: [int(v) for v in s.split(",") if v.strip()]
            lc, rc = ints(cm.group(1)), ints(cm.group(2))
            lb, rb = (ints(bm.group(1)), ints(bm.group(2))) if bm else ([], [])
            (shape, et), = _types_after_colon(text)
            A, B = _wide(a), _wide(b)
            lfree = [d for d in range(A.ndim) if d not in lc + lb]
            rfree = [d for d in range(B.ndim) if d not in rc + rb]
            letters = "abcdefghijklmnopqrstuvwxyz"
            la, rb_ = [""] * A.ndim, [""] * B.ndim
            k = 0
            for x_, y_ in zip(lb, rb):
                la[x_] = rb_[y_] = letters[k]; k += 1
            batch = "".join(la[d] for d in lb)
            for x_, y_ in zip(lc, rc):
                la[x_] = rb_[y_] = letters[k]; k += 1
            for d in lfree:
                la[d] = letters[k]; k += 1
            for d in rfree:
                rb_[d] = letters[k]; k += 1
            out = batch + "".join(la[d] for d in lfree) + "".join(rb_[d] for d in rfree)
            if not lb:
                # same sum, same float64 accumulation, through BLAS: result dims are (lhs free, rhs free)
                res = np.tensordot(A, B, axes=(lc, rc))
            else:
                res = np.einsum(f"{''.join(la)},{''.join(rb_)}->{out}", A, B)
            return make(res.reshape(shape), et)
        if short == "reduce":
            return self._reduce(op, env)
        if short == "reduce_window":
            return self._reduce_window(op, env)
        if short == "while":
            return self._while(op, env)
        if short == "all_reduce":
            # single-address-space evaluation: the operand already is the global value
            return _operands(text, env, len(name))[0]
        raise NotImplementedError(f"oracle: unsupported op {name}")

    def _reduce(self, op, env):
        text = op.text
        m = re.search(r"reduce\(\s*(%[\w#.$-]+)\s+init:\s*(%[\w#.$-]+)\s*\)", text)
        x, init = env[m.group(1)], env[m.group(2)]
        dims = tuple(int(v) for v in re.search(r"dimensions\s*=\s*\[([^\]]*)\]", text).group(1).split(",") if v.strip())
        (shape, et), = _types_after_colon(text)
        am = re.search(r"applies\s+stablehlo\.(\w+)", text)
        if am:
            kind = am.group(1)
        else:
            _, body = op.regions[0]
            kinds = [o.name.split(".", 1)[1] for o in body if o.name != "stablehlo.return"]
            assert len(kinds) == 1, "only single-op reducers are on the path"
            kind = kinds[0]
        X = _wide(x)
        i0 = _wide(init)
        if kind == "add":
            r = X.sum(axis=dims) + i0 if not (x.et == "i1") else np.logical_or(X.any(axis=dims), i0)
        elif kind == "maximum":
            r = np.maximum(X.max(axis=dims, initial=-np.inf if _is_float(x.et) else np.iinfo(X.dtype).min), i0)
        elif kind == "minimum":
            r = np.minimum(X.min(axis=dims, initial=np.inf if _is_float(x.et) else np.iinfo(X.dtype).max), i0)
        elif kind == "multiply":
            r = X.prod(axis=dims) * i0
        elif kind == "or":
            r = np.logical_or(X.any(axis=dims), i0)
        elif kind == "and":
            r = np.logical_and(X.all(axis=dims), i0)
        else:
            raise NotImplementedError(f"oracle: reducer {kind}")
        return make(np.asarray(r).reshape(shape), et)

    def _reduce_window(self, op, env):
        """stablehlo.reduce_window with a single-op combiner, base dilations of 1.  The cumulative form (Reactant's
        scan_impl!, src/TracedRArray.jl:1049-1107: the window spans one whole dimension, padded low by its extent minus
        one) is an inclusive scan; anything else (pooling windows) is evaluated position by position over the operand
        padded with the init value, in the wide type."""
        text = op.text
        names = re.findall(r"%[\w#.$-]+", text[text.index("("):text.index(")")])
        x, init = env[names[0]], env[names[1]]
        win = [int(v) for v in re.search(r"window_dimensions\s*=\s*array<i64:\s*([^>]*)>", text).group(1).split(",")]
        rank = len(win)
        pm = re.search(r"padding\s*=\s*dense<(.*?)>\s*:\s*tensor<(\d+)x2xi64>", text)
        nums = [int(v) for v in re.findall(r"-?\d+", pm.group(1))] if pm else [0]
        pad = [(nums[2 * d], nums[2 * d + 1]) for d in range(rank)] if len(nums) == 2 * rank else [(nums[0], nums[0])] * rank

        def ints(attr):
            m = re.search(attr + r"\s*=\s*array<i64:\s*([^>]*)>", text)
            return [int(v) for v in m.group(1).split(",")] if m else [1] * rank

        strides, wdil = ints("window_strides"), ints("window_dilations")
        assert all(v == 1 for v in ints("base_dilations")), "oracle: base_dilations other than 1"
        shape = list(x.a.shape)
        kinds = [o.name.split(".", 1)[1] for o in op.regions[0] if o.name != "stablehlo.return"]
        assert len(kinds) == 1, "only single-op reducers are on the path"
        kind = kinds[0]
        X, i0 = _wide(x), _wide(init)
        ufunc = {"add": np.add, "maximum": np.maximum, "minimum": np.minimum, "multiply": np.multiply}[kind]
        (oshape, et), = _types_after_colon(text)[-1:]
        axes = [d for d in range(rank) if win[d] != 1 or pad[d] != (0, 0) or strides[d] != 1]
        if not axes:
            return make(np.asarray(ufunc(X, i0)).reshape(oshape), et)
        if len(axes) == 1 and win[axes[0]] == shape[axes[0]] and pad[axes[0]] == (shape[axes[0]] - 1, 0) and strides[axes[0]] == 1 and wdil[axes[0]] == 1:
            r = ufunc(ufunc.accumulate(X, axis=axes[0]), i0)
            return make(np.asarray(r).reshape(oshape), et)
        P = np.pad(X, pad, mode="constant", constant_values=i0.item())
        r = None
        for k in np.ndindex(*win):
            sl = tuple(slice(k[d] * wdil[d], k[d] * wdil[d] + (oshape[d] - 1) * strides[d] + 1, strides[d]) for d in range(rank))
            piece = P[sl]
            assert list(piece.shape) == list(oshape), (piece.shape, oshape)
            r = piece if r is None else ufunc(r, piece)
        return make(np.asarray(r).reshape(oshape), et)

    def _while(self, op, env):
        text = op.text
        pairs = re.findall(r"(%[\w#.$-]+)\s*=\s*(%[\w#.$-]+)", text[text.index("(") + 1:text.index(")")])
        names = [p[0] for p in pairs]
        state = [env[p[1]] for p in pairs]
        cond, body = op.regions
        guard = 0
        while True:
            scope = dict(env)
            scope.update(zip(names, state))
            (c,) = self._run_block(cond, scope)
            if not bool(c.a):
                break
            scope = dict(env)
            scope.update(zip(names, state))
            state = self._run_block(body, scope)
            guard += 1
            assert guard < 1_000_000, "runaway loop"
        return list(state)


def run_module(text, inputs, func="main"):
    """Evaluate `@main` of a StableHLO module on numpy inputs (XLA layout:
    row-major over the tensor type's dims)."""
    return Interpreter(text).run(inputs, func)


# ----------------------------------------------------------------------------
# layout helpers shared by the tests (the boundary convention, restated)
# ----------------------------------------------------------------------------
def julia_to_xla(a: np.ndarray) -> np.ndarray:
    """A Julia column-major array of size (d1..dn) crosses the runtime boundary
    as a row-major tensor of dims (dn..d1) with the same bytes
    (src/xla/PJRT/Buffer.jl:9-17, src/TracedUtils.jl:511-527)."""
    return np.ascontiguousarray(np.transpose(a))


def construct_test_array(dtype, *dims):
    """src/TestUtils.jl:9-23: 1:prod(dims) (divided by prod(dims) for floats),
    reshaped column-major.  Returned as a numpy array indexed like Julia."""
    n = int(np.prod(dims))
    flat = np.arange(1, n + 1)
    if np.issubdtype(np.dtype(dtype), np.floating):
        flat = (flat.astype(dtype) / dtype(n)).astype(dtype)
    else:
        flat = flat.astype(dtype)
    return flat.reshape(dims, order="F")


def reduction_tolerance(n):
    """fp32 reduction bar: relative error <= 1e-5 * sqrt(log2 n)."""
    return 1e-5 * math.sqrt(max(1.0, math.log2(max(2, n))))
