"""CPU oracle: a NumPy restatement of StableHLO semantics for the op subset the B200 executor serves.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path imports this file; it is used by tests/, by
`__graft_entry__.smoke()` and by `bench.py`'s CPU-baseline legs as the checker / reported baseline.

Why a restatement: the reference (eaplatanios/ryft) executes these programs inside OpenXLA's CPU PJRT plugin
(OpenXLA commit 7b1be14958aac5c83f1b9f7bcdfc51fdbd29acba, crates/ryft-xla-sys/WORKSPACE:9; StableHLO 1.16.0,
crates/ryft-pjrt/src/lib.rs:575-576), which is fetched at build time and is not part of the reference tree, so it
cannot be compiled or imported here.  The semantics below follow the rules the reference documents beside each op
builder under crates/ryft-mlir/src/dialects/stable_hlo/operations/ (cited per function), which restate the published
StableHLO specification.

Pinning: tests/test_oracle_golden.py checks this evaluator against every known answer the reference's tests and doc
comments hold for these ops (README matmul, the i32 add of programs.rs:2781-2829, and the worked examples in the doc
comments of dot_general, reduce, iota, broadcast_in_dim, compare, tanh, all_reduce, all_gather).  Everything beyond
those vectors (bf16 GEMM, softmax/attention, GELU gradients at scale) is PARITY UNPINNED by the reference itself.

Numerics: dot_general multiplies exactly and accumulates in float64 (then rounds to the result element type);
elementwise ops on bf16/f16 compute in float32 and round to the element type after every op (what a CPU evaluation in
that type does); reductions accumulate in float64 for float types.  Integer and predicate ops are exact.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

try:
    import ml_dtypes
    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _BF16 = None

_DTYPES = {"i1": np.dtype(np.bool_), "i8": np.dtype(np.int8), "i16": np.dtype(np.int16), "i32": np.dtype(np.int32),
           "i64": np.dtype(np.int64), "ui8": np.dtype(np.uint8), "ui16": np.dtype(np.uint16), "ui32": np.dtype(np.uint32),
           "ui64": np.dtype(np.uint64), "f16": np.dtype(np.float16), "f32": np.dtype(np.float32), "f64": np.dtype(np.float64)}


def np_dtype(name: str) -> np.dtype:
    if name == "bf16":
        return _BF16
    return _DTYPES[name]


@dataclass
class TType:
    dims: Tuple[int, ...]
    dtype: str

    @property
    def np(self) -> np.dtype:
        return np_dtype(self.dtype)


@dataclass
class OpRec:
    name: str                      # short op name: add, dot_general, ...
    results: List[str]
    operands: List[str]
    attrs: Dict[str, object]
    result_types: List[TType]
    operand_types: List[TType] = field(default_factory=list)


@dataclass
class ModuleRec:
    args: List[Tuple[str, TType]]
    ops: List[OpRec]
    returns: List[str]


_TYPE_RE = re.compile(r"tensor<((?:\d+x)*)([a-z0-9]+)>")


def _parse_type(s: str) -> TType:
    m = _TYPE_RE.search(s)
    if not m:
        raise ValueError(f"cannot parse type in {s!r}")
    dims = tuple(int(d) for d in m.group(1).split("x") if d)
    return TType(dims, m.group(2))


def _types_in(s: str) -> List[TType]:
    return [TType(tuple(int(d) for d in m.group(1).split("x") if d), m.group(2)) for m in _TYPE_RE.finditer(s)]


def _ints(s: str) -> List[int]:
    return [int(x) for x in re.findall(r"-?\d+", s)]


def _statements(body: str) -> List[str]:
    """Splits a function body into statements; a statement may span lines while brackets are open."""
    out, cur, depth = [], "", 0
    for line in body.splitlines():
        line = line.split("//")[0].rstrip()
        if not line.strip():
            continue
        cur = (cur + " " + line.strip()) if cur else line.strip()
        depth += sum(line.count(c) for c in "({[") - sum(line.count(c) for c in ")}]")
        if depth <= 0:
            out.append(cur)
            cur, depth = "", 0
    if cur:
        out.append(cur)
    return out


def _dense_values(lit: str, t: TType) -> np.ndarray:
    """dense<...> literal -> array; hex integers are bit patterns for float types
    (crates/ryft-mlir/src/dialects/builtin/attributes/float.rs:12-24)."""
    dt = t.np
    toks = re.findall(r"0x[0-9A-Fa-f]+|true|false|[-+]?(?:\d+\.?\d*(?:[eE][-+]?\d+)?|\.\d+(?:[eE][-+]?\d+)?|inf|nan)", lit)
    vals = []
    for tok in toks:
        if tok.startswith("0x") and t.dtype in ("f32", "bf16", "f16", "f64"):
            bits = int(tok, 16)
            width = dt.itemsize
            raw = bits.to_bytes(width, "little")
            vals.append(np.frombuffer(raw, dtype=dt)[0])
        elif tok in ("true", "false"):
            vals.append(tok == "true")
        elif t.dtype.startswith("f") or t.dtype == "bf16":
            vals.append(np.float64(tok))
        else:
            vals.append(int(tok, 0))
    n = int(np.prod(t.dims)) if t.dims else 1
    arr = np.empty(len(vals), dtype=dt)
    for i, v in enumerate(vals):
        arr[i] = v
    if len(vals) == 1 and n != 1:
        return np.full(t.dims, arr[0], dtype=dt)
    return arr.reshape(t.dims)


def parse(text: str) -> ModuleRec:
    """Reads `module { func.func @main(...) { ... } }` in the printed forms of ryft-mlir
    (e.g. crates/ryft-pjrt/src/programs.rs:2492-2498)."""
    m = re.search(r"func\.func\s+(?:public\s+|private\s+)?@\w+\s*\((.*?)\)\s*(?:->\s*(.*?))?\s*(?:attributes\s*\{.*?\}\s*)?\{\n", text, re.S)
    if not m:
        raise ValueError("no func.func found")
    args = []
    for a in re.finditer(r"(%[\w#]+)\s*:\s*(tensor<[^>]*>)", m.group(1)):
        args.append((a.group(1), _parse_type(a.group(2))))
    body = text[m.end():]
    # cut at the function's closing brace: last '}' pair belongs to func and module
    depth, end = 1, len(body)
    for i, ch in enumerate(body):
        if ch == "{":
            depth += 1
        elif ch == "}":
            depth -= 1
            if depth == 0:
                end = i
                break
    ops: List[OpRec] = []
    returns: List[str] = []
    for st in _statements(body[:end]):
        if st.startswith("return") or st.startswith("func.return") or st.startswith('"func.return"'):
            returns = re.findall(r"%[\w#]+", st.split(":")[0])
            continue
        lhs, rhs = st.split("=", 1) if re.match(r"\s*%[\w#:, ]+=", st) else ("", st)
        res_names = []
        for tok in re.findall(r"%[\w#]+(?::\d+)?", lhs):
            if ":" in tok:
                base, n = tok.split(":")
                res_names += [f"{base}#{i}" for i in range(int(n))]
            else:
                res_names.append(tok)
        rhs = rhs.strip()
        gm = re.match(r'"stablehlo\.(\w+)"\((.*?)\)\s*(<\{.*?\}>)?\s*(\(\{.*\}\))?\s*(\{.*?\})?\s*:\s*(.*)$', rhs, re.S)
        if gm:
            name = gm.group(1)
            operands = re.findall(r"%[\w#]+", gm.group(2))
            props = (gm.group(3) or "") + (gm.group(5) or "")
            sig = gm.group(6)
            ins, outs = sig.split("->")
            attrs: Dict[str, object] = {}
            rg = re.search(r"replica_groups\s*=\s*dense<(.*?)>\s*:\s*tensor<(\d+)x(\d+)xi64>", props, re.S)
            if rg:
                flat = _ints(rg.group(1))
                rows, cols = int(rg.group(2)), int(rg.group(3))
                if len(flat) == 1:
                    flat = flat * (rows * cols)
                attrs["replica_groups"] = [[v for v in flat[r * cols:(r + 1) * cols] if v >= 0] for r in range(rows)]
            ag = re.search(r"all_gather_dim\s*=\s*(\d+)", props)
            if ag:
                attrs["all_gather_dim"] = int(ag.group(1))
            dm = re.search(r"dimensions\s*=\s*array<i64:?\s*([^>]*)>", props)
            if dm:
                attrs["dimensions"] = _ints(dm.group(1))
            if gm.group(4):
                bm = re.search(r"stablehlo\.(\w+)\s+%", gm.group(4))
                attrs["body"] = bm.group(1) if bm else "add"
            ops.append(OpRec(name, res_names, operands, attrs, _types_in(outs), _types_in(ins)))
            continue
        pm = re.match(r"stablehlo\.(\w+)\s*(.*)$", rhs, re.S)
        if not pm:
            raise ValueError(f"cannot parse statement: {st}")
        name, rest = pm.group(1), pm.group(2)
        attrs = {}
        head, _, sig = rest.rpartition(" : ") if " : " in rest else ("", "", rest.lstrip(": "))
        if name == "constant":
            cm = re.match(r"dense<(.*)>\s*:\s*(tensor<[^>]*>)\s*$", rest, re.S)
            t = _parse_type(cm.group(2))
            attrs["value"] = _dense_values(cm.group(1), t)
            ops.append(OpRec(name, res_names, [], attrs, [t]))
            continue
        operands = re.findall(r"%[\w#]+", head)
        tys = _types_in(sig)
        if "->" in sig:
            ins_s, outs_s = sig.split("->")
            in_t, out_t = _types_in(ins_s), _types_in(outs_s)
        elif name == "select":
            in_t, out_t = [], [tys[-1]]
        else:
            in_t, out_t = [], [tys[0]]
        if name == "iota":
            attrs["dim"] = int(re.search(r"dim\s*=\s*(\d+)", head if head else rest).group(1))
        elif name in ("broadcast_in_dim", "transpose"):
            attrs["dims"] = _ints(re.search(r"dims\s*=\s*\[([^\]]*)\]", head).group(1))
        elif name == "compare":
            attrs["direction"] = re.match(r"\s*(\w+)", head).group(1)
        elif name == "dot_general":
            bm = re.search(r"batching_dims\s*=\s*\[([^\]]*)\]\s*x\s*\[([^\]]*)\]", head)
            cm = re.search(r"contracting_dims\s*=\s*\[([^\]]*)\]\s*x\s*\[([^\]]*)\]", head)
            attrs["lb"], attrs["rb"] = (_ints(bm.group(1)), _ints(bm.group(2))) if bm else ([], [])
            attrs["lc"], attrs["rc"] = _ints(cm.group(1)), _ints(cm.group(2))
            operands = operands[:2]
        elif name == "reduce":
            rm = re.match(r"\((%[\w#]+)\s+init:\s*(%[\w#]+)\)\s*(?:applies\s+stablehlo\.(\w+)\s+)?across dimensions\s*=\s*\[([^\]]*)\]", head)
            operands = [rm.group(1), rm.group(2)]
            attrs["body"] = rm.group(3) or "add"
            attrs["dimensions"] = _ints(rm.group(4))
        ops.append(OpRec(name, res_names, operands, attrs, out_t, in_t))
    return ModuleRec(args, ops, returns)


# ---- evaluation -------------------------------------------------------------------------------------------------------
def _is_narrow_float(dt: np.dtype) -> bool:
    return dt == _BF16 or dt == np.float16


def _unary_float(fn, x: np.ndarray) -> np.ndarray:
    if _is_narrow_float(x.dtype):
        return fn(x.astype(np.float32)).astype(x.dtype)
    return fn(x).astype(x.dtype)


def _binary(fn, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    if _is_narrow_float(a.dtype):
        return fn(a.astype(np.float32), b.astype(np.float32)).astype(a.dtype)
    with np.errstate(all="ignore"):
        return fn(a, b).astype(a.dtype)


def _int_div(a, b):
    """Integer division truncates toward zero."""
    if np.issubdtype(a.dtype, np.integer):
        q = np.where(b == 0, -1, np.trunc(a.astype(np.float64) / np.where(b == 0, 1, b).astype(np.float64)))
        return q.astype(a.dtype)
    return a / b


_MONOID = {"add": np.add, "multiply": np.multiply, "maximum": np.maximum, "minimum": np.minimum, "and": np.logical_and,
           "or": np.logical_or, "xor": np.logical_xor}


def _dot_general(a: np.ndarray, b: np.ndarray, lb, rb, lc, rc, out_t: TType) -> np.ndarray:
    """result[batch..., lhs free..., rhs free...] = sum over contracting dims of lhs * rhs
    (crates/ryft-mlir/src/dialects/stable_hlo/operations/linear_algebra.rs:561-592)."""
    lf = [i for i in range(a.ndim) if i not in lb and i not in lc]
    rf = [i for i in range(b.ndim) if i not in rb and i not in rc]
    if np.issubdtype(a.dtype, np.integer) or a.dtype == np.bool_:
        acc = np.int64
    else:
        acc = np.float64
    A = np.transpose(a, list(lb) + lf + list(lc)).astype(acc)
    B = np.transpose(b, list(rb) + list(rc) + rf).astype(acc)
    bs = [a.shape[i] for i in lb]
    M = int(np.prod([a.shape[i] for i in lf])) if lf else 1
    K = int(np.prod([a.shape[i] for i in lc])) if lc else 1
    N = int(np.prod([b.shape[i] for i in rf])) if rf else 1
    nb = int(np.prod(bs)) if bs else 1
    C_ = np.matmul(A.reshape(nb, M, K), B.reshape(nb, K, N))
    return C_.reshape(out_t.dims).astype(out_t.np)


def evaluate(text_or_module, inputs_per_replica: Sequence[Sequence[np.ndarray]], fast_dot: bool = False) -> List[List[np.ndarray]]:
    """Evaluates the module for every replica (outer list) and returns each replica's outputs.

    With `fast_dot` the contraction accumulates in float32 through BLAS (used for timing the CPU baseline)."""
    mod = parse(text_or_module) if isinstance(text_or_module, str) else text_or_module
    nrep = len(inputs_per_replica)
    env: List[Dict[str, np.ndarray]] = []
    for r in range(nrep):
        e = {}
        for (name, t), arr in zip(mod.args, inputs_per_replica[r]):
            arr = np.asarray(arr)
            assert tuple(arr.shape) == t.dims and arr.dtype == t.np, (name, arr.shape, arr.dtype, t)
            e[name] = arr
        env.append(e)
    # a value is dropped after its last use, so that a full-size program does not hold every intermediate at once
    last_use: Dict[str, int] = {}
    for i, op in enumerate(mod.ops):
        for o in op.operands:
            last_use[o] = i
    keep = set(mod.returns)
    for i, op in enumerate(mod.ops):
        outs_per_rep = [_eval_op(op, [env[r][o] for o in op.operands], r, fast_dot) for r in range(nrep)] if op.name not in ("all_reduce", "all_gather") else \
            _eval_collective(op, [[env[r][o] for o in op.operands] for r in range(nrep)])
        for r in range(nrep):
            for n, v in zip(op.results, outs_per_rep[r]):
                env[r][n] = v
        for o in set(op.operands):
            if last_use.get(o) == i and o not in keep:
                for r in range(nrep):
                    env[r].pop(o, None)
    return [[env[r][n] for n in mod.returns] for r in range(nrep)]


def use_all_host_threads() -> int:
    """Lets the BLAS behind NumPy use every host core, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to
    1 for multi-process runs).  Returns the number of threads now in use (1 when the pool cannot be inspected)."""
    import os
    n = os.cpu_count() or 1
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=n)
        pools = [p.get("num_threads", 1) for p in threadpoolctl.threadpool_info() if p.get("user_api") == "blas"]
        return max(pools) if pools else 1
    except Exception:
        return 1


def _eval_collective(op: OpRec, ins: List[List[np.ndarray]]) -> List[List[np.ndarray]]:
    """all_reduce / all_gather over replica groups, cross-replica mode
    (crates/ryft-mlir/src/dialects/stable_hlo/operations/communication.rs:714-739, 807-841)."""
    nrep = len(ins)
    groups = op.attrs.get("replica_groups") or [list(range(nrep))]
    out: List[List[np.ndarray]] = [[None] * len(op.operands) for _ in range(nrep)]
    for g in groups:
        for k in range(len(op.operands)):
            if op.name == "all_reduce":
                fn = _MONOID[op.attrs.get("body", "add")]
                dt = ins[g[0]][k].dtype
                acc = ins[g[0]][k].astype(np.float64 if dt.kind == "f" or dt == _BF16 else dt)
                for r in g[1:]:
                    acc = fn(acc, ins[r][k].astype(acc.dtype))
                for r in g:
                    out[r][k] = acc.astype(dt)
            else:
                cat = np.concatenate([ins[r][k] for r in g], axis=op.attrs["all_gather_dim"])
                for r in g:
                    out[r][k] = cat
    return out


def _eval_op(op: OpRec, x: List[np.ndarray], replica: int, fast_dot: bool) -> List[np.ndarray]:
    n = op.name
    t = op.result_types[0]
    if n == "constant":
        return [op.attrs["value"]]
    if n == "iota":  # miscellaneous.rs:67-129
        shape = [1] * len(t.dims)
        shape[op.attrs["dim"]] = t.dims[op.attrs["dim"]]
        return [np.broadcast_to(np.arange(t.dims[op.attrs["dim"]]).reshape(shape), t.dims).astype(t.np)]
    if n == "replica_id":
        return [np.array(replica, dtype=np.uint32)]
    if n == "partition_id":
        return [np.array(0, dtype=np.uint32)]
    if n == "broadcast_in_dim":  # manipulation.rs:271-285: result[i] = operand[i[dims[d]]]
        dims = op.attrs["dims"]
        shape = [1] * len(t.dims)
        for d, rd in enumerate(dims):
            shape[rd] = x[0].shape[d]
        perm = np.argsort(dims) if len(dims) else []
        src = np.transpose(x[0], perm).reshape(shape) if len(dims) else x[0].reshape(shape)
        return [np.broadcast_to(src, t.dims).copy()]
    if n == "transpose":
        return [np.transpose(x[0], op.attrs["dims"]).copy()]
    if n == "reshape":
        return [x[0].reshape(t.dims)]
    if n == "convert":  # casting.rs:123: float -> narrower float rounds to nearest even; float -> int truncates
        src, dst = x[0], t.np
        if dst == np.bool_:
            return [(src.astype(np.float64) != 0) if src.dtype != np.bool_ else src]
        if (src.dtype.kind == "f" or src.dtype == _BF16) and dst.kind in "iu":
            return [np.trunc(src.astype(np.float64)).astype(dst)]
        return [src.astype(np.float32).astype(dst) if _is_narrow_float(src.dtype) else src.astype(dst)]
    if n == "compare":  # comparison.rs:136-164
        a, b = x
        if _is_narrow_float(a.dtype):
            a, b = a.astype(np.float32), b.astype(np.float32)
        fn = {"EQ": np.equal, "NE": np.not_equal, "GE": np.greater_equal, "GT": np.greater, "LE": np.less_equal, "LT": np.less}[op.attrs["direction"]]
        return [fn(a, b)]
    if n == "select":  # control_flow.rs:263
        return [np.where(x[0], x[1], x[2]).astype(t.np)]
    if n == "clamp":
        return [_binary(np.minimum, _binary(np.maximum, x[1], np.broadcast_to(x[0], x[1].shape)), np.broadcast_to(x[2], x[1].shape))]
    if n == "dot_general":
        if fast_dot and x[0].dtype != np.int64:
            a32, b32 = x[0].astype(np.float32), x[1].astype(np.float32)
            lb, rb, lc, rc = op.attrs["lb"], op.attrs["rb"], op.attrs["lc"], op.attrs["rc"]
            lf = [i for i in range(a32.ndim) if i not in lb and i not in lc]
            rf = [i for i in range(b32.ndim) if i not in rb and i not in rc]
            A = np.transpose(a32, list(lb) + lf + list(lc)); B = np.transpose(b32, list(rb) + list(rc) + rf)
            nb = int(np.prod([a32.shape[i] for i in lb])) if lb else 1
            M = int(np.prod([a32.shape[i] for i in lf])) if lf else 1
            K = int(np.prod([a32.shape[i] for i in lc])) if lc else 1
            N = int(np.prod([b32.shape[i] for i in rf])) if rf else 1
            return [np.matmul(A.reshape(nb, M, K), B.reshape(nb, K, N)).reshape(t.dims).astype(t.np)]
        return [_dot_general(x[0], x[1], op.attrs["lb"], op.attrs["rb"], op.attrs["lc"], op.attrs["rc"], t)]
    if n == "reduce":  # functional.rs:109-118 (order unspecified; the body is a monoid)
        a, init = x
        body = op.attrs["body"]
        dims = tuple(op.attrs["dimensions"])
        wide = a.astype(np.float64) if (a.dtype.kind == "f" or a.dtype == _BF16) else a
        if body == "add":
            r = wide.sum(axis=dims) + init.astype(wide.dtype)
        elif body == "multiply":
            r = wide.prod(axis=dims) * init.astype(wide.dtype)
        elif body == "maximum":
            r = np.maximum(wide.max(axis=dims) if wide.size else np.full(t.dims, -np.inf), init.astype(wide.dtype))
        elif body == "minimum":
            r = np.minimum(wide.min(axis=dims) if wide.size else np.full(t.dims, np.inf), init.astype(wide.dtype))
        elif body in ("and", "or", "xor"):
            fn = {"and": np.logical_and, "or": np.logical_or, "xor": np.logical_xor}[body]
            r = fn(fn.reduce(wide, axis=dims) if len(dims) == 1 else fn.reduce(wide.reshape(wide.shape), axis=dims), init)
        else:
            raise NotImplementedError(body)
        return [np.asarray(r).astype(t.np).reshape(t.dims)]
    # elementwise arithmetic (arithmetic.rs:190-453; comparison.rs:274-341; trigonometric.rs:157-201; exponential.rs)
    un = {"negate": np.negative, "abs": np.abs, "tanh": np.tanh, "exponential": np.exp, "log": np.log, "sqrt": np.sqrt,
          "rsqrt": lambda v: 1.0 / np.sqrt(v), "logistic": lambda v: 1.0 / (1.0 + np.exp(-v)), "sign": np.sign, "floor": np.floor,
          "ceil": np.ceil, "exponential_minus_one": np.expm1, "log_plus_one": np.log1p, "sine": np.sin, "cosine": np.cos}
    if n in un:
        with np.errstate(all="ignore"):
            return [_unary_float(un[n], x[0])]
    if n == "not":
        return [np.logical_not(x[0]) if x[0].dtype == np.bool_ else np.invert(x[0])]
    bi = {"add": np.add, "subtract": np.subtract, "multiply": np.multiply, "maximum": np.maximum, "minimum": np.minimum,
          "power": np.power, "remainder": np.fmod,
          "and": lambda a, b: np.logical_and(a, b) if a.dtype == np.bool_ else np.bitwise_and(a, b),
          "or": lambda a, b: np.logical_or(a, b) if a.dtype == np.bool_ else np.bitwise_or(a, b),
          "xor": lambda a, b: np.logical_xor(a, b) if a.dtype == np.bool_ else np.bitwise_xor(a, b)}
    if n in bi:
        return [_binary(bi[n], x[0], x[1])]
    if n == "divide":
        return [_binary(_int_div, x[0], x[1]) if x[0].dtype.kind in "iu" else _binary(np.divide, x[0], x[1])]
    raise NotImplementedError(f"stablehlo.{n}")


# ---- error metrics used by the parity tests (tolerances come from the build's north star) --------------------------------
def rel_frobenius(actual: np.ndarray, expected: np.ndarray) -> float:
    a, e = np.asarray(actual, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    d = np.linalg.norm((a - e).ravel())
    n = np.linalg.norm(e.ravel())
    return float(d / n) if n > 0 else float(d)


def max_abs_over_rms(actual: np.ndarray, expected: np.ndarray) -> float:
    a, e = np.asarray(actual, dtype=np.float64), np.asarray(expected, dtype=np.float64)
    rms = float(np.sqrt(np.mean(e.ravel() ** 2))) if e.size else 0.0
    m = float(np.max(np.abs(a - e))) if e.size else 0.0
    return m / rms if rms > 0 else m
