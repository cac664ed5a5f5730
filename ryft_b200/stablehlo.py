"""Textual StableHLO program builder.

Emits `module { func.func @main(...) ... }` text in the printed forms that ryft-mlir's op builders produce
(reference: crates/ryft-mlir/src/dialects/stable_hlo/operations/*.rs; each method below cites the printed-form test
it follows).  ryft users obtain the same text from `module.to_string()`; the reference's own PJRT tests pass such
text through `Program::Mlir` (crates/ryft-pjrt/src/programs.rs:2490-2546).

The builder is deliberately small: it names SSA values, tracks their tensor types and appends one line per op.
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class TensorType:
    dims: Tuple[int, ...]
    dtype: str  # MLIR spelling: f32, bf16, f16, i32, i1, ui32, ...

    def __str__(self) -> str:
        return "tensor<" + "".join(f"{d}x" for d in self.dims) + self.dtype + ">"


@dataclass(frozen=True)
class Value:
    name: str
    type: TensorType

    def __str__(self) -> str:
        return self.name


def _float_literal(x: float, dtype: str) -> str:
    """Floats print as `1.500000e+00`; non-finite values as hex bit patterns of the element type
    (crates/ryft-mlir/src/dialects/builtin/attributes/float.rs:12-24)."""
    if math.isinf(x) or math.isnan(x):
        bits32 = struct.unpack("<I", struct.pack("<f", x))[0]
        if dtype == "f32":
            return f"0x{bits32:08X}"
        if dtype == "bf16":
            return f"0x{bits32 >> 16:04X}"
        if dtype == "f16":
            return {"inf": "0x7C00", "-inf": "0xFC00"}.get(str(x), "0x7E00")
        if dtype == "f64":
            return f"0x{struct.unpack('<Q', struct.pack('<d', x))[0]:016X}"
    return _sci(x)


def _sci(x: float) -> str:
    # enough digits to round-trip an f32; MLIR prints the shortest form but accepts any
    return f"{x:.9e}"


class Builder:
    """Accumulates one `func.func @main`."""

    def __init__(self) -> None:
        self._args: List[Value] = []
        self._lines: List[str] = []
        self._n = 0

    # ---- plumbing -------------------------------------------------------------------------------------------
    def arg(self, dims: Sequence[int], dtype: str) -> Value:
        v = Value(f"%arg{len(self._args)}", TensorType(tuple(dims), dtype))
        self._args.append(v)
        return v

    def _new(self, t: TensorType) -> Value:
        v = Value(f"%{self._n}", t)
        self._n += 1
        return v

    def _emit(self, t: TensorType, text: str) -> Value:
        v = self._new(t)
        self._lines.append(f"    {v} = {text}")
        return v

    def build(self, *results: Value) -> str:
        """`module { func.func @main(...) -> ... { ...; return ... } }` (crates/ryft-pjrt/src/programs.rs:2492-2498)."""
        args = ", ".join(f"{a}: {a.type}" for a in self._args)
        rts = ", ".join(str(r.type) for r in results)
        ret = f"({rts})" if len(results) != 1 else rts
        body = "\n".join(self._lines)
        names = ", ".join(str(r) for r in results)
        return (
            "module {\n"
            f"  func.func @main({args}) -> {ret} {{\n"
            f"{body}\n"
            f"    return {names} : {rts}\n"
            "  }\n"
            "}\n"
        )

    # ---- elementwise ----------------------------------------------------------------------------------------
    def _binary(self, name: str, a: Value, b: Value) -> Value:
        assert a.type == b.type, (name, a.type, b.type)
        return self._emit(a.type, f"stablehlo.{name} {a}, {b} : {a.type}")  # arithmetic.rs:695

    def add(self, a, b): return self._binary("add", a, b)
    def subtract(self, a, b): return self._binary("subtract", a, b)            # arithmetic.rs:740
    def multiply(self, a, b): return self._binary("multiply", a, b)            # arithmetic.rs:785
    def divide(self, a, b): return self._binary("divide", a, b)                # arithmetic.rs:830
    def maximum(self, a, b): return self._binary("maximum", a, b)              # comparison.rs:590
    def minimum(self, a, b): return self._binary("minimum", a, b)              # comparison.rs:634
    def power(self, a, b): return self._binary("power", a, b)                  # exponential.rs:498

    def _unary(self, name: str, a: Value) -> Value:
        return self._emit(a.type, f"stablehlo.{name} {a} : {a.type}")          # trigonometric.rs:442

    def negate(self, a): return self._unary("negate", a)                       # arithmetic.rs:650
    def tanh(self, a): return self._unary("tanh", a)
    def exponential(self, a): return self._unary("exponential", a)             # exponential.rs:673
    def log(self, a): return self._unary("log", a)
    def sqrt(self, a): return self._unary("sqrt", a)
    def rsqrt(self, a): return self._unary("rsqrt", a)
    def logistic(self, a): return self._unary("logistic", a)
    def abs(self, a): return self._unary("abs", a)

    def convert(self, a: Value, dtype: str) -> Value:                          # casting.rs:456
        t = TensorType(a.type.dims, dtype)
        return self._emit(t, f"stablehlo.convert {a} : ({a.type}) -> {t}")

    def compare(self, direction: str, a: Value, b: Value, compare_type: str | None = None) -> Value:  # comparison.rs:500
        t = TensorType(a.type.dims, "i1")
        ct = f", {compare_type}" if compare_type else ""
        return self._emit(t, f"stablehlo.compare {direction}, {a}, {b}{ct} : ({a.type}, {b.type}) -> {t}")

    def select(self, p: Value, a: Value, b: Value) -> Value:                   # control_flow.rs:596
        return self._emit(a.type, f"stablehlo.select {p}, {a}, {b} : {p.type}, {a.type}")

    # ---- sources --------------------------------------------------------------------------------------------
    def constant(self, value, dims: Sequence[int], dtype: str) -> Value:       # control_flow.rs:361 (splat)
        t = TensorType(tuple(dims), dtype)
        if dtype.startswith("f") or dtype == "bf16":
            lit = _float_literal(float(value), dtype)
        elif dtype == "i1":
            lit = "true" if value else "false"
        else:
            lit = str(int(value))
        return self._emit(t, f"stablehlo.constant dense<{lit}> : {t}")

    def constant_array(self, values, dtype: str) -> Value:                     # miscellaneous.rs:1144
        import numpy as np
        arr = np.asarray(values)
        t = TensorType(tuple(arr.shape), dtype)

        def fmt(x):
            if isinstance(x, (list, tuple)) or (hasattr(x, "ndim") and x.ndim > 0):
                return "[" + ", ".join(fmt(y) for y in x) + "]"
            if dtype.startswith("f") or dtype == "bf16":
                return _float_literal(float(x), dtype)
            if dtype == "i1":
                return "true" if x else "false"
            return str(int(x))
        return self._emit(t, f"stablehlo.constant dense<{fmt(arr)}> : {t}")

    def iota(self, dim: int, dims: Sequence[int], dtype: str) -> Value:        # miscellaneous.rs:1181
        t = TensorType(tuple(dims), dtype)
        return self._emit(t, f"stablehlo.iota dim = {dim} : {t}")

    def replica_id(self) -> Value:                                             # communication.rs:168-173
        t = TensorType((), "ui32")
        return self._emit(t, f"stablehlo.replica_id : {t}")

    # ---- index manipulation ---------------------------------------------------------------------------------
    def broadcast_in_dim(self, a: Value, dims: Sequence[int], out_dims: Sequence[int]) -> Value:  # manipulation.rs:2154
        t = TensorType(tuple(out_dims), a.type.dtype)
        return self._emit(t, f"stablehlo.broadcast_in_dim {a}, dims = [{', '.join(map(str, dims))}] : ({a.type}) -> {t}")

    def transpose(self, a: Value, perm: Sequence[int]) -> Value:               # manipulation.rs:2022
        t = TensorType(tuple(a.type.dims[p] for p in perm), a.type.dtype)
        return self._emit(t, f"stablehlo.transpose {a}, dims = [{', '.join(map(str, perm))}] : ({a.type}) -> {t}")

    def reshape(self, a: Value, dims: Sequence[int]) -> Value:                 # manipulation.rs:2065
        t = TensorType(tuple(dims), a.type.dtype)
        return self._emit(t, f"stablehlo.reshape {a} : ({a.type}) -> {t}")

    # ---- contraction / reduction ----------------------------------------------------------------------------
    def dot_general(self, a: Value, b: Value, batch: Tuple[Sequence[int], Sequence[int]],
                    contract: Tuple[Sequence[int], Sequence[int]], out_dtype: str | None = None) -> Value:
        """`stablehlo.dot_general %a, %b, batching_dims = [0] x [0], contracting_dims = [2] x [1] : (T, T) -> T`
        (linear_algebra.rs:2245-2258; empty batch lists print as `[] x []`, crates/ryft-pjrt/src/devices.rs:1265-1270)."""
        lb, rb = list(batch[0]), list(batch[1])
        lc, rc = list(contract[0]), list(contract[1])
        dims = [a.type.dims[i] for i in lb]
        dims += [d for i, d in enumerate(a.type.dims) if i not in lb and i not in lc]
        dims += [d for i, d in enumerate(b.type.dims) if i not in rb and i not in rc]
        t = TensorType(tuple(dims), out_dtype or a.type.dtype)
        fmt = lambda xs: "[" + ", ".join(map(str, xs)) + "]"
        return self._emit(
            t,
            f"stablehlo.dot_general {a}, {b}, batching_dims = {fmt(lb)} x {fmt(rb)}, "
            f"contracting_dims = {fmt(lc)} x {fmt(rc)} : ({a.type}, {b.type}) -> {t}",
        )

    def reduce(self, a: Value, init: Value, body: str, dims: Sequence[int]) -> Value:  # functional.rs:534-536
        out = tuple(d for i, d in enumerate(a.type.dims) if i not in dims)
        t = TensorType(out, a.type.dtype)
        return self._emit(
            t,
            f"stablehlo.reduce({a} init: {init}) applies stablehlo.{body} across dimensions = "
            f"[{', '.join(map(str, dims))}] : ({a.type}, {init.type}) -> {t}",
        )

    # ---- collectives (generic form; communication.rs:1759-1767, 1692-1697) -----------------------------------
    def all_reduce(self, operands: Sequence[Value], replica_groups: Sequence[Sequence[int]], body: str = "add") -> List[Value]:
        rows, cols = len(replica_groups), len(replica_groups[0])
        groups = "[" + ", ".join("[" + ", ".join(map(str, g)) + "]" for g in replica_groups) + "]"
        et = TensorType((), operands[0].type.dtype)
        outs = [self._new(o.type) for o in operands]
        lhs = f"{outs[0]}" if len(outs) == 1 else f"{outs[0]}:{len(outs)}"
        if len(outs) > 1:
            # `%r:2` binds %r#0, %r#1
            base = outs[0].name
            outs = [Value(f"{base}#{i}", o.type) for i, o in enumerate(operands)]
        a, b, r = f"%ra{self._n}", f"%rb{self._n}", f"%rr{self._n}"
        self._lines.append(
            f"    {lhs} = \"stablehlo.all_reduce\"({', '.join(map(str, operands))}) "
            f"<{{replica_groups = dense<{groups}> : tensor<{rows}x{cols}xi64>}}> ({{\n"
            f"    ^bb0({a}: {et}, {b}: {et}):\n"
            f"      {r} = stablehlo.{body} {a}, {b} : {et}\n"
            f"      stablehlo.return {r} : {et}\n"
            f"    }}) : ({', '.join(str(o.type) for o in operands)}) -> "
            + (f"({', '.join(str(o.type) for o in operands)})" if len(operands) > 1 else str(operands[0].type))
        )
        return outs

    def all_gather(self, a: Value, dim: int, replica_groups: Sequence[Sequence[int]]) -> Value:
        rows, cols = len(replica_groups), len(replica_groups[0])
        groups = "[" + ", ".join("[" + ", ".join(map(str, g)) + "]" for g in replica_groups) + "]"
        dims = list(a.type.dims)
        dims[dim] *= cols
        t = TensorType(tuple(dims), a.type.dtype)
        return self._emit(
            t,
            f"\"stablehlo.all_gather\"({a}) <{{all_gather_dim = {dim} : i64, replica_groups = dense<{groups}> : "
            f"tensor<{rows}x{cols}xi64>}}> : ({a.type}) -> {t}",
        )

    # ---- helpers for scalars broadcast to a shape -------------------------------------------------------------
    def splat(self, value, like: Value) -> Value:
        return self.constant(value, like.type.dims, like.type.dtype)
