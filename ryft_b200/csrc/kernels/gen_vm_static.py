"""Generates vm_static_table.h: the table of fused-elementwise programs that are specialised at build time.

The planner lowers every fusion group to an accumulator-machine program (vm.h).  Programs listed in the table are
compiled as straight-line code (vm.cuh, VmStatic<ID>): as the epilogue of the tcgen05 GEMM, as a standalone elementwise
kernel or as a reduce prologue.  Anything else runs through the interpreter.  The table is built from the launch plans
of the benchmark programs (ryft_b200/configs.py) and a few common shapes of fusion; add a program text to `PROGRAMS`
below to specialise its fusions as well, then run

    python ryft_b200/csrc/kernels/gen_vm_static.py && python -m ryft_b200.build

Needs libb2x_kernels.so (for the planner); on a clean checkout build once with the committed table first.
"""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[2]
sys.path.insert(0, str(ROOT))


def signatures(text: str, replicas: int = 1):
    import ryft_b200
    lib = C.CDLL(str(ryft_b200.KERNELS_PATH))
    cap = 1 << 20
    out = C.create_string_buffer(cap)
    n = C.c_size_t(0)
    lib.b2x_plan_signatures.argtypes = [C.c_char_p, C.c_size_t, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    data = text.encode()
    rc = lib.b2x_plan_signatures(data, len(data), replicas, out, cap, C.byref(n))
    if rc:
        raise RuntimeError(out.value.decode())
    rows = []
    for line in out.value.decode().splitlines():
        role, bn, vec, h, n_instr, code, elems, label = line.split("|", 7)
        rows.append({"role": role, "bn": int(bn), "vec": int(vec), "hash": int(h), "n": int(n_instr),
                     "code": [tuple(int(x) for x in c.split(".")) for c in code.split(",")], "elems": [int(e) for e in elems.split(",")], "label": label})
    return rows


def programs():
    from ryft_b200 import configs
    from ryft_b200.stablehlo import Builder
    out = [(configs.c1_program(), 1), (configs.c2_program(), 1), (configs.c3_program(), 1), (configs.c3_program(causal=False), 1),
           (configs.c4_program(), 1), (configs.c4_program(replicas=1), 1), (configs.c4_program(replicas=8), 8),
           (configs.c4_program(replicas=3), 3), (configs.ew_program(), 1), (configs.red_program(), 1)]
    # plain bf16 -> f32 / bf16 / f16 GEMM results and a bias epilogue at the three tile widths
    for n in (64, 128, 256):
        for dt_in, dt_out in (("bf16", "f32"), ("bf16", "bf16"), ("f16", "f32"), ("f16", "f16")):
            b = Builder()
            x = b.arg([256, 128], dt_in); y = b.arg([128, n], dt_in)
            out.append((b.build(b.dot_general(x, y, ([], []), ([1], [0]), out_dtype=dt_out)), 1))
    # the usual dense-layer epilogues: bias, then nothing / logistic / relu / tanh-GELU, stored as bf16 (tanh is config 2's),
    # and bias alone stored as f32; at the two tile widths that large GEMMs take
    import math
    for n in (128, 2048):
        for act in ("none", "logistic", "relu", "gelu"):
            b = Builder()
            x = b.arg([256, 128], "bf16"); w = b.arg([128, n], "bf16"); bias = b.arg([n], "f32")
            y = b.add(b.dot_general(x, w, ([], []), ([1], [0]), out_dtype="f32"), b.broadcast_in_dim(bias, [1], [256, n]))
            if act == "logistic":
                y = b.logistic(y)
            elif act == "relu":
                y = b.maximum(y, b.splat(0.0, y))
            elif act == "gelu":
                c0 = math.sqrt(2.0 / math.pi)
                inner = b.multiply(b.splat(c0, y), b.add(y, b.multiply(b.splat(0.044715, y), b.multiply(b.multiply(y, y), y))))
                y = b.multiply(b.multiply(b.splat(0.5, y), y), b.add(b.splat(1.0, y), b.tanh(inner)))
            out.append((b.build(b.convert(y, "bf16")), 1))
        b = Builder()
        x = b.arg([256, 128], "bf16"); w = b.arg([128, n], "bf16"); bias = b.arg([n], "f32")
        out.append((b.build(b.add(b.dot_general(x, w, ([], []), ([1], [0]), out_dtype="f32"), b.broadcast_in_dim(bias, [1], [256, n]))), 1))
    # common standalone shapes: copy/transposed copy, scale, add, axpy-like, row/full reductions of f32 and bf16
    for dt in ("f32", "bf16"):
        b = Builder()
        x = b.arg([1024, 1024], dt); y = b.arg([1024, 1024], dt)
        zero = b.constant(0.0, [], dt)
        out.append((b.build(b.add(x, y), b.multiply(x, y), b.multiply(x, b.splat(0.5, x)), b.reduce(x, zero, "add", [1]), b.reduce(x, zero, "add", [0, 1]),
                            b.reduce(x, b.constant(float("-inf"), [], dt), "maximum", [1])), 1))
    return out


def main():
    seen = {}
    for text, reps in programs():
        for row in signatures(text, reps):
            if row["vec"] != 8:
                continue
            key = row["hash"]
            ent = seen.setdefault(key, {"row": row, "roles": set()})
            ent["roles"].add((row["role"], row["bn"]))
            # a GEMM epilogue is built for both wide tile widths: which one a problem takes depends on its K as well
            if row["role"] == "gemm_tc" and row["bn"] >= 128:
                ent["roles"].add((row["role"], 128))
                ent["roles"].add((row["role"], 256))
    entries = sorted(seen.values(), key=lambda e: (e["row"]["n"], e["row"]["hash"]))
    lines = ["// Specialised fused-elementwise programs.  GENERATED by gen_vm_static.py from the launch plans of the benchmark",
             "// programs; regenerate after changing the planner's code generation.", "#pragma once", "namespace b2x {"]
    for i, e in enumerate(entries, start=1):
        r = e["row"]
        sig = ", ".join("{%d, %d, %d, %d, %d, %d}" % c for c in r["code"])
        elems = ", ".join(str(x) for x in r["elems"]) or "0"
        lines.append(f"// {r['label']}")
        lines.append(f"template <> struct VmStatic<{i}> {{")
        lines.append(f"  static constexpr int n = {r['n']};")
        lines.append(f"  static constexpr unsigned long long hash = {r['hash']}ull;")
        lines.append(f"  __host__ __device__ static constexpr VmSig at(int i) {{ constexpr VmSig c[{r['n']}] = {{{sig}}}; return c[i]; }}")
        lines.append(f"  __host__ __device__ static constexpr uint8_t elem(int t) {{ constexpr uint8_t e[{max(len(r['elems']), 1)}] = {{{elems}}}; return e[t]; }}")
        lines.append("};")
    lines.append("__host__ inline int vm_static_lookup(uint64_t h) {")
    lines.append("  switch (h) {")
    for i, e in enumerate(entries, start=1):
        lines.append(f"    case {e['row']['hash']}ull: return {i};")
    lines.append("    default: return 0;")
    lines.append("  }")
    lines.append("}")
    lines.append("}  // namespace b2x")

    def role_list(name, pred, with_bn=False):
        items = []
        for i, e in enumerate(entries, start=1):
            for role, bn in sorted(e["roles"]):
                if pred(role):
                    items.append(f"X({i}, {bn})" if with_bn else f"X({i})")
        uniq = []
        for it in items:
            if it not in uniq:
                uniq.append(it)
        lines.append(f"#define {name}(X) " + " ".join(uniq))
    role_list("B2X_VM_STATIC_ELEMENTWISE", lambda r: r == "elementwise")
    role_list("B2X_VM_STATIC_REDUCE", lambda r: r == "reduce")
    role_list("B2X_VM_STATIC_GEMM", lambda r: r == "gemm_tc", with_bn=True)
    (HERE / "vm_static_table.h").write_text("\n".join(lines) + "\n")
    print(f"wrote {len(entries)} specialised programs")
    for i, e in enumerate(entries, start=1):
        print(i, sorted(e["roles"]), e["row"]["n"], e["row"]["label"])


if __name__ == "__main__":
    main()
