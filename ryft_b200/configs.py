"""The five benchmark programs as StableHLO text plus their seeded synthetic inputs.

Each `cN_program` returns (mlir_text, input_specs) where input_specs lists (dims, dtype) per argument, and each
`cN_inputs` draws the arguments with `numpy.random.default_rng(seed).standard_normal(float32)`, scaled and cast to
bf16 (round to nearest even, ml_dtypes) where the config says bf16.  Sizes default to the full configuration and
can be shrunk for parity tests against the CPU oracle.
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import numpy as np

from .stablehlo import Builder, Value

try:  # bf16 host arrays
    import ml_dtypes
    BF16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    ml_dtypes = None
    BF16 = None

NP_DTYPES = {"f32": np.float32, "i32": np.int32, "i1": np.bool_, "ui32": np.uint32, "f16": np.float16,
             "i8": np.int8, "ui8": np.uint8, "i16": np.int16, "ui16": np.uint16, "i64": np.int64, "f64": np.float64}


def np_dtype(name: str):
    if name == "bf16":
        return BF16
    return NP_DTYPES[name]


# ---- c1: f32 dot_general [M,K] x [K,N] -------------------------------------------------------------------------
def c1_program(M=512, K=768, N=512) -> str:
    b = Builder()
    lhs = b.arg([M, K], "f32")
    rhs = b.arg([K, N], "f32")
    out = b.dot_general(lhs, rhs, ([], []), ([1], [0]))
    return b.build(out)


def c1_inputs(M=512, K=768, N=512, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((M, K), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32)]


# ---- c2: batched bf16 dot_general + bias + tanh + convert -------------------------------------------------------
def c2_program(B=32, M=2048, K=128, N=2048) -> str:
    b = Builder()
    lhs = b.arg([B, M, K], "bf16")
    rhs = b.arg([B, K, N], "bf16")
    bias = b.arg([N], "f32")
    acc = b.dot_general(lhs, rhs, ([0], [0]), ([2], [1]), out_dtype="f32")
    bb = b.broadcast_in_dim(bias, [2], [B, M, N])
    y = b.tanh(b.add(acc, bb))
    return b.build(b.convert(y, "bf16"))


def c2_inputs(B=32, M=2048, K=128, N=2048, seed=1):
    rng = np.random.default_rng(seed)
    lhs = (rng.standard_normal((B, M, K), dtype=np.float32) / np.float32(math.sqrt(K))).astype(BF16)
    rhs = (rng.standard_normal((B, K, N), dtype=np.float32) / np.float32(math.sqrt(K))).astype(BF16)
    bias = rng.standard_normal((N,), dtype=np.float32) * np.float32(0.1)
    return [lhs, rhs, bias]


# ---- c3: causal scaled-dot-product attention written out in StableHLO -------------------------------------------
def c3_program(B=4, H=32, S=4096, D=128, causal=True) -> str:
    b = Builder()
    q = b.arg([B, H, S, D], "bf16")
    k = b.arg([B, H, S, D], "bf16")
    v = b.arg([B, H, S, D], "bf16")
    s = b.dot_general(q, k, ([0, 1], [0, 1]), ([3], [3]), out_dtype="f32")          # [B,H,S,S]
    s = b.multiply(s, b.splat(1.0 / math.sqrt(D), s))
    if causal:
        row = b.iota(0, [S, S], "i32")
        col = b.iota(1, [S, S], "i32")
        mask = b.compare("GE", row, col, "SIGNED")
        maskb = b.broadcast_in_dim(mask, [2, 3], [B, H, S, S])
        s = b.select(maskb, s, b.splat(float("-inf"), s))
    ninf = b.constant(float("-inf"), [], "f32")
    zero = b.constant(0.0, [], "f32")
    m = b.reduce(s, ninf, "maximum", [3])                                            # [B,H,S]
    e = b.exponential(b.subtract(s, b.broadcast_in_dim(m, [0, 1, 2], [B, H, S, S])))
    l = b.reduce(e, zero, "add", [3])
    p = b.divide(e, b.broadcast_in_dim(l, [0, 1, 2], [B, H, S, S]))
    p = b.convert(p, "bf16")
    o = b.dot_general(p, v, ([0, 1], [0, 1]), ([3], [2]), out_dtype="bf16")         # [B,H,S,D]
    return b.build(o)


def c3_inputs(B=4, H=32, S=4096, D=128, seed=2):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((B, H, S, D), dtype=np.float32).astype(BF16) for _ in range(3)]


# ---- c4 / c5: MLP forward + hand-written backward (+ all_reduce over replicas) -----------------------------------
def _gelu_tanh(b: Builder, h: Value) -> Tuple[Value, Value]:
    """Returns (gelu(h), tanh term) in f32."""
    c0 = math.sqrt(2.0 / math.pi)
    h3 = b.multiply(b.multiply(h, h), h)
    inner = b.multiply(b.splat(c0, h), b.add(h, b.multiply(b.splat(0.044715, h), h3)))
    t = b.tanh(inner)
    g = b.multiply(b.multiply(b.splat(0.5, h), h), b.add(b.splat(1.0, h), t))
    return g, t


def _gelu_tanh_grad(b: Builder, h: Value) -> Value:
    """d gelu / dh in f32: 0.5(1+t) + 0.5 h (1-t^2) c0 (1 + 3*0.044715 h^2)."""
    c0 = math.sqrt(2.0 / math.pi)
    h2 = b.multiply(h, h)
    inner = b.multiply(b.splat(c0, h), b.add(h, b.multiply(b.splat(0.044715, h), b.multiply(h2, h))))
    t = b.tanh(inner)
    left = b.multiply(b.splat(0.5, h), b.add(b.splat(1.0, h), t))
    sech2 = b.subtract(b.splat(1.0, h), b.multiply(t, t))
    dinner = b.multiply(b.splat(c0, h), b.add(b.splat(1.0, h), b.multiply(b.splat(3 * 0.044715, h), h2)))
    right = b.multiply(b.multiply(b.multiply(b.splat(0.5, h), h), sech2), dinner)
    return b.add(left, right)


def c4_program(T=8192, D=4096, F=16384, replicas: int = 0, trace: bool = False) -> str:
    """Forward H = X W1, A = gelu(H), Y = A W2, loss = mean(Y^2); backward dW2 = A^T dY, dA = dY W2^T,
    dH = dA * gelu'(H), dW1 = X^T dH.  With replicas > 0 the gradients go through stablehlo.all_reduce over
    all replicas and are divided by the replica count (config 5).  With `trace` the intermediates that pass between the
    GEMMs are returned as well: (dW1, dW2, loss, H, A, Y, dY, dH)."""
    b = Builder()
    x = b.arg([T, D], "bf16")
    w1 = b.arg([D, F], "bf16")
    w2 = b.arg([F, D], "bf16")
    hf = b.dot_general(x, w1, ([], []), ([1], [0]), out_dtype="f32")                 # [T,F]
    h = b.convert(hf, "bf16")                                                        # kept for the backward pass
    g, _ = _gelu_tanh(b, hf)
    a = b.convert(g, "bf16")
    y = b.dot_general(a, w2, ([], []), ([1], [0]), out_dtype="f32")                  # [T,D]
    zero = b.constant(0.0, [], "f32")
    ssq = b.reduce(b.multiply(y, y), zero, "add", [0, 1])
    n = float(T) * float(D)
    loss = b.multiply(ssq, b.constant(1.0 / n, [], "f32"))
    dy = b.convert(b.multiply(y, b.splat(2.0 / n, y)), "bf16")                       # [T,D]
    dw2 = b.dot_general(a, dy, ([], []), ([0], [0]), out_dtype="f32")                # [F,D]
    da = b.dot_general(dy, w2, ([], []), ([1], [1]), out_dtype="f32")                # [T,F]
    dh = b.convert(b.multiply(da, _gelu_tanh_grad(b, b.convert(h, "f32"))), "bf16")
    dw1 = b.dot_general(x, dh, ([], []), ([0], [0]), out_dtype="f32")                # [D,F]
    if replicas > 0:
        dw1, dw2 = b.all_reduce([dw1, dw2], [list(range(replicas))])
        inv = 1.0 / replicas
        dw1 = b.multiply(dw1, b.splat(inv, dw1))
        dw2 = b.multiply(dw2, b.splat(inv, dw2))
    if trace:
        return b.build(dw1, dw2, loss, h, a, y, dy, dh)
    return b.build(dw1, dw2, loss)


def c4_stage_programs(T=8192, D=4096, F=16384) -> dict:
    """The five GEMMs of config 4, each with the elementwise work that the planner fuses into it, as programs of their own:
    name -> (text, argument names, result names), the names being those of `c4_program(trace=True)`.  Feeding every stage
    the expected values of its inputs checks each kernel at the benchmark's size without the compounding of rounding
    differences along the chain of bf16 intermediates."""
    n = float(T) * float(D)
    out = {}
    b = Builder()
    x = b.arg([T, D], "bf16"); w1 = b.arg([D, F], "bf16")
    hf = b.dot_general(x, w1, ([], []), ([1], [0]), out_dtype="f32")
    g, _ = _gelu_tanh(b, hf)
    out["forward 1"] = (b.build(b.convert(hf, "bf16"), b.convert(g, "bf16")), ("x", "w1"), ("h", "a"))
    b = Builder()
    a = b.arg([T, F], "bf16"); w2 = b.arg([F, D], "bf16")
    y = b.dot_general(a, w2, ([], []), ([1], [0]), out_dtype="f32")
    out["forward 2"] = (b.build(y, b.convert(b.multiply(y, b.splat(2.0 / n, y)), "bf16")), ("a", "w2"), ("y", "dy"))
    b = Builder()
    a = b.arg([T, F], "bf16"); dy = b.arg([T, D], "bf16")
    out["dW2"] = (b.build(b.dot_general(a, dy, ([], []), ([0], [0]), out_dtype="f32")), ("a", "dy"), ("dw2",))
    b = Builder()
    dy = b.arg([T, D], "bf16"); w2 = b.arg([F, D], "bf16"); h = b.arg([T, F], "bf16")
    da = b.dot_general(dy, w2, ([], []), ([1], [1]), out_dtype="f32")
    out["dH"] = (b.build(b.convert(b.multiply(da, _gelu_tanh_grad(b, b.convert(h, "f32"))), "bf16")), ("dy", "w2", "h"), ("dh",))
    b = Builder()
    x = b.arg([T, D], "bf16"); dh = b.arg([T, F], "bf16")
    out["dW1"] = (b.build(b.dot_general(x, dh, ([], []), ([0], [0]), out_dtype="f32")), ("x", "dh"), ("dw1",))
    return out


def c4_inputs(T=8192, D=4096, F=16384, seed=3, replica: int | None = None):
    """Config 4: one rng, tensors drawn in argument order.  Config 5 (replica given): weights from rng(seed)
    shared by all replicas, activations from rng(seed + replica)."""
    if replica is None:
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((T, D), dtype=np.float32).astype(BF16)
        w1 = (rng.standard_normal((D, F), dtype=np.float32) * np.float32(0.02)).astype(BF16)
        w2 = (rng.standard_normal((F, D), dtype=np.float32) * np.float32(0.02)).astype(BF16)
        return [x, w1, w2]
    wr = np.random.default_rng(seed)
    w1 = (wr.standard_normal((D, F), dtype=np.float32) * np.float32(0.02)).astype(BF16)
    w2 = (wr.standard_normal((F, D), dtype=np.float32) * np.float32(0.02)).astype(BF16)
    xr = np.random.default_rng(seed + 1 + replica)
    x = xr.standard_normal((T, D), dtype=np.float32).astype(BF16)
    return [x, w1, w2]


C4_GEMM_FLOPS = lambda T, D, F: 5 * 2.0 * T * D * F


# ---- micro-configurations for the HBM-bound kernels (the epilogue chain of config 2 and the loss reduction of config 4,
# ---- standalone at their native sizes) ----------------------------------------------------------------------------------
def ew_program(B=32, M=2048, N=2048) -> str:
    """tanh(acc + bias) -> bf16 over an f32 [B, M, N] tensor: reads 4 B, writes 2 B per element."""
    b = Builder()
    acc = b.arg([B, M, N], "f32")
    bias = b.arg([N], "f32")
    y = b.tanh(b.add(acc, b.broadcast_in_dim(bias, [2], [B, M, N])))
    return b.build(b.convert(y, "bf16"))


def ew_inputs(B=32, M=2048, N=2048, seed=5):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal((B, M, N), dtype=np.float32) * np.float32(0.1), rng.standard_normal((N,), dtype=np.float32) * np.float32(0.1)]


def red_program(T=8192, D=4096) -> str:
    """sum(y * y) / (T * D) over an f32 [T, D] tensor: reads 4 B per element."""
    b = Builder()
    y = b.arg([T, D], "f32")
    ssq = b.reduce(b.multiply(y, y), b.constant(0.0, [], "f32"), "add", [0, 1])
    return b.build(b.multiply(ssq, b.constant(1.0 / (float(T) * float(D)), [], "f32")))


def red_inputs(T=8192, D=4096, seed=6):
    return [np.random.default_rng(seed).standard_normal((T, D), dtype=np.float32)]
