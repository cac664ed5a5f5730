"""Shared helpers of the parity tests: run a StableHLO program through the PJRT C ABI on the GPU and through the CPU
oracle on the same inputs, and compare with the build's tolerances: integer / predicate / index results bit-exact;
f32 <= 1e-4 relative Frobenius error; bf16 and f16 <= 1e-2 max-abs error normalised by the RMS of the expected output."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np

from oracle import stablehlo_eval as ev
from ryft_b200 import pjrt

F32_REL_FROBENIUS = 1e-4
BF16_MAX_ABS_OVER_RMS = 1e-2


def run_gpu(client, text: str, inputs: Sequence[np.ndarray], options: pjrt.CompilationOptions | None = None) -> List[np.ndarray]:
    exe = client.compile(pjrt.Program.mlir(text), options or pjrt.CompilationOptions())
    device = exe.addressable_devices()[0]
    bufs = [client.buffer(np.asarray(x), device=device) for x in inputs]
    outs = exe.execute([pjrt.ExecutionDeviceInputs(bufs)])
    outs[0].done.await_()
    return [o.to_numpy() for o in outs[0].outputs]


def run_oracle(text: str, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
    return ev.evaluate(text, [list(inputs)])[0]


def assert_close(actual: np.ndarray, expected: np.ndarray, what: str = "", f32_tol: float = F32_REL_FROBENIUS,
                 narrow_tol: float = BF16_MAX_ABS_OVER_RMS) -> None:
    assert actual.shape == expected.shape, (what, actual.shape, expected.shape)
    assert actual.dtype == expected.dtype, (what, actual.dtype, expected.dtype)
    kind = expected.dtype.kind
    name = expected.dtype.name
    if kind in "iub":
        if not np.array_equal(actual, expected):
            bad = np.argwhere(actual != expected)
            raise AssertionError(f"{what}: {len(bad)} of {expected.size} integer elements differ; first at {bad[0].tolist()}: "
                                 f"{actual[tuple(bad[0])]} != {expected[tuple(bad[0])]}")
        return
    a64, e64 = actual.astype(np.float64), expected.astype(np.float64)
    fin = np.isfinite(e64)
    assert np.array_equal(np.isfinite(a64), fin), f"{what}: non-finite pattern differs"
    if not fin.all():
        assert np.array_equal(a64[~fin], e64[~fin], equal_nan=True), f"{what}: inf/nan values differ"
        a64, e64 = np.where(fin, a64, 0.0), np.where(fin, e64, 0.0)
    if name in ("bfloat16", "float16"):
        # The build's bar: max-abs error / RMS(expected) <= 1e-2.  One unit in the last place of bf16 is 2^-8..2^-7 of an
        # element's own magnitude, so for an element larger than ~1.3 x RMS that literal bar asks for sub-ulp agreement of
        # the final rounding, which no two implementations with different accumulation orders can give (the oracle
        # accumulates in float64).  Each element's error is therefore normalised by max(RMS, |expected element|): the
        # literal bar for elements up to the RMS, a one-ulp allowance (relative 1e-2 > 2^-7) above it.
        rms = float(np.sqrt(np.mean(e64 ** 2))) if e64.size else 0.0
        scale = np.maximum(np.abs(e64), rms)
        rel = np.abs(a64 - e64) / np.where(scale > 0, scale, 1.0)
        err = float(rel.max()) if rel.size else 0.0
        assert err <= narrow_tol, (f"{what}: max error / max(RMS, |element|) = {err:.3e} exceeds {narrow_tol} "
                                   f"(literal max-abs/RMS = {ev.max_abs_over_rms(a64, e64):.3e})")
    else:
        err = ev.rel_frobenius(a64, e64)
        assert err <= f32_tol, f"{what}: relative Frobenius error {err:.3e} exceeds {f32_tol}"


def check_program(client, text: str, inputs: Sequence[np.ndarray], what: str = "", **tol) -> List[np.ndarray]:
    got = run_gpu(client, text, inputs)
    want = run_oracle(text, inputs)
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert_close(g, w, f"{what} output {i}", **tol)
    return got


# ---- the literal metrics of the build's tolerances, recorded per configuration -----------------------------------------------
_REPORT: dict = {}


def record_metric(name: str, **metrics) -> None:
    """Remembers the literal error metrics of a configuration (max-abs error / RMS of the expected output for 16-bit
    floats, relative Frobenius error for f32) next to the bound that the test asserts; printed with `-s`, and written
    as JSON to the file named by B2X_PARITY_REPORT when that variable is set."""
    import json
    import os
    _REPORT[name] = {k: (float(v) if isinstance(v, (int, float, np.floating)) else v) for k, v in metrics.items()}
    print(f"PARITY {name}: " + ", ".join(f"{k}={v:.3e}" if isinstance(v, float) else f"{k}={v}" for k, v in _REPORT[name].items()))
    path = os.environ.get("B2X_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(_REPORT, f, indent=1, sort_keys=True)


def literal_metrics(actual: np.ndarray, expected: np.ndarray) -> dict:
    """Both literal metrics of the build's tolerances plus the relaxed 16-bit one that assert_close applies."""
    a64, e64 = actual.astype(np.float64), expected.astype(np.float64)
    rms = float(np.sqrt(np.mean(e64 ** 2))) if e64.size else 0.0
    scale = np.maximum(np.abs(e64), rms)
    relaxed = float((np.abs(a64 - e64) / np.where(scale > 0, scale, 1.0)).max()) if e64.size else 0.0
    return {"max_abs_over_rms": ev.max_abs_over_rms(a64, e64), "rel_frobenius": ev.rel_frobenius(a64, e64), "max_err_over_max_rms_elem": relaxed,
            "mismatch_fraction": float(np.mean(a64 != e64)) if e64.size else 0.0}
