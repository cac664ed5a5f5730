"""Writes the golden fixtures of this folder: small instances of the five benchmark programs (and the two collective
ops) with seeded inputs and the outputs the CPU oracle computes for them.

    python tests/golden/make_golden.py

The reference's own executor (OpenXLA's PJRT plugins) cannot be run where this repository is built, so the fixtures are
made with the oracle, which itself is pinned to every known answer the reference's tests and doc comments hold for these
ops (tests/test_oracle_golden.py).  The fixtures freeze those outputs: a later change of the oracle, of the program
builders or of the input generators shows up as a difference against the committed files.
16-bit floats are stored as their bit patterns (uint16) with the dtype name beside them.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import stablehlo_eval as ev          # noqa: E402
from ryft_b200 import configs                    # noqa: E402


def cases():
    yield "c1_dot_f32", configs.c1_program(64, 96, 32), [configs.c1_inputs(64, 96, 32)]
    yield "c2_matmul_bias_tanh", configs.c2_program(2, 128, 64, 64), [configs.c2_inputs(2, 128, 64, 64)]
    yield "c3_attention_causal", configs.c3_program(1, 2, 256, 64), [configs.c3_inputs(1, 2, 256, 64)]
    yield "c3_attention_full", configs.c3_program(1, 1, 128, 128, causal=False), [configs.c3_inputs(1, 1, 128, 128)]
    yield "c4_mlp_gradients", configs.c4_program(256, 128, 384), [configs.c4_inputs(256, 128, 384)]
    yield "c5_mlp_gradients_2_replicas", configs.c4_program(64, 64, 128, replicas=2), \
        [configs.c4_inputs(64, 64, 128, seed=4, replica=r) for r in range(2)]


def pack(x: np.ndarray):
    x = np.asarray(x)
    if x.dtype.name in ("bfloat16", "float16"):
        return x.view(np.uint16), x.dtype.name
    return x, x.dtype.name


def main() -> None:
    for name, text, per_replica_inputs in cases():
        outs = ev.evaluate(text, [list(i) for i in per_replica_inputs])
        blob = {"program": np.frombuffer(text.encode(), dtype=np.uint8), "replicas": np.int64(len(per_replica_inputs))}
        for r, (ins, o) in enumerate(zip(per_replica_inputs, outs)):
            for k, x in enumerate(ins):
                blob[f"r{r}_in{k}"], blob[f"r{r}_in{k}_dtype"] = pack(x)
            for k, x in enumerate(o):
                blob[f"r{r}_out{k}"], blob[f"r{r}_out{k}_dtype"] = pack(x)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **blob)
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
