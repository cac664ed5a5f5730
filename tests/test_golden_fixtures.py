"""The committed fixtures of tests/golden/ (made by tests/golden/make_golden.py): the oracle must keep reproducing them
(CPU), and the CUDA path must match them through the PJRT C ABI (GPU)."""
import os
from pathlib import Path

import numpy as np
import pytest

from ryft_b200 import configs

from helpers import assert_close, run_oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
SINGLE = ["c1_dot_f32", "c2_matmul_bias_tanh", "c3_attention_causal", "c3_attention_full", "c4_mlp_gradients"]


def load(name):
    z = np.load(GOLDEN / (name + ".npz"))

    def arr(key):
        x, dt = z[key], str(z[key + "_dtype"])
        return x.view(configs.BF16 if dt == "bfloat16" else np.float16) if dt in ("bfloat16", "float16") else x
    n = int(z["replicas"])
    text = bytes(z["program"]).decode()
    ins = [[arr(f"r{r}_in{k}") for k in range(sum(1 for f in z.files if f.startswith(f"r{r}_in") and not f.endswith("_dtype")))] for r in range(n)]
    outs = [[arr(f"r{r}_out{k}") for k in range(sum(1 for f in z.files if f.startswith(f"r{r}_out") and not f.endswith("_dtype")))] for r in range(n)]
    return text, ins, outs


@pytest.mark.parametrize("name", SINGLE + ["c5_mlp_gradients_2_replicas"])
def test_oracle_reproduces_the_fixture(name):
    from oracle import stablehlo_eval as ev
    text, ins, outs = load(name)
    got = ev.evaluate(text, ins)
    for r in range(len(outs)):
        for k, (g, w) in enumerate(zip(got[r], outs[r])):
            # same code on the same inputs: only the BLAS library's summation order may differ between machines
            assert_close(g, w, f"{name} replica {r} output {k}", f32_tol=1e-6, narrow_tol=8e-3)


def test_fixture_programs_are_what_the_builders_emit_today():
    assert load("c2_matmul_bias_tanh")[0] == configs.c2_program(2, 128, 64, 64)
    assert load("c4_mlp_gradients")[0] == configs.c4_program(256, 128, 384)
    q, k, v = configs.c3_inputs(1, 2, 256, 64)
    assert np.array_equal(load("c3_attention_causal")[1][0][0].view(np.uint16), q.view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("name", SINGLE)
def test_cuda_path_matches_the_fixture(client, name):
    from helpers import run_gpu
    text, ins, outs = load(name)
    if name.startswith("c3"):
        # the fixtures hold the program's own rounding points; the fused kernel's differ (see test_parity_gpu.py), so the
        # fixture is checked against the op-by-op execution
        os.environ["B2X_FUSED_ATTENTION"] = "0"
    try:
        got = run_gpu(client, text, ins[0])
    finally:
        os.environ.pop("B2X_FUSED_ATTENTION", None)
    for k, (g, w) in enumerate(zip(got, outs[0])):
        assert_close(g, w, f"{name} output {k}")
