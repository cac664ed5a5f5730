"""Pins the CPU oracle to every known answer the reference holds for the hot-path ops.

Sources: README.md:88,108-137 (f32 matmul), crates/ryft-pjrt/src/programs.rs:2490-2498,2781-2829 (i32 add), and the worked
examples in the doc comments under crates/ryft-mlir/src/dialects/stable_hlo/operations/ (cited per test)."""
import numpy as np

from oracle import stablehlo_eval as ev


def run(text, *inputs, replicas=None):
    if replicas is None:
        return ev.evaluate(text, [list(inputs)])[0]
    return ev.evaluate(text, replicas)


def test_readme_matmul():
    text = """
module {
  func.func @main(%arg0: tensor<2x3xf32>, %arg1: tensor<3x2xf32>) -> tensor<2x2xf32> {
    %0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [] x [], contracting_dims = [1] x [0] : (tensor<2x3xf32>, tensor<3x2xf32>) -> tensor<2x2xf32>
    return %0 : tensor<2x2xf32>
  }
}
"""
    lhs = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    rhs = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
    (out,) = run(text, lhs, rhs)
    assert out.dtype == np.float32
    assert out.ravel().tolist() == [58.0, 64.0, 139.0, 154.0]


def test_i32_add_program():
    # the program text of crates/ryft-pjrt/src/programs.rs:2492-2498, inputs and answer of :2781-2829
    text = """
module {
  func.func @main(%arg0: tensor<2x1xi32>, %arg1: tensor<2x1xi32>) -> tensor<2x1xi32> {
    %0 = stablehlo.add %arg0, %arg1 : tensor<2x1xi32>
    return %0 : tensor<2x1xi32>
  }
}
"""
    (out,) = run(text, np.array([[7], [-1]], np.int32), np.array([[35], [-41]], np.int32))
    assert out.tobytes() == np.array([42, -42], np.int32).tobytes()


def test_dot_general_batched_identity():
    # linear_algebra.rs:671-701
    text = """
module {
  func.func @main(%lhs: tensor<2x2x2xi64>, %rhs: tensor<2x2x2xi64>) -> tensor<2x2x2xi64> {
    %result = stablehlo.dot_general %lhs, %rhs, batching_dims = [0] x [0], contracting_dims = [2] x [1] : (tensor<2x2x2xi64>, tensor<2x2x2xi64>) -> tensor<2x2x2xi64>
    return %result : tensor<2x2x2xi64>
  }
}
"""
    lhs = np.array([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], np.int64)
    rhs = np.array([[[1, 0], [0, 1]], [[1, 0], [0, 1]]], np.int64)
    (out,) = run(text, lhs, rhs)
    assert np.array_equal(out, lhs)


def test_reduce_example():
    # functional.rs:124-131
    text = """
module {
  func.func @main(%input: tensor<1x6xi32>, %init_value: tensor<i32>) -> tensor<1xi32> {
    %result = stablehlo.reduce(%input init: %init_value) applies stablehlo.add across dimensions = [1] : (tensor<1x6xi32>, tensor<i32>) -> tensor<1xi32>
    return %result : tensor<1xi32>
  }
}
"""
    (out,) = run(text, np.array([[0, 1, 2, 3, 4, 5]], np.int32), np.array(0, np.int32))
    assert out.tolist() == [15]


def test_iota_examples():
    # miscellaneous.rs:74-90
    for dim, expect in ((0, [[i] * 5 for i in range(4)]), (1, [list(range(5))] * 4)):
        text = f"""
module {{
  func.func @main() -> tensor<4x5xi32> {{
    %output = stablehlo.iota dim = {dim} : tensor<4x5xi32>
    return %output : tensor<4x5xi32>
  }}
}}
"""
        (out,) = run(text)
        assert out.tolist() == expect


def test_broadcast_in_dim_example():
    # manipulation.rs:303-310
    text = """
module {
  func.func @main(%input: tensor<1x3xi32>) -> tensor<2x3x2xi32> {
    %output = stablehlo.broadcast_in_dim %input, dims = [2, 1] : (tensor<1x3xi32>) -> tensor<2x3x2xi32>
    return %output : tensor<2x3x2xi32>
  }
}
"""
    (out,) = run(text, np.array([[1, 2, 3]], np.int32))
    assert out.tolist() == [[[1, 1], [2, 2], [3, 3]], [[1, 1], [2, 2], [3, 3]]]


def test_compare_example():
    # comparison.rs:89-94
    text = """
module {
  func.func @main(%arg0: tensor<2xf32>, %arg1: tensor<2xf32>) -> tensor<2xi1> {
    %result = stablehlo.compare GE, %arg0, %arg1, TOTALORDER : (tensor<2xf32>, tensor<2xf32>) -> tensor<2xi1>
    return %result : tensor<2xi1>
  }
}
"""
    (out,) = run(text, np.array([1.0, 3.0], np.float32), np.array([1.1, 2.9], np.float32))
    assert out.tolist() == [False, True]


def test_tanh_example():
    # trigonometric.rs:168-172
    text = """
module {
  func.func @main(%operand: tensor<3xf32>) -> tensor<3xf32> {
    %result = stablehlo.tanh %operand : tensor<3xf32>
    return %result : tensor<3xf32>
  }
}
"""
    (out,) = run(text, np.array([-1.0, 0.0, 1.0], np.float32))
    np.testing.assert_allclose(out, np.array([-0.76159416, 0.0, 0.76159416], np.float32), rtol=1e-7, atol=0)


def test_all_reduce_example():
    # communication.rs:821-841 (the printed example passes %operand0 twice; the stated results are for operand0, operand1)
    text = """
module {
  func.func @main(%operand0: tensor<4xi64>, %operand1: tensor<4xi64>) -> (tensor<4xi64>, tensor<4xi64>) {
    %result:2 = "stablehlo.all_reduce"(%operand0, %operand1) <{channel_handle = #stablehlo.channel_handle<handle = 0, type = 1>, replica_groups = dense<[[0, 1]]> : tensor<1x2xi64>}> ({
    ^bb0(%arg0: tensor<i64>, %arg1: tensor<i64>):
      %0 = stablehlo.add %arg0, %arg1 : tensor<i64>
      stablehlo.return %0 : tensor<i64>
    }) : (tensor<4xi64>, tensor<4xi64>) -> (tensor<4xi64>, tensor<4xi64>)
    return %result#0, %result#1 : tensor<4xi64>, tensor<4xi64>
  }
}
"""
    r0 = [np.array([1, 2, 3, 4], np.int64), np.array([9, 10, 11, 12], np.int64)]
    r1 = [np.array([5, 6, 7, 8], np.int64), np.array([13, 14, 15, 16], np.int64)]
    outs = run(text, replicas=[r0, r1])
    for r in range(2):
        assert outs[r][0].tolist() == [6, 8, 10, 12]
        assert outs[r][1].tolist() == [22, 24, 26, 28]


def test_all_gather_example():
    # communication.rs:722-739
    text = """
module {
  func.func @main(%operand0: tensor<2x2xi64>, %operand1: tensor<2x2xi64>) -> (tensor<2x4xi64>, tensor<2x4xi64>) {
    %result:2 = "stablehlo.all_gather"(%operand0, %operand1) <{all_gather_dim = 1 : i64, replica_groups = dense<[[0, 1]]> : tensor<1x2xi64>, channel_handle = #stablehlo.channel_handle<handle = 0, type = 0>}> : (tensor<2x2xi64>, tensor<2x2xi64>) -> (tensor<2x4xi64>, tensor<2x4xi64>)
    return %result#0, %result#1 : tensor<2x4xi64>, tensor<2x4xi64>
  }
}
"""
    r0 = [np.array([[1, 2], [3, 4]], np.int64), np.array([[11, 12], [13, 14]], np.int64)]
    r1 = [np.array([[5, 6], [7, 8]], np.int64), np.array([[15, 16], [17, 18]], np.int64)]
    outs = run(text, replicas=[r0, r1])
    for r in range(2):
        assert outs[r][0].tolist() == [[1, 2, 5, 6], [3, 4, 7, 8]]
        assert outs[r][1].tolist() == [[11, 12, 15, 16], [13, 14, 17, 18]]


def test_config_programs_evaluate_at_small_sizes():
    """The five benchmark programs run through the oracle at shrunken sizes and produce finite, sane results."""
    from ryft_b200 import configs
    (o,) = ev.evaluate(configs.c1_program(16, 24, 8), [configs.c1_inputs(16, 24, 8)])[0]
    a, b = configs.c1_inputs(16, 24, 8)
    np.testing.assert_allclose(o, a.astype(np.float64) @ b.astype(np.float64), rtol=1e-6)
    (o,) = ev.evaluate(configs.c2_program(2, 16, 8, 16), [configs.c2_inputs(2, 16, 8, 16)])[0]
    assert o.shape == (2, 16, 16) and np.all(np.abs(o.astype(np.float32)) <= 1)
    q, k, v = configs.c3_inputs(1, 2, 16, 8)
    (o,) = ev.evaluate(configs.c3_program(1, 2, 16, 8), [[q, k, v]])[0]
    # row 0 of a causal attention sees only key 0, so its output is v[0]
    np.testing.assert_array_equal(o[:, :, 0, :], v[:, :, 0, :])
    dw1, dw2, loss = ev.evaluate(configs.c4_program(32, 16, 24), [configs.c4_inputs(32, 16, 24)])[0]
    assert dw1.shape == (16, 24) and dw2.shape == (24, 16) and loss.shape == () and np.isfinite(loss)
    reps = [configs.c4_inputs(32, 16, 24, seed=4, replica=r) for r in range(2)]
    outs = ev.evaluate(configs.c4_program(32, 16, 24, replicas=2), reps)
    np.testing.assert_array_equal(outs[0][0], outs[1][0])
