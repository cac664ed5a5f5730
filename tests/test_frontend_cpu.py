"""Front end and planner, checked on the host through `b2x_plan_dump`: every printed form the reference pins parses,
fusion decisions are the intended ones, and unsupported input is rejected at compile time with the reference's error
codes (never executed on the CPU)."""
import pytest

import ryft_b200
from ryft_b200 import configs, pjrt
from ryft_b200.stablehlo import Builder


def wrap(body: str, args: str, ret: str, names: str) -> str:
    return f"module {{\n  func.func @main({args}) -> {ret} {{\n{body}\n    return {names} : {ret.strip('()')}\n  }}\n}}\n"


# one entry per printed form pinned by a reference test (file:line of that test in crates/ryft-mlir/src/dialects/stable_hlo/operations/)
PRINTED_FORMS = [
    ("arithmetic.rs:695", "%0 = stablehlo.add %arg0, %arg1 : tensor<2x2xi32>", "%arg0: tensor<2x2xi32>, %arg1: tensor<2x2xi32>", "tensor<2x2xi32>"),
    ("arithmetic.rs:740", "%0 = stablehlo.subtract %arg0, %arg1 : tensor<2x2xi32>", "%arg0: tensor<2x2xi32>, %arg1: tensor<2x2xi32>", "tensor<2x2xi32>"),
    ("arithmetic.rs:785", "%0 = stablehlo.multiply %arg0, %arg1 : tensor<2x2xi32>", "%arg0: tensor<2x2xi32>, %arg1: tensor<2x2xi32>", "tensor<2x2xi32>"),
    ("arithmetic.rs:830", "%0 = stablehlo.divide %arg0, %arg1 : tensor<2x2xf32>", "%arg0: tensor<2x2xf32>, %arg1: tensor<2x2xf32>", "tensor<2x2xf32>"),
    ("arithmetic.rs:650", "%0 = stablehlo.negate %arg0 : tensor<3xi32>", "%arg0: tensor<3xi32>", "tensor<3xi32>"),
    ("comparison.rs:590", "%0 = stablehlo.maximum %arg0, %arg1 : tensor<3xf32>", "%arg0: tensor<3xf32>, %arg1: tensor<3xf32>", "tensor<3xf32>"),
    ("comparison.rs:634", "%0 = stablehlo.minimum %arg0, %arg1 : tensor<3xf32>", "%arg0: tensor<3xf32>, %arg1: tensor<3xf32>", "tensor<3xf32>"),
    ("trigonometric.rs:442", "%0 = stablehlo.tanh %arg0 : tensor<3xf32>", "%arg0: tensor<3xf32>", "tensor<3xf32>"),
    ("exponential.rs:673", "%0 = stablehlo.exponential %arg0 : tensor<2x2xf32>", "%arg0: tensor<2x2xf32>", "tensor<2x2xf32>"),
    ("exponential.rs:540-544", "%0 = stablehlo.sqrt %arg0 {result_accuracy = #stablehlo.result_accuracy<mode = #stablehlo.result_accuracy_mode<HIGHEST>>} : tensor<2x2xf32>",
     "%arg0: tensor<2x2xf32>", "tensor<2x2xf32>"),
    ("casting.rs:456", "%0 = stablehlo.convert %arg0 : (tensor<3xi32>) -> tensor<3xf32>", "%arg0: tensor<3xi32>", "tensor<3xf32>"),
    ("comparison.rs:500", "%0 = stablehlo.compare GE, %arg0, %arg1, TOTALORDER : (tensor<3xf32>, tensor<3xf32>) -> tensor<3xi1>",
     "%arg0: tensor<3xf32>, %arg1: tensor<3xf32>", "tensor<3xi1>"),
    ("control_flow.rs:596", "%0 = stablehlo.select %arg0, %arg1, %arg2 : tensor<3x4xi1>, tensor<3x4xi32>",
     "%arg0: tensor<3x4xi1>, %arg1: tensor<3x4xi32>, %arg2: tensor<3x4xi32>", "tensor<3x4xi32>"),
    ("control_flow.rs:361", "%0 = stablehlo.constant dense<0> : tensor<2xi32>", "", "tensor<2xi32>"),
    ("miscellaneous.rs:1144", "%0 = stablehlo.constant dense<[[0, 1, 2, 3], [4, 5, 6, 7]]> : tensor<2x4xi32>", "", "tensor<2x4xi32>"),
    ("elements.rs:1335", "%0 = stablehlo.constant dense<[1.500000e+00, -2.500000e+00]> : tensor<2xf32>", "", "tensor<2xf32>"),
    ("float.rs:12-24", "%0 = stablehlo.constant dense<0xFF800000> : tensor<2xf32>", "", "tensor<2xf32>"),
    ("miscellaneous.rs:1181", "%0 = stablehlo.iota dim = 1 : tensor<4x5xi32>", "", "tensor<4x5xi32>"),
    ("manipulation.rs:2154", "%0 = stablehlo.broadcast_in_dim %arg0, dims = [2, 1] : (tensor<1x3xi32>) -> tensor<2x3x2xi32>", "%arg0: tensor<1x3xi32>", "tensor<2x3x2xi32>"),
    ("manipulation.rs:2022", "%0 = stablehlo.transpose %arg0, dims = [2, 0, 1] : (tensor<3x4x5xi32>) -> tensor<5x3x4xi32>", "%arg0: tensor<3x4x5xi32>", "tensor<5x3x4xi32>"),
    ("manipulation.rs:2065", "%0 = stablehlo.reshape %arg0 : (tensor<1x6xi32>) -> tensor<2x3xi32>", "%arg0: tensor<1x6xi32>", "tensor<2x3xi32>"),
    ("linear_algebra.rs:2245-2258",
     "%0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [0] x [0], contracting_dims = [2] x [1], algorithm = <lhs_precision_type = tf32, rhs_precision_type = tf32, "
     "accumulation_type = f32, lhs_component_count = 1, rhs_component_count = 1, num_primitive_operations = 1, allow_imprecise_accumulation = false> "
     ": (tensor<2x2x2xf32>, tensor<2x2x2xf32>) -> tensor<2x2x2xf32>", "%arg0: tensor<2x2x2xf32>, %arg1: tensor<2x2x2xf32>", "tensor<2x2x2xf32>"),
    ("devices.rs:1265-1270", "%0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [] x [], contracting_dims = [1] x [0] : (tensor<4x4xf32>, tensor<4x4xf32>) -> tensor<4x4xf32>",
     "%arg0: tensor<4x4xf32>, %arg1: tensor<4x4xf32>", "tensor<4x4xf32>"),
    ("functional.rs:534-536", "%0 = stablehlo.reduce(%arg0 init: %arg1) applies stablehlo.add across dimensions = [1] : (tensor<3x4xi32>, tensor<i32>) -> tensor<3xi32>",
     "%arg0: tensor<3x4xi32>, %arg1: tensor<i32>", "tensor<3xi32>"),
    ("communication.rs:168-173", "%0 = stablehlo.replica_id : tensor<ui32>", "", "tensor<ui32>"),
]


@pytest.mark.parametrize("where,line,args,ret", PRINTED_FORMS, ids=[p[0] for p in PRINTED_FORMS])
def test_printed_forms_parse_and_plan(where, line, args, ret):
    text = wrap("    " + line, args, ret, "%0")
    dump = ryft_b200.plan_dump(text)
    assert dump.startswith("plan main:")


def test_generic_forms_of_collectives_parse():
    # communication.rs:1759-1767 and :1692-1697
    text = """
module {
  func.func @main(%arg0: tensor<2x2xf32>, %arg1: tensor<2x2xi32>) -> (tensor<2x2xf32>, tensor<2x4xi32>) {
    %0 = "stablehlo.all_reduce"(%arg0) <{channel_handle = #stablehlo.channel_handle<handle = 1, type = 1>, replica_groups = dense<[[0, 2], [1, 3]]> : tensor<2x2xi64>, use_global_device_ids}> ({
    ^bb0(%arg2: tensor<f32>, %arg3: tensor<f32>):
      %2 = stablehlo.add %arg2, %arg3 : tensor<f32>
      stablehlo.return %2 : tensor<f32>
    }) : (tensor<2x2xf32>) -> tensor<2x2xf32>
    %1 = "stablehlo.all_gather"(%arg1) <{all_gather_dim = 1 : i64, channel_handle = #stablehlo.channel_handle<handle = 1, type = 0>, replica_groups = dense<[[0, 2], [1, 3]]> : tensor<2x2xi64>, use_global_device_ids}> : (tensor<2x2xi32>) -> tensor<2x4xi32>
    return %0, %1 : tensor<2x2xf32>, tensor<2x4xi32>
  }
}
"""
    dump = ryft_b200.plan_dump(text, num_replicas=4)
    assert "all_reduce #0" in dump and "all_gather #1" in dump and "copy:all_gather_interleave" in dump


def test_reference_add_program_plans_to_one_kernel():
    text = wrap("    %0 = stablehlo.add %arg0, %arg1 : tensor<2x1xi32>", "%arg0: tensor<2x1xi32>, %arg1: tensor<2x1xi32>", "tensor<2x1xi32>", "%0")
    dump = ryft_b200.plan_dump(text)
    assert "1 steps" in dump and "load T0; add T1; store T2;" in dump


def test_c2_epilogue_is_fused_into_the_gemm():
    dump = ryft_b200.plan_dump(configs.c2_program())
    assert "1 steps" in dump and "tcgen05" in dump
    # bias add + tanh + convert, one store in bf16 (the store rounds, so the convert carries no rounding step); the
    # bf16 value only leaves the program, so the hardware tanh is used
    assert "load acc0; add T0; tanh aux=1; cvt; store T1;" in dump
    assert "arena 0 B" in dump                                               # nothing is materialised


def test_c3_is_recognised_as_fused_attention():
    dump = ryft_b200.plan_dump(configs.c3_program())
    assert "1 steps" in dump and "attention " in dump and "BH=128 Sq=4096 Sk=4096 D=128" in dump and "causal" in dump
    assert "arena 0 B" in dump                                               # no score tensor exists
    dump = ryft_b200.plan_dump(configs.c3_program(1, 2, 256, 64, causal=False))
    assert "attention " in dump and "causal" not in dump


def test_causal_mask_is_folded_into_the_gemm_epilogue():
    # the scores of config 3 alone (no softmax behind them): iota / compare / select run as index arithmetic in the
    # epilogue of the QK^T GEMM and the mask is never materialised
    import math
    b = Builder()
    q = b.arg([2, 256, 64], "bf16"); k = b.arg([2, 256, 64], "bf16")
    s = b.dot_general(q, k, ([0], [0]), ([2], [2]), out_dtype="f32")
    s = b.multiply(s, b.splat(1.0 / math.sqrt(64), s))
    mask = b.compare("GE", b.iota(0, [256, 256], "i32"), b.iota(1, [256, 256], "i32"), "SIGNED")
    s = b.select(b.broadcast_in_dim(mask, [1, 2], [2, 256, 256]), s, b.splat(float("-inf"), s))
    dump = ryft_b200.plan_dump(b.build(s))
    assert "1 steps" in dump and "load iota1; cmp iota2 aux=2;" in dump and "select #0xff800000" in dump


def test_c4_plan_shape():
    dump = ryft_b200.plan_dump(configs.c4_program())
    assert dump.count("gemm ") == 5 and dump.count("tcgen05") == 5
    assert "6 steps" in dump                       # 5 GEMMs + the loss reduce, which scales its own result
    assert "reduce reduce:%19+epilogue(%21 )" in dump and "load acc0; mul #" in dump
    # the forward GEMM stores H and gelu(H) in bf16 from one accumulator
    first = dump.split("[1]")[0]
    assert first.count("store") == 2 and ":bf16" in first and ":f32" not in first.split("vm:")[1].split("code:")[0]


def test_c5_collectives_are_split_hoisted_and_run_in_place():
    dump = ryft_b200.plan_dump(configs.c4_program(replicas=8), num_replicas=8)
    lines = [l for l in dump.splitlines() if l.lstrip().startswith("[")]
    first_ar = next(i for i, l in enumerate(lines) if "all_reduce #0" in l)
    last_gemm = max(i for i, l in enumerate(lines) if " gemm " in l)
    assert first_ar < last_gemm, "the first gradient all-reduce must start before the last GEMM is issued"
    # the divide by the replica count (a power of two) moved in front of the collective and into the GEMM epilogue:
    # no scaling pass remains, the collectives run in place on the output buffers and nothing in the plan waits for them
    assert "elementwise fused:stablehlo.multiply:%60" not in dump and dump.count("elementwise ") == 0   # (the loss scale runs inside the reduce)
    assert "out1 -> out1" in dump and "out0 -> out0" in dump and dump.count("detached") == 2
    assert "load acc0; mul #0x3e000000; store T0;" in dump       # accumulator * 1/8 straight into the output


def test_scale_by_a_non_power_of_two_is_not_moved():
    dump = ryft_b200.plan_dump(configs.c4_program(256, 128, 384, replicas=3), num_replicas=3)
    assert dump.count("elementwise ") == 2 and "(wait #" in dump   # two gradient scaling passes behind the all-reduce


@pytest.mark.parametrize("body,needle", [
    ("    %0 = stablehlo.custom_call @foo(%arg0) : (tensor<2xf32>) -> tensor<2xf32>", "custom_call"),
    ("    %0 = stablehlo.sort %arg0 : tensor<2xf32>", "sort"),
    ('    %0 = "stablehlo.rng_bit_generator"(%arg0) : (tensor<2xf32>) -> tensor<2xf32>', "rng_bit_generator"),
])
def test_unsupported_ops_are_rejected_by_name(body, needle):
    text = wrap(body, "%arg0: tensor<2xf32>", "tensor<2xf32>", "%0")
    with pytest.raises(pjrt.PjrtError) as e:
        ryft_b200.plan_dump(text)
    assert e.value.code_name == "UNIMPLEMENTED" and needle in e.value.message


def test_bytecode_is_rejected_with_a_clear_message():
    with pytest.raises(pjrt.PjrtError) as e:
        ryft_b200.plan_dump(b"ML\xefR\x00\x01")
    assert e.value.code_name == "UNIMPLEMENTED" and "bytecode" in e.value.message


@pytest.mark.parametrize("body,args,ret", [
    ("    %0 = stablehlo.add %arg0, %arg1 : tensor<2xf32>", "%arg0: tensor<2xf32>, %arg1: tensor<3xf32>", "tensor<2xf32>"),
    ("    %0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [] x [], contracting_dims = [1] x [0] : (tensor<2x3xf32>, tensor<4x2xf32>) -> tensor<2x2xf32>",
     "%arg0: tensor<2x3xf32>, %arg1: tensor<4x2xf32>", "tensor<2x2xf32>"),
    ("    %0 = stablehlo.broadcast_in_dim %arg0, dims = [0] : (tensor<3xf32>) -> tensor<2x3xf32>", "%arg0: tensor<3xf32>", "tensor<2x3xf32>"),
])
def test_malformed_programs_are_invalid_argument(body, args, ret):
    with pytest.raises(pjrt.PjrtError) as e:
        ryft_b200.plan_dump(wrap(body, args, ret, "%0"))
    assert e.value.code_name == "INVALID_ARGUMENT"


def test_partitioning_requests_are_unimplemented():
    text = wrap("    %0 = stablehlo.add %arg0, %arg0 : tensor<2xf32>", '%arg0: tensor<2xf32> {sdy.sharding = #sdy.sharding<@mesh, [{"x"}]>}', "tensor<2xf32>", "%0")
    assert ryft_b200.plan_dump(text).startswith("plan main")     # attributes alone are accepted


def test_builder_matches_reference_program_text():
    b = Builder()
    x = b.arg([2, 1], "i32"); y = b.arg([2, 1], "i32")
    text = b.build(b.add(x, y))
    # crates/ryft-pjrt/src/programs.rs:2492-2498
    assert text == ("module {\n  func.func @main(%arg0: tensor<2x1xi32>, %arg1: tensor<2x1xi32>) -> tensor<2x1xi32> {\n"
                    "    %0 = stablehlo.add %arg0, %arg1 : tensor<2x1xi32>\n    return %0 : tensor<2x1xi32>\n  }\n}\n")


def test_oversize_fusion_groups_are_cut_instead_of_rejected():
    """A fusion group that exceeds the kernels' program limits (56 instructions, 8 tensors, 6 temporaries) is cut at an
    interior value, which becomes a kernel of its own."""
    b = Builder()
    y = x = b.arg([1024, 1024], "f32")
    for _ in range(60):
        y = b.tanh(y)
    dump = ryft_b200.plan_dump(b.build(y))
    assert dump.count("elementwise fused:") == 2 and dump.count(" tanh;") == 60
    b = Builder()
    xs = [b.arg([1024, 1024], "f32") for _ in range(10)]
    y = xs[0]
    for v in xs[1:]:
        y = b.add(y, v)
    dump = ryft_b200.plan_dump(b.build(y))
    assert dump.count("elementwise fused:") == 2 and dump.count(" add T") == 9
    # the same chain as the prologue of a reduce, and as the epilogue of a GEMM
    b = Builder()
    y = x = b.arg([1024, 1024], "f32")
    for _ in range(60):
        y = b.tanh(y)
    dump = ryft_b200.plan_dump(b.build(b.reduce(y, b.constant(0.0, [], "f32"), "add", [1])))
    assert "reduce reduce:" in dump and dump.count(" tanh;") == 60
    b = Builder()
    lhs = b.arg([256, 128], "bf16"); rhs = b.arg([128, 256], "bf16")
    y = b.dot_general(lhs, rhs, ([], []), ([1], [0]), out_dtype="f32")
    for _ in range(60):
        y = b.tanh(y)
    dump = ryft_b200.plan_dump(b.build(y))
    assert "gemm dot_general" in dump and dump.count(" tanh;") == 60


def test_empty_reductions_plan_without_dividing_by_zero():
    b = Builder()
    x = b.arg([0, 8192], "f32")
    dump = ryft_b200.plan_dump(b.build(b.reduce(x, b.constant(0.0, [], "f32"), "add", [1])))
    assert "A=0,R=8192" in dump
    import ctypes as C
    lib = C.CDLL(str(ryft_b200.KERNELS_PATH))
    lib.b2x_reduce_splits.argtypes = [C.c_int64] * 3
    assert lib.b2x_reduce_splits(0, 8192, 1) == 1 and lib.b2x_reduce_splits(0, 1 << 20, 0) == 1


def test_benchmark_programs_take_specialised_gemm_variants():
    """The kernel variant each GEMM of the benchmark programs runs, as the launcher decides it (host only)."""
    r4 = {r["label"].split("+")[0]: r for r in ryft_b200.plan_routes(configs.c4_program())}
    assert len(r4) == 5 and all(r["bn"] == 256 and r["static_id"] and r["ctas"] == 148 for r in r4.values())
    # two-store epilogues of 256-row tiles always go through shared memory (their time is not hidden behind the next tile)
    assert r4["dot_general:%0"]["transposed"] == 1 and r4["dot_general:%16"]["transposed"] == 1 and r4["dot_general:%16"]["stores"] == 2
    # long K: 256-row tiles (two MMAs per k-step share the B sub-tile), also where their last round of SMs is less full
    assert all(r["tile_rows"] == 256 and r["epi_groups"] == 2 for r in r4.values())
    assert r4["dot_general:%0"]["m_tiles"] * r4["dot_general:%0"]["n_tiles"] == 32 * 64 and r4["dot_general:%16"]["m_tiles"] * r4["dot_general:%16"]["n_tiles"] == 32 * 16
    (r2,) = ryft_b200.plan_routes(configs.c2_program())
    assert (r2["bn"], r2["epi_groups"], r2["k_blocks"], r2["stores"], r2["tile_rows"]) == (256, 1, 2, 1, 128) and r2["static_id"]
    (r1,) = ryft_b200.plan_routes(configs.c1_program())
    assert r1["K"] == 3 * 768 and r1["static_id"]
