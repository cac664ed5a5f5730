"""Data-parallel execution over several GPUs of one process: replicas meet in stablehlo.all_reduce / all_gather (NCCL).
Needs at least two GPUs; skipped otherwise.  Failure handling is exercised on the host only (a poisoned launch)."""
import numpy as np
import pytest

from oracle import stablehlo_eval as ev
from ryft_b200 import configs, pjrt
from ryft_b200.stablehlo import Builder

from helpers import assert_close

pytestmark = pytest.mark.gpu


def _n_gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


needs2 = pytest.mark.skipif(_n_gpus() < 2, reason="needs two GPUs")


def run_replicated(client, text, per_replica_inputs):
    n = len(per_replica_inputs)
    exe = client.compile(pjrt.Program.mlir(text), pjrt.CompilationOptions(replica_count=n))
    devs = exe.addressable_devices()
    assert len(devs) == n and exe.addressable_device_logical_ids() == [(r, 0) for r in range(n)]
    ins = [pjrt.ExecutionDeviceInputs([client.buffer(np.asarray(x), device=devs[r]) for x in per_replica_inputs[r]]) for r in range(n)]
    outs = exe.execute(ins)
    for o in outs:
        o.done.await_()
    return exe, [[b.to_numpy() for b in o.outputs] for o in outs]


@needs2
def test_reference_all_reduce_example_two_replicas(client):
    # crates/ryft-mlir/src/dialects/stable_hlo/operations/communication.rs:821-841 (i32 instead of i64)
    b = Builder()
    x = b.arg([4], "i32"); y = b.arg([4], "i32")
    r0, r1 = b.all_reduce([x, y], [[0, 1]])
    text = b.build(r0, r1)
    reps = [[np.array([1, 2, 3, 4], np.int32), np.array([9, 10, 11, 12], np.int32)], [np.array([5, 6, 7, 8], np.int32), np.array([13, 14, 15, 16], np.int32)]]
    _, outs = run_replicated(client, text, reps)
    for r in range(2):
        assert outs[r][0].tolist() == [6, 8, 10, 12] and outs[r][1].tolist() == [22, 24, 26, 28]


@needs2
def test_arguments_of_a_detached_all_reduce_outlive_their_handles(client):
    """An all-reduce that nothing in the program waits for runs on the communication stream after the execute call has
    returned.  Its operands are the caller's argument buffers: destroying them right away, and allocating new buffers of
    the same size over them, must not disturb the collective (the plugin orders the free behind it)."""
    b = Builder()
    x = b.arg([16 * 1024 * 1024], "f32")
    (r,) = b.all_reduce([x], [[0, 1]])
    text = b.build(r)
    exe = client.compile(pjrt.Program.mlir(text), pjrt.CompilationOptions(replica_count=2))
    devs = exe.addressable_devices()
    rng = np.random.default_rng(5)
    data = [rng.standard_normal(16 * 1024 * 1024).astype(np.float32) for _ in range(2)]
    want = data[0] + data[1]
    for _ in range(3):
        bufs = [client.buffer(data[i], device=devs[i]) for i in range(2)]
        outs = exe.execute([pjrt.ExecutionDeviceInputs([bufs[0]]), pjrt.ExecutionDeviceInputs([bufs[1]])])
        for x_ in bufs:
            x_.delete()
        del bufs
        junk = [client.buffer(np.full(16 * 1024 * 1024, 7.0, np.float32), device=devs[i]) for i in range(2)]
        for o in outs:
            o.done.await_()
            assert np.array_equal(o.outputs[0].to_numpy(), want)
        del junk


@needs2
def test_reference_all_gather_example_two_replicas(client):
    # communication.rs:722-739 (i32): gather along dim 1
    b = Builder()
    x = b.arg([2, 2], "i32")
    text = b.build(b.all_gather(x, 1, [[0, 1]]), b.all_gather(x, 0, [[0, 1]]))
    reps = [[np.array([[1, 2], [3, 4]], np.int32)], [np.array([[5, 6], [7, 8]], np.int32)]]
    _, outs = run_replicated(client, text, reps)
    for r in range(2):
        assert outs[r][0].tolist() == [[1, 2, 5, 6], [3, 4, 7, 8]]
        assert outs[r][1].tolist() == [[1, 2], [3, 4], [5, 6], [7, 8]]


@needs2
def test_data_parallel_gradient_step_matches_oracle(client):
    T, D, F = 256, 128, 384
    n = min(_n_gpus(), 4)
    text = configs.c4_program(T, D, F, replicas=n)
    reps = [configs.c4_inputs(T, D, F, seed=4, replica=r) for r in range(n)]
    _, outs = run_replicated(client, text, reps)
    want = ev.evaluate(text, reps)
    for r in range(n):
        for i in range(3):
            assert_close(outs[r][i], want[r][i], f"replica {r} output {i}")
    for r in range(1, n):   # every replica holds the same averaged gradients
        assert np.array_equal(outs[0][0], outs[r][0]) and np.array_equal(outs[0][1], outs[r][1])


@needs2
def test_replica_id_and_group_validation(client):
    b = Builder()
    x = b.arg([8], "f32")
    rid = b.convert(b.replica_id(), "f32")
    text = b.build(b.add(x, b.broadcast_in_dim(rid, [], [8])))
    _, outs = run_replicated(client, text, [[np.zeros(8, np.float32)], [np.zeros(8, np.float32)]])
    assert outs[0][0].tolist() == [0.0] * 8 and outs[1][0].tolist() == [1.0] * 8
    bad = Builder()
    y = bad.arg([4], "f32")
    (r,) = bad.all_reduce([y], [[0, 5]])
    with pytest.raises(pjrt.PjrtError) as e:
        client.compile(pjrt.Program.mlir(bad.build(r)), pjrt.CompilationOptions(replica_count=2))
    assert e.value.code_name == "INVALID_ARGUMENT"


@needs2
def test_poisoned_replica_aborts_the_whole_execution_without_touching_the_gpus(client):
    """A replica that fails before launch (injected on the host) must keep the other replica out of the collective:
    both completion events carry an error and later executions still work."""
    b = Builder()
    x = b.arg([1024], "f32")
    (r,) = b.all_reduce([x], [[0, 1]])
    text = b.build(r)
    exe = client.compile(pjrt.Program.mlir(text), pjrt.CompilationOptions(replica_count=2))
    devs = exe.addressable_devices()
    ins = [pjrt.ExecutionDeviceInputs([client.buffer(np.full(1024, r + 1, np.float32), device=devs[r])]) for r in range(2)]
    assert devs[1].poison_execution(42, 14, "rank 1 lost its heartbeat")
    outs = exe.execute(ins, launch_id=42)
    errs = []
    for o in outs:
        with pytest.raises(pjrt.PjrtError) as e:
            o.done.await_()
        errs.append(e.value)
    assert errs[1].code_name == "UNAVAILABLE" and errs[0].code_name == "ABORTED" and "replica 1" in errs[0].message
    ok = exe.execute(ins, launch_id=43)
    for o in ok:
        o.done.await_()
    assert ok[0].outputs[0].to_numpy().tolist() == [3.0] * 1024


@needs2
def test_two_replica_gradient_step_matches_the_committed_fixture(client):
    from test_golden_fixtures import load
    text, ins, outs = load("c5_mlp_gradients_2_replicas")
    _, got = run_replicated(client, text, ins)
    for r in range(2):
        for k, (g, w) in enumerate(zip(got[r], outs[r])):
            assert_close(g, w, f"c5 fixture replica {r} output {k}")


@needs2
def test_reference_collective_examples_with_i64_as_written(client):
    """The reference's worked examples of all_reduce and all_gather with the element type they are written in
    (i64, crates/ryft-mlir/src/dialects/stable_hlo/operations/communication.rs:821-841 and :722-739)."""
    b = Builder()
    x = b.arg([4], "i64"); y = b.arg([4], "i64"); g = b.arg([2, 2], "i64")
    r0, r1 = b.all_reduce([x, y], [[0, 1]])
    text = b.build(r0, r1, b.all_gather(g, 1, [[0, 1]]))
    reps = [[np.array([1, 2, 3, 4], np.int64), np.array([9, 10, 11, 12], np.int64), np.array([[1, 2], [3, 4]], np.int64)],
            [np.array([5, 6, 7, 8], np.int64), np.array([13, 14, 15, 16], np.int64), np.array([[5, 6], [7, 8]], np.int64)]]
    _, outs = run_replicated(client, text, reps)
    for r in range(2):
        assert outs[r][0].dtype == np.int64
        assert outs[r][0].tolist() == [6, 8, 10, 12] and outs[r][1].tolist() == [22, 24, 26, 28]
        assert outs[r][2].tolist() == [[1, 2, 5, 6], [3, 4, 7, 8]]
