"""The reference's own runtime tests, replayed against the plugin on a B200 (same call sequence through the C ABI):
crates/ryft-pjrt/src/programs.rs:2576-2622, 2781-2829 (execute + metadata), buffers.rs:3780-3992 (buffers),
clients.rs:1361-1392 (client), devices.rs:1194-1234, 1254-1364 (devices, poison_execution), README.md:88-137 (matmul)."""
import threading

import numpy as np
import pytest

from ryft_b200 import pjrt

pytestmark = pytest.mark.gpu

ADD_PROGRAM = """
module {
  func.func @main(%arg0: tensor<2x1xi32>, %arg1: tensor<2x1xi32>) -> tensor<2x1xi32> {
    %0 = stablehlo.add %arg0, %arg1 : tensor<2x1xi32>
    return %0 : tensor<2x1xi32>
  }
}
"""


def test_client_and_devices(client):
    assert client.platform_name() == "cuda"
    assert client.platform_version().startswith("cuda 12")
    assert client.process_index() == 0
    devs = client.devices()
    assert devs and devs == client.addressable_devices()
    d = devs[0]
    assert d.is_addressable() and d.process_index == 0 and d.id == 0
    assert "B200" in d.kind or "NVIDIA" in d.kind
    assert d.attributes()["compute_capability"] == "10.0"
    assert d.attributes()["core_count"] == 148
    stats = d.memory_statistics()
    assert stats["bytes_limit"] > 100 * 2**30
    assert client.lookup_device(0) == d
    assert client.default_device_assignment(1, 1) == [0]
    with pytest.raises(pjrt.PjrtError):
        client.default_device_assignment(len(devs) + 1, 1)


def test_loaded_executable_execute_reference_add(client):
    # crates/ryft-pjrt/src/programs.rs:2781-2829: [7, -1] + [35, -41] = [42, -42], compared as bytes
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM), pjrt.CompilationOptions())
    device = exe.addressable_devices()[0]
    lhs = client.buffer(np.array([7, -1], np.int32).tobytes(), pjrt.BufferType.S32, [2, 1], device)
    rhs = client.buffer(np.array([35, -41], np.int32).tobytes(), pjrt.BufferType.S32, [2, 1], device)
    outs = exe.execute([pjrt.ExecutionDeviceInputs([lhs, rhs])], launch_id=0)
    assert len(outs) == 1
    outs[0].done.await_()
    out = outs[0].outputs[0]
    assert out.copy_to_host().await_() == np.array([42, -42], np.int32).tobytes()
    assert out.element_type() == pjrt.BufferType.S32 and out.dimensions() == [2, 1] and not out.is_on_cpu()


def test_executable_metadata(client):
    # crates/ryft-pjrt/src/programs.rs:2576-2622
    le = client.compile(pjrt.Program.mlir(ADD_PROGRAM), pjrt.CompilationOptions())
    exe = le.executable()
    assert exe.name() == "main" and exe.num_replicas() == 1 and exe.num_partitions() == 1 and exe.num_outputs() == 1
    assert exe.output_element_types() == [pjrt.BufferType.S32] and exe.output_dimensions() == [[2, 1]]
    assert exe.output_memory_kinds() == ["device"]
    assert le.addressable_device_logical_ids() == [(0, 0)]
    assert le.device_assignment() == b"\x08\x01\x10\x01\x1a\x03\x0a\x01\x00"   # DeviceAssignmentProto{1, 1, [[0]]}
    assert exe.optimized_program().code.decode() == ADD_PROGRAM
    assert len(exe.fingerprint()) == 16
    blob = exe.serialize()
    le2 = client.deserialize_and_load(blob)
    dev = le2.addressable_devices()[0]
    a = client.buffer(np.array([[1], [2]], np.int32), device=dev)
    outs = le2.execute([pjrt.ExecutionDeviceInputs([a, a])])
    assert outs[0].outputs[0].to_numpy().ravel().tolist() == [2, 4]
    assert not le.is_deleted()
    le.delete()
    assert le.is_deleted()
    with pytest.raises(pjrt.PjrtError):
        le.execute([pjrt.ExecutionDeviceInputs([a, a])])


def test_readme_matmul(client):
    # README.md:88, 108-137: [[1,2,3],[4,5,6]] . [[7,8],[9,10],[11,12]] = [58, 64, 139, 154]
    text = """
module {
  func.func @main(%arg0: tensor<2x3xf32>, %arg1: tensor<3x2xf32>) -> tensor<2x2xf32> {
    %0 = stablehlo.dot_general %arg0, %arg1, batching_dims = [] x [], contracting_dims = [1] x [0] : (tensor<2x3xf32>, tensor<3x2xf32>) -> tensor<2x2xf32>
    return %0 : tensor<2x2xf32>
  }
}
"""
    exe = client.compile(pjrt.Program.mlir(text))
    lhs = client.buffer(np.array([[1, 2, 3], [4, 5, 6]], np.float32))
    rhs = client.buffer(np.array([[7, 8], [9, 10], [11, 12]], np.float32))
    out = exe.execute([pjrt.ExecutionDeviceInputs([lhs, rhs])])[0].outputs[0].to_numpy()
    assert out.ravel().tolist() == [58.0, 64.0, 139.0, 154.0]


def test_buffer_round_trips(client):
    # crates/ryft-pjrt/src/buffers.rs:3873-3924
    data = bytes([1, 2, 3, 4, 5, 6])
    buf = client.buffer(data, pjrt.BufferType.U8, [2, 3])
    assert buf.on_device_size_in_bytes() == 6
    assert buf.copy_to_host().await_() == data
    assert buf.copy_raw_to_host(2, 3).await_() == bytes([3, 4, 5])
    with pytest.raises(pjrt.PjrtError):
        buf.copy_raw_to_host(2, 10).await_()
    buf.ready().await_()
    other = buf.copy_to_device(buf.device())
    assert other.copy_to_host().await_() == data
    assert buf.device_pointer() != 0 and buf.device_pointer() != other.device_pointer()
    buf.delete()
    assert buf.is_deleted()
    with pytest.raises(pjrt.PjrtError):
        buf.copy_to_host()


def test_strided_host_buffer_and_large_round_trip(client):
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    t = a.T  # strides (4, 24) bytes
    buf = client.buffer(t, pjrt.BufferType.F32, t.shape, byte_strides=t.strides)
    assert np.array_equal(buf.to_numpy(), t)
    big = np.random.default_rng(0).integers(0, 255, size=(64 << 20,), dtype=np.uint8)
    assert np.array_equal(client.buffer(big).to_numpy(), big)
    empty = client.buffer(np.zeros((0, 4), np.float32))
    assert empty.to_numpy().shape == (0, 4)


def test_view_of_device_buffer_is_zero_copy(client):
    import torch
    t = torch.arange(16, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    view = client.view_of_device_buffer(t.data_ptr(), pjrt.BufferType.F32, [16], keep=t)
    assert view.device_pointer() == t.data_ptr()
    assert view.to_numpy().tolist() == list(range(16))


def test_execute_argument_validation(client):
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM))
    a = client.buffer(np.zeros((2, 1), np.int32))
    f = client.buffer(np.zeros((2, 1), np.float32))
    with pytest.raises(pjrt.PjrtError) as e:
        exe.execute([pjrt.ExecutionDeviceInputs([a])])
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(pjrt.PjrtError) as e:
        exe.execute([pjrt.ExecutionDeviceInputs([a, f])])
    assert "tensor<2x1xf32>" in e.value.message
    with pytest.raises(pjrt.PjrtError):
        exe.execute([pjrt.ExecutionDeviceInputs([a, a]), pjrt.ExecutionDeviceInputs([a, a])])
    gone = client.buffer(np.zeros((2, 1), np.int32))
    gone.delete()
    with pytest.raises(pjrt.PjrtError):
        exe.execute([pjrt.ExecutionDeviceInputs([a, gone])])


def test_compile_errors_surface_through_the_c_abi(client):
    bad = ADD_PROGRAM.replace("stablehlo.add", "stablehlo.cholesky")
    with pytest.raises(pjrt.PjrtError) as e:
        client.compile(pjrt.Program.mlir(bad))
    assert e.value.code_name == "UNIMPLEMENTED" and "cholesky" in e.value.message
    with pytest.raises(pjrt.PjrtError) as e:
        client.compile(pjrt.Program(b"HloModule m", "hlo"))
    assert e.value.code_name == "UNIMPLEMENTED"
    with pytest.raises(pjrt.PjrtError) as e:
        client.compile(pjrt.Program.mlir(ADD_PROGRAM), pjrt.CompilationOptions(replica_count=64))
    assert e.value.code_name == "INVALID_ARGUMENT"


def test_poison_execution_fails_that_launch_only(client):
    # crates/ryft-pjrt/src/devices.rs:1254-1364: the failure is injected on the host, before anything is enqueued
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM))
    dev = exe.addressable_devices()[0]
    a = client.buffer(np.ones((2, 1), np.int32), device=dev)
    assert dev.poison_execution(7, 10, "injected failure")
    outs = exe.execute([pjrt.ExecutionDeviceInputs([a, a])], launch_id=7)
    with pytest.raises(pjrt.PjrtError) as e:
        outs[0].done.await_()
    assert e.value.code_name == "ABORTED" and "injected failure" in e.value.message
    with pytest.raises(pjrt.PjrtError):
        outs[0].outputs[0].copy_to_host()
    ok = exe.execute([pjrt.ExecutionDeviceInputs([a, a])], launch_id=8)
    ok[0].done.await_()
    assert ok[0].outputs[0].to_numpy().ravel().tolist() == [2, 2]


def test_expired_device_wait_is_reported_once_as_deadline_exceeded(client):
    """A wait inside a kernel that nothing satisfies must end by itself: with one mbarrier arrival withheld (a host-side
    switch of the launcher; every other block of the kernel runs normally) the roles of that block give up after about
    a second, the kernel returns, and the execution's completion event carries DEADLINE_EXCEEDED.  The device's status
    word is cleared by that report: the next execution on the same device succeeds and is correct."""
    import os
    import time
    from ryft_b200.stablehlo import Builder
    b = Builder()
    x = b.arg([256, 128], "bf16"); y = b.arg([128, 256], "bf16")
    text = b.build(b.dot_general(x, y, ([], []), ([1], [0]), out_dtype="f32"))
    exe = client.compile(pjrt.Program.mlir(text))
    dev = exe.addressable_devices()[0]
    import ml_dtypes
    xs = np.ones((256, 128), np.float32).astype(ml_dtypes.bfloat16)
    ys = np.ones((128, 256), np.float32).astype(ml_dtypes.bfloat16)
    bufs = [client.buffer(xs, device=dev), client.buffer(ys, device=dev)]
    os.environ["B2X_DEBUG_WITHHOLD_ARRIVE"] = "1"
    try:
        t0 = time.perf_counter()
        outs = exe.execute([pjrt.ExecutionDeviceInputs(bufs)])
    finally:
        del os.environ["B2X_DEBUG_WITHHOLD_ARRIVE"]
    with pytest.raises(pjrt.PjrtError) as e:
        outs[0].done.await_()
    waited = time.perf_counter() - t0
    assert e.value.code_name == "DEADLINE_EXCEEDED" and "gave up waiting" in e.value.message
    assert waited < 20.0, f"the kernel took {waited:.1f} s to give up"
    ok = exe.execute([pjrt.ExecutionDeviceInputs(bufs)])
    ok[0].done.await_()
    assert np.array_equal(ok[0].outputs[0].to_numpy(), np.full((256, 256), 128.0, np.float32))


def test_error_buffer_propagates(client):
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM))
    a = client.buffer(np.ones((2, 1), np.int32))
    err = client.error_buffer(13, "upstream computation failed", pjrt.BufferType.S32, [2, 1])
    with pytest.raises(pjrt.PjrtError) as e:
        exe.execute([pjrt.ExecutionDeviceInputs([a, err])])
    assert e.value.code_name == "INTERNAL" and "upstream" in e.value.message


def test_completion_callback_runs_off_thread(client):
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM))
    a = client.buffer(np.ones((2, 1), np.int32))
    outs = exe.execute([pjrt.ExecutionDeviceInputs([a, a])])
    hit = threading.Event()
    seen = []
    outs[0].done.on_ready(lambda err: (seen.append(err), hit.set()))
    assert hit.wait(10)
    assert seen == [None]


def test_all_reduce_over_a_single_replica_is_identity(client):
    text = """
module {
  func.func @main(%arg0: tensor<8xf32>) -> tensor<8xf32> {
    %0 = "stablehlo.all_reduce"(%arg0) <{replica_groups = dense<[[0]]> : tensor<1x1xi64>}> ({
    ^bb0(%a: tensor<f32>, %b: tensor<f32>):
      %s = stablehlo.add %a, %b : tensor<f32>
      stablehlo.return %s : tensor<f32>
    }) : (tensor<8xf32>) -> tensor<8xf32>
    %1 = stablehlo.add %0, %0 : tensor<8xf32>
    return %1 : tensor<8xf32>
  }
}
"""
    x = np.arange(8, dtype=np.float32)
    exe = client.compile(pjrt.Program.mlir(text))
    out = exe.execute([pjrt.ExecutionDeviceInputs([client.buffer(x)])])[0].outputs[0].to_numpy()
    assert np.array_equal(out, 2 * x)


def test_step_timing_extension_records_steps_and_replays_the_last_execution(client):
    """The plugin's private step-timing extension: per-step device times of recorded executions, and `replay`, which
    enqueues the plan again with the last recorded execution's buffers (the results must come out the same)."""
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM), pjrt.CompilationOptions())
    device = exe.addressable_devices()[0]
    lhs = client.buffer(np.array([7, -1], np.int32).tobytes(), pjrt.BufferType.S32, [2, 1], device)
    rhs = client.buffer(np.array([35, -41], np.int32).tobytes(), pjrt.BufferType.S32, [2, 1], device)
    with pytest.raises(pjrt.PjrtError, match="replay needs an execution"):
        exe.replay(2)
    exe.step_timing(enable=1)
    outs = exe.execute([pjrt.ExecutionDeviceInputs([lhs, rhs])])
    outs[0].done.await_()
    steps = exe.step_timing(enable=0, collect=True)
    assert len(steps) == 1 and steps[0]["label"].startswith("elementwise") and steps[0]["executions"] == 1 and steps[0]["ms"] > 0
    assert steps[0]["kernel_launches"] == 1
    ms = exe.replay(5)
    assert 0 < ms < 100
    assert outs[0].outputs[0].copy_to_host().await_() == np.array([42, -42], np.int32).tobytes()


def test_layouts_extension_on_executables_and_buffers(client):
    """crates/ryft-pjrt/src/extensions/layouts.rs:944-990: both inputs and the output of the i32 add program have
    layout "{1,0}"; a buffer reports the same layout as the client's default for its shape."""
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM))
    e = exe.executable()
    ins, outs = e.input_layouts(), e.output_layouts()
    assert [str(l) for l in ins] == ["{1,0}", "{1,0}"]
    assert len(outs) == e.num_outputs() and [str(l) for l in outs] == ["{1,0}"]
    buf = client.buffer(np.zeros((2, 3, 4), dtype=np.float32))
    assert buf.layout() == client.default_layout(pjrt.BufferType.F32, [2, 3, 4]) and str(buf.layout()) == "{2,1,0}"


def test_memory_descriptions_extension(client):
    """crates/ryft-pjrt/src/extensions/memory_descriptions.rs:297-318: every memory description has a non-empty kind
    and a non-zero kind id; the default one is among them and matches the device's default memory."""
    dev = client.addressable_devices()[0]
    descs, default = dev.memory_descriptions()
    assert descs and all(kind and kind_id != 0 for kind, kind_id in descs)
    assert 0 <= default < len(descs) and descs[default][0] == "device"


def test_abi_version_extension_on_client_and_executable(client):
    """crates/ryft-pjrt/src/extensions/abi_version.rs:51-83: the client's runtime ABI version accepts the ABI version
    of an executable it compiled, both carry the plugin's platform id, and both survive a serialize / deserialize
    round trip; an executable deserialized from its serialized form reports the same version."""
    runtime = client.abi_version()
    exe = client.compile(pjrt.Program.mlir(ADD_PROGRAM))
    executable = exe.executable().abi_version()
    assert runtime.platform_id() == executable.platform_id() != 0
    runtime.is_compatible_with_runtime(client.abi_version())
    runtime.is_compatible_with_executable(executable)
    assert pjrt.RuntimeAbiVersion.deserialize(client.api, runtime.serialize()) == runtime
    assert pjrt.ExecutableAbiVersion.deserialize(client.api, executable.serialize()) == executable
    assert runtime.proto()["platform"] == runtime.platform_id() and runtime.proto()["version"]
    reloaded = client.deserialize_and_load(exe.executable().serialize())
    assert reloaded.executable().abi_version() == executable


def test_host_to_device_transfer_manager(client):
    """crates/ryft-pjrt/src/transfers.rs:1008-1073: chunked transfers, a failed transfer, and mixed data / literal
    transfers through `PJRT_Client_CreateBuffersForAsyncHostToDevice`."""
    device = client.addressable_devices()[0]
    spec = (pjrt.BufferType.U8, [8])

    # a successful transfer in two chunks
    manager = client.host_to_device_transfer_manager([spec], device)
    assert manager.device().id == device.id and manager.buffer_count() == 1 and manager.buffer_on_device_size_in_bytes(0) == 8
    manager.transfer_data(0, bytes([1, 3, 5, 7]), 0, False)
    manager.transfer_data(0, bytes([9, 11, 13, 15]), 4, True).await_()
    manager.add_metadata({"4": "2"})
    buffer = manager.retrieve_buffer(0)
    buffer.ready().await_()
    assert buffer.copy_to_host().await_() == bytes([1, 3, 5, 7, 9, 11, 13, 15])

    # the buffer may be retrieved, and its ready event asked for, before the last chunk is sent
    manager = client.host_to_device_transfer_manager([spec], device)
    early = manager.retrieve_buffer(0)
    ready = early.ready()
    assert not ready.ready()
    manager.transfer_data(0, bytes(range(8)), 0, True).await_()
    ready.await_()
    assert early.copy_to_host().await_() == bytes(range(8))
    with pytest.raises(pjrt.PjrtError):
        manager.retrieve_buffer(0)                      # only once
    with pytest.raises(pjrt.PjrtError):
        manager.transfer_data(0, bytes(8), 0, True)     # the buffer is complete
    with pytest.raises(pjrt.PjrtError):
        manager.buffer_on_device_size_in_bytes(1)       # out of range

    # a failed transfer
    manager = client.host_to_device_transfer_manager([spec], device)
    manager.transfer_data(0, bytes([1, 3, 5, 7]), 0, False)
    manager.set_error(0, 10, "test error")              # ABORTED
    buffer = manager.retrieve_buffer(0)
    with pytest.raises(pjrt.PjrtError) as e:
        buffer.ready().await_()
    assert e.value.code == 10 and "test error" in str(e.value)

    # data and literal transfers mixed; a second literal for a complete buffer is refused
    manager = client.host_to_device_transfer_manager([spec, spec], device)
    assert manager.buffer_count() == 2 and manager.buffer_on_device_size_in_bytes(1) == 8
    manager.transfer_data(0, bytes(range(1, 9)), 0, True).await_()
    manager.transfer_literal(1, bytes(range(20, 28)), *spec).await_()
    with pytest.raises(pjrt.PjrtError):
        manager.transfer_literal(1, bytes(range(30, 38)), *spec)
    b0, b1 = manager.retrieve_buffer(0), manager.retrieve_buffer(1)
    b0.ready().await_(); b1.ready().await_()
    assert b0.copy_to_host().await_() == bytes(range(1, 9)) and b1.copy_to_host().await_() == bytes(range(20, 28))
    with pytest.raises(pjrt.PjrtError):
        manager.transfer_literal(0, bytes(4), pjrt.BufferType.U8, [4])      # wrong shape

    # a manager destroyed before a buffer's last transfer leaves an error buffer behind, not a waiter
    manager = client.host_to_device_transfer_manager([spec], device)
    orphan = manager.retrieve_buffer(0)
    manager.close()
    with pytest.raises(pjrt.PjrtError):
        orphan.ready().await_()
