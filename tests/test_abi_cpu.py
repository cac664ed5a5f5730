"""The C-ABI boundary, checked without a GPU: the libraries load, export what include/*.h declares, the PJRT_Api
table has the reference's layout and version, and the host-only entry points (errors, events, plugin attributes)
behave as ryft-pjrt's tests expect (crates/ryft-pjrt/src/lib.rs:548-591, events.rs:566-648)."""
import ctypes as C
import re
import subprocess
import threading
from pathlib import Path

import pytest

import ryft_b200
from ryft_b200 import pjrt

ROOT = Path(__file__).resolve().parent.parent


def _exports(path):
    out = subprocess.run(["nm", "-D", "--defined-only", str(path)], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def test_libraries_exist_and_load():
    assert ryft_b200.PLUGIN_PATH.exists(), "build the native library: python -m ryft_b200.build"
    assert ryft_b200.KERNELS_PATH.exists()
    C.CDLL(str(ryft_b200.PLUGIN_PATH))
    C.CDLL(str(ryft_b200.KERNELS_PATH))


def test_plugin_exports_only_get_pjrt_api():
    # the reference's plugins export exactly this symbol (crates/ryft-xla-sys/pjrt_plugin_version_script.lds:1-7)
    assert _exports(ryft_b200.PLUGIN_PATH) == {"GetPjrtApi"}


def test_kernel_library_exports_every_declared_entry_point():
    header = (ROOT / "include" / "b2x_kernels.h").read_text()
    declared = set(re.findall(r"B2X_API\s+\w+\s+(b2x_\w+)\(", header))
    assert len(declared) >= 8
    assert declared <= _exports(ryft_b200.KERNELS_PATH)


def test_api_table_layout_and_version(plugin):
    names = pjrt.api_function_names()
    assert len(names) == 135                      # crates/ryft-pjrt/src/lib.rs:222-363
    assert names[0] == "PJRT_Error_Destroy" and names[-1] == "PJRT_Executable_ParameterMemoryKinds"
    assert plugin.version() == (0, 104)           # crates/ryft-pjrt/src/versions.rs:33-34
    assert plugin.api.struct_size == 16 + 24 + 8 * 135
    must = ["Client_Destroy", "Buffer_Destroy", "Event_Destroy", "Executable_Destroy", "LoadedExecutable_Destroy", "ExecuteContext_Destroy",
            "Error_Destroy", "Error_Message", "Error_GetCode", "Plugin_Initialize", "Client_Compile", "LoadedExecutable_Execute",
            "Client_BufferFromHostBuffer", "Buffer_ToHostBuffer", "Event_Await", "Event_OnReady"]
    for m in must:
        assert plugin.api.has(m), m
    # optional subsystems stay NULL, which ryft maps to Unimplemented (crates/ryft-pjrt/src/macros.rs:36-44)
    assert not plugin.api.has("TopologyDescription_Create")
    with pytest.raises(pjrt.PjrtError) as e:
        plugin.api.call("TopologyDescription_Create", pjrt.A["Plugin_Initialize"]())
    assert e.value.code == 12


def test_plugin_attributes(plugin):
    # crates/ryft-pjrt/src/lib.rs:575-577
    assert plugin.attribute("stablehlo_current_version") == [1, 16, 0]
    assert plugin.attribute("stablehlo_minimum_version") == [0, 9, 0]
    assert plugin.attribute("xla_version") == 2
    with pytest.raises(pjrt.PjrtError) as e:
        plugin.attribute("__missing__")
    assert e.value.code == 5 and "__missing__" in e.value.message


def test_load_plugin_is_cached():
    assert pjrt.load_plugin(ryft_b200.PLUGIN_PATH) is pjrt.load_plugin(ryft_b200.PLUGIN_PATH)


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        pjrt.Plugin(tmp_path / "libpjrt-plugin-cuda-13.so")


def test_event_set_await_on_ready(plugin):
    # crates/ryft-pjrt/src/events.rs:566-648
    ev = pjrt.Event.create(plugin.api)
    assert not ev.ready()
    seen = []
    ev.on_ready(lambda err: seen.append(("before", err)))
    ev.set()
    assert ev.ready() and ev.error() is None
    ev.on_ready(lambda err: seen.append(("after", err)))
    assert seen == [("before", None), ("after", None)]
    ev.await_()
    with pytest.raises(pjrt.PjrtError):
        ev.set()                                   # an event can be set only once


def test_event_error_propagates_code_and_message(plugin):
    ev = pjrt.Event.create(plugin.api)
    got = []
    ev.on_ready(lambda err: got.append(err))
    ev.set(10, "replica 1 never joined")
    assert got[0].code == 10 and got[0].message == "replica 1 never joined"
    err = ev.error()
    assert err.code == 10
    with pytest.raises(pjrt.PjrtError) as e:
        ev.await_()
    assert e.value.code_name == "ABORTED"


def test_event_await_from_another_thread(plugin):
    ev = pjrt.Event.create(plugin.api)
    t = threading.Timer(0.05, ev.set)
    t.start()
    ev.await_()
    t.join()
    assert ev.ready()


def test_compile_options_wire_format():
    # field numbers of crates/ryft-xla-sys/src/protos.rs:3298-3346, 2391-2417, 2340-2354
    lib = C.CDLL(str(ryft_b200.KERNELS_PATH))
    lib.b2x_debug_parse_compile_options.argtypes = [C.c_char_p, C.c_size_t, C.POINTER(C.c_int64), C.c_size_t]
    out = (C.c_int64 * 16)()
    blob = pjrt.CompilationOptions(replica_count=4, partition_count=1, device_assignment=[3, 2, 1, 0], precision=2).encode()
    assert lib.b2x_debug_parse_compile_options(blob, len(blob), out, 16) == 0
    assert list(out[:5]) == [4, 1, -1, 2, 4] and list(out[5:9]) == [3, 2, 1, 0]
    blob = pjrt.CompilationOptions().encode()
    assert lib.b2x_debug_parse_compile_options(blob, len(blob), out, 16) == 0
    assert list(out[:5]) == [1, 1, -1, 0, 0]
    assert lib.b2x_debug_parse_compile_options(b"\x1a\x7f", 2, out, 16) == 3   # truncated message is rejected


def test_client_create_without_gpu_fails_without_fallback(plugin):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(pjrt.PjrtError) as e:
        plugin.client()
    assert e.value.code_name == "FAILED_PRECONDITION" and "no CPU execution path" in e.value.message


def test_layouts_extension_default_layout_and_serialization(plugin):
    """crates/ryft-pjrt/src/extensions/layouts.rs:829-841: the default layout of an f32 [2,3,4] buffer renders as
    "{2,1,0}".  The extension answers from the dimensions alone, so this runs without a device."""
    import ctypes as C
    api = plugin.api
    ext = api.extension(pjrt.EXTENSION_TYPE_LAYOUTS)
    assert ext, "layouts extension missing from the extension chain"
    assert api.extension(pjrt.EXTENSION_TYPE_MEMORY_DESCRIPTIONS) and api.extension(pjrt.EXTENSION_TYPE_STREAM)
    slots = [bool(C.c_void_p.from_address(ext + 24 + 8 * i).value) for i in range(7)]
    assert slots == [True, True, True, True, False, True, True]      # no topology objects in this plugin

    class _NoClient:
        handle = None
    fake = pjrt.Client.__new__(pjrt.Client)
    fake.api, fake.handle = api, None
    layout = fake.default_layout(pjrt.BufferType.F32, [2, 3, 4])
    assert str(layout) == "{2,1,0}" and repr(layout) == "Layout[{2,1,0}]" and layout.minor_to_major() == [2, 1, 0]
    assert str(fake.default_layout(pjrt.BufferType.BF16, [5, 7])) == "{1,0}"
    assert str(fake.default_layout(pjrt.BufferType.S32, [])) == "{}"
    assert layout == fake.default_layout(pjrt.BufferType.F32, [9, 9, 9])
    with pytest.raises(pjrt.PjrtError):
        fake.default_layout(0, [1])                                   # PJRT_Buffer_Type_INVALID


def _proto(platform: int, payload: bytes) -> bytes:
    def varint(v):
        out = bytearray()
        while v >= 0x80:
            out.append((v & 0x7F) | 0x80); v >>= 7
        out.append(v)
        return bytes(out)
    return varint(1 << 3) + varint(platform) + varint((2 << 3) | 2) + varint(len(payload)) + payload


def test_abi_version_extension_round_trip_and_compatibility(plugin):
    """crates/ryft-pjrt/src/extensions/abi_version.rs:184-230, 262-324: versions deserialize from the
    `{platform, version}` message, serialize back to the same bytes, report their platform id and are checked against
    each other.  The reference has no plugin that offers the extension (abi_version.rs:776-782), so the expectations
    here are this plugin's rules: same platform and SM architecture; a runtime reads executables of its own
    serialization generation or older, and talks to runtimes of its own generation.  No device is needed."""
    import ctypes as C
    api = plugin.api
    ext = api.extension(pjrt.EXTENSION_TYPE_ABI_VERSION)
    assert ext, "ABI-version extension missing from the extension chain"
    assert all(C.c_void_p.from_address(ext + 24 + 8 * i).value for i in range(12))
    platform = 0x6232785F63756461
    current = _proto(platform, bytes([1, 100]))
    rt = pjrt.RuntimeAbiVersion.deserialize(api, current)
    assert rt.platform_id() == platform and rt.serialize() == current
    assert rt.proto() == {"platform": platform, "version": bytes([1, 100])}
    assert rt == pjrt.RuntimeAbiVersion.deserialize(api, current) and hash(rt) == hash(pjrt.RuntimeAbiVersion.deserialize(api, current))
    ex = pjrt.ExecutableAbiVersion.deserialize(api, current)
    assert ex.platform_id() == platform and ex.serialize() == current
    rt.is_compatible_with_runtime(rt)
    rt.is_compatible_with_executable(ex)
    older = pjrt.ExecutableAbiVersion.deserialize(api, _proto(platform, bytes([0, 100])))
    rt.is_compatible_with_executable(older)
    for payload, what in ((bytes([2, 100]), "generation"), (bytes([1, 90]), "SM 90")):
        with pytest.raises(pjrt.PjrtError) as e:
            rt.is_compatible_with_executable(pjrt.ExecutableAbiVersion.deserialize(api, _proto(platform, payload)))
        assert e.value.code_name == "FAILED_PRECONDITION" and what in e.value.message
    with pytest.raises(pjrt.PjrtError) as e:
        rt.is_compatible_with_runtime(pjrt.RuntimeAbiVersion.deserialize(api, _proto(platform, bytes([0, 100]))))
    assert e.value.code_name == "FAILED_PRECONDITION"
    for bad in (_proto(platform + 1, bytes([1, 100])), _proto(platform, b""), _proto(platform, bytes([1])), b"\x08", b"\x12\x05ab"):
        with pytest.raises(pjrt.PjrtError) as e:
            pjrt.RuntimeAbiVersion.deserialize(api, bad)
        assert e.value.code_name == "INVALID_ARGUMENT"
        with pytest.raises(pjrt.PjrtError):
            pjrt.ExecutableAbiVersion.deserialize(api, bad)
