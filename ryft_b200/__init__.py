"""B200-native executor for ryft's StableHLO programs, behind the PJRT C API.

`ryft_b200.pjrt` mirrors the ryft-pjrt host surface over the plugin (`lib/libpjrt-plugin-cuda-13.so`);
`ryft_b200.stablehlo` builds program text in the forms ryft-mlir prints; `ryft_b200.configs` holds the benchmark
programs.  The native libraries are built in-tree by `python -m ryft_b200.build`; nothing here computes on the CPU.
"""
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"
PLUGIN_PATH = LIB_DIR / "libpjrt-plugin-cuda-13.so"
KERNELS_PATH = LIB_DIR / "libb2x_kernels.so"


def plan_dump(mlir_text: str, num_replicas: int = 1) -> str:
    """Compiles `mlir_text` on the host and returns the launch plan as text (no GPU needed).  Raises
    pjrt.PjrtError with the plugin's error code when the program is rejected."""
    import ctypes as C
    from .pjrt import PjrtError
    if not KERNELS_PATH.exists():
        raise FileNotFoundError(f"{KERNELS_PATH} is missing: run `python -m ryft_b200.build`")
    lib = C.CDLL(str(KERNELS_PATH))
    data = mlir_text.encode() if isinstance(mlir_text, str) else bytes(mlir_text)
    cap = 1 << 20
    out = C.create_string_buffer(cap)
    n = C.c_size_t(0)
    lib.b2x_plan_dump.argtypes = [C.c_char_p, C.c_size_t, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    code = lib.b2x_plan_dump(data, len(data), num_replicas, out, cap, C.byref(n))
    text = out.value.decode("utf-8", "replace")
    if code:
        raise PjrtError(code, text)
    return text


def plan_routes(mlir_text: str, num_replicas: int = 1) -> list:
    """For every tensor-core GEMM step of the program's launch plan, the kernel variant the launcher will pick (no GPU
    needed): a list of dicts with the problem size, tile width `bn`, the id of the build-time specialised epilogue
    (`static_id`, 0 = interpreted), `epi_groups`, `transposed`, `group_m`, tile counts, `stores`, `ctas` and `tile_rows`
    (128, or 256 for the tall tiles of long-K problems)."""
    import ctypes as C
    from .pjrt import PjrtError
    if not KERNELS_PATH.exists():
        raise FileNotFoundError(f"{KERNELS_PATH} is missing: run `python -m ryft_b200.build`")
    lib = C.CDLL(str(KERNELS_PATH))
    data = mlir_text.encode() if isinstance(mlir_text, str) else bytes(mlir_text)
    cap = 1 << 20
    out = C.create_string_buffer(cap)
    n = C.c_size_t(0)
    lib.b2x_plan_routes.argtypes = [C.c_char_p, C.c_size_t, C.c_int, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t)]
    code = lib.b2x_plan_routes(data, len(data), num_replicas, out, cap, C.byref(n))
    text = out.value.decode("utf-8", "replace")
    if code:
        raise PjrtError(code, text)
    keys = ("M", "N", "K", "batch", "bn", "static_id", "epi_groups", "transposed", "group_m", "m_tiles", "n_tiles", "k_blocks", "stores", "ctas", "tile_rows")
    rows = []
    for line in text.splitlines():
        parts = line.split("|")
        row = {"label": parts[0]}
        row.update({k: int(v) for k, v in zip(keys, parts[1:])})
        rows.append(row)
    return rows
