"""ctypes mirror of include/b2x_kernels.h: the kernel-level C ABI in libb2x_kernels.so.

Used by kernel-level tests and micro-benchmarks; device memory is supplied by the caller (any allocator: torch, a PJRT
buffer's device pointer, ...).  Raises if the library has not been built: there is no fallback."""
from __future__ import annotations

import ctypes as C

from . import KERNELS_PATH

MAX_INSTR, MAX_TENSORS, MAX_DIMS = 56, 8, 5

# opcodes / enums of csrc/kernels/vm.h
VM_LOAD, VM_SAVE, VM_STORE, VM_ADD, VM_SUB, VM_RSUB, VM_MUL = 1, 2, 3, 4, 5, 6, 7
VM_SRC_TEMP, VM_SRC_TENSOR, VM_SRC_IMM = 1, 2, 3
VM_F32, VM_S32, VM_U32 = 0, 1, 2
EL_S32, EL_U32, EL_BF16, EL_F32 = 3, 7, 10, 11
MONOID_ADD, MONOID_MUL, MONOID_MAX, MONOID_MIN = 0, 1, 2, 3
REDUCE_NOALLOC_MAX_PARTIALS = 16384


class VmInstr(C.Structure):
    _fields_ = [("op", C.c_uint8), ("src_kind", C.c_uint8), ("src_idx", C.c_uint8), ("aux", C.c_uint8), ("tc", C.c_uint8), ("rnd", C.c_uint8),
                ("pad0", C.c_uint8), ("pad1", C.c_uint8), ("imm", C.c_uint32)]


class VmTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * MAX_DIMS), ("elem", C.c_uint8), ("pad", C.c_uint8 * 7)]


class VmProgram(C.Structure):
    _fields_ = [("n_instr", C.c_int32), ("n_tensors", C.c_int32), ("n_dims", C.c_int32), ("pad", C.c_int32), ("dim", C.c_int64 * MAX_DIMS),
                ("tensors", VmTensor * MAX_TENSORS), ("code", VmInstr * MAX_INSTR)]


class ReduceArgs(C.Structure):
    _fields_ = [("A", C.c_int64), ("R", C.c_int64), ("B", C.c_int64), ("monoid", C.c_uint8), ("cls", C.c_uint8), ("out_elem", C.c_uint8),
                ("init_elem", C.c_uint8), ("init_imm", C.c_uint32), ("init_ptr", C.c_void_p), ("out", C.c_void_p), ("scratch", C.c_void_p),
                ("vec", C.c_int), ("host_post", C.c_void_p)]


def load() -> C.CDLL:
    if not KERNELS_PATH.exists():
        raise FileNotFoundError(f"{KERNELS_PATH} is missing: run `python -m ryft_b200.build`")
    lib = C.CDLL(str(KERNELS_PATH))
    lib.b2x_reduce_splits.argtypes = [C.c_int64, C.c_int64, C.c_int64]
    lib.b2x_launch_reduce.argtypes = [C.POINTER(VmProgram), C.POINTER(ReduceArgs), C.c_void_p]
    lib.b2x_launch_reduce_noalloc.argtypes = [C.POINTER(VmProgram), C.POINTER(ReduceArgs), C.c_void_p, C.c_char_p, C.c_size_t]
    lib.b2x_launch_elementwise.argtypes = [C.POINTER(VmProgram), C.c_int64, C.c_int, C.c_void_p]
    lib.b2x_kernel_launch_count.restype = C.c_int64
    return lib


def load_tensor_program(ptr: int, n_elements: int, elem: int = EL_F32, cls: int = VM_F32) -> VmProgram:
    """A one-instruction program that reads a contiguous tensor (the prologue of a plain reduction)."""
    p = VmProgram()
    p.n_instr, p.n_tensors, p.n_dims = 1, 1, 1
    p.dim[0] = n_elements
    p.tensors[0].ptr = ptr
    p.tensors[0].stride[0] = 1
    p.tensors[0].elem = elem
    p.code[0].op, p.code[0].src_kind, p.code[0].src_idx, p.code[0].tc = VM_LOAD, VM_SRC_TENSOR, 0, cls
    return p
