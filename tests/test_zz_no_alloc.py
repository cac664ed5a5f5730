"""The reduction entry point for callers that cannot allocate device memory (an embedding runtime that owns the
allocator, a serving loop that cannot take an allocation stall): `b2x_launch_reduce_noalloc` keeps its partial results
in a fixed array inside the library.  It must give what `b2x_launch_reduce` gives with caller-provided scratch, call
after call, and refuse reductions whose partials do not fit.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_reduce_matches_the_scratch_variant_on_two_calls_in_a_row():
    import torch
    from ryft_b200 import kernels as K
    lib = K.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    n = 3_000_000 * 8
    splits = lib.b2x_reduce_splits(1, n, 1)
    assert splits > 1, "the case must exercise the partials buffer"
    scratch = torch.empty(splits, dtype=torch.float32, device=dev)
    out_ref = torch.zeros(1, dtype=torch.float32, device=dev)
    out_new = torch.zeros(1, dtype=torch.float32, device=dev)
    err = C.create_string_buffer(256)
    for call, seed in enumerate((1, 2)):
        g = torch.Generator(device=dev).manual_seed(seed)
        x = torch.randn(n, dtype=torch.float32, device=dev, generator=g)
        prog = K.load_tensor_program(x.data_ptr(), n)
        args = K.ReduceArgs(A=1, R=n, B=1, monoid=K.MONOID_ADD, cls=K.VM_F32, out_elem=K.EL_F32, init_elem=K.EL_F32, init_imm=0,
                            init_ptr=None, out=out_ref.data_ptr(), scratch=scratch.data_ptr(), vec=8)
        assert lib.b2x_launch_reduce(C.byref(prog), C.byref(args), stream) == 0
        args.out = out_new.data_ptr()
        args.scratch = None                              # ignored by the allocation-free entry point
        rc = lib.b2x_launch_reduce_noalloc(C.byref(prog), C.byref(args), stream, err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        ref, new = float(out_ref.item()), float(out_new.item())
        exact = float(x.double().sum().item())
        # same kernel, same split: identical bits; and both within the f32 tolerance of the parity tests
        assert new == ref, (call, new, ref)
        assert abs(new - exact) <= 1e-4 * max(1.0, float(x.double().norm().item())), (call, new, exact)


def test_noalloc_reduce_refuses_what_does_not_fit():
    import torch
    from ryft_b200 import kernels as K
    lib = K.load()
    torch.cuda.set_device(0)
    # 200 rows x 1 column block each split 3 ways fits; make a case whose partial count exceeds the built-in buffer
    A, R, B = 2, 1 << 22, 8192
    need = A * lib.b2x_reduce_splits(A, R, B) * B
    assert need > K.REDUCE_NOALLOC_MAX_PARTIALS
    prog = K.load_tensor_program(0, A * R * B)
    args = K.ReduceArgs(A=A, R=R, B=B, monoid=K.MONOID_ADD, cls=K.VM_F32, out_elem=K.EL_F32, init_elem=K.EL_F32, vec=8)
    err = C.create_string_buffer(256)
    rc = lib.b2x_launch_reduce_noalloc(C.byref(prog), C.byref(args), None, err, 256)
    assert rc != 0 and b"partial results" in err.value
