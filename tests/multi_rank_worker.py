"""One rank of the CPU multi-rank tests (launched by torch.distributed.run with the gloo backend).

Exercises the host side of the one-process-per-GPU configuration without a GPU: the key-value callbacks that carry the
NCCL unique id from rank 0 to the other ranks (`PJRT_Client_Create`'s kv_get / kv_put,
crates/ryft-pjrt/src/clients.rs:698-825), driven exactly as the plugin drives them (through the C function pointers),
over the same torch.distributed store `bench.py` uses.
"""
import ctypes as C
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch
import torch.distributed as dist

from ryft_b200 import pjrt


def call_put(cb: pjrt.KvCallbacks, key: bytes, value: bytes) -> None:
    a = pjrt.KvCallbacks.PUT()
    a.struct_size = C.sizeof(a)
    kb, vb = C.create_string_buffer(key, len(key)), C.create_string_buffer(value, len(value))
    a.key, a.key_size, a.value, a.value_size = C.addressof(kb), len(key), C.addressof(vb), len(value)
    err = C.CFUNCTYPE(C.c_void_p, C.c_void_p)(cb.put_ptr.value)(C.addressof(a))
    assert not err


def call_get(cb: pjrt.KvCallbacks, key: bytes, timeout_ms: int) -> bytes:
    a = pjrt.KvCallbacks.GET()
    a.struct_size = C.sizeof(a)
    kb = C.create_string_buffer(key, len(key))
    a.key, a.key_size, a.timeout_in_ms = C.addressof(kb), len(key), timeout_ms
    err = C.CFUNCTYPE(C.c_void_p, C.c_void_p)(cb.get_ptr.value)(C.addressof(a))
    assert not err
    out = C.string_at(a.value, a.value_size)
    assert len(cb.live) == 1                      # the value is kept alive for the plugin ...
    C.CFUNCTYPE(None, C.c_void_p)(a.value_deleter_callback)(a.value)
    assert len(cb.live) == 0                      # ... until it calls the deleter it was handed
    return out


def main() -> None:
    dist.init_process_group(backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from torch.distributed.distributed_c10d import _get_default_store
    store = pjrt.TorchStoreKeyValueStore(dist.PrefixStore("b2x", _get_default_store()))
    cb = pjrt.KvCallbacks(store)
    # the rendezvous the plugin performs: rank 0 publishes a 128-byte id, every other rank blocks until it is there
    ident = bytes((7 * i + 3) % 256 for i in range(128))
    if rank == 0:
        call_put(cb, b"b2x/nccl_id/0", ident)
    got = call_get(cb, b"b2x/nccl_id/0", 20000)
    assert got == ident, (rank, got[:8])
    # every rank publishes its device list, every rank reads all of them (global device ids = process * local + l)
    call_put(cb, f"b2x/devices/{rank}".encode(), bytes([rank, 1]))
    seen = [call_get(cb, f"b2x/devices/{r}".encode(), 20000) for r in range(world)]
    assert seen == [bytes([r, 1]) for r in range(world)]
    # shard bookkeeping used by bench.py: every rank draws its own tokens and the same weights
    from ryft_b200 import configs
    x0, w1, _ = configs.c4_inputs(8, 16, 32, seed=4, replica=0)
    xr, w1r, _ = configs.c4_inputs(8, 16, 32, seed=4, replica=rank)
    same_w = torch.tensor([float((w1.astype("float32") == w1r.astype("float32")).all())])
    differs = torch.tensor([float(rank == 0 or not (x0.astype("float32") == xr.astype("float32")).all())])
    dist.all_reduce(same_w, op=dist.ReduceOp.MIN)
    dist.all_reduce(differs, op=dist.ReduceOp.MIN)
    assert same_w.item() == 1.0 and differs.item() == 1.0
    dist.barrier()
    if rank == 0:
        print("MULTI_RANK_OK", world, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
