#!/usr/bin/env python
"""Benchmark of the StableHLO hot path through the PJRT C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config c5|c4|c2|c3|c1]

Own arm.  A step is one execution of the data-parallel gradient program (config 5 of BASELINE.json: the MLP forward +
hand-written backward of config 4 on an 8192-token shard per replica, then stablehlo.all_reduce over the f32
gradients and a divide by the replica count) on synthetic seeded inputs.  One process per GPU (torchrun for N > 1):
every rank creates a PJRT client over its GPU with `node_id`/`num_nodes`, and the plugin's NCCL communicator is
bootstrapped through the PJRT key-value callbacks backed by the torch.distributed store.  `value` is whole-job TFLOP/s
(algorithmic GEMM flops of all replicas / max-over-ranks device time, inputs resident in HBM, CUDA events on the
plugin's compute stream).  `e2e` runs the same step through the same API from pinned host memory: the activations are
copied host->device and the loss device->host inside the timed region.

Parity.  What was timed is also checked: the gradients and the loss of the last timed step against the CPU oracle at
full size (rank 0), and for N > 1 the all-reduced gradients against an independent all-reduce of the per-rank gradients,
bit-identity of the results across ranks, and a small pre-flight data-parallel step against the oracle.  The outcome is
the `parity` object of the JSON line; a failed check makes the process exit non-zero after printing the line.

Reference arm (--impl reference).  The reference executes these programs in OpenXLA's CPU plugin, which cannot be built
here, so this arm times the CPU oracle (oracle/stablehlo_eval.py, a NumPy restatement; BLAS on all host cores) on a
bounded token sample of the same program.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
import zlib
from pathlib import Path

# The CPU legs (oracle check, CPU baseline, reference arm) run on rank 0 and should use every host core; a multi-process
# launcher exports OMP_NUM_THREADS=1, which must not leak into them.
if os.environ.get("RANK", "0") == "0":
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

T_FULL, D_FULL, F_FULL = 8192, 4096, 16384
METRIC = "DP step TFLOP/s (dot_general GEMM flops of the config-4 gradient step, all replicas)"


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def _dist():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def _max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _barrier(world: int):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def program_for(config: str, n_replicas: int):
    from ryft_b200 import configs
    if config in ("c5", "c4"):
        text = configs.c4_program(T_FULL, D_FULL, F_FULL, replicas=n_replicas if config == "c5" else 0)
        flops = configs.C4_GEMM_FLOPS(T_FULL, D_FULL, F_FULL)
        return text, flops
    if config == "c2":
        return configs.c2_program(), 2.0 * 32 * 2048 * 128 * 2048
    if config == "c3":
        return configs.c3_program(), 2.0 * 4 * 32 * 128 * 4096 * 4097
    if config == "c1":
        return configs.c1_program(), 2.0 * 512 * 768 * 512
    if config == "ew":
        return configs.ew_program(), 2.0 * 32 * 2048 * 2048        # counted as 2 flops per element; the metric that matters is GB/s
    if config == "red":
        return configs.red_program(), 2.0 * 8192 * 4096
    raise SystemExit(f"unknown config {config}")


def inputs_for(config: str, replica: int):
    from ryft_b200 import configs
    if config == "c5":
        return configs.c4_inputs(T_FULL, D_FULL, F_FULL, seed=4, replica=replica)
    if config == "c4":
        return configs.c4_inputs(T_FULL, D_FULL, F_FULL)
    return {"c2": configs.c2_inputs, "c3": configs.c3_inputs, "c1": configs.c1_inputs, "ew": configs.ew_inputs, "red": configs.red_inputs}[config]()


# DRAM traffic of the dominant kernel per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of that
# kernel on this workload (a profiler cannot run inside a timed bench, so the measured figures are recorded here and must
# be re-measured when the kernel changes).  For c5/c4 it is the mean over the five GEMM launches of one step.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {
    "c5": 1.20e9,      # (1.43 + 1.14 + 1.17 + 1.19 + 1.05) GB / 5
    "c4": 1.20e9,
    "c2": 249.0e6,
    "c3": 519.1e6,     # k_attention_pw: 403.1 MB read + 115.9 MB written
    "ew": 771.0e6,
    "red": 138.7e6,    # 134.3 MB read + 4.4 MB written
}


def time_device(client, exe, bufs, steps: int, warmup: int, world: int, stream_handle: int, local: int):
    """W untimed + K timed executions; CUDA events on the plugin's compute stream; returns (ms_total, step timings)."""
    import torch
    from ryft_b200 import pjrt
    s = torch.cuda.ExternalStream(stream_handle, device=local)
    last = None
    for _ in range(warmup):
        last = exe.execute([pjrt.ExecutionDeviceInputs(bufs)])
    if last:
        last[0].done.await_()
    _barrier(world)
    exe.step_timing(enable=1)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(s)
    for _ in range(steps):
        last = exe.execute([pjrt.ExecutionDeviceInputs(bufs)])
    # a step ends when its last output exists (a trailing all-reduce runs on the communication stream)
    for out in last[0].outputs:
        out.wait_until_ready_on_stream(stream_handle)
    t1.record(s)
    last[0].done.await_()
    t1.synchronize()
    _barrier(world)
    ms = float(t0.elapsed_time(t1))
    timings = exe.step_timing(enable=0, collect=True)
    return ms, timings, last


def replay_ms_per_execution(exe, last, times: int):
    """Device milliseconds of one execution when the plan is enqueued `times` more times back to back by the plugin itself
    (step-timing extension, `replay`): the kernels' own duration, without the tens of microseconds of host work that a
    PJRT execution costs between launches.  `last` keeps the replayed execution's output buffers alive.  None for plans
    with collectives."""
    from ryft_b200 import pjrt
    try:
        exe.replay(3)
        return exe.replay(times) / times
    except pjrt.PjrtError:
        return None
    finally:
        del last



PARITY_TOL = 1e-4          # relative Frobenius error of f32 results, relative error of the scalar loss
# dW1 sits behind three bf16 roundings (H/A, dY, dH), each of which turns a relative difference d of its input into about
# sqrt(d * 2^-8): two CPU evaluations of the oracle that differ only in how the contractions accumulate (float32 BLAS
# against float64) are 4.5e-4 apart on dW1 (1e-5 on dW2, 0 on the loss), and the truncating accumulation of the tensor
# cores (a relative shift of -1e-9 * K per GEMM) puts this build at 1.1e-3.  Every single GEMM of the step meets 1e-4
# when it is fed the oracle's inputs (tests/test_parity_gpu.py checks that at full size).
PARITY_TOL_DW1_CHAIN = 3e-3


def _rel_fro(a: np.ndarray, e: np.ndarray) -> float:
    """Relative Frobenius error, accumulated blockwise in float64 so that 64 M-element gradients need no f64 copy."""
    a, e = a.reshape(-1), e.reshape(-1)
    num = den = 0.0
    step = 1 << 24
    for i in range(0, e.size, step):
        x = e[i:i + step].astype(np.float64)
        d = a[i:i + step].astype(np.float64) - x
        num += float(d @ d); den += float(x @ x)
    return float(np.sqrt(num / den)) if den > 0 else float(np.sqrt(num))


def _run_to_numpy(exe, bufs):
    from ryft_b200 import pjrt
    outs = exe.execute([pjrt.ExecutionDeviceInputs(bufs)])
    outs[0].done.await_()
    return [o.to_numpy() for o in outs[0].outputs]


def parity_check(client, dev, exe, bufs, host_inputs, n_rep: int, rank: int, world: int) -> tuple:
    """Checks the results of the timed program.  Returns (parity dict, cpu seconds of the full-size oracle run or None).

    N = 1: the step's dW1, dW2 and loss against the CPU oracle on the same inputs at full size.
    N > 1: (a) a small data-parallel step (same program text, reduced sizes) on all ranks against the oracle evaluating all
    replicas, (b) the full-size all-reduced gradients against torch.distributed's all-reduce of the per-rank gradients
    (computed by the same program without the collective), (c) bit-identity of the all-reduced results across ranks, and
    (d) rank 0's per-rank gradients and loss against the oracle at full size."""
    import torch
    from oracle import stablehlo_eval as ev
    from ryft_b200 import configs, pjrt
    res = {"checked": True, "tolerance": PARITY_TOL}
    rels = []
    got = _run_to_numpy(exe, bufs)                       # dW1, dW2 (all-reduced and divided when N > 1), loss
    local = got
    if world > 1:
        import torch.distributed as dist
        # (a) pre-flight: small sizes, every rank its own shard, oracle over all replicas on rank 0
        t, d, f = 256, 128, 384
        small = client.compile(pjrt.Program.mlir(configs.c4_program(t, d, f, replicas=n_rep)), pjrt.CompilationOptions(replica_count=n_rep))
        sm_in = configs.c4_inputs(t, d, f, seed=4, replica=rank)
        sm_got = _run_to_numpy(small, [client.buffer(x, device=dev) for x in sm_in])
        if rank == 0:
            want = ev.evaluate(configs.c4_program(t, d, f, replicas=n_rep), [configs.c4_inputs(t, d, f, seed=4, replica=r) for r in range(n_rep)])[0]
            res["preflight_dw1_rel"] = _rel_fro(sm_got[0], want[0])     # behind the chain of bf16 roundings, like the full-size dW1
            res["preflight_dw2_rel"] = _rel_fro(sm_got[1], want[1])
            res["preflight_loss_rel"] = abs(float(sm_got[2]) - float(want[2])) / abs(float(want[2]))
            rels += [res["preflight_dw2_rel"], res["preflight_loss_rel"]]
        # (b) full size: the plugin's all-reduce against an independent one over the per-rank gradients
        exe_local = client.compile(pjrt.Program.mlir(configs.c4_program(T_FULL, D_FULL, F_FULL)))
        local = _run_to_numpy(exe_local, bufs)
        worst = 0.0
        for k in (0, 1):
            ref = torch.from_numpy(local[k]).cuda()
            dist.all_reduce(ref)
            ref /= world
            worst = max(worst, _rel_fro(got[k], ref.cpu().numpy()))
            del ref
        res["allreduce_vs_independent_rel"] = _max_over_ranks(worst, world)
        rels.append(res["allreduce_vs_independent_rel"])
        # (c) every rank must hold the same bits
        sums = [zlib.crc32(memoryview(np.ascontiguousarray(got[k])).cast("B")) for k in (0, 1)] + \
               [zlib.crc32(memoryview(np.ascontiguousarray(sm_got[k])).cast("B")) for k in (0, 1)]
        all_sums = [None] * world
        dist.all_gather_object(all_sums, sums)
        res["ranks_identical"] = all(s == all_sums[0] for s in all_sums)
    oracle_s = None
    if rank == 0:
        # (d) / N = 1: full-size oracle on this rank's inputs (f32 BLAS accumulation on all host threads)
        threads = ev.use_all_host_threads()
        text = configs.c4_program(T_FULL, D_FULL, F_FULL)
        t0 = time.perf_counter()
        want = ev.evaluate(text, [host_inputs], fast_dot=True)[0]
        oracle_s = time.perf_counter() - t0
        res["dw1_rel_frobenius"] = _rel_fro(local[0], want[0])
        res["dw2_rel_frobenius"] = _rel_fro(local[1], want[1])
        res["loss"] = float(local[2]); res["loss_oracle"] = float(want[2])
        res["loss_rel"] = abs(float(local[2]) - float(want[2])) / abs(float(want[2]))
        res["oracle_seconds"] = oracle_s; res["oracle_threads"] = threads
        tight = rels + [res["dw2_rel_frobenius"], res["loss_rel"]]
        res["max_rel"] = max(tight + [res["dw1_rel_frobenius"]])
        res["tolerance_dw1_behind_three_bf16_roundings"] = PARITY_TOL_DW1_CHAIN
        res["ok"] = bool(max(tight) <= PARITY_TOL and res["dw1_rel_frobenius"] <= PARITY_TOL_DW1_CHAIN and
                         res.get("preflight_dw1_rel", 0.0) <= PARITY_TOL_DW1_CHAIN and res.get("ranks_identical", True))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    return res, oracle_s


def run_own(args) -> dict:
    import torch
    from ryft_b200 import configs, pjrt
    rank, world, local = _dist()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    torch.cuda.set_device(local)
    kv = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        # rank 0 spends tens of seconds in the CPU oracle while the others wait at a barrier; five minutes bound a lost peer
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
        from torch.distributed.distributed_c10d import _get_default_store
        kv = pjrt.TorchStoreKeyValueStore(torch.distributed.PrefixStore("b2x", _get_default_store()))
    plugin = pjrt.load_cuda_13_plugin()
    client = plugin.client({"visible_devices": [local], "node_id": rank, "num_nodes": world}, kv_store=kv)
    config = args.config
    n_rep = world if config == "c5" else 1
    text, flops_per_replica = program_for(config, n_rep)
    exe = client.compile(pjrt.Program.mlir(text), pjrt.CompilationOptions(replica_count=n_rep))
    dev = exe.addressable_devices()[0]
    stream = dev.compute_stream()
    host_inputs = inputs_for(config, rank)
    bufs = [client.buffer(x, device=dev) for x in host_inputs]
    launches_per_exec = int(exe.executable().cost_analysis()["kernel launches"])

    sampler = ClockSampler(local)
    sampler.start()
    ms, timings, last = time_device(client, exe, bufs, args.steps, args.warmup, world, stream, local)
    # single-kernel plans are shorter than the host work of an execution: their kernel is timed by back-to-back replays
    replay_ms = replay_ms_per_execution(exe, last, max(args.steps, 20)) if world == 1 and len(timings) == 1 else None
    clocks = sampler.stop()
    ms = _max_over_ranks(ms, world)
    total_flops = flops_per_replica * n_rep * args.steps
    value = total_flops / (ms * 1e-3) / 1e12

    # ---- end to end: activations from pinned host memory each step, loss read back each step ----
    e2e = None
    if config in ("c5", "c4"):
        x = host_inputs[0]
        pinned = torch.empty(x.size, dtype=torch.uint16).pin_memory()
        pinned.numpy()[:] = x.reshape(-1).view(np.uint16)
        loss_host = np.zeros(4, dtype=np.uint8)
        e2e_steps = max(3, min(args.steps, 20))

        def upload():
            # asynchronous copy from pinned host memory on the plugin's transfer stream (ImmutableUntilTransferCompletes)
            return client.buffer(pinned.data_ptr(), pjrt.BufferType.BF16, list(x.shape), device=dev, semantics=1)

        host = {"upload": 0.0, "execute": 0.0, "readback": 0.0, "wait": 0.0}
        upload_each = []   # host milliseconds of every upload call of the timed loop (a slow one = the pool had to grow)

        def run_steps(n):
            # the input pipeline of a training loop: step i+1's tokens are uploaded while step i computes, and with
            # --e2e-depth 2 step i+1 is also enqueued before the host waits for loss i.  Every step uploads its own 64 MiB
            # of tokens and has its own loss read back inside the timed region.  Host time is split by stage: what the
            # enqueue calls cost (upload, execute, readback) and how long the host then sat waiting for the device.
            for k in host:
                host[k] = 0.0
            del upload_each[:]
            c = time.perf_counter
            xb = upload()
            pending = None
            hosts = [np.zeros(4, dtype=np.uint8), np.zeros(4, dtype=np.uint8)]
            for i in range(n):
                t0 = c()
                outs = exe.execute([pjrt.ExecutionDeviceInputs([xb, bufs[1], bufs[2]])])
                t1 = c()
                if i + 1 < n:
                    xb = upload()
                t2 = c()
                ev = outs[0].outputs[2].copy_to_host(hosts[i & 1])
                t3 = c()
                if args.e2e_depth <= 1:
                    ev.await_()
                else:
                    if pending is not None:
                        pending.await_()
                    pending = ev
                t4 = c()
                host["execute"] += t1 - t0; host["upload"] += t2 - t1; host["readback"] += t3 - t2; host["wait"] += t4 - t3
                upload_each.append(round((t2 - t1) * 1e3, 3))
            if pending is not None:
                pending.await_()
            loss_host[:] = hosts[(n - 1) & 1]
        # enough untimed steps for the stream-ordered memory pool to hold every token buffer the pipelined loop keeps alive
        run_steps(max(args.warmup, 4))
        # the upload alone, for reading the end-to-end figure: when it takes longer than a step, the host link bounds e2e
        t_up = time.perf_counter()
        upload().ready().await_()
        h2d_ms = (time.perf_counter() - t_up) * 1e3
        _barrier(world)
        w0 = time.perf_counter()
        run_steps(e2e_steps)
        _barrier(world)
        wall = _max_over_ranks(time.perf_counter() - w0, world)
        e2e = {"value": flops_per_replica * n_rep * e2e_steps / wall / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(x.nbytes) * n_rep,
               "d2h_bytes_per_step": 4 * n_rep, "ms_per_step": wall / e2e_steps * 1e3, "loss": float(loss_host.view(np.float32)[0]),
               "h2d_alone_ms": h2d_ms, "h2d_alone_gb_per_s": x.nbytes / (h2d_ms * 1e-3) / 1e9,
               "host_ms_per_step": {k: v / e2e_steps * 1e3 for k, v in host.items()}, "upload_call_ms_each": list(upload_each),
               "results_left_on_device": "dW1 and dW2 (512 MiB of f32 gradients) stay in HBM for the optimiser; only the loss is read back"}

    # ---- roofline of the dominant kernel (tcgen05 GEMM) from the per-step CUDA events of the timed region ----
    peaks = _peaks()
    gemm_ms = sum(t["ms"] for t in timings if t["label"].startswith("gemm_tc"))
    gemm_flops = sum(t["flops"] for t in timings if t["label"].startswith("gemm_tc")) * args.steps
    gemm_launches = sum(1 for t in timings if t["label"].startswith("gemm_tc")) * args.steps
    roofline = None
    if gemm_ms > 0:
        achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "k_gemm_tc (tcgen05, 128xBN tiles)", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                    "peak_source": f"{peaks['source']} (sustained cuBLAS bf16)", "avg_launch_ms": gemm_ms / max(gemm_launches, 1)}
    hbm_cfg = {"ew": (32 * 2048 * 2048 * 6.0 + 8192, "elementwise", "k_elementwise (fused add + tanh + convert)"),
               "red": (8192 * 4096 * 4.0, "reduce", "k_reduce_rows_direct (sum of squares, partial sums folded and scaled in the same launch)")}
    if config in hbm_cfg:
        algo_bytes, prefix, kname = hbm_cfg[config]
        k_ms = sum(t["ms"] for t in timings if t["label"].startswith(prefix) and t["bytes"] > 1e6) / args.steps
        if replay_ms:
            k_ms = replay_ms
        if k_ms > 0:
            gbs = algo_bytes / (k_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": kname, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                        "traffic": None, "peak_source": peaks["source"], "avg_launch_ms": k_ms}
    if config == "c3":
        a_ms = sum(t["ms"] for t in timings if t["label"].startswith("attention")) / args.steps
        if replay_ms:
            a_ms = replay_ms
        if a_ms > 0:
            achieved = flops_per_replica / (a_ms * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": "k_attention_pw (tcgen05, online softmax, two workers per SM)", "achieved": achieved,
                        "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops_sustained"], "traffic": None,
                        "peak_source": f"{peaks['source']} (sustained cuBLAS bf16)", "avg_launch_ms": a_ms}
    if config == "c2" and gemm_ms > 0:
        algo_bytes = 301_998_080.0
        k_ms = replay_ms if replay_ms else gemm_ms / max(gemm_launches, 1)
        gbs = algo_bytes / (k_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "k_gemm_tc + fused bias/tanh/convert epilogue", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"], "avg_launch_ms": k_ms}

    if roofline is not None:
        roofline["traffic"] = NCU_TRAFFIC_BYTES_PER_LAUNCH.get(config)
        roofline["timing"] = ("launches enqueued back to back by the plugin (step-timing extension, replay), one pair of CUDA events around all of them"
                              if replay_ms and config in ("ew", "red", "c2", "c3") else "CUDA events around every launch of the timed region")
        if replay_ms:
            roofline["replayed_ms_per_execution"] = replay_ms
            roofline["replay_host_ms_per_execution"] = getattr(exe, "last_replay_host_ms", 0.0) / max(args.steps, 20)
    line = {
        "metric": METRIC if config in ("c5", "c4") else f"{config} TFLOP/s",
        "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "steps_per_s": args.steps / (ms * 1e-3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 operands, f32 accumulate", "data": "synthetic (seeded N(0,1) activations, N(0,0.02) weights)",
        "config": config_for(config, n_rep),
        "gpu_launches": launches_per_exec * args.steps, "clocks": clocks,
        "steps_breakdown": [{"label": t["label"], "ms_per_step": t["ms"] / max(t["executions"], 1)} for t in timings],
    }
    if e2e:
        line["e2e"] = e2e
    if roofline:
        line["roofline"] = roofline
    if config == "c5" and world > 1:
        line["collectives"] = collective_figures(client, dev, timings, world, stream, local)
    parity, oracle_s = None, None
    if config == "c5" and not args.no_parity:
        parity, oracle_s = parity_check(client, dev, exe, bufs, host_inputs, n_rep, rank, world)
        line["parity"] = parity
    elif config == "c5":
        line["parity"] = {"checked": False, "why": "--no-parity"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        if oracle_s:
            # the oracle run of the parity check is the CPU baseline: the whole step, all tokens, on the host's cores
            line["cpu_baseline"] = {"value": flops_per_replica / oracle_s / 1e12, "unit": "TFLOP/s", "cores": parity.get("oracle_threads") or os.cpu_count(),
                                    "kind": "port", "seconds": oracle_s,
                                    "sample": f"one full step (all {T_FULL} tokens, d={D_FULL}, ff={F_FULL}); NumPy oracle, f32 BLAS GEMMs on all host threads, "
                                              "elementwise ops single-threaded"}
        else:
            line["cpu_baseline"] = cpu_baseline(config)
    if rank == 0 and world == 1 and config == "c5" and not args.no_extras:
        line["extra"] = extras(client, peaks, local)
    client.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return line if rank == 0 else None


def collective_figures(client, dev, timings, world: int, stream_handle: int, local: int) -> dict:
    """Bus bandwidth of the gradient all-reduce, 2 (n - 1) / n x bytes / time with CUDA events on the communication
    stream: inside the timed step, where it shares the GPU with the GEMMs it overlaps, and alone (a program that only
    all-reduces one 256 MiB f32 gradient)."""
    from ryft_b200 import pjrt
    from ryft_b200.stablehlo import Builder
    factor = 2.0 * (world - 1) / world
    inside = [t for t in timings if t["label"].startswith("collective")]
    out = {"bytes_per_all_reduce": D_FULL * F_FULL * 4, "ranks": world,
           "overlapped_ms": [t["ms"] / max(t["executions"], 1) for t in inside]}
    out["overlapped_bus_gbs"] = [factor * out["bytes_per_all_reduce"] / (ms * 1e-3) / 1e9 for ms in out["overlapped_ms"] if ms > 0]
    b = Builder()
    g = b.arg([D_FULL, F_FULL], "f32")
    (r,) = b.all_reduce([g], [list(range(world))])
    exe = client.compile(pjrt.Program.mlir(b.build(r)), pjrt.CompilationOptions(replica_count=world))
    buf = client.buffer(np.zeros((D_FULL, F_FULL), np.float32), device=dev)
    ms, t2, _ = time_device(client, exe, [buf], 5, 3, world, stream_handle, local)
    alone = [t["ms"] / max(t["executions"], 1) for t in t2 if t["label"].startswith("collective")]
    ms_alone = _max_over_ranks(alone[0] if alone else ms / 5, world)
    out["alone_ms"] = ms_alone
    out["alone_bus_gbs"] = factor * out["bytes_per_all_reduce"] / (ms_alone * 1e-3) / 1e9
    return out


def extras(client, peaks, local) -> dict:
    """dot_general (config 2) and attention (config 3) at full size, timed briefly on the same GPU."""
    from ryft_b200 import pjrt
    out = {}
    for cfg, steps in (("c2", 20), ("c3", 5), ("c1", 20), ("ew", 10), ("red", 20)):
        try:
            text, flops = program_for(cfg, 1)
            exe = client.compile(pjrt.Program.mlir(text))
            dev = exe.addressable_devices()[0]
            bufs = [client.buffer(x, device=dev) for x in inputs_for(cfg, 0)]
            ms, timings, last = time_device(client, exe, bufs, steps, 3, 1, dev.compute_stream(), local)
            # ms_per_step: executions issued one by one through the API (host work between launches included);
            # kernel_ms: the same plan replayed back to back by the plugin, i.e. the kernel's own duration
            kernel_ms = replay_ms_per_execution(exe, last, max(steps, 20)) if len(timings) == 1 else None
            del last
            out[cfg] = {"ms_per_step": ms / steps, "kernel_ms": kernel_ms, "tflops": flops / ((kernel_ms or ms / steps) * 1e-3) / 1e12,
                        "steps_breakdown": [{"label": t["label"], "ms_per_step": t["ms"] / max(t["executions"], 1)} for t in timings]}
            algo = {"c2": 301_998_080.0, "ew": 32 * 2048 * 2048 * 6.0 + 8192, "red": 8192 * 4096 * 4.0}.get(cfg)
            if algo:
                out[cfg]["hbm_gbs"] = algo / ((kernel_ms or ms / steps) * 1e-3) / 1e9
                out[cfg]["hbm_frac"] = out[cfg]["hbm_gbs"] / peaks["hbm_gbs"]
                out[cfg]["hbm_frac_through_api"] = algo * steps / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]
            del bufs, exe
        except Exception as e:  # report, never hide
            out[cfg] = {"error": str(e)}
    return out


def config_for(config: str, n_rep: int) -> dict:
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": {"c5": c5_workload(n_rep),
                         "c4": "config 4: MLP fwd+bwd gradient step on one GPU", "c2": "config 2: batched bf16 dot_general + bias + tanh + convert",
                         "c3": "config 3: causal attention written out in StableHLO", "c1": "config 1: f32 dot_general 512x768x512",
                         "ew": "micro: config 2's epilogue chain standalone, tanh(f32[32,2048,2048] + bias) -> bf16",
                         "red": "micro: config 4's loss reduction standalone, sum of squares of f32[8192,4096]"}[config],
            "replicas": n_rep, "parallelism": f"dp{n_rep}", "l2": "inputs (>= 320 MiB per step) exceed the 126 MB L2; no flush needed"}


def c5_workload(n_rep: int) -> str:
    return (f"config 5: MLP fwd+bwd gradient step, tokens {T_FULL} x d {D_FULL} x ff {F_FULL} per replica, all_reduce(sum) of "
            f"f32 dW1+dW2 ({2 * D_FULL * F_FULL * 4} B) over {n_rep} replica(s), divide by replica count")


def cpu_baseline(config: str, target_seconds: float = 12.0) -> dict:
    """The oracle timed on the host cores on a bounded sample of the workload: the token count is cut so that the run
    takes about `target_seconds` on this host (a 512-token probe sets the rate; the full 8192 tokens if the host is fast
    enough)."""
    from oracle import stablehlo_eval as ev
    from ryft_b200 import configs
    if config not in ("c5", "c4"):
        return {"value": None, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "sample": "not timed for this config"}

    def run(tokens: int) -> float:
        text = configs.c4_program(tokens, D_FULL, F_FULL)
        ins = configs.c4_inputs(tokens, D_FULL, F_FULL, seed=4)
        mod = ev.parse(text)
        t0 = time.perf_counter()
        ev.evaluate(mod, [ins], fast_dot=True)
        return time.perf_counter() - t0
    probe = run(512)
    tokens = int(min(T_FULL, max(512, 512 * target_seconds / max(probe, 1e-3)))) // 512 * 512
    dt = run(tokens) if tokens > 512 else probe
    flops = configs.C4_GEMM_FLOPS(tokens, D_FULL, F_FULL)
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "seconds": dt,
            "sample": f"{tokens} of {T_FULL} tokens, full d={D_FULL} ff={F_FULL}; NumPy oracle, f32 BLAS GEMMs on all host threads"}


def run_reference(args) -> dict:
    """The CPU arm: the oracle on the host's cores, every step a bounded token sample of one replica's program.  With N
    replicas the reference's CPU plugin would run them on the same host cores, so the whole-job rate on the host equals
    one replica's rate; that rate is the value."""
    rank, world, _ = _dist()
    if rank != 0:
        return None
    from oracle import stablehlo_eval as ev
    from ryft_b200 import configs
    threads = ev.use_all_host_threads()
    sample = args.ref_tokens
    text = configs.c4_program(sample, D_FULL, F_FULL)
    ins = configs.c4_inputs(sample, D_FULL, F_FULL, seed=4)
    mod = ev.parse(text)
    flops = configs.C4_GEMM_FLOPS(sample, D_FULL, F_FULL)
    for _ in range(args.warmup):
        ev.evaluate(mod, [ins], fast_dot=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ev.evaluate(mod, [ins], fast_dot=True)
    dt = time.perf_counter() - t0
    value = flops * args.steps / dt / 1e12
    n_rep = max(args.gpus, 1)
    sample_txt = (f"{sample} of {T_FULL} tokens per step, full d={D_FULL} ff={F_FULL}, one replica's program (replicas would share these cores, so the "
                  f"whole-job rate equals this rate); NumPy oracle (port of StableHLO semantics), f32 BLAS on {threads} host threads; rank 0 only")
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 operands, f32 accumulate",
            "data": "synthetic (seeded N(0,1) activations, N(0,0.02) weights)",
            "config": config_for("c5", n_rep),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample_txt},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference runs this path inside OpenXLA's CPU PJRT plugin, which cannot be built or fetched in this environment; the CPU oracle is timed instead"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--config", default="c5", choices=["c1", "c2", "c3", "c4", "c5", "ew", "red"])
    ap.add_argument("--e2e-depth", type=int, default=2, help="steps the end-to-end loop keeps in flight (1 or 2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed program (profiling runs)")
    ap.add_argument("--ref-tokens", type=int, default=2048, help="tokens per step of the CPU reference arm")
    ap.add_argument("--no-extras", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "own":
        args.warmup = 3
    # libraries (NCCL, the CUDA runtime) may print banners to stdout: keep stdout for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        line = run_reference(args) if args.impl == "reference" else run_own(args)
    except BaseException:
        # a rank that fails must not linger (threads of the plugin, communicators): the launcher ends the other ranks only
        # once this process is gone, and they may be waiting for it inside a collective
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(1)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    if line is not None:
        print(json.dumps(line), flush=True)
        if line.get("parity", {}).get("checked") and line["parity"].get("ok") is False:
            print("parity check failed: " + json.dumps(line["parity"]), file=sys.stderr)
            sys.exit(3)


if __name__ == "__main__":
    main()
