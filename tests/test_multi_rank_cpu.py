"""World-size-2 tests of the one-process-per-GPU host logic, on CPU with the gloo backend."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(args, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port())] + args
    env = dict(os.environ, OMP_NUM_THREADS="4")
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_kv_callbacks_rendezvous_between_two_ranks():
    r = _torchrun([os.path.join("tests", "multi_rank_worker.py")])
    assert r.returncode == 0, r.stderr[-3000:]
    assert "MULTI_RANK_OK 2" in r.stdout


def test_reference_arm_prints_one_line_from_rank_zero_only():
    r = _torchrun(["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"])
    assert r.returncode == 0, r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["unit"] == "TFLOP/s"
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port" and line["value"] > 0
