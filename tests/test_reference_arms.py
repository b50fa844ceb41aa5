"""The benchmark's reference arms for the composed configs (stock torch.distributed.pipelining + DDP / DTensor /
all_to_all_single) run end to end on gloo ranks with tiny shapes and print the benchmark's JSON line."""
import json
import math
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("config,inner,parallelism,vocab", [
    ("gpt2-pp4dp2", 2, "pp2xdp2", 512),
    ("llama13b-tp4pp2", 2, "tp2xpp2", 512),
    ("mixtral-pp2ep4", 2, "pp2xep2", 512),
])
def test_composed_reference_arm_runs_on_cpu_ranks(config, inner, parallelism, vocab):
    env = dict(os.environ, PIPPY_REF_DEVICE="cpu", PIPPY_REF_TINY="1", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "bench.py"), "--impl", "reference",
           "--config", config, "--inner", str(inner), "--gpus", "4", "--layers", "2", "--seq", "32", "--batch", "8",
           "--microbatches", "2", "--steps", "2", "--warmup", "1"]
    out = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    rec = json.loads(lines[0])
    assert "unavailable" not in rec, rec
    assert rec["impl"] == "reference" and rec["reference_system"] == "torch.distributed.pipelining"
    assert rec["config"]["name"] == config and rec["config"]["parallelism"].startswith(parallelism)
    assert rec["value"] > 0 and rec["e2e"]["value"] > 0 and rec["e2e"]["h2d_bytes_per_step"] > 0
    # two optimizer steps from a random start: the loss is still close to that of a uniform guess
    assert abs(rec["final_loss"] - math.log(vocab)) < 1.0
