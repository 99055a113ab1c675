"""Data parallel over NCCL on two GPUs of one box: after three steps both ranks hold bit-identical parameters (the spread the
bench line also reports) although they started from different seeds, the parameters moved, the losses are finite and fall.
Skipped on a box with one GPU; the arithmetic of the wrapper (averaged gradients against a single-process run) is covered on
CPU ranks by test_dp_gloo.py."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_gpu_ranks_end_with_identical_parameters(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = tmp_path / "rank0.json"
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "dp_nccl_worker.py"), str(out)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    logs = []
    for p in procs:
        try:
            logs.append(p.communicate(timeout=300)[0].decode(errors="replace"))
        except subprocess.TimeoutExpired:
            p.kill()
            logs.append("timed out")
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)[-3000:]
    got = json.loads(out.read_text())
    assert got["spread"] == 0.0, got["spread"]
    assert got["moved"] > 1e-4 and got["buckets"] >= 2
    assert all(l == l and abs(l) < 1e3 for l in got["losses"]) and got["losses"][-1] < got["losses"][0]
