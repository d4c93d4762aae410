"""Failure detection without any GPU fault: host-made failures over gloo-style child processes, and a
bounded device wait that runs out and reports through the error word."""

import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, world=3, port=29840):
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "health_worker.py"), mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    res = {}
    for o in outs:
        for line in o.splitlines():
            if line.startswith("HEALTH_RESULT "):
                d = json.loads(line[len("HEALTH_RESULT "):])
                res[d["rank"]] = d
    return res, outs


def test_survivors_learn_of_a_rank_that_raised():
    res, outs = _run("raise", port=29840)
    assert res[1]["detected"][0] == "self", outs
    for r in (0, 2):
        # a survivor may first see another survivor leave; the reason chain still names the root cause
        assert res[r]["detected"] is not None and res[r]["detected"][0] in (0, 1, 2), outs
        assert "injected host failure" in res[r]["detected"][1] and res[r]["steps"] < 400


def test_survivors_notice_a_silent_rank_by_heartbeat():
    res, outs = _run("silent", port=29850)
    for r in (0, 2):
        assert res[r]["detected"] is not None, outs
        assert "no heartbeat" in res[r]["detected"][1]
    assert any(res[r]["detected"][0] == 1 for r in (0, 2)), outs


@pytest.mark.gpu
def test_bounded_device_wait_times_out_and_context_survives():
    from modular_b200 import ops
    from modular_b200._native import lib

    L = lib()
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    ok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    L.tp_wait_flag(flag, 1, 50, 777, ok)            # nothing ever sets the flag: the wait runs out after 50 ms
    torch.cuda.synchronize()
    assert int(ok) == 0 and L.read_error_flag(True) == 777
    flag[0] = 3
    L.tp_wait_flag(flag, 2, 50, 778, ok)
    torch.cuda.synchronize()
    assert int(ok) == 1 and L.read_error_flag(True) == 0
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)      # the context is still healthy
    w = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    y = ops.linear(x, w)
    assert torch.allclose(y.float(), x.float() @ w.float().t(), atol=1.0, rtol=0.05)
    ops.check_device_error()
