"""Expert parallelism: the EP layer must reproduce the single-rank MoE layer.

CPU: two gloo ranks exercise the host exchange. GPU: 2 (and 4) ranks exercise the peer-memory
dispatch / combine kernels, in bf16 and with fp8-quantised dispatch.
"""

import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(world: int, backend: str, *extra, port: int):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "ep_worker.py"),
           backend, *extra]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    line = [l for l in p.stdout.splitlines() if l.startswith("EP_RESULT ")][-1]
    return json.loads(line[len("EP_RESULT "):])


def test_ep_host_exchange_matches_full_layer():
    res = _run(2, "gloo", port=29611)
    for r in res:
        assert max(r["errs"]) < 2e-2, r


@pytest.mark.gpu
@pytest.mark.parametrize("world,mode", [(2, "bf16"), (2, "fp8"), (2, "fp8experts"), (4, "bf16"), (2, "deepseek"),
                                        (2, "engine"), (4, "fp8experts")])
def test_ep_kernels_match_full_layer(world, mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    res = _run(world, "nccl", *([mode] if mode != "bf16" else []), port=29620 + world)
    tol = 6e-2 if mode in ("fp8", "fp8experts") else 3e-2
    for r in res:
        assert r["dropped"] == 0
        assert max(r["errs"]) < tol, r
