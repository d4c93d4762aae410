"""Child process of test_failure_detection.py (gloo, CPU): ranks step together; one rank fails on the host."""

import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    mode = sys.argv[1]          # "raise" | "silent"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, rank == 0, wait_for_workers=True)
    from modular_b200.parallel.health import PeerFailure, RankHealth

    health = RankHealth(store, rank, world, interval_s=0.05, timeout_s=1.5)
    result = {"rank": rank, "steps": 0, "detected": None}
    # start stepping only when every rank is up (a real job does this with its first collective)
    store.add("ready", 1)
    while int(store.add("ready", 0)) < world:
        time.sleep(0.01)
    try:
        with health.guard():
            for step in range(400):
                health.check()
                if rank == 1 and step == 5:
                    if mode == "raise":
                        raise RuntimeError("injected host failure")
                    health._stop.set()          # stops beating without saying goodbye
                    time.sleep(4.0)
                    os._exit(0)
                time.sleep(0.02)                # the "step" (no collective: the peers must not need one to notice)
                result["steps"] = step + 1
    except PeerFailure as e:
        result["detected"] = [e.rank, e.reason]
    except RuntimeError as e:
        result["detected"] = ["self", str(e)]
    print("HEALTH_RESULT " + json.dumps(result), flush=True)
    time.sleep(0.3 if rank else 1.0)            # rank 0 hosts the store: let the others finish reading


if __name__ == "__main__":
    main()
