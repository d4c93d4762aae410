"""Tensor-parallel model worker: one process per GPU behind one serving endpoint.

The model worker that owns the ZMQ queues is rank 0. It starts ``world - 1`` follower processes; every rank
builds its shard of the model and runs the *same* scheduler on the *same* requests, so all ranks construct
identical batches and meet in the kernels' collectives without any per-step negotiation. The only thing that has
to travel is the input: once per loop iteration rank 0 broadcasts the requests and cancellations it drained from
the API process (as the msgpack frames of ``worker_interface/codec.py``, over a gloo group so the control plane
never touches the GPUs' streams), and every rank enqueues them before its ``run_iteration``. Followers discard
their outputs; rank 0 answers the API process.

Reference: the reference drives all GPUs of a replica from one process and one compiled graph
(max/python/max/serve/pipelines/model_worker.py:213, nn/transformer/distributed_transformer.py:297); with one
process per GPU the lock-step scheduler plays that role.
"""

from __future__ import annotations

import copy
import os
import queue
import socket
from typing import Optional

from .worker_interface import codec


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rank_config(pipeline_config, rank: int, world: int):
    pc = copy.deepcopy(pipeline_config)
    if pc.expert_parallel_degree > 1:
        pc.ep_rank = rank
    else:
        pc.tp_size, pc.tp_rank = world, rank
    return pc


def init_distributed(rank: int, world: int, port: int, device_index: int):
    """NCCL group for the kernels' bootstrap, gloo group for the control plane."""
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.cuda.set_device(device_index)
    dist.init_process_group("nccl", device_id=torch.device("cuda", device_index), rank=rank, world_size=world)
    return dist.new_group(backend="gloo")


class LockstepFeed:
    """Replicates rank 0's request stream on every rank (see the module docstring)."""

    def __init__(self, ctl_group, rank: int):
        self.group, self.rank = ctl_group, rank
        self.requests: "queue.SimpleQueue" = queue.SimpleQueue()
        self.cancels: "queue.SimpleQueue" = queue.SimpleQueue()

    def exchange(self, new_ctxs=(), cancels=(), stop: bool = False) -> bool:
        """Rank 0 passes what it drained; every rank returns with the same items in its local queues.
        Returns False when rank 0 asked the group to stop."""
        import torch.distributed as dist

        box = [None]
        if self.rank == 0:
            box[0] = {"new": [codec.encode(c) for c in new_ctxs], "cancel": list(cancels), "stop": stop}
        dist.broadcast_object_list(box, src=0, group=self.group)
        msg = box[0]
        for frame in msg["new"]:
            self.requests.put_nowait(codec.decode(frame))
        for rid in msg["cancel"]:
            self.cancels.put_nowait(rid)
        return not msg["stop"]


class ShardedFeed:
    """Expert parallelism with data-parallel attention behind one endpoint: rank 0 deals the requests it drained to
    the ranks in turn (every rank hears about every request, keeps its own), and after every iteration the ranks
    exchange what they produced: rank 0 forwards all outputs to the API process, and every rank learns whether any
    rank still has work, because a step is an exchange that all ranks must take part in (ranks without requests
    run idle steps, see ``DeepseekV3Model.idle_step``).

    Reference: the data-parallel replicas of one process in max/python/max/serve/scheduler/text_batch_constructor.py
    (:1318 replica assignment) and dp_padding.py:45 (idle replicas run dummy batches)."""

    def __init__(self, ctl_group, rank: int, world: int):
        self.group, self.rank, self.world = ctl_group, rank, world
        self.requests: "queue.SimpleQueue" = queue.SimpleQueue()
        self.cancels: "queue.SimpleQueue" = queue.SimpleQueue()
        # rank 0 deals every new request to the rank with the fewest outstanding tokens (prompt tokens not yet
        # encoded weigh in full, a decoding request as one token per step), as the reference balances context
        # encoding over its data-parallel replicas (scheduler/batch_constructor/text_batch_constructor.py:566-594)
        self._outstanding = [0] * world
        self._owner_cost: dict = {}
        self.any_busy = False
        self.arrived = 0
        self.iterations = 0
        self.rank_loads: list = [None] * world     # latest expert-load slice of every rank (rank 0 keeps them)

    def exchange(self, new_ctxs=(), cancels=(), stop: bool = False) -> bool:
        import torch.distributed as dist

        box = [None]
        if self.rank == 0:
            frames = []
            for c in new_ctxs:
                owner = min(range(self.world), key=lambda r: (self._outstanding[r], r))
                cost = int(c.tokens.prompt_len) + int(c.max_new_tokens_effective)
                self._outstanding[owner] += cost
                self._owner_cost[c.request_id] = (owner, cost)
                frames.append((owner, codec.encode(c)))
            box[0] = {"new": frames, "cancel": list(cancels), "stop": stop}
        dist.broadcast_object_list(box, src=0, group=self.group)
        msg = box[0]
        for owner, frame in msg["new"]:
            if owner == self.rank:
                self.requests.put_nowait(codec.decode(frame))
        for rid in msg["cancel"]:
            self.cancels.put_nowait(rid)       # unknown ids are ignored by the scheduler
        self.arrived = len(msg["new"])
        return not msg["stop"]

    LOAD_EVERY = 64        # iterations between expert-load snapshots

    def gather(self, outputs: list, busy: bool, load=None) -> list:
        """Every rank contributes the response batches of its iteration (and now and then its expert-load slice,
        the input of the load balancer); returns all responses on rank 0 (an empty list elsewhere) and records
        whether any rank is still busy."""
        import torch.distributed as dist

        mine = {"out": [codec.encode(o) for o in outputs], "busy": bool(busy), "load": load}
        got = [None] * self.world
        dist.all_gather_object(got, mine, group=self.group)
        self.any_busy = any(g["busy"] for g in got)
        if self.rank != 0:
            return []
        for r, g in enumerate(got):
            if g.get("load") is not None:
                self.rank_loads[r] = g["load"]
        responses = [codec.decode(f) for g in got for f in g["out"]]
        for batch in responses:
            for rid, o in batch.items():
                if o.is_done and rid in self._owner_cost:
                    owner, cost = self._owner_cost.pop(rid)
                    self._outstanding[owner] -= cost
        return responses


def _drain_simple(q) -> list:
    out = []
    while True:
        try:
            out.append(q.get_nowait())
        except queue.Empty:
            return out


def ep_iteration(feed: ShardedFeed, sched, model, out_queue: "queue.SimpleQueue", new=(), cancels=(), stop=False):
    """One loop iteration of an expert-parallel rank. Returns (keep going, response batches for the API process
    (rank 0 only), whether this iteration did anything)."""
    if not feed.exchange(new, cancels, stop):
        return False, [], False
    active = feed.any_busy or feed.arrived > 0
    if active:
        calls = getattr(model, "forward_calls", 0)
        sched.run_iteration()
        if getattr(model, "forward_calls", 0) == calls:
            model.idle_step()
    load = None
    if active:
        feed.iterations += 1
        if feed.iterations % feed.LOAD_EVERY == 1 and hasattr(model, "expert_load"):
            load = model.expert_load()          # the same iterations on every rank: the counter advances in step
    responses = feed.gather(_drain_simple(out_queue), sched.has_work() or not feed.requests.empty(), load)
    return True, responses, active


def ep_follower_main(rank: int, world: int, port: int, factory, pipeline_config, settings) -> None:
    """Entry point of ranks 1..world-1 of an expert-parallel engine (spawned by rank 0)."""
    import logging
    import time
    import traceback

    from .model_worker import scheduler_config_from
    from .scheduler import TokenGenerationScheduler

    logging.basicConfig(level=getattr(logging, str(settings.log_level).upper(), logging.INFO),
                        format=f"%(asctime)s ep-rank-{rank} %(levelname)s %(name)s: %(message)s")
    try:
        pc = rank_config(pipeline_config, rank, world)
        ctl = init_distributed(rank, world, port, pc.model.device_ids[rank])
        llm = factory(pc)
        feed = ShardedFeed(ctl, rank, world)
        out_q: "queue.SimpleQueue" = queue.SimpleQueue()
        sched = TokenGenerationScheduler(scheduler_config_from(pc, llm), llm.pipeline, llm.kv, feed.requests, out_q,
                                         feed.cancels)
        while True:
            go, _, active = ep_iteration(feed, sched, llm.model, out_q)
            if not go:
                break
            if not active:
                time.sleep(0.001)
    except BaseException:  # noqa: BLE001
        traceback.print_exc()
        os._exit(1)


class _NullQueue:
    def put_nowait(self, _obj) -> None:
        pass


def follower_main(rank: int, world: int, port: int, factory, pipeline_config, settings) -> None:
    """Entry point of ranks 1..world-1 (spawned by rank 0)."""
    import logging
    import traceback

    from .model_worker import scheduler_config_from
    from .scheduler import TokenGenerationScheduler

    logging.basicConfig(level=getattr(logging, str(settings.log_level).upper(), logging.INFO),
                        format=f"%(asctime)s tp-rank-{rank} %(levelname)s %(name)s: %(message)s")
    try:
        pc = rank_config(pipeline_config, rank, world)
        ctl = init_distributed(rank, world, port, pc.model.device_ids[rank])
        llm = factory(pc)
        feed = LockstepFeed(ctl, rank)
        sched = TokenGenerationScheduler(scheduler_config_from(pc, llm), llm.pipeline, llm.kv, feed.requests,
                                         _NullQueue(), feed.cancels)
        while feed.exchange():
            sched.run_iteration()
    except BaseException:  # noqa: BLE001
        traceback.print_exc()
        os._exit(1)


def start_followers(world: int, port: int, factory, pipeline_config, settings, main=None) -> list:
    import multiprocessing as mp

    ctx = mp.get_context("spawn")
    procs = []
    for r in range(1, world):
        p = ctx.Process(target=main or follower_main, args=(r, world, port, factory, pipeline_config, settings), daemon=True,
                        name=f"rank-{r}")
        p.start()
        procs.append(p)
    return procs
