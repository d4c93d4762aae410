"""ZMQ PUSH/PULL queues with a ``queue.Queue``-like API (``put_nowait`` / ``get_nowait``); frames are msgpack
(see ``codec.py``), never pickle."""

from __future__ import annotations

import os
import queue
import tempfile
import uuid
from dataclasses import dataclass

import zmq

from . import codec


def generate_ipc_path(tag: str = "q") -> str:
    d = os.path.join(tempfile.gettempdir(), "mb200-ipc")
    os.makedirs(d, exist_ok=True)
    return f"ipc://{d}/{tag}-{os.getpid()}-{uuid.uuid4().hex[:12]}"


@dataclass(frozen=True)
class ZmqQueueSpec:
    """Picklable description of a queue endpoint; each process opens its own socket end."""

    path: str

    @classmethod
    def create(cls, tag: str) -> "ZmqQueueSpec":
        return cls(generate_ipc_path(tag))

    def push(self, bind: bool = False) -> "ZmqPushSocket":
        return ZmqPushSocket(self.path, bind)

    def pull(self, bind: bool = True) -> "ZmqPullSocket":
        return ZmqPullSocket(self.path, bind)


class _Base:
    def __init__(self, path: str, kind: int, bind: bool):
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(kind)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.path = path
        if bind:
            self.sock.bind(path)
        else:
            self.sock.connect(path)

    def close(self) -> None:
        self.sock.close(0)


class ZmqPushSocket(_Base):
    def __init__(self, path: str, bind: bool = False):
        super().__init__(path, zmq.PUSH, bind)

    def put_nowait(self, obj) -> None:
        try:
            self.sock.send(codec.encode(obj), flags=zmq.NOBLOCK)
        except zmq.Again as e:
            raise queue.Full() from e

    put = put_nowait


class ZmqPullSocket(_Base):
    def __init__(self, path: str, bind: bool = True):
        super().__init__(path, zmq.PULL, bind)

    def get_nowait(self):
        try:
            return codec.decode(self.sock.recv(flags=zmq.NOBLOCK))
        except zmq.Again as e:
            raise queue.Empty() from e

    def get(self, timeout_s: float = None):
        if timeout_s is not None and not self.sock.poll(int(timeout_s * 1000)):
            raise queue.Empty()
        return codec.decode(self.sock.recv())

    def empty(self) -> bool:
        return not self.sock.poll(0)
