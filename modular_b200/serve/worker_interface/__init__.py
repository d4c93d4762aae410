"""API process <-> model worker transport.

``WorkerQueues`` is the triple (request, response, cancel). The in-process flavour uses
``queue.SimpleQueue``; the multi-process flavour uses ZMQ PUSH/PULL sockets over ``ipc://``
endpoints (reference: max/python/max/serve/worker_interface/__init__.py:62,123;
zmq_interface.py:50; _zmq_queue.py).
"""

from .zmq_queue import ZmqPullSocket, ZmqPushSocket, ZmqQueueSpec, generate_ipc_path  # noqa: F401
from .interface import ModelWorkerProxy, ReplicaRouter, RequestQueueFull, WorkerGone, WorkerQueues  # noqa: F401
