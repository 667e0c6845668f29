"""In-process communicator for tests: N ranks are threads of one process that meet at a barrier for
every collective.  Faults can be injected on the host: a rank that never joins (`drop_rank`), a delay,
or an exception, so failure handling is exercised without touching a GPU."""
from __future__ import annotations

import threading
import time

import torch


class CommTimeout(RuntimeError):
    pass


class _Hub:
    def __init__(self, world_size: int, timeout_s: float):
        self.n = world_size
        self.timeout = timeout_s
        self.cv = threading.Condition()
        self.slots = {}
        self.round = {}
        self.dropped = set()
        self.delay = {}

    def exchange(self, rank: int, key: str, value):
        """All-to-all of one value per rank; returns the list ordered by rank."""
        if rank in self.dropped:
            raise CommTimeout(f"rank {rank} was dropped by the test")
        if rank in self.delay:
            time.sleep(self.delay[rank])
        with self.cv:
            r = self.round.get((key, rank), 0)
            self.round[(key, rank)] = r + 1
            box = self.slots.setdefault((key, r), {})
            box[rank] = value
            self.cv.notify_all()
            deadline = time.monotonic() + self.timeout
            while len(box) < self.n:
                left = deadline - time.monotonic()
                if left <= 0:
                    missing = sorted(set(range(self.n)) - set(box))
                    raise CommTimeout(f"collective {key!r} timed out waiting for ranks {missing}")
                self.cv.wait(left)
            return [box[i] for i in range(self.n)]


class FakeComm:
    def __init__(self, hub: _Hub, rank: int):
        self.hub, self.rank, self.world_size = hub, rank, hub.n

    def all_reduce(self, t):
        parts = self.hub.exchange(self.rank, "ar", t.clone())
        out = parts[0].clone()
        for p in parts[1:]:
            out += p
        t.copy_(out)
        return t

    def all_gather(self, t):
        return [p.clone() for p in self.hub.exchange(self.rank, "ag", t.clone())]

    def broadcast(self, t, src=0):
        t.copy_(self.hub.exchange(self.rank, "bc", t.clone())[src])
        return t

    def broadcast_object(self, obj, src=0):
        return self.hub.exchange(self.rank, "bo", obj)[src]

    def barrier(self):
        self.hub.exchange(self.rank, "ba", None)


def make_fake_world(world_size: int, timeout_s: float = 20.0):
    hub = _Hub(world_size, timeout_s)
    return hub, [FakeComm(hub, r) for r in range(world_size)]


def run_ranks(world_size: int, fn, timeout_s: float = 60.0, hub_timeout_s: float = 20.0):
    """Runs fn(comm) on `world_size` threads; returns (results, errors) ordered by rank."""
    hub, comms = make_fake_world(world_size, hub_timeout_s)
    results, errors = [None] * world_size, [None] * world_size

    def work(r):
        try:
            results[r] = fn(comms[r])
        except BaseException as e:     # noqa: BLE001  (reported to the test)
            errors[r] = e
    threads = [threading.Thread(target=work, args=(r,), daemon=True) for r in range(world_size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s)
    return results, errors, hub
