"""Host-side peer watchdog: every rank publishes a heartbeat in the rendezvous key-value store and watches
the others'.  A rank whose counter has not moved for `timeout_s` is reported as lost, so the survivors learn
of a dead peer on the host, BEFORE their next launch, instead of inside a collective (where the fused
kernels would only notice through their bounded waits, and NCCL through its process-group timeout).

The reference has no failure detection: a dead rank leaves the others blocked in NCCL until the 600 s
process-group timeout (engine/parallel.py:35-40).

The store can be any `torch.distributed.Store` (TCPStore of the torchrun rendezvous, FileStore, or an
in-process HashStore in tests).  Store errors (the rank hosting the store is gone) count as the loss of
rank `store_owner`.
"""
from __future__ import annotations

import threading
import time


class PeerLostError(RuntimeError):
    def __init__(self, ranks):
        self.ranks = sorted(ranks)
        super().__init__(f"tensor-parallel peer(s) {self.ranks} stopped sending heartbeats")


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, *, interval_s: float = 0.5, timeout_s: float = 5.0,
                 prefix: str = "ti_hb", store_owner: int = 0, clock=time.monotonic, on_lost=None):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self.prefix, self.store_owner = prefix, store_owner
        self.clock, self.on_lost = clock, on_lost
        self.lost: set = set()
        self._beats = 0
        self._seen = {}            # rank -> (last counter value, time it changed)
        self._stop = threading.Event()
        self._thread = None
        self._lock = threading.Lock()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    # one round: publish, then look at every peer.  Separate from the thread so tests can drive it with a fake clock.
    def tick(self):
        now = self.clock()
        try:
            self._beats += 1
            self.store.set(self._key(self.rank), str(self._beats))
            for r in range(self.world):
                if r == self.rank or r in self.lost:
                    continue
                val = self.store.get(self._key(r)).decode() if self.store.check([self._key(r)]) else None
                last = self._seen.get(r)
                if last is None or last[0] != val:
                    self._seen[r] = (val, now)            # first look, or the counter moved
                elif now - last[1] > self.timeout_s:
                    self._report(r)
        except Exception:                                  # the store itself is gone
            if self.store_owner != self.rank:
                self._report(self.store_owner)

    def _report(self, r: int):
        with self._lock:
            if r in self.lost:
                return
            self.lost.add(r)
        if self.on_lost is not None:
            self.on_lost(r)

    def _run(self):
        while not self._stop.wait(self.interval_s):
            self.tick()

    def start(self):
        if self._thread is None:
            self.tick()
            self._thread = threading.Thread(target=self._run, name="ti-heartbeat", daemon=True)
            self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1)
            self._thread = None

    def check(self):
        """Raises PeerLostError if a peer has been reported lost.  Called by the engine before every step."""
        if self.lost:
            raise PeerLostError(self.lost)


def default_store():
    """The key-value store of the current torch.distributed rendezvous, or None."""
    try:
        import torch.distributed as dist
        from torch.distributed import distributed_c10d as c10d
        if dist.is_initialized():
            return c10d._get_default_store()
    except Exception:
        pass
    return None
