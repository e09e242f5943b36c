"""Host-side liveness of the ranks of the collective path.

The fused kernels wait for their peers with bounded device waits (a lost peer ends the call with
``Status::Timeout`` after ``wait_limit_s``), but a rank that is known to be gone should not be waited for at
all: nothing may be in flight towards it. ``Membership`` is a heartbeat over a ``torch.distributed`` store
(the counterpart of the master's registry-as-liveness on the RPC path, pico-ps/service/Client.cpp:364-368):
every rank publishes the step it is about to run, and ``wait_all`` returns only when every peer has
announced the same step. A peer that announced its departure (``leave``) or stays silent longer than
``timeout_s`` raises :class:`RankLost` on the others BEFORE they launch, so they can re-plan (restore the
lost shards from their mirror with ``ReplicaSet.restore`` or from a dump, or re-shard onto the survivors).

A rank leaves only between steps, with none of its kernels or collectives in flight.
"""
from __future__ import annotations

import time
from typing import Iterable, List, Optional


class RankLost(RuntimeError):
    def __init__(self, ranks: Iterable[int], left: Iterable[int] = ()):
        self.ranks = sorted(set(ranks))
        self.left = sorted(set(left))       # the subset that announced its departure
        super().__init__(f"ranks {self.ranks} are gone (announced: {self.left})")


class Membership:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "psb/hb", poll_s: float = 0.002):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix, self.poll_s = timeout_s, prefix, poll_s
        self.gone: List[int] = []           # ranks already reported lost: not waited for again
        self.store.set(self._key(rank), "0")

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Announce that this rank is about to run ``step`` (monotonic)."""
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        """Announce a clean departure (call between steps, after the last kernel has completed)."""
        self.store.set(self._key(self.rank), "left")

    def _read(self, r: int) -> Optional[str]:
        if not self.store.check([self._key(r)]):
            return None
        return self.store.get(self._key(r)).decode()

    def wait_all(self, step: int, peers: Optional[Iterable[int]] = None) -> None:
        """Block until every live peer has announced ``step`` (or a later one). Raises :class:`RankLost` with
        the peers that left or stayed silent for ``timeout_s``; they are remembered in ``gone``."""
        pending = [r for r in (peers if peers is not None else range(self.world)) if r != self.rank and r not in self.gone]
        left: List[int] = []
        deadline = time.monotonic() + self.timeout_s
        while pending:
            still = []
            for r in pending:
                v = self._read(r)
                if v == "left":
                    left.append(r)
                elif v is None or int(v) < step:
                    still.append(r)
            pending = still
            if not pending or time.monotonic() > deadline:
                break
            time.sleep(self.poll_s)
        lost = left + pending
        if lost:
            self.gone.extend(lost)
            raise RankLost(lost, left)

    def step(self, step: int) -> None:
        """``beat`` + ``wait_all``: call right before the collective launches of a step."""
        self.beat(step)
        self.wait_all(step)

    def survivors(self) -> List[int]:
        return [r for r in range(self.world) if r not in self.gone]
