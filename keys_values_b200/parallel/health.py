"""Host-side failure detection between steps.

Every rank publishes a heartbeat (the number of the step it has finished, or the reason why it
gave up) in the key-value store of the process group. Before a rank launches the collectives of
its next step it publishes its own heartbeat and waits for those of its peers (`enter_step`): a peer that has not reached the step within
the grace time, or that has published a failure, raises :class:`RankFailure` here, on the host,
instead of leaving this rank inside a collective that can never complete. A rank leaves only
between steps, with none of its kernels or collectives in flight; restart is ``--resume auto``.

The reference has no rank failure detection (only the OOM retry of
``keys_values/long_context.py:333-363``); this module is the host half of the bounded-wait /
status-word scheme of the device code.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    """Raised on the surviving ranks. ``ranks`` maps each failed rank to what is known about it."""

    def __init__(self, ranks: Dict[int, str]):
        self.ranks = dict(ranks)
        super().__init__("rank failure detected on the host: " + ", ".join(f"rank {r}: {why}" for r, why in sorted(ranks.items())))


class RankHealth:
    def __init__(self, rank: int, world_size: int, store=None, prefix: str = "kvb200/health", poll_s: float = 0.05):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store, self.rank, self.world_size = store, rank, world_size
        self.prefix, self.poll_s = prefix, poll_s
        self.store.set(self._key(rank), "-1")

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/step/{rank}"

    def _fail_key(self, rank: int) -> str:
        return f"{self.prefix}/failed/{rank}"

    # ------------------------------------------------------------------ publish
    def beat(self, step: int) -> None:
        """This rank has finished ``step`` (all of its kernels and collectives are done)."""
        self.store.set(self._key(self.rank), str(int(step)))

    def mark_failed(self, reason: str) -> None:
        """This rank gives up (call it from the exception handler, between steps)."""
        self.store.set(self._fail_key(self.rank), reason[:500] or "failed")

    # -------------------------------------------------------------------- check
    def _peer_state(self, r: int) -> (Optional[str], int):
        failed = None
        try:
            if self.store.check([self._fail_key(r)]):
                failed = self.store.get(self._fail_key(r)).decode()
            step = -1
            if self.store.check([self._key(r)]):
                step = int(self.store.get(self._key(r)).decode())
        except Exception as ex:  # the process that serves the store is gone
            raise RankFailure({0: f"key-value store unreachable: {type(ex).__name__}"}) from ex
        return failed, step

    def laggards(self, step: int, grace_s: float = 5.0) -> Dict[int, str]:
        """Peers that have not finished ``step`` after ``grace_s`` seconds, or that have failed."""
        deadline = time.monotonic() + grace_s
        bad: Dict[int, str] = {}
        while True:
            bad = {}
            for r in range(self.world_size):
                if r == self.rank:
                    continue
                failed, s = self._peer_state(r)
                if failed is not None:
                    bad[r] = f"reported: {failed}"
                elif s < step:
                    bad[r] = f"heartbeat at step {s}, expected {step}"
            reported = any(v.startswith("reported") for v in bad.values())
            if not bad or reported or time.monotonic() >= deadline:
                return bad
            time.sleep(self.poll_s)

    def assert_alive(self, step: int, grace_s: float = 5.0) -> None:
        """Call before launching the collectives of step ``step + 1``."""
        bad = self.laggards(step, grace_s)
        if bad:
            raise RankFailure(bad)

    def enter_step(self, step: int, grace_s: float = 5.0) -> None:
        """Host-side rendezvous before the collectives of ``step`` are launched: announces that this
        rank enters ``step`` (i.e. has finished ``step − 1``) and waits until every peer has done the
        same. A peer that does not arrive within ``grace_s`` seconds, or that has reported a failure,
        raises :class:`RankFailure`, so no rank launches a collective that a lost peer will never join."""
        self.beat(step - 1)
        self.assert_alive(step - 1, grace_s)

    def failed_ranks(self) -> List[int]:
        return [r for r in range(self.world_size) if self.store.check([self._fail_key(r)])]
