"""Automatic spill policy for a :class:`SparseTable` with a pinned-host cold tier.

``ColdTierPolicy`` keeps the number of rows in HBM under a budget: every ``interval`` steps it looks at the
distribution of one row section (by default the first optimizer slot, e.g. the Adagrad accumulator, which grows
with the gradient a key has received), picks the threshold that frees the required fraction, and spills the rows
below it. ``pull`` brings back the cold rows of the batch first (synchronously, or staged one step ahead with
``stage_next``). The role of the capacity management around the reference's persistent-memory tier
(pico-ps/storage/DCPmemory.h:324-513 holds what does not fit DRAM); the policy itself is new.
"""
from __future__ import annotations

from typing import Optional

import torch

from .sparse import SparseTable


class ColdTierPolicy:
    def __init__(self, table: SparseTable, hbm_budget_rows: int, cold_capacity_rows: int, *, section: int = 1,
                 interval: int = 100, headroom: float = 0.1, sample_rows: int = 1 << 16):
        if not table.is_cuda:
            raise RuntimeError("the cold tier sits under a GPU table")
        self.table = table
        self.budget = int(hbm_budget_rows)
        self.section = int(section)
        self.interval = int(interval)
        self.headroom = float(headroom)
        self.sample_rows = int(sample_rows)
        self.steps = 0
        self.spilled_total = 0
        self.fetched_total = 0
        self._staged = False
        if not hasattr(table, "cold"):
            table.enable_cold_tier(cold_capacity_rows)

    # ------------------------------------------------------------------------------------------
    def _threshold_for(self, fraction: float) -> float:
        """Value of the section mean below which about ``fraction`` of the rows lie (from a sample window)."""
        dim = self.table.dim
        for _, rows in self.table.export(batch=self.sample_rows):
            sec = rows[:, self.section * dim:(self.section + 1) * dim].mean(dim=1)
            return float(torch.quantile(sec.float(), min(max(fraction, 0.0), 1.0)).item())
        return float("-inf")

    def maybe_spill(self) -> int:
        """Call once per step. Spills when the table is over budget at an interval boundary; returns rows spilled."""
        self.steps += 1
        if self.steps % self.interval:
            return 0
        n = self.table.size()
        if n <= self.budget:
            return 0
        # free down to (1 - headroom) * budget so that the next interval has room to grow
        target = int(self.budget * (1.0 - self.headroom))
        fraction = (n - target) / n
        thr = self._threshold_for(fraction)
        spilled = self.table.spill_cold(self.section, thr)
        self.spilled_total += spilled
        return spilled

    def stage_next(self, next_keys_host: torch.Tensor) -> None:
        """Start fetching the cold rows of the NEXT batch while the current step computes."""
        self.table.prefetch_cold_async(next_keys_host)
        self._staged = True

    def pull(self, keys: torch.Tensor, keys_host: Optional[torch.Tensor] = None, **kw) -> torch.Tensor:
        """``table.pull`` preceded by the return of the batch's cold rows: the staged ones if ``stage_next`` ran for
        this batch, and whatever else of ``keys_host`` (default: a host copy of ``keys``) is still cold."""
        if self._staged:
            self.fetched_total += self.table.commit_prefetch()
            self._staged = False
        if self.table.cold.size():
            self.fetched_total += self.table.prefetch_cold(keys_host if keys_host is not None else keys.cpu())
        return self.table.pull(keys, **kw)
