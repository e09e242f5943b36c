"""Incremental sync from a collective (training) table to a predictor table of the service layer.

The training job holds its embeddings in a ``SparseTable`` on its GPUs; the serving side is a table of the RPC
path (``parameter_server_b200.service``) that predictors pull from. ``PredictorSync`` ships the rows that changed
since the last round - every rank its own - through a ``SyncHandler`` of the predictor table, in blocks, and
clears the marks only after every block of the round was accepted, so a failed round is sent again in full.

Parity: the trainer -> predictor path of the reference, pico-ps/handler/SyncHandler.h:36-74 (``sync_pred``: stream
the increment in blocks, rewind on failure) and pico-ps/operator/SyncOperator.h:102-260 (``to_sync_value`` picks
what of a row travels; apply = overwrite), with the double-buffered increment of
pico-ps/service/IncrementStorage.h:11-43 replaced by the table's per-row dirty marks.

The dirty marks are the ones ``ReplicaSet.sync`` uses: a table syncs to a mirror or to a predictor, not both.
"""
from typing import Callable, Optional

import torch

from ..ops.sparse import SparseTable
from ..utils.status import raise_if_error


class PredictorSync:
    """``PredictorSync(table, handler)``; ``handler`` is a ``service.SyncHandler`` of the predictor table.

    Args:
        to_sync_value: ``fn(keys, rows) -> rows`` picks what of a row travels (default: the whole row, which needs
            the same optimizer on both sides; ``embedding_only`` sends the first ``dim`` floats, for predictor
            tables created with the ``set`` or ``sum`` optimizer).
        block: rows per message (default: the handler's ``block_size``).
    """

    def __init__(self, table: SparseTable, handler, *, embedding_only: bool = False,
                 to_sync_value: Optional[Callable] = None, block: Optional[int] = None, timeout_ms: int = 30000):
        self.table, self.handler = table, handler
        self.block = int(block or handler.block_size())
        self.timeout_ms = int(timeout_ms)
        if to_sync_value is None and embedding_only:
            dim = table.dim
            to_sync_value = lambda k, r: r[:, :dim]   # noqa: E731
        self.to_sync_value = to_sync_value
        self._full_next = True                        # the first round ships everything
        self.rounds = self.rows_sent = self.failed_rounds = 0
        table.table.enable_dirty_tracking()

    def sync(self) -> int:
        """One round: ship this rank's changed rows. Returns rows sent; raises ``StatusError`` when the predictor
        refused a block (the marks stay, the next round sends the increment again)."""
        t = self.table
        sent = 0
        try:
            for k, r in t.export(batch=max(self.block, 1 << 14), dirty_only=not self._full_next):
                if self.to_sync_value is not None:
                    r = self.to_sync_value(k, r)
                kn = k.cpu().numpy()
                rn = r.contiguous().cpu().float().numpy()
                for off in range(0, len(kn), self.block):
                    raise_if_error(self.handler.sync_block(kn[off:off + self.block], rn[off:off + self.block], self.timeout_ms))
                    sent += len(kn[off:off + self.block])
        except Exception:
            self.failed_rounds += 1
            raise
        if t.is_cuda:
            raise_if_error(t.table.clear_dirty(torch.cuda.current_stream().cuda_stream))
        else:
            t.table.clear_dirty()
        self._full_next = False
        self.rounds += 1
        self.rows_sent += sent
        return sent
