"""Multi-GPU plumbing: process-group helpers and the NCCL-only baselines of the fused paths."""
from .nccl_baseline import NcclDenseTable, NcclSparseTable  # noqa: F401
from .migrate import PeerInbox, ReplicaSet, reshard  # noqa: F401
from . import checkpoint  # noqa: F401
from .membership import Membership, RankLost  # noqa: F401
from .predictor_sync import PredictorSync  # noqa: F401
