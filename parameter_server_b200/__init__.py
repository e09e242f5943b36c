"""parameter_server_b200: a Blackwell-native parameter server.

Sharded sparse tables (int64 key -> fp32 row + optimizer slots) and dense tables live in the HBM of
the GPUs of one box; pull / push run as fused sm_100a kernels that move keys, rows and gradients
through NVLink peer memory. The package keeps the reference's layering:
``storage -> operator -> handler -> service -> controller`` (pico-ps/{storage,operator,handler,
service,controller}/), with the torch-facing modules in ``ops``, ``models`` and ``parallel``.
"""
from ._lib import C  # noqa: F401
from .utils.status import Status, StatusCode, StatusError  # noqa: F401
from .ops.optim import make_opt_config, OPTIMIZERS  # noqa: F401
from .ops.sparse import SparseTable, sparse_lookup  # noqa: F401
from .ops.dense import DenseTable  # noqa: F401

__version__ = "0.1.0"
