"""Model families trained against the parameter server: DLRM (sparse + dense tables) and a GPT-style
decoder (dense tables)."""
from .dlrm import DLRM, DLRMConfig, SyntheticCTR, field_keys  # noqa: F401
