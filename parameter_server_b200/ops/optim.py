"""Update rules of sparse and dense tables.

The reference leaves the rule to user overrides of ``store_push_value`` / ``init_store_value``
(pico-ps/operator/SparsePushOperator.h:433-448); here they are concrete device functors selected
by name in the operator config.
"""
from __future__ import annotations

from .._lib import C

OPTIMIZERS = {
    "sgd": C.OPT_SGD,
    "adagrad": C.OPT_ADAGRAD,
    "ftrl": C.OPT_FTRL,
    "adam": C.OPT_ADAM,
    "adamw": C.OPT_ADAM,
    "sum": C.OPT_SUM,
    "set": C.OPT_SET,
}

_FIELDS = ("lr", "eps", "l1", "l2", "alpha", "beta", "beta1", "beta2", "weight_decay", "slot_init0", "slot_init1")


def make_opt_config(name: str = "sgd", **kw) -> "C.OptConfig":
    """Build an ``OptConfig``. Aliases: ``init_accumulator`` (Adagrad) -> ``slot_init0``."""
    name = name.lower()
    if name not in OPTIMIZERS:
        raise ValueError(f"unknown optimizer {name!r}; choose from {sorted(OPTIMIZERS)}")
    c = C.OptConfig()
    c.type = OPTIMIZERS[name]
    if name == "adagrad":
        c.eps = 1e-10
    if "init_accumulator" in kw:
        kw["slot_init0"] = kw.pop("init_accumulator")
    for k, v in kw.items():
        if k not in _FIELDS:
            raise ValueError(f"unknown optimizer option {k!r}")
        setattr(c, k, float(v))
    return c


def set_adam_step(cfg: "C.OptConfig", step: int) -> None:
    """Bias-correction terms of Adam for (1-based) step ``step``."""
    cfg.bias_corr1 = 1.0 - cfg.beta1 ** step
    cfg.bias_corr2 = 1.0 - cfg.beta2 ** step
