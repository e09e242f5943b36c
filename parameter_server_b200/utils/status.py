"""Status helpers on top of the native ``Status`` (codes of pico-ps/common/Status.h:15-29)."""
from __future__ import annotations

from .._lib import C

Status = C.Status
StatusCode = C.StatusCode


class StatusError(RuntimeError):
    """Raised by the convenience API when an operation ends with a non-OK status."""

    def __init__(self, status):
        super().__init__(str(status))
        self.status = status

    @property
    def code(self):
        return self.status.code()


def ok() -> "C.Status":
    return C.Status()


def make(code, msg: str = "") -> "C.Status":
    return C.Status(code, msg)


def raise_if_error(st) -> None:
    if not st.ok():
        raise StatusError(st)
