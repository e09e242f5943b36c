"""Service layer: master, servers, clients, handlers, controller, model objects, in-process PS.

These are the native classes of ``csrc/service``, ``csrc/handler``, ``csrc/controller``,
``csrc/model`` and ``csrc/native_ps`` (the layers L5-L7 of the reference: pico-ps/service,
pico-ps/handler, pico-ps/controller, pico-ps/model, pico-ps/native_ps). Every process of a job
creates a :class:`Client` (and, if it holds shards, a :class:`Server`) pointing at one
:class:`Master`. The built-in operators are registered under the library name ``"psb"``.
"""
from __future__ import annotations

import json
from typing import Dict, Iterable, List, Optional, Sequence

from .._lib import C

Master = C.Master
MasterClient = C.MasterClient
Server = C.Server
ServerConfig = C.ServerConfig
Client = C.Client
PullHandler = C.PullHandler
PullGroup = C.PullGroup
PushGroup = C.PushGroup
PushHandler = C.PushHandler
ForEachHandler = C.ForEachHandler
EraseIfHandler = C.EraseIfHandler
DumpHandler = C.DumpHandler
LoadHandler = C.LoadHandler
UpdateContextHandler = C.UpdateContextHandler
SyncHandler = C.SyncHandler
TableSyncer = C.TableSyncer
set_hadoop_bin = C.set_hadoop_bin
set_log_level = C.set_log_level


def log_to_python(logger_name: str = "parameter_server_b200") -> None:
    """Route the native runtime's log lines into the ``logging`` module (levels map DEBUG..ERROR)."""
    import logging

    logger = logging.getLogger(logger_name)
    levels = [logging.DEBUG, logging.INFO, logging.WARNING, logging.ERROR]
    C.set_log_sink(lambda level, msg: logger.log(levels[min(level, 3)], msg))
UDFHandler = C.UDFHandler
Controller = C.Controller
OpSpec = C.OpSpec
NativePS = C.NativePS
NativePullHandler = C.NativePullHandler
NativeLoadHandler = C.NativeLoadHandler
TableDescriptor = C.TableDescriptor
register_udf = C.register_udf

LIB = "psb"

#: operator keys used by :func:`standard_ops`
PULL, PULL_RO, PUSH, FOREACH, ERASE, DUMP, LOAD, UPDATE_CTX, SYNC = (
    "pull", "pull_ro", "push", "for_each", "erase_if", "dump", "load", "update_ctx", "sync")


def storage_config(nodes: Dict[int, Sequence[int]], op_config: dict, table_name: str = "") -> str:
    """Storage config JSON: ``nodes`` maps a server's node id to the shard ids it holds."""
    return json.dumps({
        "nodes": [{"g_rank": int(n), "shard_list": [int(s) for s in shards]} for n, shards in nodes.items()],
        "op_config": op_config,
        "table_name": table_name,
    })


def nodes_json(nodes: Dict[int, Sequence[int]]) -> str:
    return json.dumps([{"g_rank": int(n), "shard_list": [int(s) for s in shards]} for n, shards in nodes.items()])


def config_to_json(text: str) -> str:
    """A config text as the native layer reads it, as JSON: operator and storage configs may be written as JSON or as
    YAML (block mappings / sequences, flow sequences, scalars, comments)."""
    return C.config_to_json(text)


def standard_ops(compress: str = "", block_size: int = 1000) -> List["C.OpSpec"]:
    """The usual operator set of a sparse table (what the reference's tests register one by one)."""
    c = json.dumps({"compress_algorithm": compress, "block_size": block_size})
    return [
        OpSpec(PULL, LIB, "SparseTablePullOperator", "{}"),
        OpSpec(PULL_RO, LIB, "SparseTablePullOperator", json.dumps({"read_only": True})),
        OpSpec(PUSH, LIB, "SparseTablePushOperator", "{}"),
        OpSpec(FOREACH, LIB, "ForEachOperator", "{}"),
        OpSpec(ERASE, LIB, "EraseIfOperator", "{}"),
        OpSpec(DUMP, LIB, "DumpOperator", c),
        OpSpec(LOAD, LIB, "LoadOperator", c),
        OpSpec(UPDATE_CTX, LIB, "ShardUpdateContextOperator", "{}"),
        OpSpec(SYNC, LIB, "KVSyncOperator", c),
    ]


def check(st) -> None:
    from ..utils.status import raise_if_error

    raise_if_error(st)


class Pending:
    """A handler call in flight: the start / ``wait()`` pattern of the reference's handlers
    (pico-ps/handler/Handler.h:40-83: ``pull(...)`` sends, ``wait()`` blocks until the answers are in).

    ``start(handler.pull, keys)`` returns at once; the call runs on a thread of its own (the bindings release the GIL
    while they wait for the servers, so several calls really overlap), and ``wait()`` hands back what the call
    returned or raises what it raised. One handler object carries one call at a time, as in the reference: use one
    handler per call in flight.
    """

    def __init__(self, fn, *args, **kwargs):
        import threading

        self._result = None
        self._error: Optional[BaseException] = None

        def run():
            try:
                self._result = fn(*args, **kwargs)
            except BaseException as e:  # noqa: BLE001 - handed to the waiter
                self._error = e

        self._thread = threading.Thread(target=run, daemon=True)
        self._thread.start()

    def done(self) -> bool:
        return not self._thread.is_alive()

    def wait(self, timeout: Optional[float] = None):
        self._thread.join(timeout)
        if self._thread.is_alive():
            raise TimeoutError("the call is still in flight")
        if self._error is not None:
            raise self._error
        return self._result


def start(fn, *args, **kwargs) -> Pending:
    """``start(PullHandler(...).pull, keys)`` -> :class:`Pending`."""
    return Pending(fn, *args, **kwargs)
