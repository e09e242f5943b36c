"""The documents name classes and methods of the Python API; every `Class.method` they mention must exist."""
import os
import re

import parameter_server_b200 as P
from parameter_server_b200 import parallel
from parameter_server_b200 import service as S
from parameter_server_b200.parallel import checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OWNERS = {name: getattr(S, name) for name in
          ["Client", "Controller", "PullHandler", "PushHandler", "ForEachHandler", "EraseIfHandler", "DumpHandler", "LoadHandler",
           "UpdateContextHandler", "SyncHandler", "UDFHandler", "Server", "ServerConfig", "MasterClient", "NativePS",
           "NativePullHandler", "NativeLoadHandler", "TableSyncer"]}
OWNERS.update(SparseTable=P.SparseTable, DenseTable=P.DenseTable, service=S, parallel=parallel, checkpoint=checkpoint)
OWNERS["parallel.checkpoint"] = checkpoint


def _mentions(text):
    for owner, names in re.findall(r"`((?:parallel\.)?[A-Za-z_]+)\.([a-z_]+(?: / [a-z_]+)*)", text):
        if owner in OWNERS:
            for name in names.split(" / "):
                if name not in ("py", "md", "h", "cu", "cpp"):        # `checkpoint.py` is a file, not a call
                    yield owner, name


def test_every_method_that_the_documents_name_exists():
    missing = []
    for doc in ("README.md", "docs/migration.md", "docs/operators.md", "docs/availability.md", "docs/overview.md", "docs/testing.md"):
        text = open(os.path.join(ROOT, doc)).read()
        for owner, name in _mentions(text):
            if not hasattr(OWNERS[owner], name):
                missing.append(f"{doc}: {owner}.{name}")
    assert not missing, sorted(set(missing))
