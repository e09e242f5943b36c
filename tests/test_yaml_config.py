"""Configs written as YAML: the reference reads its operator and storage configs with a YAML reader
(pico-ps/service/Context.cpp:14-25); here the native config parser accepts JSON or a YAML subset."""
import json

import numpy as np
import pytest
import yaml

from parameter_server_b200 import service as S

DOCS = [
    "dim: 4\noptimizer: sum\ninit_range: 0.0\n",
    "a: 1\nb:\n  c: [1, 2, 3]\n  d: 'x y'\n  e: \"q: r\"\nf: true\ng: ~\nh: -2.5e-3\n",
    "nodes:\n  - g_rank: 0\n    shard_list: [0, 1]\n  - g_rank: 7\n    shard_list: []\nop_config:\n  dim: 8   # comment\n  tags:\n  - a\n  - b\n",
    "# only a comment\nkey: value # trailing\nurl: hdfs://host/path\nempty:\nlist:\n  -\n  - 3\n",
    "limits: {soft: 10, hard: 20}\nnested: [[1, 2], [3]]\nflag: no\n",
]


@pytest.mark.parametrize("doc", DOCS)
def test_yaml_subset_agrees_with_pyyaml(doc):
    assert json.loads(S.config_to_json(doc)) == yaml.safe_load(doc)


def test_json_is_still_json_and_bad_input_is_an_error():
    assert json.loads(S.config_to_json('{"a": [1, 2, {"b": null}]}')) == {"a": [1, 2, {"b": None}]}
    assert S.config_to_json("") == "{}"
    for bad in ("a: 1\n\tb: 2", "just a line without a key\n", "a: [1, 2", "a:\n    b: 1\n  c: 2\n"):
        with pytest.raises(RuntimeError):
            S.config_to_json(bad)


def test_a_table_created_and_used_from_yaml_configs():
    master = S.Master()
    servers = [S.Server(master.address()) for _ in range(2)]
    client = S.Client(master.address())
    try:
        ids = [s.node_id() for s in servers]
        storage_yaml = f"""
table_name: yaml_table
nodes:
  - g_rank: {ids[0]}
    shard_list: [0, 2]
  - g_rank: {ids[1]}
    shard_list: [1, 3]
op_config:
  dim: 4
  optimizer: sum       # w += g
  init_range: 0.0
"""
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", storage_yaml)
        assert st.ok(), st
        st, h_pull = client.register_handler("pull", S.LIB, "SparseTablePullOperator", "read_only: false\n", sid)
        assert st.ok(), st
        st, h_ro = client.register_handler("pull_ro", S.LIB, "SparseTablePullOperator", "read_only: yes", sid)
        assert st.ok(), st
        st, h_push = client.register_handler("push", S.LIB, "SparseTablePushOperator", "", sid)
        assert st.ok(), st
        pull, ro, push = S.PullHandler(client, sid, h_pull), S.PullHandler(client, sid, h_ro), S.PushHandler(client, sid, h_push)
        keys = np.arange(100, dtype=np.int64)
        st, v = pull.pull(keys)
        assert st.ok() and (v == 0).all()
        st = push.async_push(keys, np.ones((100, 4), dtype=np.float32))
        assert st.ok(), st
        st, v = ro.pull(np.arange(200, dtype=np.int64))          # the read-only handler never inserts
        assert st.ok() and (v[:100] == 1).all() and (v[100:] == 0).all()
        st, v = pull.pull(keys)
        assert st.ok() and (v == 1).all()
        bad, _ = client.register_handler("x", S.LIB, "SparseTablePullOperator", "read_only: [1, 2", sid)
        assert not bad.ok()
    finally:
        for s in servers:
            s.stop()
        master.stop()


def _scalars():
    from hypothesis import strategies as st
    plain = st.text(alphabet="abcdefghijklmnopqrstuvwxyzABCXYZ_0123456789./-", min_size=1, max_size=12).filter(
        lambda s: s[0].isalpha() and s.lower() not in ("true", "false", "yes", "no", "on", "off", "null", "y", "n"))
    return st.one_of(st.integers(-10**9, 10**9), st.booleans(), st.none(), plain,
                     st.floats(allow_nan=False, allow_infinity=False, width=32).map(lambda x: round(x, 3)))


def test_generated_documents_round_trip_like_pyyaml():
    """Nested mappings / sequences of scalars, written by PyYAML in block style, read back by the native parser."""
    from hypothesis import given, settings, strategies as st
    keys = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_", min_size=1, max_size=8).filter(
        lambda s: s not in ("true", "false", "yes", "no", "on", "off", "null", "y", "n"))
    tree = st.recursive(_scalars(), lambda ch: st.one_of(st.lists(ch, max_size=4), st.dictionaries(keys, ch, max_size=4)), max_leaves=12)
    docs = st.dictionaries(keys, tree, min_size=1, max_size=5)

    @settings(max_examples=200, deadline=None)
    @given(docs)
    def check(doc):
        text = yaml.safe_dump(doc, default_flow_style=False)
        got = json.loads(S.config_to_json(text))
        assert got == yaml.safe_load(text), text

    check()
