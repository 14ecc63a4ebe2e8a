"""Grammar engine: GBNF parsing, masks over a byte vocabulary, JSON object and JSON-Schema lowering."""
import json

import numpy as np
import pytest

from sllm_b200.engine.grammar import (JSON_OBJECT_GBNF, CompiledGrammar, GrammarError, schema_to_gbnf)
from sllm_b200.frontend.text import ByteTokenizer, TokenByteTable

TK = ByteTokenizer()
TABLE = TokenByteTable(TK).bytes


def accepts(gbnf, text, complete=True):
    g = CompiledGrammar(gbnf, TABLE)
    st = g.new_state()
    for t in TK.encode(text, allow_special=False):
        m = st.mask()
        if not m[t] or not st.accept(t):
            return False
    return st.is_complete() if complete else True


def test_gbnf_basics_and_masks():
    g = 'root ::= "yes" | "no" [0-9]+\n'
    assert accepts(g, "yes") and accepts(g, "no42") and not accepts(g, "no") and not accepts(g, "maybe")
    cg = CompiledGrammar(g, TABLE)
    st = cg.new_state()
    m = st.mask()
    assert set(np.nonzero(m)[0].tolist()) == {ord("y"), ord("n")}
    assert not st.mask(eos_ids=(TK.eos_token_id,))[TK.eos_token_id]
    for ch in "yes":
        assert st.accept(ord(ch))
    assert st.is_complete() and st.mask(eos_ids=(TK.eos_token_id,))[TK.eos_token_id] == 1
    assert st.mask().sum() == 0
    c = st.clone()
    assert not c.accept(ord("x")) and st.is_complete()


def test_repetitions_groups_classes_and_utf8():
    g = 'root ::= item ("," item){1,2}\nitem ::= [a-c]{2} | "é" | [^\\x00-\\x7f]\n'
    assert accepts(g, "ab,cc") and accepts(g, "é,ab,é") and not accepts(g, "ab") and not accepts(g, "ab,ab,ab,ab")
    assert accepts(g, "€,ab")           # multi-byte code point split across byte tokens
    with pytest.raises(GrammarError):
        CompiledGrammar('root ::= missing\n', TABLE)
    with pytest.raises(GrammarError):
        CompiledGrammar('root ::= "unterminated\n', TABLE)


def test_json_object_mode_limits():
    assert accepts(JSON_OBJECT_GBNF, '{"a": 1, "b": [true, null], "c": {"d": "x"}}')
    assert accepts(JSON_OBJECT_GBNF, "{}")
    assert not accepts(JSON_OBJECT_GBNF, '{"a": [[1]]}')                       # depth > 1
    assert not accepts(JSON_OBJECT_GBNF, '{"a":1,"b":2,"c":3,"d":4,"e":5}')    # more than four members
    assert not accepts(JSON_OBJECT_GBNF, '[1]')
    assert not accepts(JSON_OBJECT_GBNF, '{"a": "' + "x" * 65 + '"}')


def test_json_schema_lowering():
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                                "tags": {"type": "array", "items": {"enum": ["a", "b"]}},
                                                "kind": {"anyOf": [{"const": "x"}, {"type": "null"}]}},
              "required": ["name", "age"], "additionalProperties": False}
    g = schema_to_gbnf(schema)
    assert accepts(g, '{"name": "bob", "age": 42}')
    assert accepts(g, '{"name":"bob","age":-3,"tags":["a","b"],"kind":null}')
    assert not accepts(g, '{"age": 42, "name": "bob"}')         # declaration order is fixed
    assert not accepts(g, '{"name": "bob"}')
    assert not accepts(g, '{"name": "bob", "age": 1.5}')
    ref = {"$defs": {"p": {"type": "boolean"}}, "type": "array", "items": {"$ref": "#/$defs/p"}}
    assert accepts(schema_to_gbnf(ref), "[true, false]")
    for bad in ({"type": "string", "pattern": "a+"}, {"type": "object", "properties": {}, "additionalProperties": True},
                {"allOf": []}, {"$ref": "http://x"}, {"$defs": {"a": {"$ref": "#/$defs/a"}}, "$ref": "#/$defs/a"},
                {"type": "string", "minLength": 2}):
        with pytest.raises(GrammarError):
            schema_to_gbnf(bad)


def test_mask_cache_and_stats():
    g = CompiledGrammar(JSON_OBJECT_GBNF, TABLE)
    st = g.new_state()
    st.accept_text('{"k": "')
    m1 = st.mask()
    st.accept(ord("a"))
    m2 = st.mask()
    assert m1[ord("z")] and m2[ord("z")] and not m1[0x01]
    s = g.stats()
    assert s["rules"] > 5 and s["dfa_states"] > 3 and s["trie_nodes"] >= 256
