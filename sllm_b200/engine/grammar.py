"""Grammar-constrained decoding front end: GBNF text, the bounded JSON-object grammar, and the
fail-closed JSON-Schema lowerer, on top of the native automaton (csrc/host/grammar.cpp).

Reference behaviour: crates/sllm-core/src/grammar.rs and docs/api/openai-compatibility.md:111-131 -
`json_object` allows depth 1, up to four members / items per container, strings and numbers up to 64
characters, whitespace runs up to 16 bytes; `json_schema` supports only $ref to local $defs, $defs, type,
properties, required, additionalProperties:false, items, enum, const, anyOf and rejects everything else.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Optional

import numpy as np

from ..ops import _lib

MAX_SCHEMA_BYTES = 64 * 1024
MAX_SCHEMA_DEPTH = 16
MAX_ENUM = 256
MAX_PROPERTIES = 64


class GrammarError(ValueError):
    pass


WS = 'ws ::= [ \\t\\n\\r]{0,16}\n'
JSON_PRIMITIVES = (
    'string ::= "\\"" char{0,64} "\\""\n'
    'char ::= [^"\\\\\\x00-\\x1f] | "\\\\" (["\\\\/bfnrt] | "u" [0-9a-fA-F]{4})\n'
    'number ::= "-"? ("0" | [1-9] [0-9]{0,15}) ("." [0-9]{1,16})? ([eE] [-+]? [0-9]{1,3})?\n'
    'integer ::= "-"? ("0" | [1-9] [0-9]{0,17})\n'
    'boolean ::= "true" | "false"\n'
    'null ::= "null"\n')

JSON_OBJECT_GBNF = (
    'root ::= ws object ws\n'
    'object ::= "{" ws (member (ws "," ws member){0,3})? ws "}"\n'
    'member ::= string ws ":" ws value\n'
    'value ::= scalar | flatobject | flatarray\n'
    'scalar ::= string | number | boolean | null\n'
    'flatobject ::= "{" ws (flatmember (ws "," ws flatmember){0,3})? ws "}"\n'
    'flatmember ::= string ws ":" ws scalar\n'
    'flatarray ::= "[" ws (scalar (ws "," ws scalar){0,3})? ws "]"\n' + JSON_PRIMITIVES + WS)

_ALLOWED_KEYS = {"$ref", "$defs", "type", "properties", "required", "additionalProperties", "items", "enum", "const",
                 "anyOf", "title", "description"}


def _lit(s: str) -> str:
    out = []
    for ch in s:
        o = ord(ch)
        if ch in '"\\':
            out.append("\\" + ch)
        elif o < 0x20:
            out.append(f"\\x{o:02x}")
        else:
            out.append(ch)
    return '"' + "".join(out) + '"'


def schema_to_gbnf(schema: dict) -> str:
    """Lowers the supported JSON-Schema subset to GBNF; anything else raises GrammarError."""
    if len(json.dumps(schema).encode()) > MAX_SCHEMA_BYTES:
        raise GrammarError("schema larger than 64 KiB")
    defs = schema.get("$defs", {}) if isinstance(schema, dict) else {}
    if not isinstance(defs, dict):
        raise GrammarError("$defs must be an object")
    rules: dict = {}
    counter = [0]

    def fresh(prefix: str) -> str:
        counter[0] += 1
        return f"{prefix}{counter[0]}"

    def lower(node, depth: int, stack: tuple) -> str:
        if depth > MAX_SCHEMA_DEPTH:
            raise GrammarError("schema nesting too deep")
        if not isinstance(node, dict):
            raise GrammarError("schema nodes must be objects")
        unknown = set(node) - _ALLOWED_KEYS
        if unknown:
            raise GrammarError(f"unsupported schema keyword: {sorted(unknown)[0]}")
        if "$ref" in node:
            ref = node["$ref"]
            if not isinstance(ref, str) or not ref.startswith("#/$defs/") or ref[8:] not in defs:
                raise GrammarError("only $ref to a local $defs entry is supported")
            name = ref[8:]
            if name in stack:
                raise GrammarError("recursive $ref is not supported")
            return lower(defs[name], depth + 1, stack + (name,))
        if "const" in node:
            return _lit(json.dumps(node["const"], ensure_ascii=False, separators=(",", ":")))
        if "enum" in node:
            vals = node["enum"]
            if not isinstance(vals, list) or not vals or len(vals) > MAX_ENUM:
                raise GrammarError("enum must hold 1..256 values")
            return "(" + " | ".join(_lit(json.dumps(v, ensure_ascii=False, separators=(",", ":"))) for v in vals) + ")"
        if "anyOf" in node:
            alts = node["anyOf"]
            if not isinstance(alts, list) or not alts or len(alts) > MAX_ENUM:
                raise GrammarError("anyOf must hold 1..256 schemas")
            return "(" + " | ".join(lower(a, depth + 1, stack) for a in alts) + ")"
        t = node.get("type")
        if isinstance(t, list):
            return "(" + " | ".join(lower({**node, "type": x}, depth + 1, stack) for x in t) + ")"
        if t == "object":
            props = node.get("properties", {})
            if not isinstance(props, dict) or len(props) > MAX_PROPERTIES:
                raise GrammarError("too many properties")
            if node.get("additionalProperties", False) is not False:
                raise GrammarError("additionalProperties must be false")
            required = node.get("required", [])
            if not isinstance(required, list) or any(r not in props for r in required):
                raise GrammarError("required must list declared properties")
            name = fresh("obj")
            parts = []
            first = True
            # properties are emitted in declaration order; optional ones may be skipped
            for key, sub in props.items():
                item = f'{_lit(json.dumps(key))} ws ":" ws {lower(sub, depth + 1, stack)}'
                if key in required:
                    parts.append((item if first else f'ws "," ws {item}'))
                    first = False
                else:
                    if first and not any(k in required for k in list(props)[list(props).index(key) + 1:]):
                        parts.append(f'({item})?')       # may be the only member
                        first = False if False else first
                    elif first:
                        raise GrammarError("optional properties before the first required one are not supported")
                    else:
                        parts.append(f'(ws "," ws {item})?')
            rules[name] = '"{" ws ' + " ".join(parts) + ' ws "}"' if parts else '"{" ws "}"'
            return name
        if t == "array":
            items = node.get("items")
            if items is None:
                raise GrammarError("array schemas need items")
            name = fresh("arr")
            it = lower(items, depth + 1, stack)
            rules[name] = f'"[" ws ({it} (ws "," ws {it}){{0,15}})? ws "]"'
            return name
        if t in ("string", "number", "integer", "boolean", "null"):
            return t
        raise GrammarError("schema needs a supported type, enum, const, anyOf or $ref")

    root = lower(schema, 0, ())
    text = f"root ::= ws {root} ws\n" + "".join(f"{k} ::= {v}\n" for k, v in rules.items()) + JSON_PRIMITIVES + WS
    return text


def _host():
    lib = _lib.host()
    if not getattr(lib, "_grammar_ready", False):
        lib.sllm_grammar_create.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]
        lib.sllm_grammar_set_vocab.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib.sllm_grammar_mask.argtypes = [C.c_int, C.c_void_p, C.c_int]
        lib.sllm_grammar_accept_bytes.argtypes = [C.c_int, C.c_char_p, C.c_int]
        lib.sllm_grammar_stats.argtypes = [C.c_int, C.c_void_p]
        lib._grammar_ready = True
    return lib


class CompiledGrammar:
    """A grammar bound to a vocabulary (token byte table)."""

    def __init__(self, gbnf: str, token_bytes: list, root: str = "root"):
        lib = _host()
        err = C.create_string_buffer(512)
        self.h = lib.sllm_grammar_create(gbnf.encode("utf-8"), root.encode(), err, 512)
        if self.h <= 0:
            raise GrammarError(err.value.decode() or "grammar rejected")
        self.n = len(token_bytes)
        blob = b"".join(token_bytes)
        offs = np.zeros(self.n + 1, dtype=np.uint32)
        np.cumsum([len(b) for b in token_bytes], out=offs[1:])
        self._blob = np.frombuffer(blob, dtype=np.uint8).copy() if blob else np.zeros(1, dtype=np.uint8)
        rc = lib.sllm_grammar_set_vocab(self.h, self.n, self._blob.ctypes.data, offs.ctypes.data)
        if rc:
            lib.sllm_grammar_destroy(self.h)
            raise GrammarError(f"vocabulary rejected ({rc})")

    def new_state(self) -> "GrammarState":
        return GrammarState(self)

    def stats(self) -> dict:
        out = (C.c_longlong * 3)()
        _host().sllm_grammar_stats(self.h, out)
        return {"rules": out[0], "dfa_states": out[1], "trie_nodes": out[2]}

    def close(self):
        if self.h > 0:
            _host().sllm_grammar_destroy(self.h)
            self.h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GrammarState:
    def __init__(self, grammar: CompiledGrammar, handle: Optional[int] = None):
        self.g = grammar
        self.s = handle if handle is not None else _host().sllm_grammar_state_new(grammar.h)
        if self.s <= 0:
            raise GrammarError("could not create a grammar state")

    def mask(self, eos_ids=()) -> np.ndarray:
        """uint8[vocab]; end-of-sequence tokens are allowed exactly when the text is a complete sentence."""
        m = np.zeros(self.g.n, dtype=np.uint8)
        _host().sllm_grammar_mask(self.s, m.ctypes.data, self.g.n)
        if eos_ids and self.is_complete():
            for e in eos_ids:
                if 0 <= e < self.g.n:
                    m[e] = 1
        return m

    def accept(self, token: int) -> bool:
        return _host().sllm_grammar_accept(self.s, int(token)) == 0

    def accept_text(self, text: str) -> bool:
        b = text.encode("utf-8")
        return _host().sllm_grammar_accept_bytes(self.s, b, len(b)) == 0

    def is_complete(self) -> bool:
        return _host().sllm_grammar_is_complete(self.s) == 1

    def clone(self) -> "GrammarState":
        return GrammarState(self.g, _host().sllm_grammar_state_clone(self.s))

    def __del__(self):
        try:
            if self.s > 0:
                _host().sllm_grammar_state_free(self.s)
        except Exception:
            pass
