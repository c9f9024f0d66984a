"""JSON Schema -> regular expression, for schema-constrained decoding on top of the regex grammar.

Covers what serving APIs send in practice: ``type`` (string / integer / number / boolean / null / object /
array, or a list of them), ``enum`` and ``const``, ``properties`` with ``required`` (properties are emitted
in declaration order; optional ones may be left out), ``additionalProperties: false`` semantics (nothing
beyond the declared properties), ``items`` with ``minItems`` / ``maxItems``, string ``minLength`` /
``maxLength`` / ``pattern``, ``anyOf`` / ``oneOf``, local ``$ref`` into ``$defs`` / ``definitions``.
Whitespace between tokens is limited to ``whitespace`` (default: at most one blank or newline) so that a
model cannot stall in padding.  Recursion through ``$ref`` is unrolled to ``max_depth`` levels.
(reference: the reference hands JSON schemas to xgrammar through vLLM's structured-output manager,
src/vllm_torchtpu/runner/structured_decoding_manager.py; this is the own, regex-based route)"""
from __future__ import annotations

import json
import re

WS = r"[ \n]?"
STRING_CHAR = r'(?:[^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'
INTEGER = r"-?(?:0|[1-9][0-9]*)"
NUMBER = INTEGER + r"(?:\.[0-9]+)?(?:[eE][+-]?[0-9]+)?"


def _literal(value) -> str:
    return re.escape(json.dumps(value, ensure_ascii=False, separators=(",", ":")))


def _string(schema: dict) -> str:
    if "pattern" in schema:
        pat = schema["pattern"]
        pat = pat[1:] if pat.startswith("^") else pat
        pat = pat[:-1] if pat.endswith("$") and not pat.endswith(r"\$") else pat
        return '"(?:' + pat + ')"'
    lo, hi = schema.get("minLength", 0), schema.get("maxLength")
    rep = f"{{{lo},{hi}}}" if hi is not None else (f"{{{lo},}}" if lo else "*")
    return '"' + STRING_CHAR + rep + '"'


def _array(schema: dict, ctx) -> str:
    item = ctx.build(schema.get("items", {}))
    lo, hi = schema.get("minItems", 0), schema.get("maxItems")
    sep = WS + "," + WS
    if hi is not None and hi == 0:
        return r"\[" + WS + r"\]"
    more_hi = "" if hi is None else str(max(hi - 1, 0))
    more_lo = max(lo - 1, 0)
    body = f"(?:{item})(?:{sep}(?:{item})){{{more_lo},{more_hi}}}"
    if lo == 0:
        body = f"(?:{body})?"
    return r"\[" + WS + body + WS + r"\]"


def _object(schema: dict, ctx) -> str:
    props = schema.get("properties")
    if not props:
        if schema.get("additionalProperties") is False:
            return r"\{" + WS + r"\}"
        # free-form object: string keys, any JSON value (bounded nesting)
        val = ctx.any_value()
        pair = _string({}) + WS + ":" + WS + f"(?:{val})"
        return r"\{" + WS + f"(?:{pair}(?:{WS},{WS}{pair})*)?" + WS + r"\}"
    required = set(schema.get("required", []))
    sep = WS + "," + WS
    parts = [(name, _literal(name) + WS + ":" + WS + f"(?:{ctx.build(sub)})", name in required)
             for name, sub in props.items()]
    # properties in declaration order; an optional one may be skipped.  The pattern after the first emitted
    # property is "(, next)" per remaining property; alternatives enumerate which property comes first.
    def tail(i: int) -> str:
        out = ""
        for _, pat, req in parts[i:]:
            out += f"{sep}{pat}" if req else f"(?:{sep}{pat})?"
        return out
    alts = []
    for i, (_, pat, req) in enumerate(parts):
        alts.append(pat + tail(i + 1))
        if req:
            break                         # nothing after a required property can be the first one
    body = "(?:" + "|".join(alts) + ")"
    if not required:
        body += "?"
    return r"\{" + WS + body + WS + r"\}"


class _Ctx:
    def __init__(self, root: dict, max_depth: int):
        self.root, self.max_depth, self.depth = root, max_depth, 0

    def any_value(self, depth: int = 2) -> str:
        scalars = [_string({}), NUMBER, "true", "false", "null"]
        if depth == 0:
            return "|".join(scalars)
        inner = self.any_value(depth - 1)
        arr = r"\[" + WS + f"(?:(?:{inner})(?:{WS},{WS}(?:{inner}))*)?" + WS + r"\]"
        pair = _string({}) + WS + ":" + WS + f"(?:{inner})"
        obj = r"\{" + WS + f"(?:{pair}(?:{WS},{WS}{pair})*)?" + WS + r"\}"
        return "|".join(scalars + [arr, obj])

    def resolve(self, ref: str) -> dict:
        if not ref.startswith("#/"):
            raise ValueError(f"only local $ref is supported, got {ref!r}")
        node = self.root
        for part in ref[2:].split("/"):
            node = node[part.replace("~1", "/").replace("~0", "~")]
        return node

    def build(self, schema) -> str:
        if schema is True or schema == {}:
            return self.any_value()
        if schema is False:
            raise ValueError("a schema that accepts nothing cannot be generated from")
        if "$ref" in schema:
            if self.depth >= self.max_depth:
                raise ValueError(f"$ref recursion deeper than {self.max_depth}")
            self.depth += 1
            try:
                return self.build(self.resolve(schema["$ref"]))
            finally:
                self.depth -= 1
        if "const" in schema:
            return _literal(schema["const"])
        if "enum" in schema:
            return "(?:" + "|".join(_literal(v) for v in schema["enum"]) + ")"
        for key in ("anyOf", "oneOf"):
            if key in schema:
                return "(?:" + "|".join(f"(?:{self.build(s)})" for s in schema[key]) + ")"
        t = schema.get("type")
        if isinstance(t, list):
            return "(?:" + "|".join(f"(?:{self.build({**schema, 'type': one})})" for one in t) + ")"
        if t == "string":
            return _string(schema)
        if t == "integer":
            return INTEGER
        if t == "number":
            return NUMBER
        if t == "boolean":
            return "(?:true|false)"
        if t == "null":
            return "null"
        if t == "array":
            return _array(schema, self)
        if t == "object" or "properties" in schema:
            return _object(schema, self)
        if t is None:
            return self.any_value()
        raise ValueError(f"unsupported schema type {t!r}")


def schema_to_regex(schema, max_depth: int = 4) -> str:
    """Regular expression (Python ``regex`` syntax) matching exactly the JSON texts the schema admits under
    the restrictions in the module docstring."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    return _Ctx(schema, max_depth).build(schema)


JSON_OBJECT = None


def any_json_object_regex() -> str:
    """``response_format = json_object``: any JSON object, nesting bounded."""
    global JSON_OBJECT
    if JSON_OBJECT is None:
        JSON_OBJECT = _object({}, _Ctx({}, 4))
    return JSON_OBJECT
