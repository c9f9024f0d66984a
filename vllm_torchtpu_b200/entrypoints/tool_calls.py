"""Function calling for the chat endpoint.

Two ways a completion becomes ``tool_calls``:

* ``tool_choice`` names a function (or is ``"required"``): the completion is constrained by structured decoding to
  the JSON the call needs (the function's parameter schema, or an array of {name, parameters} objects over all
  tools), so it parses by construction.
* ``tool_choice`` is ``"auto"``: the model decides; calls written in the Hermes convention
  (``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``, the format Qwen and Hermes templates teach) are
  taken out of the text.

The tools are handed to the tokenizer's chat template (``tools=``), which is where a model learns about them.
"""
from __future__ import annotations

import json
import re
import uuid
from typing import Optional

_TOOL_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*(?:</tool_call>|$)", re.S)


def validate_tools(body: dict) -> tuple:
    """(tools, choice) with choice one of None, "none", "auto", "required" or a function name."""
    tools = body.get("tools") or []
    choice = body.get("tool_choice")
    if not tools:
        if choice not in (None, "none", "auto"):
            raise ValueError("tool_choice needs tools")
        return [], None
    names = []
    for t in tools:
        fn = (t or {}).get("function") if isinstance(t, dict) else None
        if not isinstance(fn, dict) or t.get("type", "function") != "function" or not fn.get("name"):
            raise ValueError("each tool must be {'type': 'function', 'function': {'name': ..., 'parameters': ...}}")
        names.append(fn["name"])
    if choice is None:
        choice = "auto"
    if isinstance(choice, dict):
        name = (choice.get("function") or {}).get("name")
        if name not in names:
            raise ValueError(f"tool_choice names an unknown function {name!r}")
        return tools, name
    if choice not in ("none", "auto", "required"):
        raise ValueError("tool_choice must be 'none', 'auto', 'required' or a named function")
    return tools, choice


def _params(tool: dict) -> dict:
    return tool["function"].get("parameters") or {"type": "object", "properties": {}}


def structured_spec_for(tools: list, choice) -> Optional[dict]:
    """The structured-decoding spec that forces a call, or None when the model is free."""
    if choice in (None, "none", "auto"):
        return None
    if choice == "required":
        one = [{"type": "object", "properties": {"name": {"enum": [t["function"]["name"]]}, "parameters": _params(t)},
                "required": ["name", "parameters"]} for t in tools]
        return {"json": {"type": "array", "minItems": 1, "items": {"anyOf": one} if len(one) > 1 else one[0]}}
    tool = next(t for t in tools if t["function"]["name"] == choice)
    return {"json": _params(tool)}


def _call(name: str, arguments) -> dict:
    args = arguments if isinstance(arguments, str) else json.dumps(arguments)
    return {"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function", "function": {"name": name, "arguments": args}}


def extract_tool_calls(text: str, tools: list, choice) -> tuple:
    """(content left for the message or None, list of tool calls)."""
    if not tools or choice in (None, "none"):
        return text, []
    if choice == "required":
        try:
            items = json.loads(text)
            return None, [_call(it["name"], it.get("parameters", {})) for it in items]
        except (ValueError, KeyError, TypeError):
            return text, []
    if choice != "auto":
        try:
            return None, [_call(choice, json.loads(text))]
        except ValueError:
            return text, []
    names = {t["function"]["name"] for t in tools}
    calls = []
    for m in _TOOL_CALL.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except ValueError:
            continue
        if isinstance(obj, dict) and obj.get("name") in names:
            calls.append(_call(obj["name"], obj.get("arguments", obj.get("parameters", {}))))
    if not calls:
        return text, []
    rest = _TOOL_CALL.sub("", text).strip()
    return (rest or None), calls
