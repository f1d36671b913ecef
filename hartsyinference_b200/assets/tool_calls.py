"""Tool calls in model output: the formats chat models emit, parsed into (name, JSON arguments).

* Hermes / Qwen:   ``<tool_call>{"name": "f", "arguments": {...}}</tool_call>`` (any number of them)
* Mistral:         ``[TOOL_CALLS] [{"name": "f", "arguments": {...}}, ...]``
* Llama 3.x:       the whole reply is one JSON object ``{"name": "f", "parameters": {...}}``
  (optionally behind ``<|python_tag|>``)

``forced_prefix`` builds the text that forces a call of one tool: the reply is started for the model.

Reference: src/HartsyInference.LLM (TextRequest.Tools / ForceToolId, StopReason.ToolCall,
TextChunkKind.NativeToolCall).
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass
from typing import Optional


@dataclass
class ToolCall:
    id: str
    name: str
    arguments: str           # JSON text, as the OpenAI API carries it

    def to_openai(self) -> dict:
        return {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}


_TAGGED = re.compile(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", re.S)


def _one(obj) -> Optional[ToolCall]:
    if not isinstance(obj, dict) or not isinstance(obj.get("name"), str):
        return None
    args = obj.get("arguments", obj.get("parameters", {}))
    if isinstance(args, str):
        try:
            json.loads(args)
        except ValueError:
            return None
        text = args
    else:
        text = json.dumps(args, ensure_ascii=False)
    return ToolCall("call_" + uuid.uuid4().hex[:24], obj["name"], text)


def parse_tool_calls(text: str, known: Optional[set] = None) -> tuple[str, list[ToolCall]]:
    """-> (the reply without the call syntax, calls). ``known`` (tool names offered) filters out JSON
    that merely looks like a call."""
    calls: list[ToolCall] = []
    rest = text

    def keep(c: Optional[ToolCall]) -> bool:
        return c is not None and (known is None or c.name in known)

    if "<tool_call>" in text:
        for m in _TAGGED.finditer(text):
            try:
                c = _one(json.loads(m.group(1)))
            except ValueError:
                c = None
            if keep(c):
                calls.append(c)
        if calls:
            rest = _TAGGED.sub("", text)
    elif "[TOOL_CALLS]" in text:
        head, _, tail = text.partition("[TOOL_CALLS]")
        try:
            arr, end = json.JSONDecoder().raw_decode(tail.lstrip())
            for obj in arr if isinstance(arr, list) else [arr]:
                c = _one(obj)
                if keep(c):
                    calls.append(c)
            if calls:
                rest = head + tail.lstrip()[end:]
        except ValueError:
            pass
    else:
        body = text.strip()
        if body.startswith("<|python_tag|>"):
            body = body[len("<|python_tag|>"):].strip()
        if body.startswith("{") and body.endswith("}"):
            try:
                c = _one(json.loads(body))
            except ValueError:
                c = None
            if keep(c) and ("parameters" in body or "arguments" in body):
                calls.append(c)
                rest = ""
    return rest.strip() if calls else text, calls


def tool_names(tools: Optional[list]) -> set:
    out = set()
    for t in tools or []:
        fn = t.get("function", t) if isinstance(t, dict) else {}
        if isinstance(fn.get("name"), str):
            out.add(fn["name"])
    return out


def forced_prefix(tool_id: str) -> str:
    """The start of a reply that can only continue as a call of ``tool_id`` (Hermes / Qwen syntax)."""
    return '<tool_call>\n{"name": "' + tool_id + '", "arguments": '
