"""Parser of the qwen3_coder tool-call text format into OpenAI tool calls:

    <function=NAME>
    <parameter=KEY>
    VALUE
    </parameter>
    </function>

Tolerant of truncation (a missing closing tag ends the value at the next tag or the end) and of nested
angle brackets inside values; values are coerced with the tool's JSON schema when one is given
(reference behaviour: server/qwserve/tool_calls.py:87-138)."""
import json
import re
import uuid
from typing import Any, Dict, List, Optional

_FN = re.compile(r"<function=([^>\n]+)>")
_PARAM = re.compile(r"<parameter=([^>\n]+)>")


def _coerce(value: str, schema: Optional[dict]) -> Any:
    v = value.strip("\n")
    ty = (schema or {}).get("type")
    if isinstance(ty, list):
        ty = next((t for t in ty if t != "null"), None)
    try:
        if ty == "integer":
            return int(v.strip())
        if ty == "number":
            return float(v.strip())
        if ty == "boolean":
            return v.strip().lower() in ("true", "1", "yes")
        if ty in ("object", "array"):
            return json.loads(v)
        if ty == "string":
            return v
    except (ValueError, json.JSONDecodeError):
        return v
    if ty is None:
        try:
            return json.loads(v)
        except (ValueError, json.JSONDecodeError):
            return v
    return v


def parse_tool_call(text: str, tools: Optional[List[dict]] = None) -> Optional[Dict[str, Any]]:
    m = _FN.search(text)
    if not m:
        return None
    name = m.group(1).strip()
    body = text[m.end():]
    end = body.find("</function>")
    if end >= 0:
        body = body[:end]
    props = {}
    for t in tools or []:
        f = t.get("function", t)
        if f.get("name") == name:
            props = (f.get("parameters") or {}).get("properties", {}) or {}
    args: Dict[str, Any] = {}
    pos = 0
    while True:
        pm = _PARAM.search(body, pos)
        if not pm:
            break
        key = pm.group(1).strip()
        start = pm.end()
        close = body.find("</parameter>", start)
        nxt = _PARAM.search(body, start)
        if close < 0 or (nxt and nxt.start() < close):
            stop = nxt.start() if nxt else len(body)        # truncated value: ends at the next parameter
            pos = stop
        else:
            stop = close
            pos = close + len("</parameter>")
        args[key] = _coerce(body[start:stop], props.get(key))
    return {"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
            "function": {"name": name, "arguments": json.dumps(args, ensure_ascii=False)}}
