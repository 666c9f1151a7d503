"""Tool-call extraction and reasoning split for chat completions.

Models emit tool calls in family-specific text formats; the server turns them into OpenAI ``tool_calls`` entries and
strips them from ``content``.  Reasoning models wrap their chain of thought in ``<think>…</think>``; it is returned as
``reasoning_content``.  ``StreamSplitter`` does the reasoning split incrementally for SSE.
Reference: crates/plowrt/src/serve/tools/ (per-family parsers, fixtures tests/fixtures/toolcall/*), serve/reasoning.rs,
serve/think.rs, docs/serving-openai-compat.md."""
from __future__ import annotations

import json
import re
import uuid


def _call(name, args) -> dict:
    if not isinstance(args, str):
        args = json.dumps(args, ensure_ascii=False)
    return {"id": f"call_{uuid.uuid4().hex[:24]}", "type": "function", "function": {"name": name, "arguments": args}}


def _json_calls(obj) -> list:
    objs = obj if isinstance(obj, list) else [obj]
    out = []
    for o in objs:
        if isinstance(o, dict) and "name" in o:
            out.append(_call(o["name"], o.get("arguments", o.get("parameters", {}))))
    return out


def parse_hermes(text: str):
    """<tool_call>{"name": ..., "arguments": {...}}</tool_call>  (Hermes, Qwen2.5/3)"""
    calls = []
    for m in re.finditer(r"<tool_call>\s*(.*?)\s*</tool_call>", text, re.S):
        try:
            calls += _json_calls(json.loads(m.group(1)))
        except json.JSONDecodeError:
            return None
    return (re.sub(r"<tool_call>.*?</tool_call>", "", text, flags=re.S).strip(), calls) if calls else None


def parse_llama3(text: str):
    """<|python_tag|>{"name": ..., "parameters": {...}}  or a bare JSON object / ';'-separated objects (Llama 3.x)"""
    body = text.split("<|python_tag|>", 1)[1] if "<|python_tag|>" in text else text
    body = body.replace("<|eom_id|>", "").replace("<|eot_id|>", "").strip()
    if not body.startswith("{"):
        return None
    calls = []
    for part in re.split(r";\s*(?=\{)", body):
        try:
            calls += _json_calls(json.loads(part))
        except json.JSONDecodeError:
            return None
    return ("", calls) if calls else None


def parse_mistral(text: str):
    """[TOOL_CALLS][{"name": ..., "arguments": {...}}, ...]  (Mistral / Mixtral)"""
    if "[TOOL_CALLS]" not in text:
        return None
    head, body = text.split("[TOOL_CALLS]", 1)
    try:
        obj, _ = json.JSONDecoder().raw_decode(body.strip())
    except json.JSONDecodeError:
        return None
    calls = _json_calls(obj)
    return (head.strip(), calls) if calls else None


def parse_deepseek(text: str):
    """<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{...}\\n```<｜tool▁call▁end｜>…  (DeepSeek V3/R1)"""
    if "<｜tool▁calls▁begin｜>" not in text:
        return None
    head = text.split("<｜tool▁calls▁begin｜>", 1)[0]
    calls = []
    for m in re.finditer(r"<｜tool▁call▁begin｜>(?:function)?<｜tool▁sep｜>([^\n]+)\n```json\n(.*?)\n```<｜tool▁call▁end｜>", text, re.S):
        calls.append(_call(m.group(1).strip(), m.group(2).strip()))
    return (head.strip(), calls) if calls else None


def parse_glm(text: str):
    """<tool_call>NAME\\n<arg_key>k</arg_key>\\n<arg_value>v</arg_value>…</tool_call>  (GLM-4.5 / GLM-5 family)"""
    calls = []
    for m in re.finditer(r"<tool_call>\s*([^\n<]+)\n(.*?)</tool_call>", text, re.S):
        keys = re.findall(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", m.group(2), re.S)
        if not keys and m.group(2).strip():
            return None
        args = {}
        for k, v in keys:
            try:
                args[k.strip()] = json.loads(v)
            except json.JSONDecodeError:
                args[k.strip()] = v
        calls.append(_call(m.group(1).strip(), args))
    return (re.sub(r"<tool_call>.*?</tool_call>", "", text, flags=re.S).strip(), calls) if calls else None


def parse_kimi(text: str):
    """<|tool_call_begin|>functions.NAME:0<|tool_call_argument_begin|>{...}<|tool_call_end|>  (Kimi K2)"""
    calls = []
    for m in re.finditer(r"<\|tool_call_begin\|>\s*(?:functions\.)?([\w.\-]+?)(?::\d+)?\s*<\|tool_call_argument_begin\|>(.*?)<\|tool_call_end\|>", text, re.S):
        calls.append(_call(m.group(1), m.group(2).strip()))
    if not calls:
        return None
    head = text.split("<|tool_calls_section_begin|>", 1)[0] if "<|tool_calls_section_begin|>" in text else text.split("<|tool_call_begin|>", 1)[0]
    return head.strip(), calls


def parse_gptoss(text: str):
    """<|channel|>commentary to=functions.NAME <|constrain|>json<|message|>{...}<|call|>  (gpt-oss harmony)"""
    calls = []
    for m in re.finditer(r"to=functions\.([\w.\-]+)[^<]*(?:<\|constrain\|>\w+)?<\|message\|>(.*?)(?:<\|call\|>|$)", text, re.S):
        calls.append(_call(m.group(1), m.group(2).strip()))
    if not calls:
        return None
    final = re.search(r"<\|channel\|>final<\|message\|>(.*?)(?:<\|end\|>|<\|return\|>|$)", text, re.S)
    return (final.group(1).strip() if final else ""), calls


PARSERS = {"hermes": parse_hermes, "qwen": parse_hermes, "llama3": parse_llama3, "mistral": parse_mistral,
           "deepseek": parse_deepseek, "glm": parse_glm, "kimi": parse_kimi, "gptoss": parse_gptoss}

FAMILY_OF_MODEL_TYPE = {"llama": "llama3", "qwen2": "hermes", "qwen3": "hermes", "qwen3_moe": "hermes", "qwen3_next": "hermes",
                        "mistral": "mistral", "mixtral": "mistral", "deepseek_v3": "deepseek", "glm_moe_dsa": "glm", "glm4_moe": "glm",
                        "kimi_k2": "kimi", "gpt_oss": "gptoss"}


def extract_tool_calls(text: str, family: str | None = None):
    """(content, tool_calls): with a family, only that parser; otherwise the first parser that recognises the text."""
    order = [PARSERS[family]] if family in PARSERS else [parse_deepseek, parse_kimi, parse_gptoss, parse_mistral, parse_glm, parse_hermes, parse_llama3]
    for p in order:
        r = p(text)
        if r is not None:
            return r
    return text, []


def split_reasoning(text: str, open_tag="<think>", close_tag="</think>", starts_in_reasoning=False):
    """(reasoning, content).  ``starts_in_reasoning``: the template already opened the block in the prompt."""
    if open_tag in text:
        pre, rest = text.split(open_tag, 1)
        if close_tag in rest:
            r, post = rest.split(close_tag, 1)
            return r.strip(), (pre + post).strip()
        return rest.strip(), pre.strip()              # generation ended inside the block
    if starts_in_reasoning:
        if close_tag in text:
            r, post = text.split(close_tag, 1)
            return r.strip(), post.strip()
        return text.strip(), ""
    return None, text


class StreamSplitter:
    """Incremental reasoning split: feed text deltas, get (reasoning_delta, content_delta) back.  Text that might be the
    beginning of a tag is held back until it is decided."""

    def __init__(self, open_tag="<think>", close_tag="</think>", starts_in_reasoning=False):
        self.open, self.close = open_tag, close_tag
        self.in_reasoning = starts_in_reasoning
        self.seen_open = starts_in_reasoning
        self.buf = ""

    def _held(self, s: str, tag: str) -> int:
        for n in range(min(len(tag) - 1, len(s)), 0, -1):
            if tag.startswith(s[-n:]):
                return n
        return 0

    def feed(self, delta: str, final: bool = False):
        self.buf += delta
        r_out, c_out = "", ""
        while True:
            tag = self.close if self.in_reasoning else self.open
            if not self.in_reasoning and self.seen_open:
                tag = None                           # one block per message: after it closes everything is content
            if tag and tag in self.buf:
                pre, self.buf = self.buf.split(tag, 1)
                if self.in_reasoning:
                    r_out += pre
                else:
                    c_out += pre
                    self.seen_open = True
                self.in_reasoning = not self.in_reasoning
                continue
            hold = 0 if (final or not tag) else self._held(self.buf, tag)
            emit, self.buf = (self.buf[:len(self.buf) - hold], self.buf[len(self.buf) - hold:]) if hold else (self.buf, "")
            if self.in_reasoning:
                r_out += emit
            else:
                c_out += emit
            return r_out, c_out
