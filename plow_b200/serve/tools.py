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


def parse_qwen3_coder(text: str):
    """<tool_call><function=NAME><parameter=k>v</parameter>…</function></tool_call>  (Qwen3-Coder XML form)"""
    calls = []
    for m in re.finditer(r"<function=([\w.\-]+)>(.*?)</function>", text, re.S):
        args = {}
        for k, v in re.findall(r"<parameter=([\w.\-]+)>\n?(.*?)\n?</parameter>", m.group(2), re.S):
            try:
                args[k] = json.loads(v)
            except json.JSONDecodeError:
                args[k] = v
        calls.append(_call(m.group(1), args))
    if not calls:
        return None
    head = re.sub(r"<tool_call>.*?</tool_call>|<function=.*?</function>", "", text, flags=re.S)
    return head.strip(), calls


def _py_value(node):
    import ast
    if isinstance(node, ast.Constant):
        return node.value
    if isinstance(node, (ast.List, ast.Tuple)):
        return [_py_value(e) for e in node.elts]
    if isinstance(node, ast.Dict):
        return {_py_value(k): _py_value(v) for k, v in zip(node.keys, node.values)}
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
        return -_py_value(node.operand)
    if isinstance(node, ast.Name) and node.id in ("true", "false", "null", "True", "False", "None"):
        return {"true": True, "false": False, "null": None, "True": True, "False": False, "None": None}[node.id]
    raise ValueError("not a literal")


def parse_pythonic(text: str):
    """[get_weather(city="Paris", days=3), other(x=[1, 2])]  (Llama 4 / pythonic tool calls: a list of call expressions)"""
    import ast
    body = text.strip().replace("<|python_start|>", "").replace("<|python_end|>", "").strip()
    if not (body.startswith("[") and body.endswith("]")):
        return None
    try:
        tree = ast.parse(body, mode="eval").body
        if not isinstance(tree, ast.List) or not tree.elts:
            return None
        calls = []
        for e in tree.elts:
            if not isinstance(e, ast.Call) or e.args:
                return None
            name = ast.unparse(e.func)
            calls.append(_call(name, {kw.arg: _py_value(kw.value) for kw in e.keywords}))
    except (SyntaxError, ValueError):
        return None
    return "", calls


def parse_granite(text: str):
    """<|tool_call|>[{"name": ..., "arguments": {...}}]  or  <tool_call>[...]  (Granite 3.x)"""
    for tag in ("<|tool_call|>", "<tool_call>["):
        if tag in text:
            head, body = text.split(tag, 1)
            body = ("[" + body) if tag.endswith("[") else body
            try:
                obj, _ = json.JSONDecoder().raw_decode(body.strip())
            except json.JSONDecodeError:
                return None
            calls = _json_calls(obj)
            return (head.strip(), calls) if calls else None
    return None


def parse_phi4(text: str):
    """functools[{"name": ..., "arguments": {...}}, ...]  (Phi-4-mini)"""
    if "functools[" not in text:
        return None
    head, body = text.split("functools", 1)
    try:
        obj, _ = json.JSONDecoder().raw_decode(body.strip())
    except json.JSONDecodeError:
        return None
    calls = _json_calls(obj)
    return (head.strip(), calls) if calls else None


def parse_minimax(text: str):
    """<tool_calls>\n{"name": ..., "arguments": {...}}\n{...}\n</tool_calls>  (MiniMax: one JSON object per line)"""
    m = re.search(r"<tool_calls>\s*(.*?)\s*</tool_calls>", text, re.S)
    if not m:
        return None
    calls = []
    for line in m.group(1).splitlines():
        line = line.strip()
        if not line:
            continue
        try:
            calls += _json_calls(json.loads(line))
        except json.JSONDecodeError:
            return None
    return (text[:m.start()] + text[m.end():]).strip(), calls if calls else None


def parse_internlm(text: str):
    """<|action_start|><|plugin|>{"name": ..., "parameters": {...}}<|action_end|>  (InternLM 2.5 / 3)"""
    calls = []
    for m in re.finditer(r"<\|action_start\|><\|plugin\|>\s*(.*?)\s*<\|action_end\|>", text, re.S):
        try:
            calls += _json_calls(json.loads(m.group(1)))
        except json.JSONDecodeError:
            return None
    return (text.split("<|action_start|>", 1)[0].strip(), calls) if calls else None


def parse_json_list(text: str):
    """A bare JSON list of {"name", "arguments"} objects, optionally fenced  (xLAM, Jamba, Hunyuan-style plain JSON)"""
    body = text.strip()
    m = re.fullmatch(r"```(?:json)?\s*(.*?)\s*```", body, re.S)
    if m:
        body = m.group(1)
    if not body.startswith("["):
        return None
    try:
        obj = json.loads(body)
    except json.JSONDecodeError:
        return None
    calls = _json_calls(obj) if isinstance(obj, list) and all(isinstance(o, dict) and "name" in o for o in obj) else []
    return ("", calls) if calls else None


PARSERS = {"qwen3_coder": parse_qwen3_coder, "pythonic": parse_pythonic, "llama4": parse_pythonic, "granite": parse_granite,
           "phi4": parse_phi4, "minimax": parse_minimax, "internlm": parse_internlm, "json": parse_json_list, "xlam": parse_json_list,
           "hermes": parse_hermes, "qwen": parse_hermes, "llama3": parse_llama3, "mistral": parse_mistral,
           "deepseek": parse_deepseek, "glm": parse_glm, "kimi": parse_kimi, "gptoss": parse_gptoss}

FAMILY_OF_MODEL_TYPE = {"llama": "llama3", "qwen2": "hermes", "qwen3": "hermes", "qwen3_moe": "hermes", "qwen3_next": "hermes",
                        "mistral": "mistral", "mixtral": "mistral", "deepseek_v3": "deepseek", "glm_moe_dsa": "glm", "glm4_moe": "glm",
                        "kimi_k2": "kimi", "gpt_oss": "gptoss", "llama4": "pythonic", "granite": "granite", "phi3": "phi4",
                        "minimax": "minimax", "internlm2": "internlm", "internlm3": "internlm"}


def extract_tool_calls(text: str, family: str | None = None):
    """(content, tool_calls): with a family, only that parser; otherwise the first parser that recognises the text."""
    order = [PARSERS[family]] if family in PARSERS else [parse_deepseek, parse_kimi, parse_gptoss, parse_mistral, parse_granite, parse_phi4,
                                                         parse_minimax, parse_internlm, parse_qwen3_coder, parse_glm, parse_hermes,
                                                         parse_llama3, parse_pythonic, parse_json_list]
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
