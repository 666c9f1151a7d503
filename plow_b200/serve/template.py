"""Chat templates: the checkpoint's Jinja template rendered in a transformers-compatible sandbox
(``raise_exception``, ``strftime_now``, ``tojson``, Python str/dict methods), with a plain
role-tagged fallback when the checkpoint ships none (reference: crates/plowrt/src/serve/template.rs,
docs/serving-openai-compat.md:7-60)."""
from __future__ import annotations

import datetime
import json
from pathlib import Path

from jinja2 import StrictUndefined, TemplateError
from jinja2.sandbox import ImmutableSandboxedEnvironment

FALLBACK = ("{% for m in messages %}<|{{ m['role'] }}|>\n{{ m['content'] }}\n{% endfor %}"
            "{% if add_generation_prompt %}<|assistant|>\n{% endif %}")


class ChatTemplateError(ValueError):
    pass


def _raise(msg):
    raise ChatTemplateError(msg)


class ChatTemplate:
    def __init__(self, source: str | None = None, bos_token: str = "", eos_token: str = ""):
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, undefined=StrictUndefined)
        env.globals["raise_exception"] = _raise
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        env.filters["tojson"] = lambda v, indent=None, **kw: json.dumps(v, indent=indent, ensure_ascii=False)
        self.source = source or FALLBACK
        self.tpl = env.from_string(self.source)
        self.bos, self.eos = bos_token, eos_token

    @staticmethod
    def from_assets(assets_dir) -> "ChatTemplate":
        d = Path(assets_dir)
        src, bos, eos = None, "", ""
        if (d / "chat_template.jinja").exists():
            src = (d / "chat_template.jinja").read_text()
        if (d / "tokenizer_config.json").exists():
            tc = json.loads((d / "tokenizer_config.json").read_text())
            src = src or tc.get("chat_template")
            tok = lambda v: v.get("content", "") if isinstance(v, dict) else (v or "")
            bos, eos = tok(tc.get("bos_token")), tok(tc.get("eos_token"))
        return ChatTemplate(src, bos, eos)

    def render(self, messages: list, tools: list | None = None, add_generation_prompt: bool = True, **kw) -> str:
        for m in messages:
            c = m.get("content")
            if isinstance(c, list):   # OpenAI content parts -> text
                m["content"] = "".join(p.get("text", "") for p in c if p.get("type") == "text")
            elif c is None:
                m["content"] = ""
        try:
            return self.tpl.render(messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                                   bos_token=self.bos, eos_token=self.eos, **kw)
        except TemplateError as e:
            raise ChatTemplateError(str(e)) from e
