"""Guided decoding: constrain generation to a grammar by filtering the candidate tokens of every step.

``JsonPrefix`` is an incremental recogniser of JSON text (RFC 8259) that answers "is this still the prefix of a valid
JSON document?" one character at a time; ``GuidedJson`` keeps one per request and, given a step's logits, returns the
highest-scoring token among the top candidates whose text keeps the prefix valid (end-of-sequence once the document
is complete).  Used for ``response_format: {"type": "json_object"}``.  Reference: crates/plowrt/src/text/guided.rs."""
from __future__ import annotations

import copy

import numpy as np

_WS = " \t\n\r"
_LITERALS = ("true", "false", "null")


class JsonPrefix:
    """Character-level pushdown recogniser.  ``require_object``: the document must be an object."""

    def __init__(self, require_object: bool = True):
        self.stack = []            # 'obj_key', 'obj_colon', 'obj_value', 'obj_next', 'arr_value', 'arr_next'
        self.mode = "value"        # value | string | escape | unicode | number | literal | done
        self.is_key = False
        self.buf = ""              # literal / number / unicode digits in progress
        self.started = False
        self.require_object = require_object
        self.after_comma = False   # inside an object right after ',': a key must follow, '}' would be a trailing comma

    @property
    def complete(self) -> bool:
        return self.mode == "done" or (self.mode == "number" and not self.stack and self._number_ok(self.buf) and not self.require_object)

    def clone(self) -> "JsonPrefix":
        c = copy.copy(self)
        c.stack = list(self.stack)
        return c

    @staticmethod
    def _number_prefix_ok(s: str) -> bool:
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)?(\.\d*)?([eE][+-]?\d*)?", s) is not None and s not in ("",) and \
            not re.fullmatch(r"-?\.\d*.*", s) and (not ("e" in s.lower()) or re.search(r"\d", s.split("e")[0].split("E")[0]) is not None)

    @staticmethod
    def _number_ok(s: str) -> bool:
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?", s) is not None

    def _value_done(self) -> None:
        if not self.stack:
            self.mode = "done"
            return
        top = self.stack[-1]
        if top == "obj_value":
            self.stack[-1] = "obj_next"
        elif top == "arr_value":
            self.stack[-1] = "arr_next"
        self.mode = "between"

    def feed(self, ch: str) -> bool:
        m = self.mode
        if m == "done":
            return ch in _WS
        if m == "string":
            if ch == "\\":
                self.mode = "escape"
            elif ch == '"':
                if self.is_key:
                    self.stack[-1] = "obj_colon"
                    self.mode = "between"
                else:
                    self._value_done()
            elif ord(ch) < 0x20:
                return False
            return True
        if m == "escape":
            if ch in '"\\/bfnrt':
                self.mode = "string"
                return True
            if ch == "u":
                self.mode, self.buf = "unicode", ""
                return True
            return False
        if m == "unicode":
            if ch not in "0123456789abcdefABCDEF":
                return False
            self.buf += ch
            if len(self.buf) == 4:
                self.mode = "string"
            return True
        if m == "literal":
            self.buf += ch
            if any(l.startswith(self.buf) for l in _LITERALS):
                if self.buf in _LITERALS:
                    self._value_done()
                return True
            return False
        if m == "number":
            if self._number_prefix_ok(self.buf + ch):
                self.buf += ch
                return True
            if not self._number_ok(self.buf):
                return False
            self._value_done()           # the number ended; this character belongs to what follows
            return self.feed(ch)
        if ch in _WS:
            return True
        if m == "value":
            if not self.started and self.require_object and ch != "{":
                return False
            self.started = True
            if ch == "{":
                self.stack.append("obj_key")
                self.after_comma = False
                self.mode = "between"
            elif ch == "[":
                self.stack.append("arr_value")
                self.mode = "value_or_close"
            elif ch == '"':
                self.mode, self.is_key = "string", False
            elif ch in "-0123456789":
                self.mode, self.buf = "number", ch
            elif ch in "tfn":
                self.mode, self.buf = "literal", ch
            else:
                return False
            return True
        if m == "value_or_close":
            if ch == "]":
                self.stack.pop()
                self._value_done()
                return True
            self.mode = "value"
            return self.feed(ch)
        # between tokens inside a container
        top = self.stack[-1] if self.stack else None
        if top == "obj_key":
            if ch == '"':
                self.mode, self.is_key, self.after_comma = "string", True, False
                return True
            if ch == "}" and not self.after_comma:
                self.stack.pop()
                self._value_done()
                return True
            return False
        if top == "obj_colon":
            if ch == ":":
                self.stack[-1] = "obj_value"
                self.mode = "value"
                return True
            return False
        if top == "obj_next":
            if ch == ",":
                self.stack[-1] = "obj_key"
                self.after_comma = True
                return True
            if ch == "}":
                self.stack.pop()
                self._value_done()
                return True
            return False
        if top == "arr_next":
            if ch == ",":
                self.stack[-1] = "arr_value"
                self.mode = "value"
                return True
            if ch == "]":
                self.stack.pop()
                self._value_done()
                return True
            return False
        return False

    def feed_text(self, s: str) -> bool:
        for ch in s:
            if not self.feed(ch):
                return False
        return True


class GuidedJson:
    def __init__(self, decode_token, eos_id: int, top_candidates: int = 64):
        """decode_token(id) -> text of one token; eos_id is emitted once the document is complete."""
        self.decode_token, self.eos_id, self.top = decode_token, eos_id, top_candidates
        self.state = JsonPrefix()

    def pick(self, logits: np.ndarray) -> int:
        if self.state.complete:
            return self.eos_id
        order = np.argsort(-logits)
        for tok in order[:self.top].tolist() + [None]:
            if tok is None:
                break
            text = self.decode_token(tok)
            if not text:
                continue
            trial = self.state.clone()
            if trial.feed_text(text):
                self.state = trial
                return int(tok)
        # nothing among the top candidates fits: close the document with the cheapest valid continuation
        for text_tok in order.tolist():
            text = self.decode_token(text_tok)
            trial = self.state.clone()
            if text and trial.feed_text(text):
                self.state = trial
                return int(text_tok)
        return self.eos_id
