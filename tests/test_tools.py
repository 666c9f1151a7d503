"""Tool-call parsers per model family and the reasoning split (whole-message and streaming)."""
import json


def test_family_parsers():
    from plow_b200.serve import tools as t
    c, calls = t.extract_tool_calls('Sure.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>', "hermes")
    assert c == "Sure." and calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Paris"}
    c, calls = t.extract_tool_calls('<|python_tag|>{"name": "f", "parameters": {"x": 1}}; {"name": "g", "parameters": {}}<|eom_id|>', "llama3")
    assert [k["function"]["name"] for k in calls] == ["f", "g"]
    c, calls = t.extract_tool_calls('ok [TOOL_CALLS][{"name": "add", "arguments": {"a": 1, "b": 2}}]', "mistral")
    assert c == "ok" and json.loads(calls[0]["function"]["arguments"])["b"] == 2
    ds = 'Let me check.<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>search\n```json\n{"q": "b200"}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>'
    c, calls = t.extract_tool_calls(ds)                      # family detected from the text
    assert c == "Let me check." and calls[0]["function"]["name"] == "search"
    glm = '<tool_call>lookup\n<arg_key>id</arg_key>\n<arg_value>42</arg_value>\n<arg_key>name</arg_key>\n<arg_value>plow</arg_value>\n</tool_call>'
    c, calls = t.extract_tool_calls(glm, "glm")
    assert json.loads(calls[0]["function"]["arguments"]) == {"id": 42, "name": "plow"}
    kimi = '<|tool_calls_section_begin|><|tool_call_begin|>functions.run:0<|tool_call_argument_begin|>{"cmd": "ls"}<|tool_call_end|><|tool_calls_section_end|>'
    c, calls = t.extract_tool_calls(kimi)
    assert calls[0]["function"]["name"] == "run" and c == ""
    oss = '<|channel|>commentary to=functions.get_time <|constrain|>json<|message|>{"tz": "UTC"}<|call|>'
    c, calls = t.extract_tool_calls(oss, "gptoss")
    assert calls[0]["function"]["name"] == "get_time"
    assert t.extract_tool_calls("just text") == ("just text", [])
    assert t.extract_tool_calls('<tool_call>{broken</tool_call>', "hermes") == ('<tool_call>{broken</tool_call>', [])


def test_reasoning_split_whole_and_streaming():
    from plow_b200.serve import tools as t
    assert t.split_reasoning("<think>a b</think>answer") == ("a b", "answer")
    assert t.split_reasoning("no tags") == (None, "no tags")
    assert t.split_reasoning("plan</think>go", starts_in_reasoning=True) == ("plan", "go")
    assert t.split_reasoning("<think>cut off") == ("cut off", "")
    s = t.StreamSplitter()
    pieces = ["<th", "ink>step", " one</th", "ink>The ans", "wer <b>"]
    r, c = "", ""
    for i, p in enumerate(pieces):
        dr, dc = s.feed(p, final=i == len(pieces) - 1)
        r += dr
        c += dc
    assert r == "step one" and c == "The answer <b>"


def test_json_prefix_recogniser_and_guided_pick():
    import numpy as np
    from plow_b200.text.guided import GuidedJson, JsonPrefix
    good = ['{"a": 1}', '{"a": [1, 2, {"b": null}], "c": "x\\n"}', '{}', '{"k": [], "z": {}}', '{"a": -1.5e3, "b": false}  ']
    bad = ['{"a": 1,}', '[1]', '{"a" 1}', '{"a": 01}', '{"a": 1} x', '{,', '{"a": tru3}']
    for s in good:
        p = JsonPrefix()
        assert p.feed_text(s) and p.complete, s
    for s in bad:
        assert not JsonPrefix().feed_text(s), s
    p = JsonPrefix()
    assert p.feed_text('{"a": tru') and not p.complete
    # a byte-level "model" that prefers garbage: the guide still produces a valid document
    vocab = [chr(c) for c in range(32, 127)]
    g = GuidedJson(lambda t: vocab[t] if t < len(vocab) else "", eos_id=len(vocab), top_candidates=16)
    rng = np.random.default_rng(0)
    text = ""
    for step in range(200):
        logits = rng.standard_normal(len(vocab) + 1)
        if step > 12:
            logits[vocab.index("}")] += 6.0          # the model eventually wants to close
            logits[vocab.index('"')] += 3.0
        tok = g.pick(logits)
        if tok == len(vocab):
            break
        text += vocab[tok]
    import json
    assert isinstance(json.loads(text), dict), text


def test_more_tool_call_families():
    import json
    from plow_b200.serve import tools as t

    def args(c):
        return json.loads(c["function"]["arguments"])
    content, calls = t.extract_tool_calls('I will look.\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>', "qwen3_coder")
    assert content == "I will look." and calls[0]["function"]["name"] == "get_weather" and args(calls[0]) == {"city": "Paris", "days": 3}
    content, calls = t.extract_tool_calls('[get_weather(city="Paris", days=3), lookup(ids=[1, 2], exact=True, opts={"k": -1.5})]', "pythonic")
    assert content == "" and [c["function"]["name"] for c in calls] == ["get_weather", "lookup"]
    assert args(calls[1]) == {"ids": [1, 2], "exact": True, "opts": {"k": -1.5}}
    assert t.parse_pythonic("[1, 2, 3]") is None and t.parse_pythonic("[f(1)]") is None and t.parse_pythonic("[os.system('x')") is None
    content, calls = t.extract_tool_calls('<|tool_call|>[{"name": "f", "arguments": {"a": 1}}]', "granite")
    assert content == "" and args(calls[0]) == {"a": 1}
    content, calls = t.extract_tool_calls('Sure. functools[{"name": "f", "arguments": {"a": 1}}, {"name": "g", "arguments": {}}]', "phi4")
    assert content == "Sure." and len(calls) == 2
    content, calls = t.extract_tool_calls('ok\n<tool_calls>\n{"name": "f", "arguments": {"a": 1}}\n{"name": "g", "arguments": {"b": "x"}}\n</tool_calls>', "minimax")
    assert content == "ok" and args(calls[1]) == {"b": "x"}
    content, calls = t.extract_tool_calls('thinking<|action_start|><|plugin|>{"name": "f", "parameters": {"a": 1}}<|action_end|>', "internlm")
    assert content == "thinking" and args(calls[0]) == {"a": 1}
    content, calls = t.extract_tool_calls('```json\n[{"name": "f", "arguments": {"a": 1}}]\n```', "xlam")
    assert content == "" and calls[0]["function"]["name"] == "f"
    # without a family the text itself decides, and plain prose stays prose
    for text, name in (('functools[{"name": "f", "arguments": {}}]', "f"), ('[g(x=1)]', "g"),
                       ('<|action_start|><|plugin|>{"name": "h", "parameters": {}}<|action_end|>', "h")):
        assert t.extract_tool_calls(text)[1][0]["function"]["name"] == name
    assert t.extract_tool_calls("The list [1, 2, 3] has three items.") == ("The list [1, 2, 3] has three items.", [])
    assert len(set(t.PARSERS.values())) >= 14
