"""Chat templates, output parsing (reasoning split, XML and JSON tool calls, incremental stream parser) and the JSON
Schema subset validator: pure host code, checked against hand-written expectations and against each other."""
import json
import random

import pytest

from hipengine_b200.chat.templates import render_chat, render_chatml, render_gemma, render_tool_call_xml
from hipengine_b200.server import json_schema as JS
from hipengine_b200.server.chat_output import ChatStreamParser, parse_chat_output, parse_tool_body, split_reasoning

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {
    "type": "object", "properties": {"city": {"type": "string"}, "days": {"type": "integer"}}, "required": ["city"]}}}]


def test_chatml_rendering_roles_tools_and_generation_prompt():
    msgs = [{"role": "developer", "content": "be terse"}, {"role": "user", "content": [{"type": "text", "text": "hi "},
                                                                                     {"type": "text", "text": "there"}]},
            {"role": "assistant", "content": "", "tool_calls": [{"id": "c1", "type": "function", "function": {
                "name": "get_weather", "arguments": json.dumps({"city": "Oslo", "days": 2})}}]},
            {"role": "tool", "tool_call_id": "c1", "content": "sunny"}]
    p = render_chatml(msgs, tools=TOOLS, enable_thinking=True)
    assert p.startswith("<|im_start|>system\nbe terse\n\n") and '"name": "get_weather"' in p.split("<|im_end|>")[0]
    assert "<|im_start|>user\nhi there<|im_end|>" in p
    assert "<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n<parameter=days>\n2\n</parameter>" in p
    assert "<|im_start|>user\n<tool_response>\nsunny\n</tool_response><|im_end|>" in p
    assert p.endswith("<|im_start|>assistant\n<think>\n")
    assert render_chatml(msgs[:2], enable_thinking=False).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert not render_chatml(msgs[:2], add_generation_prompt=False).endswith("assistant\n")
    with pytest.raises(ValueError, match="unknown chat role"):
        render_chatml([{"role": "narrator", "content": "x"}])
    # a call rendered by the template parses back to the same call
    back = parse_tool_body(render_tool_call_xml("get_weather", {"city": "Oslo", "days": 2, "opts": {"a": [1, 2]}})
                           .replace("<tool_call>", "").replace("</tool_call>", ""))
    assert back.name == "get_weather" and back.arguments == {"city": "Oslo", "days": 2, "opts": {"a": [1, 2]}}


def test_gemma_rendering_and_dispatch():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "u1"}, {"role": "assistant", "content": "a1"},
            {"role": "user", "content": "u2"}]
    g = render_gemma(msgs)
    assert g == ("<bos><start_of_turn>user\nS\n\nu1<end_of_turn>\n<start_of_turn>model\na1<end_of_turn>\n"
                 "<start_of_turn>user\nu2<end_of_turn>\n<start_of_turn>model\n")
    assert render_chat(msgs, arch="gemma4") == g and render_chat(msgs, arch="qwen35").startswith("<|im_start|>system")
    tpl = "{% for m in messages %}[{{ m.role }}:{{ m.content }}]{% endfor %}{% if add_generation_prompt %}>{% endif %}"
    assert render_chat(msgs[1:3], jinja_template=tpl) == "[user:u1][assistant:a1]>"


def test_reasoning_split_and_tool_call_parsing():
    assert split_reasoning("plain") == (None, "plain", True)
    assert split_reasoning("<think>\nwhy\n</think>\n\nanswer") == ("why", "answer", True)
    assert split_reasoning("why</think>answer", starts_in_think=True) == ("why", "answer", True)
    assert split_reasoning("never closes", starts_in_think=True) == ("never closes", "", False)
    text = ("r1</think>\n\nLet me check.\n<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n"
            "<parameter=days>\n3\n</parameter>\n</function>\n</tool_call>\n"
            '<tool_call>{"name": "get_weather", "arguments": {"city": "Rome"}}</tool_call>')
    p = parse_chat_output(text, starts_in_think=True)
    assert p.reasoning == "r1" and p.content == "Let me check." and p.thinking_closed
    assert [(c.name, c.arguments) for c in p.tool_calls] == [("get_weather", {"city": "Oslo", "days": 3}),
                                                             ("get_weather", {"city": "Rome"})]
    assert p.tool_calls[0].id != p.tool_calls[1].id
    assert json.loads(p.tool_calls[0].to_openai(0)["function"]["arguments"]) == {"city": "Oslo", "days": 3}
    bad = parse_chat_output("<tool_call>not a call</tool_call>")
    assert bad.tool_calls[0].error and bad.tool_calls[0].name == ""
    cut = parse_chat_output("x<tool_call>\n<function=get_weather>\n<parameter=city>\nOs")      # cut by the length limit
    assert len(cut.tool_calls) == 1 and cut.content == "x"
    assert parse_chat_output("a <tool_call>b</tool_call>", parse_tools=False).content == "a <tool_call>b</tool_call>"
    strs = parse_tool_body("<function=f><parameter=s>\n7\n</parameter><parameter=z>\n007\n</parameter>"
                           "<parameter=t>\nhello world\n</parameter></function>")
    assert strs.arguments == {"s": 7, "z": "007", "t": "hello world"}    # JSON values are decoded, other text stays text


@pytest.mark.parametrize("starts_in_think", [False, True])
def test_stream_parser_agrees_with_the_whole_text_parser_under_any_chunking(starts_in_think):
    body = ("thinking about it\nstill</think>\n\nThe answer < 5 and <b>bold</b>.\n"
            "<tool_call>\n<function=get_weather>\n<parameter=city>\nOslo\n</parameter>\n</function>\n</tool_call>\n"
            "after the call <tool_call>\n<function=get_weather>\n<parameter=city>\nRome\n</parameter>\n</function>\n"
            "</tool_call>")
    text = body if starts_in_think else "<think>\n" + body
    whole = parse_chat_output(text, starts_in_think)
    rng = random.Random(3)
    for trial in range(60):
        cuts = sorted(rng.sample(range(1, len(text)), rng.randrange(0, 25))) if trial else list(range(1, len(text)))
        pieces = [text[a:b] for a, b in zip([0] + cuts, cuts + [len(text)])]
        sp = ChatStreamParser(starts_in_think)
        think, answer, calls = "", "", []
        for i, piece in enumerate(pieces):
            for phase, delta in sp.feed(piece, final=i == len(pieces) - 1):
                if phase == "think":
                    think += delta
                elif phase == "answer":
                    answer += delta
                else:
                    calls.append(delta)
        assert think.strip("\n") == whole.reasoning
        assert answer.replace("\n", "").replace(" ", "") == whole.content.replace("\n", "").replace(" ", "")
        names = [c["function"]["name"] for c in calls if "name" in c["function"]]
        assert names == [c.name for c in whole.tool_calls]
        args = [json.loads(c["function"]["arguments"]) for c in calls if c["function"].get("arguments")]
        assert args == [c.arguments for c in whole.tool_calls]
        assert [c.arguments for c in sp.calls] == [c.arguments for c in whole.tool_calls]
        assert "<think" not in answer and "</think" not in think and "<tool_call" not in answer


def test_json_schema_subset_validator():
    schema = {"type": "object", "required": ["name", "age"], "additionalProperties": False,
              "properties": {"name": {"type": "string", "minLength": 2, "pattern": "^[A-Z]"},
                             "age": {"type": "integer", "minimum": 0, "maximum": 150},
                             "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "minItems": 1, "uniqueItems": True},
                             "kind": {"const": "person"},
                             "contact": {"oneOf": [{"type": "object", "required": ["email"]},
                                                   {"type": "object", "required": ["phone"]}]},
                             "ref": {"$ref": "#/$defs/id"}},
              "$defs": {"id": {"type": "string", "maxLength": 4}},
              "if": {"properties": {"age": {"maximum": 17}}}, "then": {"required": ["guardian"]}}
    JS.check_schema(schema)
    ok = {"name": "Ann", "age": 30, "tags": ["a"], "kind": "person", "contact": {"email": "x"}, "ref": "ab12"}
    assert JS.validate(ok, schema) == []
    cases = [({"name": "Ann"}, "age"), (dict(ok, extra=1), "extra"), (dict(ok, name="a"), "name"),
             (dict(ok, name="ann"), "pattern"), (dict(ok, age=200), "age"), (dict(ok, age=3.5), "age"),
             (dict(ok, tags=[]), "tags"), (dict(ok, tags=["c"]), "tags"), (dict(ok, kind="robot"), "kind"),
             (dict(ok, contact={"email": 1, "phone": 2}), "contact"), (dict(ok, ref="toolong"), "ref"),
             (dict(ok, age=10), "guardian")]
    for inst, needle in cases:
        errs = JS.validate(inst, schema)
        assert errs and any(needle in e for e in errs), (inst, errs)
    assert JS.validate(True, {"type": "integer"})                       # a boolean is not an integer
    assert JS.validate(5, {"not": {"type": "string"}}) == [] and JS.validate("s", {"not": {"type": "string"}})
    assert JS.validate(7, {"anyOf": [{"type": "string"}, {"minimum": 5}]}) == []
    assert JS.validate([1, "a"], {"allOf": [{"type": "array"}, {"items": {"type": "integer"}}]})
    for bad in ({"type": "object", "patternProperties": {"^x": {}}}, {"$ref": "http://elsewhere/schema"},
                {"type": "frobnicate"}, {"type": ["string", "nope"]}, {"properties": {"a": {"contains": {}}}},
                {"anyOf": [{"pattern": "("}]}, {"$ref": "#/$defs/missing"}, {"items": 3}):
        with pytest.raises(JS.SchemaError):
            JS.check_schema(bad)
    # a property NAMED like a keyword is not a keyword
    JS.check_schema({"type": "object", "properties": {"contains": {"type": "string"}, "type": {"enum": ["a"]},
                                                      "patternProperties": {"type": "integer"}}})
    JS.check_schema(True)
