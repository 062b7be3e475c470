"""Chat prompt rendering.

Qwen-family models use the ChatML frame (``<|im_start|>role\\ncontent<|im_end|>``) with a prompt-injected
tool block and ``<tool_call><function=NAME><parameter=K>V</parameter></function></tool_call>`` call syntax;
thinking is opened with ``<think>`` in the assistant turn (behaviour described in the reference's
``docs/API.md:495,1495-1600``; model-owned templates live in ``hipengine/chat/*.py``).  Gemma 4 uses
``<start_of_turn>role`` frames.  A GGUF-embedded Jinja template (``tokenizer.chat_template``) takes
precedence when present.
"""
from __future__ import annotations

import json
from typing import Any, Mapping, Optional, Sequence

VALID_ROLES = ("system", "developer", "user", "assistant", "tool")

TOOL_PREAMBLE = (
    "# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
    "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n{tools}\n</tools>\n\n"
    "For each function call, return the call within <tool_call></tool_call> XML tags:\n"
    "<tool_call>\n<function=example_function>\n<parameter=example_parameter>\nvalue\n</parameter>\n"
    "</function>\n</tool_call>"
)


def _content_text(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    parts = []
    for p in content:
        if isinstance(p, Mapping):
            if p.get("type") == "text":
                parts.append(str(p.get("text", "")))
            elif p.get("type") in ("image_url", "image"):
                parts.append("<|vision_start|><|image_pad|><|vision_end|>")
        else:
            parts.append(str(p))
    return "".join(parts)


def render_tool_call_xml(name: str, arguments: Mapping[str, Any]) -> str:
    lines = ["<tool_call>", f"<function={name}>"]
    for k, v in arguments.items():
        sv = v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)
        lines += [f"<parameter={k}>", sv, "</parameter>"]
    lines += ["</function>", "</tool_call>"]
    return "\n".join(lines)


def render_chatml(messages: Sequence[Mapping[str, Any]], tools: Optional[Sequence[Mapping[str, Any]]] = None,
                  add_generation_prompt: bool = True, enable_thinking: bool = True) -> str:
    out = []
    msgs = list(messages)
    sys_text = ""
    if msgs and msgs[0].get("role") in ("system", "developer"):
        sys_text = _content_text(msgs[0].get("content"))
        msgs = msgs[1:]
    if tools:
        tool_lines = "\n".join(json.dumps(t, ensure_ascii=False) for t in tools)
        sys_text = (sys_text + "\n\n" if sys_text else "") + TOOL_PREAMBLE.format(tools=tool_lines)
    if sys_text:
        out.append(f"<|im_start|>system\n{sys_text}<|im_end|>\n")
    for m in msgs:
        role = m.get("role")
        if role not in VALID_ROLES:
            raise ValueError(f"unknown chat role {role!r}")
        text = _content_text(m.get("content"))
        if role == "assistant":
            body = text
            for tc in m.get("tool_calls") or ():
                fn = tc.get("function", {})
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except Exception:
                        args = {"_raw": args}
                body += ("\n" if body else "") + render_tool_call_xml(fn.get("name", ""), args)
            out.append(f"<|im_start|>assistant\n{body}<|im_end|>\n")
        elif role == "tool":
            out.append(f"<|im_start|>user\n<tool_response>\n{text}\n</tool_response><|im_end|>\n")
        else:
            r = "system" if role == "developer" else role
            out.append(f"<|im_start|>{r}\n{text}<|im_end|>\n")
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
        out.append("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n")
    return "".join(out)


def render_gemma(messages: Sequence[Mapping[str, Any]], add_generation_prompt: bool = True) -> str:
    out = ["<bos>"]
    sys_text = ""
    for m in messages:
        role = m.get("role")
        text = _content_text(m.get("content"))
        if role in ("system", "developer"):
            sys_text = text
            continue
        r = "model" if role == "assistant" else "user"
        if r == "user" and sys_text:
            text = sys_text + "\n\n" + text
            sys_text = ""
        out.append(f"<start_of_turn>{r}\n{text}<end_of_turn>\n")
    if add_generation_prompt:
        out.append("<start_of_turn>model\n")
    return "".join(out)


def render_chat(messages: Sequence[Mapping[str, Any]], tools=None, enable_thinking: bool = True,
                arch: str = "qwen35", jinja_template: Optional[str] = None, add_generation_prompt: bool = True) -> str:
    if jinja_template:
        try:
            import jinja2
            env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
            env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
            return env.from_string(jinja_template).render(messages=list(messages), tools=tools,
                                                          add_generation_prompt=add_generation_prompt,
                                                          enable_thinking=enable_thinking)
        except ImportError:
            pass
    if arch.startswith("gemma"):
        return render_gemma(messages, add_generation_prompt)
    return render_chatml(messages, tools, add_generation_prompt, enable_thinking)
