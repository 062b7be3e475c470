"""Request-owned grammar constraints.

Two parts, as in the reference (``hipengine/generation/grammar.py``): (1) a generator that turns the JSON-schema
parameter blocks of OpenAI tool definitions into a Lark-syntax grammar for the Qwen XML tool-call format
(``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``), and (2) a matcher
that masks logits token by token.  The matcher delegates to ``llguidance`` (``LLMatcher`` / ``LLTokenizer``) when
that package is importable; in images without it ``grammar_available()`` is False and requests carrying a grammar
are refused before generation with ``unsupported_parameter`` (the server and ``SamplingParams`` check this), so a
constraint is never silently dropped.  The generator is pure Python and always available: the tool-call result
policy uses the same schema walk to validate arguments after generation.
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Mapping, Optional, Sequence

_NAME_OK = re.compile(r"^[A-Za-z_][A-Za-z0-9_\-\.]*$")


def grammar_available() -> bool:
    try:
        import llguidance  # noqa: F401
        return True
    except Exception:
        return False


def _lit(s: str) -> str:
    return json.dumps(s)


def _value_rule(schema: Mapping[str, Any], name: str, rules: Dict[str, str]) -> str:
    """Adds rules for one parameter value and returns the rule name.  Scalars are written bare inside the
    <parameter> element; objects and arrays as JSON."""
    t = schema.get("type")
    if "enum" in schema:
        rules[name] = " | ".join(_lit(v if isinstance(v, str) else json.dumps(v)) for v in schema["enum"])
    elif t == "integer":
        rules[name] = "/-?(0|[1-9][0-9]*)/"
    elif t == "number":
        rules[name] = "/-?(0|[1-9][0-9]*)(\\.[0-9]+)?([eE][+-]?[0-9]+)?/"
    elif t == "boolean":
        rules[name] = '"true" | "false"'
    elif t == "string":
        rules[name] = "/[^<]*/"                      # any text up to the closing tag
    elif t in ("object", "array"):
        rules[name] = "json_value"
        rules.setdefault("json_value", 'json_object | json_array | json_string | json_number | "true" | "false" | "null"')
        rules.setdefault("json_object", '"{" [json_pair ("," json_pair)*] "}"')
        rules.setdefault("json_pair", 'json_string ":" json_value')
        rules.setdefault("json_array", '"[" [json_value ("," json_value)*] "]"')
        rules.setdefault("json_string", '/"([^"\\\\]|\\\\.)*"/')
        rules.setdefault("json_number", "/-?(0|[1-9][0-9]*)(\\.[0-9]+)?([eE][+-]?[0-9]+)?/")
    else:
        rules[name] = "/[^<]*/"
    return name


def tool_call_grammar(tools: Sequence[Mapping[str, Any]], allow_text_before: bool = True,
                      parallel: bool = True, only: Optional[str] = None) -> str:
    """Lark grammar accepting zero or more XML tool calls to the given functions (optionally after free text).

    Required parameters must appear, in the order of the schema's ``properties``; optional ones may be omitted.
    ``only`` restricts the grammar to one function name (``tool_choice`` naming a function)."""
    rules: Dict[str, str] = {}
    fn_rules: List[str] = []
    for ti, tool in enumerate(tools):
        fn = tool.get("function", tool)
        fname = fn.get("name", "")
        if not _NAME_OK.match(fname):
            raise ValueError(f"tool name {fname!r} cannot be expressed in the tool-call grammar")
        if only is not None and fname != only:
            continue
        params = fn.get("parameters") or {}
        props = params.get("properties") or {}
        required = set(params.get("required") or [])
        parts: List[str] = []
        for pi, (key, sch) in enumerate(props.items()):
            if not _NAME_OK.match(key):
                raise ValueError(f"parameter name {key!r} cannot be expressed in the tool-call grammar")
            vr = _value_rule(sch or {}, f"v_{ti}_{pi}", rules)
            pr = f"p_{ti}_{pi}"
            rules[pr] = f'{_lit("<parameter=" + key + ">")} ws {vr} ws "</parameter>" ws'
            parts.append(pr if key in required else f"[{pr}]")
        body = " ".join(parts) if parts else ""
        rules[f"f_{ti}"] = f'{_lit("<function=" + fname + ">")} ws {body} "</function>"'.replace("  ", " ")
        fn_rules.append(f"f_{ti}")
    if not fn_rules:
        raise ValueError("no tool matches the requested tool choice")
    rules["call"] = '"<tool_call>" ws (' + " | ".join(fn_rules) + ') ws "</tool_call>"'
    many = "call (ws call)*" if parallel else "call"
    start = f"[text] {many}" if allow_text_before else many
    lines = [f"start: {start}", "text: /[^<]+/", "ws: /[ \\t\\n]*/"]
    for k in sorted(rules):
        lines.append(f"{k}: {rules[k]}")
    return "\n".join(lines) + "\n"


class GrammarMatcher:
    """Token-level matcher over an ``llguidance`` grammar.  Only constructible when the package is present."""

    def __init__(self, lark_grammar: str, vocab: Sequence[bytes], eos_token_id: int):
        if not grammar_available():
            raise RuntimeError("grammar constraints need the llguidance package, which is not installed")
        import llguidance
        self._ll = llguidance
        self.tokenizer = llguidance.LLTokenizer(llguidance.TokenizerWrapper(
            _VocabAdapter(vocab, eos_token_id)))
        self.matcher = llguidance.LLMatcher(self.tokenizer, llguidance.LLMatcher.grammar_from_lark(lark_grammar))

    def allowed_mask(self):
        return self.matcher.compute_logit_bias()

    def accept(self, token_id: int) -> bool:
        return bool(self.matcher.consume_token(int(token_id)))

    def finished(self) -> bool:
        return bool(self.matcher.is_stopped())


class _VocabAdapter:
    def __init__(self, vocab: Sequence[bytes], eos: int):
        self.tokens = list(vocab)
        self.eos_token_id = eos
        self.bos_token_id = None
        self.special_token_ids = [eos]

    def __call__(self, s: str) -> List[int]:
        raise NotImplementedError("canonical tokenisation is not needed for masking")
