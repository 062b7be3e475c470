"""Pure request lowering: OpenAI request fields -> rendered prompt + ``SamplingParams`` + post-validation plan.

Covers what the reference lowers in ``chat_completions`` (``hipengine/server/api.py:8069`` and helpers;
behaviour in ``docs/API.md:1495-1830``): stop strings -> token sequences, thinking controls -> close-token
budget, ``response_format`` / ``guided_*`` -> JSON close forcing plus result validation, tools -> prompt block
and name constraint, user grammars rejected before generation.
"""
from __future__ import annotations

import json
import re
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..chat.templates import VALID_ROLES, render_chat
from ..generation.constraints import ToolCallConstraintSpec
from ..llm import SamplingParams
from . import json_schema as JS
from .chat_output import THINK_CLOSE, ParsedOutput, ToolCall
from .errors import APIError
from .schemas import ChatCompletionRequest, CompletionRequest

EFFORT_BUDGET = {"none": 0, "minimal": 128, "low": 512, "medium": 2048, "high": 8192}


@dataclass
class ResultPlan:
    """What to check on the finished output."""
    json_mode: Optional[str] = None                 # json_object | json_schema
    schema: Optional[Dict[str, Any]] = None
    regex: Optional[str] = None
    choices: Optional[List[str]] = None
    tools: Dict[str, Dict[str, Any]] = field(default_factory=dict)     # name -> parameters schema
    tool_mode: str = "none"                          # none | auto | required | specific
    tool_specific: Optional[str] = None
    strict_tools: bool = False
    hard_error: bool = False
    starts_in_think: bool = False


def _stops(stop, tokenizer) -> Tuple[Tuple[int, ...], ...]:
    if not stop:
        return ()
    items = [stop] if isinstance(stop, str) else list(stop)
    if len(items) > 8:
        raise APIError("unsupported_parameter", "at most 8 stop sequences are supported", "stop")
    return tuple(tuple(tokenizer.encode(s)) for s in items if s)


def _bias(logit_bias) -> Dict[int, float]:
    out = {}
    for k, v in (logit_bias or {}).items():
        try:
            out[int(k)] = float(v)
        except Exception:
            raise APIError("unsupported_parameter", f"logit_bias key {k!r} is not a token id", "logit_bias") from None
    return out


def _deadline(timeout_ms: Optional[int]) -> Optional[float]:
    """Wall-clock deadline of a request's ``timeout_ms``; zero or absent means none, a negative value is refused."""
    if timeout_ms is None or timeout_ms == 0:
        return None
    if timeout_ms < 0:
        raise APIError("unsupported_parameter", "timeout_ms must be >= 0", "timeout_ms")
    return time.time() + timeout_ms / 1e3


def _params(**kw) -> SamplingParams:
    """``SamplingParams`` from request fields; a value the sampler refuses (negative temperature, top_p outside (0, 1],
    a negative count ...) is the client's error, not the server's."""
    try:
        if int(kw.get("max_tokens", 1)) < 1:
            raise ValueError("max_tokens must be at least 1 (a request always produces a token)")
        return SamplingParams(**kw)
    except (ValueError, TypeError) as exc:
        raise APIError("unsupported_parameter", f"invalid sampling parameter: {exc}") from None


def validate_messages(messages: Sequence[Any]) -> None:
    """Role and tool-transcript rules (``hipengine/server/chat_validation.py``)."""
    if not messages:
        raise APIError("invalid_request", "messages must not be empty", "messages")
    open_calls: Dict[str, bool] = {}
    for i, m in enumerate(messages):
        role = m.role
        if role not in VALID_ROLES:
            raise APIError("invalid_request", f"messages[{i}].role {role!r} is not supported", f"messages[{i}].role")
        if role == "assistant":
            open_calls = {tc.get("id"): True for tc in (m.tool_calls or []) if tc.get("id")}
        elif role == "tool":
            if not m.tool_call_id:
                raise APIError("invalid_request", f"messages[{i}] (tool) needs tool_call_id", f"messages[{i}].tool_call_id")
            if m.tool_call_id not in open_calls:
                raise APIError("invalid_request", f"messages[{i}].tool_call_id does not answer a preceding tool call",
                               f"messages[{i}].tool_call_id")
    if messages[-1].role == "assistant" and not messages[-1].content and not messages[-1].tool_calls:
        raise APIError("invalid_request", "the last message must not be an empty assistant turn", "messages")


def build_completion_params(req: CompletionRequest, tokenizer, default_max: int = 16) -> SamplingParams:
    if req.n < 1 or req.n > 16:
        raise APIError("unsupported_parameter", "n must be in [1, 16]", "n")
    deadline = _deadline(req.timeout_ms)
    return _params(
        max_tokens=req.max_tokens if req.max_tokens is not None else default_max,
        temperature=req.temperature if req.temperature is not None else 1.0,
        top_p=req.top_p if req.top_p is not None else 1.0, top_k=req.top_k or 0, min_p=req.min_p or 0.0,
        presence_penalty=req.presence_penalty, frequency_penalty=req.frequency_penalty,
        repetition_penalty=req.repetition_penalty, logit_bias=_bias(req.logit_bias),
        stop_token_sequences=_stops(req.stop, tokenizer), stop_token_ids=tuple(req.stop_token_ids or ()),
        seed=req.seed, ignore_eos=req.ignore_eos, min_tokens=req.min_tokens, deadline_at=deadline,
        logprobs=req.logprobs is not None, top_logprobs=min(int(req.logprobs or 0), 20),
        speculative_mtp=bool(req.speculative_mtp))


def build_chat(req: ChatCompletionRequest, tokenizer, arch: str, default_max: int = 4096,
               jinja_template: Optional[str] = None) -> Tuple[str, SamplingParams, ResultPlan]:
    if req.grammar is not None or req.guided_grammar is not None:
        raise APIError("unsupported_parameter", "user-supplied grammars are not accepted", "grammar")
    if req.n < 1 or req.n > 16:
        raise APIError("unsupported_parameter", "n must be in [1, 16]", "n")
    if req.top_logprobs is not None and not req.logprobs:
        raise APIError("unsupported_parameter", "top_logprobs requires logprobs=true", "top_logprobs")
    if req.top_logprobs is not None and not (0 <= req.top_logprobs <= 20):
        raise APIError("unsupported_parameter", "top_logprobs must be in [0, 20]", "top_logprobs")
    validate_messages(req.messages)
    # media parts are parsed under hard limits first; the text-only models served here cannot use them, and dropping
    # them silently would answer another question than the one asked
    from .multimodal import MediaError, extract_media
    try:
        media = extract_media(req.messages)
    except MediaError as exc:
        raise APIError("invalid_request", str(exc), exc.param) from None
    if media:
        raise APIError("unsupported_feature",
                       f"the served model is text-only: {len(media)} media part(s) were validated but cannot be used",
                       f"messages[{media[0].message_index}].content[{media[0].part_index}]",
                       extra={"media": [m.as_dict() for m in media]})
    plan = ResultPlan(hard_error=req.invalid_tool_call_error_mode == "hard_error")

    # ---- thinking controls
    kwargs = req.chat_template_kwargs or {}
    enable_thinking = req.enable_thinking if req.enable_thinking is not None else kwargs.get("enable_thinking", True)
    if req.reasoning_effort is not None:
        if req.reasoning_effort not in EFFORT_BUDGET:
            raise APIError("unsupported_parameter", f"reasoning_effort must be one of {sorted(EFFORT_BUDGET)}",
                           "reasoning_effort")
        if req.reasoning_effort == "none":
            enable_thinking = False
    budget = req.thinking_token_budget if req.thinking_token_budget is not None else req.max_think_tokens
    if budget is None and req.reasoning_effort in EFFORT_BUDGET and enable_thinking:
        budget = EFFORT_BUDGET[req.reasoning_effort]
    plan.starts_in_think = bool(enable_thinking) and not arch.startswith("gemma")

    # ---- tools
    tools = None
    constraint = None
    if req.tools:
        tools = [t.model_dump(exclude_none=True) for t in req.tools]
        for t in req.tools:
            if t.type != "function":
                raise APIError("unsupported_parameter", "only function tools are supported", "tools")
            params = t.function.parameters or {"type": "object"}
            try:
                JS.check_schema(params)
            except JS.SchemaError as exc:
                raise APIError("unsupported_parameter", f"tool {t.function.name!r}: {exc}", "tools") from None
            plan.tools[t.function.name] = params
            plan.strict_tools = plan.strict_tools or bool(t.function.strict)
        choice = req.tool_choice if req.tool_choice is not None else "auto"
        if isinstance(choice, dict):
            name = (choice.get("function") or {}).get("name")
            if name not in plan.tools:
                raise APIError("unsupported_parameter", f"tool_choice names unknown function {name!r}", "tool_choice")
            plan.tool_mode, plan.tool_specific = "specific", name
        elif choice in ("auto", "required", "none"):
            plan.tool_mode = choice
        else:
            raise APIError("unsupported_parameter", f"tool_choice {choice!r} is not supported", "tool_choice")
        if plan.tool_mode == "none":
            tools = None
        else:
            import json as _json
            strict = plan.tool_mode in ("required", "specific")
            constraint = ToolCallConstraintSpec(
                tuple(plan.tools), plan.tool_mode, plan.tool_specific,
                tools_json=_json.dumps([t.model_dump() if hasattr(t, "model_dump") else t for t in req.tools])
                if strict else None)
    elif req.tool_choice not in (None, "none", "auto"):
        raise APIError("unsupported_parameter", "tool_choice requires tools", "tool_choice")

    # ---- structured output
    json_hint = ""
    rf = req.response_format
    schema = None
    if rf is not None and rf.type not in ("text", "json_object", "json_schema"):
        raise APIError("unsupported_parameter", f"response_format.type {rf.type!r} is not supported", "response_format")
    if rf is not None and rf.type == "json_schema":
        js = rf.json_schema or {}
        schema = js.get("schema", js)
        plan.json_mode = "json_schema"
    elif rf is not None and rf.type == "json_object":
        plan.json_mode = "json_object"
    if req.guided_json is not None:
        schema = json.loads(req.guided_json) if isinstance(req.guided_json, str) else req.guided_json
        plan.json_mode = "json_schema"
    if schema is not None:
        try:
            JS.check_schema(schema)
        except JS.SchemaError as exc:
            raise APIError("unsupported_parameter", f"response schema: {exc}", "response_format") from None
        plan.schema = schema
        json_hint = "\n\nRespond with one JSON object that conforms to this JSON Schema:\n" + json.dumps(schema)
    elif plan.json_mode == "json_object":
        json_hint = "\n\nRespond with one JSON object and nothing else."
    if req.guided_regex is not None:
        try:
            re.compile(req.guided_regex)
        except re.error as exc:
            raise APIError("unsupported_parameter", f"guided_regex: {exc}", "guided_regex") from None
        plan.regex = req.guided_regex
    if req.guided_choice:
        plan.choices = list(req.guided_choice)
        json_hint += "\n\nAnswer with exactly one of: " + ", ".join(plan.choices)

    msgs = [m.model_dump(exclude_none=True) for m in req.messages]
    if json_hint:
        if msgs and msgs[0]["role"] in ("system", "developer") and isinstance(msgs[0].get("content"), str):
            msgs[0] = dict(msgs[0], content=msgs[0]["content"] + json_hint)
        else:
            msgs.insert(0, {"role": "system", "content": json_hint.strip()})
    prompt = render_chat(msgs, tools=tools, enable_thinking=bool(enable_thinking), arch=arch,
                         jinja_template=jinja_template)

    max_tokens = req.max_completion_tokens if req.max_completion_tokens is not None else req.max_tokens
    if max_tokens is None:
        max_tokens = default_max
    close_ids: Tuple[int, ...] = ()
    hard_cap = None
    if plan.starts_in_think:
        close_ids = tuple(tokenizer.encode(THINK_CLOSE))
        if budget is not None:
            hard_cap = max(0, int(budget))
            if req.min_answer_tokens:
                hard_cap = min(hard_cap, max(0, max_tokens - int(req.min_answer_tokens)))
    deadline = _deadline(req.timeout_ms)
    sp = _params(
        max_tokens=max_tokens, temperature=req.temperature if req.temperature is not None else 1.0,
        top_p=req.top_p if req.top_p is not None else 1.0, top_k=req.top_k or 0, min_p=req.min_p or 0.0,
        presence_penalty=req.presence_penalty, frequency_penalty=req.frequency_penalty,
        repetition_penalty=req.repetition_penalty, logit_bias=_bias(req.logit_bias),
        stop_token_sequences=_stops(req.stop, tokenizer), stop_token_ids=tuple(req.stop_token_ids or ()),
        seed=req.seed, ignore_eos=req.ignore_eos, deadline_at=deadline, logprobs=req.logprobs,
        top_logprobs=int(req.top_logprobs or 0), json_object_close_forcing=plan.json_mode is not None and not plan.starts_in_think,
        tool_call_constraint=constraint, thinking_close_token_ids=close_ids if hard_cap is not None else (),
        thinking_hard_token_cap=hard_cap, thinking_soft_close_window=int(req.soft_close_window or 0),
        speculative_mtp=bool(req.speculative_mtp))
    return prompt, sp, plan


def apply_result_policy(parsed: ParsedOutput, plan: ResultPlan) -> Tuple[ParsedOutput, Optional[Dict[str, Any]]]:
    """Validate parsed output against the plan.  Returns (possibly emptied output, finish_details or None)."""
    # tools
    if plan.tool_mode in ("required", "specific") and not parsed.tool_calls:
        return parsed, {"reason": "tool_required_not_satisfied", "message": "the model produced no tool call"}
    for call in parsed.tool_calls:
        if call.error or call.name not in plan.tools or (plan.tool_mode == "specific" and call.name != plan.tool_specific):
            msg = call.error or f"unknown function {call.name!r}"
            if plan.hard_error:
                raise APIError("invalid_tool_call", msg)
            return parsed, {"reason": "invalid_tool_call", "message": msg}
        errs = JS.validate(call.arguments, plan.tools[call.name])
        if errs:
            if plan.hard_error:
                raise APIError("invalid_tool_call", "; ".join(errs[:3]))
            return parsed, {"reason": "invalid_tool_call", "message": "; ".join(errs[:3])}
    # structured output
    if plan.json_mode is not None and not parsed.tool_calls:
        try:
            obj = json.loads(parsed.content)
            if not isinstance(obj, dict):
                raise ValueError("root value is not an object")
        except Exception as exc:
            parsed.content = ""
            return parsed, {"reason": "schema_violation", "message": f"output is not a JSON object: {exc}"}
        if plan.schema is not None:
            errs = JS.validate(obj, plan.schema)
            if errs:
                parsed.content = ""
                return parsed, {"reason": "schema_violation", "message": "; ".join(errs[:3])}
    if plan.regex is not None and re.fullmatch(plan.regex, parsed.content.strip()) is None:
        return parsed, {"reason": "schema_violation", "message": "output does not match guided_regex"}
    if plan.choices is not None and parsed.content.strip() not in plan.choices:
        return parsed, {"reason": "schema_violation", "message": "output is not one of guided_choice"}
    return parsed, None
