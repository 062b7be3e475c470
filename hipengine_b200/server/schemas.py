"""OpenAI-compatible request schemas (pydantic, ``extra="allow"``).

Field inventory follows the reference (``hipengine/server/schemas.py:52-150``): ``CompletionRequest`` and
``ChatCompletionRequest`` with tools, tool_choice, reasoning/thinking controls, response_format and the
guided_* family, logprobs, stream_options, timeout_ms, continuation/session ids and the speculative switch.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

from pydantic import BaseModel, ConfigDict, Field


class _Base(BaseModel):
    model_config = ConfigDict(extra="allow")


class StreamOptions(_Base):
    include_usage: bool = False
    include_hipengine: bool = False


class CompletionRequest(_Base):
    model: Optional[str] = None
    prompt: Union[str, List[str], List[int], List[List[int]]] = ""
    max_tokens: Optional[int] = 16
    temperature: Optional[float] = 1.0
    top_p: Optional[float] = 1.0
    top_k: Optional[int] = 0
    min_p: Optional[float] = 0.0
    n: int = 1
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    logprobs: Optional[int] = None
    echo: bool = False
    stop: Optional[Union[str, List[str]]] = None
    stop_token_ids: Optional[List[int]] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[Dict[str, float]] = None
    seed: Optional[int] = None
    ignore_eos: bool = False
    min_tokens: int = 0
    timeout_ms: Optional[int] = None
    user: Optional[str] = None
    speculative_mtp: Optional[bool] = None


class FunctionDef(_Base):
    name: str
    description: Optional[str] = None
    parameters: Optional[Dict[str, Any]] = None
    strict: Optional[bool] = None


class ToolDef(_Base):
    type: str = "function"
    function: FunctionDef


class ResponseFormat(_Base):
    type: str = "text"                      # text | json_object | json_schema
    json_schema: Optional[Dict[str, Any]] = None


class ChatMessage(_Base):
    role: str
    content: Optional[Union[str, List[Dict[str, Any]]]] = None
    name: Optional[str] = None
    tool_calls: Optional[List[Dict[str, Any]]] = None
    tool_call_id: Optional[str] = None
    reasoning_content: Optional[str] = None


class ChatCompletionRequest(_Base):
    model: Optional[str] = None
    messages: List[ChatMessage] = Field(default_factory=list)
    max_tokens: Optional[int] = None
    max_completion_tokens: Optional[int] = None
    temperature: Optional[float] = 1.0
    top_p: Optional[float] = 1.0
    top_k: Optional[int] = 0
    min_p: Optional[float] = 0.0
    n: int = 1
    stream: bool = False
    stream_options: Optional[StreamOptions] = None
    stop: Optional[Union[str, List[str]]] = None
    stop_token_ids: Optional[List[int]] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[Dict[str, float]] = None
    seed: Optional[int] = None
    logprobs: bool = False
    top_logprobs: Optional[int] = None
    tools: Optional[List[ToolDef]] = None
    tool_choice: Optional[Union[str, Dict[str, Any]]] = None
    parallel_tool_calls: Optional[bool] = True
    response_format: Optional[ResponseFormat] = None
    guided_json: Optional[Union[str, Dict[str, Any]]] = None
    guided_regex: Optional[str] = None
    guided_choice: Optional[List[str]] = None
    guided_grammar: Optional[str] = None
    grammar: Optional[Any] = None
    reasoning_effort: Optional[str] = None
    enable_thinking: Optional[bool] = None
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    thinking_token_budget: Optional[int] = None
    max_think_tokens: Optional[int] = None
    min_answer_tokens: Optional[int] = None
    hard_think_cap: Optional[bool] = None
    soft_close_window: Optional[int] = None
    invalid_tool_call_error_mode: Optional[str] = None
    timeout_ms: Optional[int] = None
    continuation_id: Optional[str] = None
    session: Optional[Union[str, Dict[str, Any]]] = None
    speculative_mtp: Optional[bool] = None
    ignore_eos: bool = False
    user: Optional[str] = None


class TokenizeRequest(_Base):
    model: Optional[str] = None
    text: Optional[str] = None
    prompt: Optional[str] = None
    messages: Optional[List[ChatMessage]] = None
    max_tokens: Optional[int] = None            # fit_context: would prompt + max_tokens fit?


class DetokenizeRequest(_Base):
    model: Optional[str] = None
    tokens: List[int] = Field(default_factory=list)
