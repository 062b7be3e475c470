"""Canonical error codes and the OpenAI-style error envelope.

``{"error": {message, type, code, param, hipengine: {code, status, retryable}}}`` with the reference's code
table (``docs/API.md:2026-2062`` of the reference): unsupported_parameter 400, unsupported_feature 501,
invalid_tool_call 400, schema_violation 422, invalid_continuation 400, continuation_expired 410,
context_overflow 400, deadline_exceeded 408, cancelled 499, engine_busy 429, engine_unavailable 503,
internal_error 500, execution_failed 500, model_unavailable 404, routing_failed 502.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

CODES: Dict[str, tuple] = {
    "unsupported_parameter": (400, "invalid_request_error", False),
    "invalid_request": (400, "invalid_request_error", False),
    "unsupported_feature": (501, "invalid_request_error", False),
    "invalid_tool_call": (400, "invalid_request_error", False),
    "schema_violation": (422, "invalid_request_error", False),
    "invalid_continuation": (400, "invalid_request_error", False),
    "continuation_expired": (410, "invalid_request_error", False),
    "context_overflow": (400, "invalid_request_error", False),
    "deadline_exceeded": (408, "timeout_error", True),
    "cancelled": (499, "cancelled_error", False),
    "engine_busy": (429, "rate_limit_error", True),
    "engine_unavailable": (503, "service_unavailable_error", True),
    "internal_error": (500, "server_error", False),
    "execution_failed": (500, "server_error", True),
    "model_unavailable": (404, "invalid_request_error", False),
    "routing_failed": (502, "server_error", True),
    "unauthorized": (401, "authentication_error", False),
    "not_found": (404, "invalid_request_error", False),
    "method_not_allowed": (405, "invalid_request_error", False),
}


class APIError(Exception):
    def __init__(self, code: str, message: str, param: Optional[str] = None, extra: Optional[Dict[str, Any]] = None,
                 retry_after: Optional[float] = None):
        super().__init__(message)
        self.code = code if code in CODES else "internal_error"
        self.message = message
        self.param = param
        self.extra = extra or {}
        self.retry_after = retry_after

    @property
    def status(self) -> int:
        return CODES[self.code][0]

    def body(self) -> Dict[str, Any]:
        status, typ, retryable = CODES[self.code]
        he = {"code": self.code, "status": status, "retryable": retryable}
        he.update(self.extra)
        return {"error": {"message": self.message, "type": typ, "code": self.code, "param": self.param,
                          "hipengine": he}}


def classify_engine_error(message: str) -> str:
    """Map an engine-side failure string to a canonical code."""
    m = message or ""
    for code in ("context_overflow", "engine_busy", "engine_unavailable", "deadline_exceeded", "execution_failed",
                 "cancelled"):
        if code in m:
            return code
    return "internal_error"
