"""The API error envelope and status / code matrix (docs/api/openai-compatibility.md:133-158 of the reference)."""
from __future__ import annotations

from typing import Optional


class ApiError(Exception):
    def __init__(self, status: int, code: str, message: str, param: Optional[str] = None,
                 err_type: str = "invalid_request_error"):
        super().__init__(message)
        self.status, self.code, self.message, self.param, self.err_type = status, code, message, param, err_type

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.err_type, "param": self.param, "code": self.code}}


def invalid_json(msg="request body is not valid JSON"):
    return ApiError(400, "invalid_json", msg)


def invalid_value(msg, param=None):
    return ApiError(400, "invalid_value", msg, param)


def unsupported(msg, param=None):
    return ApiError(400, "unsupported_parameter", msg, param)


def unauthorized():
    return ApiError(401, "invalid_api_key", "invalid or missing API key")


def forbidden():
    return ApiError(403, "insufficient_permissions", "the key does not grant this role")


def model_not_found(alias):
    return ApiError(404, "model_not_found", "the requested model is not served", "model")


def not_found(msg="not found"):
    return ApiError(404, "not_found", msg)


def too_large():
    return ApiError(413, "request_too_large", "request body exceeds the 96 MiB limit")


def rate_limited(msg="the request queue is full"):
    return ApiError(429, "rate_limit_exceeded", msg, err_type="rate_limit_error")


def unavailable(msg="the model is not ready"):
    return ApiError(503, "service_unavailable", msg, err_type="server_error")


def server_error(msg="generation failed"):
    return ApiError(500, "server_error", msg, err_type="server_error")
