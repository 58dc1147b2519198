"""Error envelope ``{"error": {"message", "type", "code"}}`` and the error catalogue.
Parity: reference ``metal_marlin/serving/errors.py`` and ``metal_marlin/serving/server.py:42-70``."""
from __future__ import annotations


class ServingError(Exception):
    status_code = 500
    error_type = "server_error"
    code = "internal_error"

    def __init__(self, message: str = ""):
        super().__init__(message or self.code)
        self.message = message or self.code

    def to_dict(self) -> dict:
        return {"error": {"message": self.message, "type": self.error_type, "code": self.code}}


class ModelNotLoaded(ServingError):
    status_code, error_type, code = 503, "service_unavailable", "model_not_loaded"


class InvalidRequest(ServingError):
    status_code, error_type, code = 400, "invalid_request_error", "invalid_request"


class ModelNotFound(ServingError):
    status_code, error_type, code = 404, "invalid_request_error", "model_not_found"


class RateLimitExceeded(ServingError):
    status_code, error_type, code = 429, "rate_limit_error", "rate_limit_exceeded"


class ContextLengthExceeded(ServingError):
    status_code, error_type, code = 400, "invalid_request_error", "context_length_exceeded"


class RequestTimeout(ServingError):
    status_code, error_type, code = 504, "timeout_error", "request_timeout"
