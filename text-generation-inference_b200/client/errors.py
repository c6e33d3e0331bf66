"""Exceptions raised by the HTTP client, one per ``error_type`` the router reports.

Same taxonomy as ``clients/python/text_generation/errors.py`` of the reference so that
callers can switch clients without changing their ``except`` clauses.
"""
from __future__ import annotations

from typing import Dict, Optional


class ClientError(Exception):
    """Base class; ``status`` is the HTTP status code when there was a response."""

    def __init__(self, message: str, status: Optional[int] = None):
        super().__init__(message)
        self.message, self.status = message, status


class ValidationError(ClientError):
    """The request was rejected before scheduling (bad parameter, input too long ...)."""


class GenerationError(ClientError):
    """The shard failed while generating."""


class OverloadedError(ClientError):
    """The router's concurrency limit was reached (HTTP 429)."""


class IncompleteGenerationError(ClientError):
    """The generation stopped before a full answer could be produced."""


class BadRequestError(ClientError):
    pass


class ShardNotReadyError(ClientError):
    pass


class ShardTimeoutError(ClientError):
    pass


class NotFoundError(ClientError):
    pass


class RateLimitExceededError(ClientError):
    pass


class NotSupportedError(ClientError):
    pass


class UnknownError(ClientError):
    pass


_BY_TYPE = {
    "validation": ValidationError,
    "generation": GenerationError,
    "overloaded": OverloadedError,
    "incomplete_generation": IncompleteGenerationError,
    "unhealthy": ShardNotReadyError,
}
_BY_STATUS = {400: BadRequestError, 403: ShardNotReadyError, 404: NotFoundError, 422: ValidationError,
              424: GenerationError, 429: OverloadedError, 503: ShardNotReadyError, 504: ShardTimeoutError}


def error_from_payload(payload: Dict, status: Optional[int] = None) -> ClientError:
    """Build the exception for an error body ``{"error": ..., "error_type": ...}``."""
    message = str(payload.get("error") or payload.get("message") or payload)
    kind = payload.get("error_type")
    cls = _BY_TYPE.get(kind) or _BY_STATUS.get(status or 0) or UnknownError
    return cls(message, status)
