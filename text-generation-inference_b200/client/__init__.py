"""Python HTTP client of the router (sync and asyncio), with typed requests, responses and errors."""
from .client import AsyncClient, Client
from .errors import ClientError
from .types import (ChatComplete, ChatCompletionChunk, Completion, Details, FinishReason, Grammar, GrammarType,
                    Message, Parameters, Request, Response, StreamResponse, Token, Tool)

__all__ = ["AsyncClient", "Client", "ClientError", "ChatComplete", "ChatCompletionChunk", "Completion", "Details",
           "FinishReason", "Grammar", "GrammarType", "Message", "Parameters", "Request", "Response",
           "StreamResponse", "Token", "Tool"]
