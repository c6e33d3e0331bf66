"""Synchronous and asynchronous HTTP clients of the router.

Counterpart of ``clients/python/text_generation/client.py`` in the reference (``Client`` /
``AsyncClient`` with ``generate``, ``generate_stream``, ``chat``; here also ``completion``,
``tokenize``, ``info``, ``health``).  The synchronous client uses ``requests``, the asynchronous
one ``aiohttp``; streaming responses are server-sent events, one JSON object per ``data:`` line.
"""
from __future__ import annotations

import json
from typing import Any, AsyncIterator, Dict, Iterator, List, Optional, Union

from .errors import ClientError, error_from_payload
from .types import (ChatComplete, ChatCompletionChunk, ChatRequest, Completion, CompletionRequest, Grammar, Message,
                    Parameters, Request, Response, StreamResponse, Tool)


def _parameters(**kw) -> Parameters:
    stop = kw.pop("stop_sequences", None)
    kw["stop"] = list(stop) if stop else []
    return Parameters(**{k: v for k, v in kw.items() if v is not None or k in ("stop",)})


def _sse_payloads(lines) -> Iterator[Dict[str, Any]]:
    """Decode an iterable of byte lines of an event stream into JSON payloads."""
    for raw in lines:
        if not raw:
            continue
        line = raw.decode("utf-8") if isinstance(raw, (bytes, bytearray)) else raw
        line = line.strip()
        if not line.startswith("data:"):
            continue
        body = line[5:].strip()
        if body == "[DONE]":
            return
        yield json.loads(body)


def _raise_for(payload: Any, status: int):
    if status != 200:
        if not isinstance(payload, dict):
            payload = {"error": str(payload)}
        raise error_from_payload(payload, status)


class Client:
    """Blocking client.

    >>> client = Client("http://127.0.0.1:3000")
    >>> client.generate("Why is the sky blue?", max_new_tokens=20).generated_text
    >>> for event in client.generate_stream("Why is the sky blue?"):
    ...     print(event.token.text, end="")
    """

    def __init__(self, base_url: str, headers: Optional[Dict[str, str]] = None, cookies: Optional[Dict[str, str]] = None,
                 timeout: float = 60.0):
        self.base_url = base_url.rstrip("/")
        self.headers, self.cookies, self.timeout = headers or {}, cookies, timeout

    # ---- plumbing ------------------------------------------------------------------------------
    def _post(self, path: str, body: Dict[str, Any], stream: bool = False):
        import requests

        return requests.post(self.base_url + path, json=body, headers=self.headers, cookies=self.cookies,
                             timeout=self.timeout, stream=stream)

    def _get(self, path: str):
        import requests

        return requests.get(self.base_url + path, headers=self.headers, cookies=self.cookies, timeout=self.timeout)

    @staticmethod
    def _json(resp):
        try:
            return resp.json()
        except Exception:
            return {"error": resp.text}

    # ---- native API ----------------------------------------------------------------------------
    def generate(self, prompt: str, do_sample: bool = False, max_new_tokens: Optional[int] = None,
                 best_of: Optional[int] = None, repetition_penalty: Optional[float] = None,
                 frequency_penalty: Optional[float] = None, return_full_text: bool = False, seed: Optional[int] = None,
                 stop_sequences: Optional[List[str]] = None, temperature: Optional[float] = None,
                 top_k: Optional[int] = None, top_p: Optional[float] = None, truncate: Optional[int] = None,
                 typical_p: Optional[float] = None, watermark: bool = False, decoder_input_details: bool = False,
                 top_n_tokens: Optional[int] = None, grammar: Optional[Grammar] = None,
                 adapter_id: Optional[str] = None, details: bool = True) -> Response:
        params = _parameters(best_of=best_of, details=details, do_sample=do_sample, max_new_tokens=max_new_tokens,
                             repetition_penalty=repetition_penalty, frequency_penalty=frequency_penalty,
                             return_full_text=return_full_text, seed=seed, stop_sequences=stop_sequences,
                             temperature=temperature, top_k=top_k, top_p=top_p, truncate=truncate, typical_p=typical_p,
                             watermark=watermark, decoder_input_details=decoder_input_details,
                             top_n_tokens=top_n_tokens, grammar=grammar, adapter_id=adapter_id)
        req = Request(inputs=prompt, stream=False, parameters=params)
        resp = self._post("/generate", req.model_dump(exclude_none=True))
        payload = self._json(resp)
        _raise_for(payload, resp.status_code)
        if isinstance(payload, list):
            payload = payload[0]
        return Response(**payload)

    def generate_stream(self, prompt: str, do_sample: bool = False, max_new_tokens: Optional[int] = None,
                        repetition_penalty: Optional[float] = None, frequency_penalty: Optional[float] = None,
                        return_full_text: bool = False, seed: Optional[int] = None,
                        stop_sequences: Optional[List[str]] = None, temperature: Optional[float] = None,
                        top_k: Optional[int] = None, top_p: Optional[float] = None, truncate: Optional[int] = None,
                        typical_p: Optional[float] = None, watermark: bool = False,
                        top_n_tokens: Optional[int] = None, grammar: Optional[Grammar] = None,
                        adapter_id: Optional[str] = None) -> Iterator[StreamResponse]:
        params = _parameters(details=True, do_sample=do_sample, max_new_tokens=max_new_tokens,
                             repetition_penalty=repetition_penalty, frequency_penalty=frequency_penalty,
                             return_full_text=return_full_text, seed=seed, stop_sequences=stop_sequences,
                             temperature=temperature, top_k=top_k, top_p=top_p, truncate=truncate, typical_p=typical_p,
                             watermark=watermark, top_n_tokens=top_n_tokens, grammar=grammar, adapter_id=adapter_id)
        req = Request(inputs=prompt, stream=True, parameters=params)
        resp = self._post("/generate_stream", req.model_dump(exclude_none=True), stream=True)
        if resp.status_code != 200:
            _raise_for(self._json(resp), resp.status_code)
        for payload in _sse_payloads(resp.iter_lines()):
            if "error" in payload and "token" not in payload:
                raise error_from_payload(payload, resp.status_code)
            yield StreamResponse(**payload)

    # ---- OpenAI-compatible API -------------------------------------------------------------------
    def chat(self, messages: List[Union[Message, Dict[str, Any]]], stream: bool = False, **kw
             ) -> Union[ChatComplete, Iterator[ChatCompletionChunk]]:
        tools = kw.pop("tools", None)
        req = ChatRequest(messages=[m if isinstance(m, Message) else Message(**m) for m in messages], stream=stream,
                          tools=[t if isinstance(t, Tool) else Tool(**t) for t in tools] if tools else None, **kw)
        body = req.model_dump(exclude_none=True)
        if not stream:
            resp = self._post("/v1/chat/completions", body)
            payload = self._json(resp)
            _raise_for(payload, resp.status_code)
            return ChatComplete(**payload)
        return self._chat_stream(body)

    def _chat_stream(self, body) -> Iterator[ChatCompletionChunk]:
        resp = self._post("/v1/chat/completions", body, stream=True)
        if resp.status_code != 200:
            _raise_for(self._json(resp), resp.status_code)
        for payload in _sse_payloads(resp.iter_lines()):
            if "error" in payload and "choices" not in payload:
                raise error_from_payload(payload, resp.status_code)
            yield ChatCompletionChunk(**payload)

    def completion(self, prompt: Union[str, List[str]], **kw) -> Completion:
        req = CompletionRequest(prompt=prompt, stream=False, **kw)
        resp = self._post("/v1/completions", req.model_dump(exclude_none=True))
        payload = self._json(resp)
        _raise_for(payload, resp.status_code)
        return Completion(**payload)

    # ---- utility routes --------------------------------------------------------------------------
    def tokenize(self, prompt: str) -> List[Dict[str, Any]]:
        resp = self._post("/tokenize", {"inputs": prompt})
        payload = self._json(resp)
        _raise_for(payload, resp.status_code)
        return payload

    def info(self) -> Dict[str, Any]:
        resp = self._get("/info")
        payload = self._json(resp)
        _raise_for(payload, resp.status_code)
        return payload

    def health(self) -> bool:
        try:
            return self._get("/health").status_code == 200
        except Exception:
            return False


class AsyncClient:
    """``asyncio`` twin of :class:`Client` (same methods, awaitable / async iterators)."""

    def __init__(self, base_url: str, headers: Optional[Dict[str, str]] = None, cookies: Optional[Dict[str, str]] = None,
                 timeout: float = 60.0):
        self.base_url = base_url.rstrip("/")
        self.headers, self.cookies, self.timeout = headers or {}, cookies, timeout

    def _session(self):
        import aiohttp

        return aiohttp.ClientSession(headers=self.headers, cookies=self.cookies,
                                     timeout=aiohttp.ClientTimeout(total=self.timeout))

    async def _post_json(self, path: str, body: Dict[str, Any]):
        async with self._session() as session:
            async with session.post(self.base_url + path, json=body) as resp:
                try:
                    payload = await resp.json(content_type=None)
                except Exception:
                    payload = {"error": await resp.text()}
                _raise_for(payload, resp.status)
                return payload

    async def _post_stream(self, path: str, body: Dict[str, Any]) -> AsyncIterator[Dict[str, Any]]:
        async with self._session() as session:
            async with session.post(self.base_url + path, json=body) as resp:
                if resp.status != 200:
                    try:
                        payload = await resp.json(content_type=None)
                    except Exception:
                        payload = {"error": await resp.text()}
                    _raise_for(payload, resp.status)
                async for raw in resp.content:
                    for payload in _sse_payloads([raw]):
                        yield payload

    async def generate(self, prompt: str, details: bool = True, **kw) -> Response:
        kw.setdefault("stop_sequences", None)
        req = Request(inputs=prompt, stream=False, parameters=_parameters(details=details, **kw))
        payload = await self._post_json("/generate", req.model_dump(exclude_none=True))
        if isinstance(payload, list):
            payload = payload[0]
        return Response(**payload)

    async def generate_stream(self, prompt: str, **kw) -> AsyncIterator[StreamResponse]:
        kw.setdefault("stop_sequences", None)
        req = Request(inputs=prompt, stream=True, parameters=_parameters(details=True, **kw))
        async for payload in self._post_stream("/generate_stream", req.model_dump(exclude_none=True)):
            if "error" in payload and "token" not in payload:
                raise error_from_payload(payload)
            yield StreamResponse(**payload)

    async def chat(self, messages: List[Union[Message, Dict[str, Any]]], **kw) -> ChatComplete:
        req = ChatRequest(messages=[m if isinstance(m, Message) else Message(**m) for m in messages], stream=False, **kw)
        return ChatComplete(**await self._post_json("/v1/chat/completions", req.model_dump(exclude_none=True)))

    async def chat_stream(self, messages: List[Union[Message, Dict[str, Any]]], **kw) -> AsyncIterator[ChatCompletionChunk]:
        req = ChatRequest(messages=[m if isinstance(m, Message) else Message(**m) for m in messages], stream=True, **kw)
        async for payload in self._post_stream("/v1/chat/completions", req.model_dump(exclude_none=True)):
            if "error" in payload and "choices" not in payload:
                raise error_from_payload(payload)
            yield ChatCompletionChunk(**payload)

    async def completion(self, prompt: Union[str, List[str]], **kw) -> Completion:
        req = CompletionRequest(prompt=prompt, stream=False, **kw)
        return Completion(**await self._post_json("/v1/completions", req.model_dump(exclude_none=True)))


__all__ = ["Client", "AsyncClient", "ClientError"]
