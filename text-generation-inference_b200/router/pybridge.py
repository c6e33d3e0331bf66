"""Python helpers called from the C++ router through its embedded interpreter.

The router itself (HTTP, validation, scheduling, block allocation) is native; what it borrows from
Python are the two things that already exist as maintained libraries there: the Hugging Face
tokenizer of the model and a full Jinja implementation for chat templates (the reference embeds
`tokenizers` and `minijinja` in its Rust router, with the same Python fallback for tokenizers it
cannot load natively, router/src/lib.rs:29-110).  Every entry point takes one JSON string and
returns one JSON string, which keeps the C API surface in the router tiny.
"""
from __future__ import annotations

import datetime
import json
import os
from typing import Any, Dict, List, Optional

_STATE: Dict[str, Any] = {}


def _ok(**kw) -> str:
    return json.dumps({"ok": True, **kw})


def _err(msg: str, kind: str = "validation") -> str:
    return json.dumps({"ok": False, "error": msg, "error_type": kind})


def load(arg: str) -> str:
    a = json.loads(arg)
    path = a.get("tokenizer_name") or a.get("model_id")
    from tgi_b200.utils.tokenizer import load_tokenizer

    tok = load_tokenizer(path, a.get("revision"), False, vocab_size=a.get("vocab_size", 259))
    _STATE["tokenizer"] = tok
    cfg: Dict[str, Any] = {}
    for name in ("config.json", "tokenizer_config.json", "generation_config.json"):
        f = os.path.join(path or "", name)
        if path and os.path.exists(f):
            with open(f) as fh:
                cfg[name] = json.load(fh)
    _STATE["config"] = cfg
    tc = cfg.get("tokenizer_config.json", {})
    # A stand-alone chat_template.json overrides the tokenizer's template (server.rs:1662-1689); vision-language
    # checkpoints also keep theirs in processor_config.json, newer ones in chat_template.jinja.
    standalone = None
    if path:
        for name in ("chat_template.json", "processor_config.json"):
            f = os.path.join(path, name)
            if standalone is None and os.path.exists(f):
                try:
                    with open(f) as fh:
                        standalone = json.load(fh).get("chat_template")
                except (OSError, ValueError):
                    standalone = None
        f = os.path.join(path, "chat_template.jinja")
        if standalone is None and os.path.exists(f):
            with open(f) as fh:
                standalone = fh.read()
    template = (a.get("chat_template") or standalone or getattr(tok, "chat_template", None)
                or tc.get("chat_template"))
    if isinstance(template, list):  # named templates: take "default"
        template = next((t["template"] for t in template if t.get("name") == "default"), template[0]["template"])
    _STATE["chat_template"] = template
    _STATE["bos_token"] = _tok_str(tc.get("bos_token")) or getattr(tok, "bos_token", None)
    _STATE["eos_token"] = _tok_str(tc.get("eos_token")) or getattr(tok, "eos_token", None)
    model_cfg = cfg.get("config.json", {})
    return _ok(model_type=model_cfg.get("model_type"), has_chat_template=template is not None,
               bos_token=_STATE["bos_token"] if isinstance(_STATE["bos_token"], str) else None,
               is_hf_tokenizer=hasattr(tok, "convert_tokens_to_ids"),
               max_position_embeddings=model_cfg.get("max_position_embeddings"),
               vocab_size=model_cfg.get("vocab_size"))


def _tok_str(t) -> Optional[str]:
    if isinstance(t, dict):
        return t.get("content")
    return t


def encode(arg: str) -> str:
    a = json.loads(arg)
    tok = _STATE["tokenizer"]
    text = a["text"]
    add = a.get("add_special_tokens", True)
    truncate = a.get("truncate")
    if a.get("offsets") and hasattr(tok, "encode_plus"):
        enc = tok(text, add_special_tokens=add, return_offsets_mapping=True)
        ids, offs = list(enc["input_ids"]), [list(o) for o in enc["offset_mapping"]]
    else:
        ids = list(tok(text, add_special_tokens=add)["input_ids"])
        offs = None
    if truncate and len(ids) > truncate:
        ids = ids[-truncate:]
        if offs:
            offs = offs[-truncate:]
    out = {"ids": ids}
    if a.get("offsets"):
        toks = []
        for i, t in enumerate(ids):
            if offs:
                s, e = offs[i]
                toks.append({"id": t, "text": text[s:e], "start": s, "stop": e})
            else:
                toks.append({"id": t, "text": tok.decode([t]), "start": 0, "stop": 0})
        out["tokens"] = toks
    return _ok(**out)


def decode(arg: str) -> str:
    a = json.loads(arg)
    return _ok(text=_STATE["tokenizer"].decode(a["ids"], skip_special_tokens=a.get("skip_special_tokens", True)))


def _jinja_env():
    env = _STATE.get("jinja_env")
    if env is None:
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(message):
            raise jinja2.exceptions.TemplateError(message)

        def strftime_now(fmt):
            return datetime.datetime.now().strftime(fmt)

        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True,
                                            extensions=["jinja2.ext.loopcontrols"])
        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = strftime_now
        env.filters["tojson"] = lambda v, indent=None, **kw: json.dumps(v, indent=indent, ensure_ascii=False)
        _STATE["jinja_env"] = env
    return env


def apply_chat_template(arg: str) -> str:
    """Render the model's chat template over OpenAI-style messages (+ tools), like the reference's
    ChatTemplate::apply (router/src/infer/chat_template.rs:27-136): messages with list content are
    flattened to text with image placeholders, tools are passed to templates that know about them
    and otherwise described in the last user message through `tool_prompt`."""
    a = json.loads(arg)
    template = _STATE.get("chat_template")
    if template is None:
        return _err("Template error: no chat template is defined for this model", "template_error")
    messages = a["messages"]
    tools = a.get("tools")
    tool_prompt = a.get("tool_prompt") or ""
    # templates of some models use python-only idioms
    template = template.replace("{% generation %}", "").replace("{% endgeneration %}", "")
    template = template.replace("[::-1]", "|reverse")
    norm = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list):
            parts = []
            for ch in c:
                if ch.get("type") == "text":
                    parts.append(ch.get("text", ""))
                elif ch.get("type") == "image_url":
                    parts.append(f"![]({ch['image_url']['url']})")
            m["content"] = "".join(parts)
        norm.append(m)
    uses_tools = "tools" in template
    if tools and norm:
        # the last message carries the tool prompt; templates without a tools section also get the tool list there
        # (chat_template.rs:83-105: "\n---\n" + tools + "\n" + prompt, or "\n---\n" + prompt)
        if uses_tools:
            text = f"\n---\n{tool_prompt}"
        else:
            text = f"\n---\n{json.dumps(tools, ensure_ascii=False, separators=(',', ':'))}\n{tool_prompt}"
        norm[-1] = dict(norm[-1])
        norm[-1]["content"] = f"{norm[-1].get('content') or ''}{text}"
    try:
        tpl = _jinja_env().from_string(template)
        rendered = tpl.render(messages=norm, bos_token=_STATE.get("bos_token") or "",
                              eos_token=_STATE.get("eos_token") or "",
                              add_generation_prompt=a.get("add_generation_prompt", True),
                              tools=tools if uses_tools else None, tools_in_user_message=False,
                              guideline=a.get("guideline"))
    except Exception as err:  # noqa: BLE001
        return _err(f"Template error: {err}", "template_error")
    # assistant prefill: a trailing assistant message is continued, not closed.  The rendered text is cut right after
    # the last occurrence of that message's content (chat_template.rs:120-136, after the text-generation pipeline of
    # transformers), which drops the end-of-turn marker and the generation prompt the template added behind it.
    if norm and norm[-1].get("role") == "assistant" and isinstance(norm[-1].get("content"), str) and norm[-1]["content"]:
        content = norm[-1]["content"]
        at = rendered.rfind(content)
        if at >= 0:
            rendered = rendered[:at + len(content)].rstrip()
    return _ok(text=rendered)


def compile_grammar(arg: str) -> str:
    """Validate a grammar and bring it to the form sent to the shards: JSON schemas are checked and
    compiled to a regular expression (router/src/validation.rs:348-412 does this with outlines-core)."""
    a = json.loads(arg)
    kind, value = a["type"], a["value"]
    try:
        if kind in ("json", "json_object", "json_schema"):
            if isinstance(value, str):
                value = json.loads(value)
            if kind == "json_schema" and isinstance(value, dict) and "schema" in value:
                value = value["schema"]
            if not isinstance(value, dict):
                return _err("Grammar must be a valid JSON object")
            from outlines_core.json_schema import build_regex_from_schema

            return _ok(grammar=build_regex_from_schema(json.dumps(value)), grammar_type=2)
        if kind == "regex":
            import re

            re.compile(value)
            return _ok(grammar=value, grammar_type=2)
    except Exception as err:  # noqa: BLE001
        return _err(f"Grammar error: {err}")
    return _err(f"unknown grammar type {kind}")
