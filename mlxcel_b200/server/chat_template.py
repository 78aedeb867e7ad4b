"""Chat-template rendering.

A sandboxed Jinja2 environment with the helpers HF chat templates expect
(``raise_exception``, ``strftime_now``, ``tojson``), like the reference's minijinja environment
(src/server/chat_template.rs:15-45), one render funnel for every route
(src/server/chat_front.rs) and ``chat_template_kwargs`` pass-through
(``enable_thinking``, ``reasoning_effort`` …).
"""
from __future__ import annotations

import datetime
import json

from jinja2 import StrictUndefined  # noqa: F401
from jinja2.exceptions import TemplateError
from jinja2.sandbox import ImmutableSandboxedEnvironment

CHATML = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n"
    "{% if m['content'] is string %}{{ m['content'] }}{% else %}"
    "{% for p in m['content'] %}{% if p['type'] == 'text' %}{{ p['text'] }}{% endif %}{% endfor %}{% endif %}"
    "<|im_end|>\n{% endfor %}{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}"
)


class TemplateRenderError(ValueError):
    pass


def _raise(msg):
    raise TemplateRenderError(str(msg))


def _tojson(v, ensure_ascii=False, indent=None, **kw):
    return json.dumps(v, ensure_ascii=ensure_ascii, indent=indent)


def _env() -> ImmutableSandboxedEnvironment:
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
    env.globals["raise_exception"] = _raise
    env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
    env.filters["tojson"] = _tojson
    return env


_ENV = _env()
_CACHE: dict[str, object] = {}


def template_signature(template: str | None) -> str:
    import hashlib
    return hashlib.sha256((template or CHATML).encode()).hexdigest()[:16]


def normalize_messages(messages: list[dict]) -> list[dict]:
    """Flatten OpenAI content parts to text where the template wants strings; keep tool fields."""
    out = []
    for m in messages:
        m = dict(m)
        c = m.get("content")
        if isinstance(c, list) and all(isinstance(p, dict) and p.get("type") == "text" for p in c):
            m["content"] = "".join(p.get("text", "") for p in c)
        if c is None:
            m["content"] = ""
        for tc in m.get("tool_calls") or []:
            fn = tc.get("function", {})
            if isinstance(fn.get("arguments"), str):
                try:
                    fn["arguments"] = json.loads(fn["arguments"])
                except Exception:
                    pass
        out.append(m)
    return out


_IMAGE_PART_TYPES = ("image_url", "image", "input_image")


_AUDIO_PART_TYPES = ("input_audio", "audio_url", "audio")


def extract_media(messages: list[dict], placeholder: str, template: str | None, audio: bool = False) -> tuple[list[dict], list]:
    """Pull the images out of OpenAI-style content parts. Returns the messages to render and the image
    sources in prompt order. A template that handles ``{"type": "image"}`` parts itself (the templates
    vision-language checkpoints ship) gets them in that form; otherwise every image part becomes the
    model's placeholder text inside a flattened string content."""
    kinds = _AUDIO_PART_TYPES if audio else _IMAGE_PART_TYPES
    tag = "audio" if audio else "image"
    native = bool(template) and (f"'{tag}'" in template or f'"{tag}"' in template)
    out, images = [], []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list) or not any(isinstance(p, dict) and p.get("type") in kinds for p in c):
            out.append(m)
            continue
        parts, text = [], ""
        for p in c:
            kind = p.get("type") if isinstance(p, dict) else None
            if kind in kinds:
                src = (p.get("input_audio") or p.get("audio_url") or p.get("audio") or p.get("url")) if audio else \
                    (p.get("image_url") or p.get("image") or p.get("url"))
                if isinstance(src, dict):
                    src = src.get("data") or src.get("url")
                if src is None:
                    raise TemplateRenderError(f"an {tag} part carries no data")
                images.append(src)
                parts.append({"type": tag})
                text += placeholder
            elif kind in ("text", "input_text"):
                parts.append({"type": "text", "text": p.get("text", "")})
                text += p.get("text", "")
        m = dict(m)
        m["content"] = parts if native else text
        out.append(m)
    return out, images


def render_chat(messages: list[dict], template: str | None = None, *, add_generation_prompt: bool = True,
                tools: list | None = None, bos_token: str = "", eos_token: str = "", **kwargs) -> str:
    src = template or CHATML
    tpl = _CACHE.get(src)
    if tpl is None:
        try:
            tpl = _ENV.from_string(src)
        except TemplateError as e:
            raise TemplateRenderError(f"invalid chat template: {e}") from e
        _CACHE[src] = tpl
    try:
        return tpl.render(messages=normalize_messages(messages), add_generation_prompt=add_generation_prompt,
                          tools=tools, bos_token=bos_token or "", eos_token=eos_token or "", **kwargs)
    except TemplateRenderError:
        raise
    except Exception as e:  # template runtime error (undefined access, sandbox violation ...)
        raise TemplateRenderError(f"chat template failed: {e}") from e
