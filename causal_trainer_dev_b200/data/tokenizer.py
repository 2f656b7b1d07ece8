"""Tokenizer and chat-template front end of the data pipeline.

A thin, training-only wrapper around the serialized fast ``tokenizer.json`` (executed by the
``tokenizers`` wheel; repository Python is never imported) with sandboxed Jinja chat
templates.  Behaviour follows the reference (src/causal_trainer/data/tokenizer.py:27-533):

* ``{% generation %}…{% endgeneration %}`` blocks mark assistant text; their *character*
  spans are mapped to tokens by interval overlap, so a block that ends in whitespace the
  tokenizer drops cannot spill supervision onto the next turn;
* an assistant message with ``"loss": false`` keeps its tokens but loses its span (this
  needs exactly one generation block per assistant message);
* ``chat_template.jinja`` / ``chat_templates/*.jinja`` on disk override the template of
  ``tokenizer_config.json``; ``tool_use`` is picked when tools are passed;
* raw tokenisation never inserts special tokens; asking for it raises.
"""
from __future__ import annotations

import contextvars
import json
from datetime import datetime
from functools import lru_cache
from pathlib import Path
from typing import Any, Mapping, Sequence

import jinja2
from jinja2.ext import Extension
from jinja2.sandbox import ImmutableSandboxedEnvironment

ChatTemplate = str | dict[str, str] | None


class _SpanRecorder:
    """Collects rendered text and the character spans of kept generation blocks."""

    def __init__(self, keep_flags: Sequence[bool] | None):
        self.pieces: list[str] = []
        self.length = 0
        self.spans: list[tuple[int, int]] = []
        self.keep_flags = None if keep_flags is None else tuple(keep_flags)
        self.blocks_seen = 0

    def push(self, text: str) -> None:
        self.pieces.append(text)
        self.length += len(text)

    def on_block(self, rendered: str) -> None:
        keep = True
        if self.keep_flags is not None:
            if self.blocks_seen >= len(self.keep_flags):
                raise ValueError("message-level loss requires exactly one generation block per assistant message")
            keep = self.keep_flags[self.blocks_seen]
        self.blocks_seen += 1
        if keep:
            self.spans.append((self.length, self.length + len(rendered)))

    def finish(self) -> None:
        if self.keep_flags is not None and self.blocks_seen != len(self.keep_flags):
            raise ValueError("message-level loss requires exactly one generation block per assistant message")


_ACTIVE_RECORDER: contextvars.ContextVar[_SpanRecorder | None] = contextvars.ContextVar("ctb_span_recorder", default=None)


class GenerationBlocks(Extension):
    """Jinja extension implementing ``{% generation %}``: transparent, but reports its output."""

    tags = {"generation"}

    def parse(self, parser: Any) -> jinja2.nodes.CallBlock:
        lineno = next(parser.stream).lineno
        body = parser.parse_statements(["name:endgeneration"], drop_needle=True)
        return jinja2.nodes.CallBlock(self.call_method("_emit"), [], [], body).set_lineno(lineno)

    def _emit(self, caller: Any) -> str:
        rendered = caller()
        recorder = _ACTIVE_RECORDER.get()
        if recorder is not None:
            recorder.on_block(rendered)
        return rendered


def _raise_exception(message: str) -> None:
    raise jinja2.exceptions.TemplateError(message)


def _tojson(value: Any, ensure_ascii: bool = False, indent: int | None = None,
            separators: tuple[str, str] | None = None, sort_keys: bool = False) -> str:
    return json.dumps(value, ensure_ascii=ensure_ascii, indent=indent, separators=separators, sort_keys=sort_keys)


@lru_cache(maxsize=128)
def compile_chat_template(source: str) -> jinja2.Template:
    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True,
                                        extensions=[GenerationBlocks, jinja2.ext.loopcontrols])
    env.filters["tojson"] = _tojson
    env.globals["raise_exception"] = _raise_exception
    env.globals["strftime_now"] = lambda fmt: datetime.now().strftime(fmt)
    return env.from_string(source)


def _json(path: Path) -> Any:
    try:
        return json.loads(path.read_text(encoding="utf-8"))
    except json.JSONDecodeError as exc:
        raise ValueError(f"invalid JSON in {path}: {exc}") from exc


def _json_object(path: Path) -> dict[str, Any]:
    value = _json(path)
    if not isinstance(value, dict):
        raise ValueError(f"{path} must contain a JSON object")
    return value


def normalize_chat_template(value: Any, source: str) -> ChatTemplate:
    if value is None or isinstance(value, str):
        return value
    if isinstance(value, Mapping):
        if set(value) == {"chat_template"}:
            return normalize_chat_template(value["chat_template"], source)
        if any(not isinstance(k, str) or not isinstance(v, str) for k, v in value.items()):
            raise ValueError(f"{source} chat template mapping must contain string names and templates")
        return dict(value)
    if isinstance(value, Sequence) and not isinstance(value, (str, bytes)):
        out: dict[str, str] = {}
        for entry in value:
            if not isinstance(entry, Mapping):
                raise ValueError(f"{source} chat template list entries must be mappings")
            name, template = entry.get("name"), entry.get("template")
            if not isinstance(name, str) or not isinstance(template, str):
                raise ValueError(f"{source} chat template entries require string name/template fields")
            out[name] = template
        return out
    raise ValueError(f"unsupported chat template value in {source}")


def _token_text(value: Any, name: str) -> str | list[str]:
    if isinstance(value, str):
        return value
    if isinstance(value, Mapping) and isinstance(value.get("content"), str):
        return value["content"]
    if isinstance(value, Sequence) and not isinstance(value, (str, bytes)):
        items = [_token_text(v, name) for v in value]
        if any(not isinstance(v, str) for v in items):
            raise ValueError(f"special token {name!r} must be a string or list of strings")
        return items
    raise ValueError(f"special token {name!r} has an unsupported serialized value")


def special_tokens_from_config(config: Mapping[str, Any]) -> dict[str, str | list[str]]:
    out: dict[str, str | list[str]] = {}
    for name, value in config.items():
        if (name.endswith("_token") or name == "additional_special_tokens") and value is not None:
            out[name] = _token_text(value, name)
    extra = config.get("extra_special_tokens")
    if extra is not None:
        if not isinstance(extra, Mapping):
            raise ValueError("extra_special_tokens must be a mapping")
        for name, value in extra.items():
            if not isinstance(name, str):
                raise ValueError("extra special-token names must be strings")
            out[name] = _token_text(value, name)
    return out


class TrainingTokenizer:
    supports_message_loss = True

    def __init__(self, backend: Any, *, chat_template: ChatTemplate = None,
                 special_tokens: Mapping[str, str | list[str]] | None = None):
        self._backend = backend
        self.chat_template = chat_template
        self.special_tokens_map = dict(special_tokens or {})
        self._id_overrides: dict[str, int] = {}

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_directory(cls, source: str | Path) -> "TrainingTokenizer":
        from tokenizers import Tokenizer

        d = Path(source)
        tok = d / "tokenizer.json"
        if not tok.is_file():
            raise FileNotFoundError(f"missing {tok}; this trainer requires a serialized fast tokenizer.json")
        backend = Tokenizer.from_file(str(tok))
        config: dict[str, Any] = _json_object(d / "tokenizer_config.json") if (d / "tokenizer_config.json").is_file() else {}
        special: dict[str, str | list[str]] = {}
        if (d / "special_tokens_map.json").is_file():
            special.update(special_tokens_from_config(_json_object(d / "special_tokens_map.json")))
        special.update(special_tokens_from_config(config))
        template = normalize_chat_template(config.get("chat_template"), str(d / "tokenizer_config.json"))
        if template is None and (d / "chat_template.json").is_file():
            template = normalize_chat_template(_json(d / "chat_template.json"), str(d / "chat_template.json"))
        on_disk: dict[str, str] = {}
        if (d / "chat_template.jinja").is_file():
            on_disk["default"] = (d / "chat_template.jinja").read_text(encoding="utf-8")
        if (d / "chat_templates").is_dir():
            for p in sorted((d / "chat_templates").glob("*.jinja")):
                if p.is_file():
                    on_disk[p.stem] = p.read_text(encoding="utf-8")
        if on_disk:  # standalone Jinja files win over tokenizer_config.json
            template = on_disk["default"] if set(on_disk) == {"default"} else on_disk
        return cls(backend, chat_template=template, special_tokens=special)

    # ------------------------------------------------------------------ vocabulary
    def __len__(self) -> int:
        return int(self._backend.get_vocab_size(with_added_tokens=True))

    def get_vocab(self) -> dict[str, int]:
        return self._backend.get_vocab(with_added_tokens=True)

    def decode(self, ids: list[int]) -> str:
        return self._backend.decode(ids, skip_special_tokens=False)

    def token_to_id(self, token: str) -> int | None:
        value = self._backend.token_to_id(token)
        return None if value is None else int(value)

    def _special_id(self, name: str) -> int | None:
        if name in self._id_overrides:
            return self._id_overrides[name]
        token = self.special_tokens_map.get(name)
        return self.token_to_id(token) if isinstance(token, str) else None

    def _set_special_id(self, name: str, value: int | None) -> None:
        if value is None:
            self._id_overrides.pop(name, None)
            return
        if isinstance(value, bool) or not isinstance(value, int) or value < 0:
            raise ValueError(f"{name}_id must be a non-negative integer")
        token = self._backend.id_to_token(value)
        if token is None:
            raise ValueError(f"{name}_id={value} is not present in tokenizer.json")
        self._id_overrides[name] = value
        self.special_tokens_map[name] = token

    pad_token_id = property(lambda self: self._special_id("pad_token"),
                            lambda self, v: self._set_special_id("pad_token", v))
    eos_token_id = property(lambda self: self._special_id("eos_token"),
                            lambda self, v: self._set_special_id("eos_token", v))

    def validate_model_vocabulary(self, model_vocab_size: int) -> None:
        if isinstance(model_vocab_size, bool) or not isinstance(model_vocab_size, int) or model_vocab_size <= 0:
            raise ValueError("model_vocab_size must be a positive integer")
        largest = max((int(i) for i in self.get_vocab().values()), default=-1)
        if largest >= model_vocab_size:
            raise ValueError(f"tokenizer contains token id {largest}, outside model vocab_size={model_vocab_size}")

    # ------------------------------------------------------------------ encoding
    def _encode(self, text: str, *, add_special_tokens: bool, truncation: bool, max_length: int | None):
        if not isinstance(text, str):
            raise TypeError("the training tokenizer accepts one string at a time")
        if add_special_tokens:
            raise ValueError("automatic special-token insertion is unsupported; templates must add tokens explicitly")
        enc = self._backend.encode(text, add_special_tokens=False)
        if truncation:
            if isinstance(max_length, bool) or not isinstance(max_length, int) or max_length <= 0:
                raise ValueError("truncation requires a positive max_length")
            enc.truncate(max_length, stride=0, direction="right")
        return enc

    def __call__(self, text: str, *, add_special_tokens: bool = False, return_attention_mask: bool = True,
                 truncation: bool = False, max_length: int | None = None, **kwargs: Any) -> dict[str, list[int]]:
        if kwargs:
            raise TypeError(f"unsupported tokenizer arguments: {', '.join(sorted(kwargs))}")
        enc = self._encode(text, add_special_tokens=add_special_tokens, truncation=truncation, max_length=max_length)
        out = {"input_ids": list(enc.ids)}
        if return_attention_mask:
            out["attention_mask"] = list(enc.attention_mask)
        return out

    # ------------------------------------------------------------------ chat templates
    def get_chat_template(self, chat_template: str | None = None,
                          tools: Sequence[Mapping[str, Any]] | None = None) -> str:
        configured = self.chat_template
        if isinstance(configured, dict):
            if chat_template is not None and chat_template in configured:
                return configured[chat_template]
            if chat_template is None:
                if tools is not None and "tool_use" in configured:
                    return configured["tool_use"]
                if "default" in configured:
                    return configured["default"]
                raise ValueError(f"multiple chat templates are available but none is default: {sorted(configured)}")
        elif chat_template is None and configured is not None:
            return configured
        if chat_template is None:
            raise ValueError("messages training requires a chat template")
        return chat_template

    @staticmethod
    def render_with_spans(template: jinja2.Template, values: Mapping[str, Any],
                          keep_flags: Sequence[bool] | None = None) -> tuple[str, list[tuple[int, int]]]:
        if _ACTIVE_RECORDER.get() is not None:
            raise RuntimeError("assistant span tracker is already active")
        recorder = _SpanRecorder(keep_flags)
        token = _ACTIVE_RECORDER.set(recorder)
        try:
            for piece in template.generate(**values):
                recorder.push(piece)
            recorder.finish()
        finally:
            _ACTIVE_RECORDER.reset(token)
        return "".join(recorder.pieces), recorder.spans

    def apply_chat_template(self, conversation: Sequence[Mapping[str, Any]], tools=None, documents=None,
                            chat_template: str | None = None, add_generation_prompt: bool = False,
                            continue_final_message: bool | str = False, tokenize: bool = True,
                            padding: bool | str = False, truncation: bool = False, max_length: int | None = None,
                            return_tensors: str | None = None, return_dict: bool = True,
                            return_assistant_tokens_mask: bool = False,
                            tokenizer_kwargs: Mapping[str, Any] | None = None, **kwargs: Any):
        if not isinstance(conversation, Sequence) or isinstance(conversation, (str, bytes)) or not conversation:
            raise ValueError("conversation must be a non-empty sequence of message mappings")
        if any(not isinstance(m, Mapping) for m in conversation):
            raise ValueError("batched conversations are not supported by the training tokenizer")
        if continue_final_message:
            raise ValueError("continue_final_message is outside the training tokenizer contract")
        if padding not in (False, "do_not_pad"):
            raise ValueError("chat-template padding is handled by the trainer, not the tokenizer")
        if return_tensors is not None:
            raise ValueError("the training tokenizer returns Python lists only")
        if return_assistant_tokens_mask and not (tokenize and return_dict):
            raise ValueError("return_assistant_tokens_mask requires tokenize=True and return_dict=True")
        if tokenizer_kwargs and set(tokenizer_kwargs) - {"return_attention_mask"}:
            raise TypeError("unsupported tokenizer_kwargs: "
                            + ", ".join(sorted(set(tokenizer_kwargs) - {"return_attention_mask"})))
        tool_list = None
        if tools is not None:
            if not isinstance(tools, Sequence) or isinstance(tools, (str, bytes)):
                raise ValueError("tools must be a sequence of JSON-schema mappings")
            if any(not isinstance(t, Mapping) for t in tools):
                raise ValueError("tools must contain JSON-schema mappings; Python callables are unsupported")
            tool_list = [dict(t) for t in tools]
        if documents is not None and any(not isinstance(d, Mapping) for d in documents):
            raise ValueError("documents must contain mappings")
        template = compile_chat_template(self.get_chat_template(chat_template, tool_list))
        flags = [m.get("loss") is not False for m in conversation if m.get("role") == "assistant"]
        keep_flags = flags if False in flags else None
        values = {**self.special_tokens_map, **kwargs, "messages": list(conversation), "tools": tool_list,
                  "documents": None if documents is None else list(documents),
                  "add_generation_prompt": add_generation_prompt}
        if return_assistant_tokens_mask:
            rendered, spans = self.render_with_spans(template, values, keep_flags)
        else:
            rendered, spans = template.render(**values), []
        if not tokenize:
            return rendered
        enc = self._encode(rendered, add_special_tokens=False, truncation=truncation, max_length=max_length)
        ids = list(enc.ids)
        if not return_dict:
            return ids
        out = {"input_ids": ids, "attention_mask": list(enc.attention_mask)}
        if return_assistant_tokens_mask:
            mask = [0] * len(ids)
            for c0, c1 in spans:
                if c1 <= c0:
                    continue
                for i, (t0, t1) in enumerate(enc.offsets):
                    if t1 > t0 and t0 < c1 and t1 > c0:
                        mask[i] = 1
            out["assistant_masks"] = mask
        return out
