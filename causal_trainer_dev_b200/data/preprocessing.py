"""Record preprocessing: raw text or chat messages -> aligned per-token fields.

One :class:`Preprocessor` is configured per run and turns source records into
``{"input_ids", "attention_mask"[, "assistant_masks", "position_ids", "loss_weights"]}``.
Rules kept from the reference (src/causal_trainer/data/preprocessing.py):

* raw text is tokenised with truncation and **no** special tokens or EOS (``:273-291``);
* messages go through the chat template; with an assistant-only mode the conversation is
  rendered untruncated, spans are mapped to tokens, ``last_assistant_only_loss`` keeps the
  final contiguous span, and the example is cut right after its last assistant token that
  has a valid predecessor inside ``max_sequence_length`` (``:181-244, 494-573``);
* EndPrompt appends a terminal anchor prompt whose position ids sit at the *end* of a logical
  context of length ``L(i) = min + ((i*1103515245 + 12345) & 0x7FFFFFFF) % (max-min+1)``,
  with separate loss weights for context and prompt tokens (``:35-64, 347-414``);
* examples without any positive-weight target are dropped; dropping everything is an error
  unless ``allow_empty``.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Any, Iterable, Mapping, Sequence

TokenizedExample = dict[str, list]


class RowTable(list):
    """A list of row dictionaries that also answers the column-wise questions code written against
    ``datasets.Dataset`` asks: ``table["input_ids"]`` is that column as a list, ``column_names`` the
    keys of the rows, and ``cache_files`` is empty because rows are never spilled to Arrow files."""

    def __init__(self, rows=(), columns: Sequence[str] | None = None):
        super().__init__(rows)
        self._columns = list(columns) if columns is not None else None   # the schema of an empty table

    def __getitem__(self, index):
        if isinstance(index, str):
            return [row[index] for row in self]
        if isinstance(index, slice):
            return RowTable(super().__getitem__(index), self._columns)
        return super().__getitem__(index)

    @property
    def column_names(self) -> list[str]:
        if self._columns is not None:
            return list(self._columns)
        return list(self[0]) if len(self) else []

    @property
    def features(self) -> dict[str, str]:
        """Element type per column (``loss_weights`` is ``float32``, every other field ``int64``), the
        plain-dictionary counterpart of a ``datasets.Features`` of sequences."""
        return {name: ("float32" if name == "loss_weights" else "int64") for name in self.column_names}

    @property
    def cache_files(self) -> list:
        return []
_ASSISTANT_KEYS = ("assistant_masks", "assistant_mask", "assistant_tokens_mask")
_ALL_FILTERED = ("All examples were filtered out because none contained a valid positive-weight training target "
                 "within max_sequence_length. Increase the limit or filter/shorten the source data.")


@dataclass(frozen=True)
class EndPromptSettings:
    logical_length_min: int
    logical_length_max: int
    prompts: tuple[str, ...]
    prompt_loss_weight: float = 0.1
    context_loss_weight: float = 1.0

    def __post_init__(self) -> None:
        if self.logical_length_min <= 0 or self.logical_length_max <= 0:
            raise ValueError("EndPrompt logical lengths must be positive")
        if self.logical_length_min > self.logical_length_max:
            raise ValueError("EndPrompt minimum logical length cannot exceed its maximum")
        if not self.prompts or any(not isinstance(p, str) or not p for p in self.prompts):
            raise ValueError("EndPrompt requires at least one non-empty prompt")
        weights = (self.context_loss_weight, self.prompt_loss_weight)
        if any(not math.isfinite(w) or w < 0.0 for w in weights):
            raise ValueError("EndPrompt loss weights must be finite and non-negative")
        if not any(w > 0.0 for w in weights):
            raise ValueError("at least one EndPrompt loss weight must be positive")

    def logical_length_for_row(self, index: int) -> int:
        span = self.logical_length_max - self.logical_length_min + 1
        if span == 1:
            return self.logical_length_min
        return self.logical_length_min + ((int(index) * 1_103_515_245 + 12_345) & 0x7FFFFFFF) % span


# ----------------------------------------------------------------------------------------- helpers
def _ints(value: Any, name: str) -> list[int]:
    if hasattr(value, "tolist"):
        value = value.tolist()
    if isinstance(value, tuple):
        value = list(value)
    if not isinstance(value, list):
        raise ValueError(f"Tokenizer field {name!r} must be a one-dimensional sequence.")
    if value and isinstance(value[0], (list, tuple)):
        if len(value) != 1:
            raise ValueError(f"Tokenizer field {name!r} unexpectedly contains a batch.")
        value = list(value[0])
    try:
        return [int(v) for v in value]
    except (TypeError, ValueError) as exc:
        raise ValueError(f"Tokenizer field {name!r} must contain integers.") from exc


def normalize_tokenizer_output(encoded: Mapping[str, Any], require_assistant_mask: bool) -> TokenizedExample:
    if not isinstance(encoded, Mapping) or "input_ids" not in encoded:
        raise ValueError("Tokenizer output must be a mapping containing 'input_ids'.")
    ids = _ints(encoded["input_ids"], "input_ids")
    if not ids:
        raise ValueError("Tokenization produced an empty sequence.")
    mask = _ints(encoded["attention_mask"], "attention_mask") if "attention_mask" in encoded else [1] * len(ids)
    if len(mask) != len(ids):
        raise ValueError("attention_mask and input_ids must have the same length.")
    if any(v not in (0, 1) for v in mask):
        raise ValueError("attention_mask must contain only binary 0/1 values.")
    out: TokenizedExample = {"input_ids": ids, "attention_mask": mask}
    key = next((k for k in _ASSISTANT_KEYS if k in encoded), None)
    if require_assistant_mask:
        if key is None:
            raise ValueError("Assistant loss masking requires a chat template that returns an assistant token mask. "
                             "Add {% generation %} blocks to the tokenizer chat template.")
        am = _ints(encoded[key], key)
        if len(am) != len(ids):
            raise ValueError("assistant mask and input_ids must have the same length.")
        if any(v not in (0, 1) for v in am):
            raise ValueError("assistant mask must contain only binary 0/1 values.")
        out["assistant_masks"] = am
    return out


def keep_last_span(mask: Sequence[int]) -> list[int]:
    out = [0] * len(mask)
    stop = next((i for i in range(len(mask) - 1, -1, -1) if int(mask[i]) != 0), None)
    if stop is None:
        return out
    start = stop
    while start > 0 and int(mask[start - 1]) != 0:
        start -= 1
    out[start:stop + 1] = [1] * (stop - start + 1)
    return out


def trainable_assistant_indices(ex: Mapping[str, Any], limit: int | None = None) -> list[int]:
    """Assistant target positions whose predecessor and themselves are valid tokens."""
    ids, mask, am = ex.get("input_ids"), ex.get("attention_mask"), ex.get("assistant_masks")
    if ids is None or mask is None or am is None:
        return []
    n = min(len(ids), len(mask), len(am))
    if limit is not None:
        n = min(n, limit)
    return [i for i in range(1, n) if int(am[i]) != 0 and int(mask[i - 1]) == 1 and int(mask[i]) == 1]


def has_effective_loss_target(ex: Mapping[str, Any]) -> bool:
    ids, mask = ex.get("input_ids"), ex.get("attention_mask")
    if ids is None or mask is None:
        return False
    weights = ex.get("loss_weights")
    n = min(len(ids), len(mask)) if weights is None else min(len(ids), len(mask), len(weights))
    return any(int(mask[i - 1]) == 1 and int(mask[i]) == 1 and (weights is None or float(weights[i]) > 0.0)
               for i in range(1, n))


def positions_from_mask(mask: Sequence[int]) -> list[int]:
    out, cur = [], 0
    for v in mask:
        if int(v) == 1:
            out.append(cur)
            cur += 1
        else:
            out.append(0)
            cur = 0
    return out


def _empty_like(ex: TokenizedExample) -> TokenizedExample:
    return {k: [] for k in ex}


def _validate_messages(messages: Any) -> list[Mapping[str, Any]]:
    if not isinstance(messages, Sequence) or isinstance(messages, (str, bytes)) or not messages:
        raise ValueError("A messages example must be a non-empty sequence of role/content mappings.")
    out = list(messages)
    for i, m in enumerate(out):
        if not isinstance(m, Mapping):
            raise ValueError(f"messages[{i}] must be a mapping.")
        if "role" not in m or "content" not in m:
            raise ValueError(f"messages[{i}] must contain both 'role' and 'content'.")
    return out


# ----------------------------------------------------------------------------------------- preprocessor
@dataclass
class Preprocessor:
    tokenizer: Any
    dataset_text_field: str
    max_sequence_length: int
    assistant_only_loss: bool = False
    last_assistant_only_loss: bool = False
    endprompt: EndPromptSettings | None = None

    def __post_init__(self) -> None:
        if self.max_sequence_length <= 0:
            raise ValueError("max_sequence_length must be positive.")
        if self.assistant_only_loss and self.last_assistant_only_loss:
            raise ValueError("assistant_only_loss and last_assistant_only_loss are mutually exclusive")

    @property
    def assistant_mode(self) -> str | None:
        if self.last_assistant_only_loss:
            return "last_assistant_only_loss"
        return "assistant_only_loss" if self.assistant_only_loss else None

    # ---- raw text ----
    def tokenize_raw_text(self, text: str, max_length: int | None = None) -> TokenizedExample:
        if not isinstance(text, str):
            raise ValueError("Raw text examples must be strings.")
        enc = self.tokenizer(text, add_special_tokens=False, return_attention_mask=True, truncation=True,
                             max_length=self.max_sequence_length if max_length is None else max_length)
        return normalize_tokenizer_output(enc, require_assistant_mask=False)

    # ---- messages ----
    def tokenize_messages(self, messages: Any, *, max_length: int | None = None, tools: Any = None,
                          chat_template_kwargs: Mapping[str, Any] | None = None) -> TokenizedExample:
        limit = self.max_sequence_length if max_length is None else max_length
        mode = self.assistant_mode
        msgs = _validate_messages(messages)
        disabled = False
        if mode is not None:
            for i, m in enumerate(msgs):
                if m.get("role") == "assistant":
                    v = m.get("loss")
                    if v is not None and type(v) is not bool:
                        raise ValueError(f"messages[{i}].loss must be a boolean or null.")
                    disabled |= v is False
        apply = getattr(self.tokenizer, "apply_chat_template", None)
        if not callable(apply):
            raise ValueError("The tokenizer must provide apply_chat_template for messages training.")
        if disabled and not getattr(self.tokenizer, "supports_message_loss", False):
            raise ValueError("The tokenizer does not support assistant message loss=false.")
        if isinstance(tools, str):
            tools = json.loads(tools)
        elif isinstance(tools, list):
            tools = [json.loads(t) if isinstance(t, str) else t for t in tools]
        opts = dict(chat_template_kwargs or {})
        # Spans are recovered on the untruncated rendering; all fields are cut together afterwards.
        opts.update(tokenize=True, return_dict=True, return_attention_mask=True,
                    return_assistant_tokens_mask=mode is not None,
                    truncation=mode is None, max_length=None if mode is not None else limit)
        if tools is not None:
            opts["tools"] = tools
        out = normalize_tokenizer_output(apply(msgs, **opts), require_assistant_mask=mode is not None)
        if mode is None:
            return out
        if not any(out["assistant_masks"]):
            if any(m.get("role") == "assistant" and m.get("loss") is not False and bool(m.get("content")) for m in msgs):
                raise ValueError(
                    f"{mode} was requested, but the tokenized example contains no assistant tokens despite having "
                    "assistant content. Check that the tokenizer chat template contains {% generation %} blocks.")
            return _empty_like(out)
        if self.last_assistant_only_loss:
            final_disabled = next((m.get("loss") is False for m in reversed(msgs) if m.get("role") == "assistant"), False)
            out["assistant_masks"] = [0] * len(out["assistant_masks"]) if final_disabled else keep_last_span(
                out["assistant_masks"])
        idx = trainable_assistant_indices(out, limit)
        if not idx:
            return _empty_like(out)
        return {k: v[:idx[-1] + 1] for k, v in out.items()}

    # ---- EndPrompt ----
    def _prompt_ids(self, example_index: int) -> list[int]:
        s = self.endprompt
        if self.max_sequence_length <= 1:
            raise ValueError("max_sequence_length must be greater than one for EndPrompt")
        if s.logical_length_min < self.max_sequence_length:
            raise ValueError("EndPrompt logical lengths must be at least max_sequence_length")
        text = s.prompts[int(example_index) % len(s.prompts)]
        enc = self.tokenizer(text, add_special_tokens=False, return_attention_mask=False)
        ids = _ints(enc["input_ids"], "EndPrompt prompt.input_ids")
        if not ids:
            raise ValueError("EndPrompt terminal prompt tokenized to an empty sequence")
        if len(ids) >= self.max_sequence_length:
            raise ValueError("EndPrompt terminal prompt must be shorter than max_sequence_length; "
                             f"got {len(ids)} tokens for length {self.max_sequence_length}")
        if len(ids) > s.logical_length_min:
            raise ValueError("EndPrompt prompt is longer than the minimum logical length")
        return ids

    def _append_endprompt(self, ctx: TokenizedExample, prompt: list[int], example_index: int,
                          assistant: bool) -> TokenizedExample:
        s = self.endprompt
        if assistant and not trainable_assistant_indices(ctx):
            empty = _empty_like(ctx)
            empty["position_ids"], empty["loss_weights"] = [], []
            return empty
        ids = [int(v) for v in ctx["input_ids"]]
        mask = [int(v) for v in ctx["attention_mask"]]
        logical = s.logical_length_for_row(example_index)
        out: TokenizedExample = {k: list(v) for k, v in ctx.items()}
        out["input_ids"] = ids + list(prompt)
        out["attention_mask"] = mask + [1] * len(prompt)
        out["position_ids"] = positions_from_mask(mask) + list(range(logical - len(prompt), logical))
        if assistant:
            am = [int(v) for v in ctx["assistant_masks"]]
            out["assistant_masks"] = am + [0] * len(prompt)
            weights = [float(s.context_loss_weight) * float(a) * float(m) for a, m in zip(am, mask, strict=True)]
        else:
            weights = [float(s.context_loss_weight) * float(m) for m in mask]
        out["loss_weights"] = weights + [float(s.prompt_loss_weight)] * len(prompt)
        return out if has_effective_loss_target(out) else _empty_like(out)

    # ---- one example ----
    def __call__(self, example: Mapping[str, Any], example_index: int = 0) -> TokenizedExample:
        if self.dataset_text_field not in example:
            raise KeyError(f"Dataset example does not contain field {self.dataset_text_field!r}.")
        value = example[self.dataset_text_field]
        mode = self.assistant_mode
        if isinstance(value, str):
            if mode is not None:
                raise ValueError(f"{mode} is supported only for messages examples, not raw text.")
            if self.endprompt is None:
                return self.tokenize_raw_text(value)
            prompt = self._prompt_ids(example_index)
            budget = self.max_sequence_length - len(prompt)
            enc = self.tokenizer(value, add_special_tokens=False, return_attention_mask=False, truncation=True,
                                 max_length=budget)
            ctx_ids = _ints(enc["input_ids"], "EndPrompt context.input_ids")
            if len(ctx_ids) > budget:
                raise ValueError("EndPrompt context tokenizer ignored its truncation budget")
            return self._append_endprompt({"input_ids": ctx_ids, "attention_mask": [1] * len(ctx_ids)}, prompt,
                                          example_index, assistant=False)
        kw = dict(tools=example.get("tools"), chat_template_kwargs=example.get("chat_template_kwargs"))
        if self.endprompt is None:
            return self.tokenize_messages(value, **kw)
        prompt = self._prompt_ids(example_index)
        budget = self.max_sequence_length - len(prompt)
        ctx = self.tokenize_messages(value, max_length=budget, **kw)
        if len(ctx.get("input_ids", ())) > budget:
            raise ValueError("EndPrompt chat tokenizer ignored its truncation budget")
        return self._append_endprompt(ctx, prompt, example_index, assistant=mode is not None)

    def keep(self, ex: Mapping[str, Any]) -> bool:
        return ((self.assistant_mode is None or bool(trainable_assistant_indices(ex)))
                and (self.endprompt is None or has_effective_loss_target(ex)))

    # ---- many examples ----
    def run(self, records: Iterable[Mapping[str, Any]], *, example_index_offset: int = 0, allow_empty: bool = False,
            num_workers: int | None = None) -> list[TokenizedExample]:
        """Tokenises and filters ``records`` (in order); ``num_workers`` fans out over processes."""
        indexed = list(enumerate(records, start=example_index_offset))
        if num_workers and num_workers > 1 and len(indexed) > 4 * num_workers:
            import multiprocessing as mp

            with mp.get_context("fork").Pool(num_workers, initializer=_install_worker, initargs=(self,)) as pool:
                out = pool.map(_worker_call, indexed, chunksize=max(1, len(indexed) // (8 * num_workers)))
        else:
            out = [self(rec, i) for i, rec in indexed]
        if self.assistant_mode is not None or self.endprompt is not None:
            out = [ex for ex in out if self.keep(ex)]
            if not out and not allow_empty:
                raise ValueError(_ALL_FILTERED)
        return out


_WORKER: Preprocessor | None = None


def _install_worker(pre: Preprocessor) -> None:
    global _WORKER
    _WORKER = pre


def _worker_call(item: tuple[int, Mapping[str, Any]]) -> TokenizedExample:
    return _WORKER(item[1], item[0])


# ---- one example at a time, as plain functions (src/causal_trainer/data/preprocessing.py:273-640) ----
def tokenize_raw_text(text: str, tokenizer, *, max_sequence_length: int) -> TokenizedExample:
    """Raw text: no special tokens are added, truncation at ``max_sequence_length``."""
    return Preprocessor(tokenizer, "text", max_sequence_length).tokenize_raw_text(text)


def tokenize_messages(messages, tokenizer, *, max_sequence_length: int, assistant_only_loss: bool = False,
                      last_assistant_only_loss: bool = False, tools: Any = None,
                      chat_template_kwargs: Mapping[str, Any] | None = None) -> TokenizedExample:
    """A conversation through the chat template, with the assistant mask the loss mode asks for."""
    pre = Preprocessor(tokenizer, "messages", max_sequence_length, assistant_only_loss, last_assistant_only_loss)
    return pre.tokenize_messages(messages, tools=tools, chat_template_kwargs=chat_template_kwargs)


def tokenize_endprompt_text(text: str, tokenizer, *, max_sequence_length: int, settings: EndPromptSettings,
                            example_index: int) -> TokenizedExample:
    """Raw text with this row's prompt anchored at its logical position."""
    if not isinstance(text, str):
        raise ValueError("EndPrompt is supported only for raw string records")
    return Preprocessor(tokenizer, "text", max_sequence_length, endprompt=settings)({"text": text}, example_index)


def tokenize_endprompt_messages(messages, tokenizer, *, max_sequence_length: int, assistant_only_loss: bool,
                                last_assistant_only_loss: bool = False, settings: EndPromptSettings,
                                example_index: int, tools: Any = None,
                                chat_template_kwargs: Mapping[str, Any] | None = None) -> TokenizedExample:
    """A conversation followed by this row's prompt."""
    pre = Preprocessor(tokenizer, "messages", max_sequence_length, assistant_only_loss, last_assistant_only_loss,
                       settings)
    return pre({"messages": messages, "tools": tools, "chat_template_kwargs": chat_template_kwargs}, example_index)


def preprocess_example(example: Mapping[str, Any], tokenizer, *, dataset_text_field: str, max_sequence_length: int,
                       assistant_only_loss: bool = False, last_assistant_only_loss: bool = False,
                       endprompt: EndPromptSettings | None = None, example_index: int = 0) -> TokenizedExample:
    """One record; a string field is raw text, a sequence of mappings a conversation."""
    return Preprocessor(tokenizer, dataset_text_field, max_sequence_length, assistant_only_loss,
                        last_assistant_only_loss, endprompt)(example, example_index)


def preprocess_records(records, tokenizer, *, dataset_text_field: str, max_sequence_length: int,
                       assistant_only_loss: bool = False, last_assistant_only_loss: bool = False,
                       endprompt: EndPromptSettings | None = None, example_index_offset: int = 0,
                       allow_empty: bool = False, num_workers: int | None = None) -> list[TokenizedExample]:
    """Functional face of :class:`Preprocessor` (accepts any iterable, ``datasets.Dataset`` included)."""
    pre = Preprocessor(tokenizer, dataset_text_field, max_sequence_length, assistant_only_loss,
                       last_assistant_only_loss, endprompt)
    # the output schema is fixed by the options, not inferred from the first row, so a shard whose
    # rows were all filtered out still merges with its siblings (src/causal_trainer/data/preprocessing.py:827-836)
    columns = ["input_ids", "attention_mask"]
    if assistant_only_loss or last_assistant_only_loss:
        columns.append("assistant_masks")
    if endprompt is not None:
        columns += ["position_ids", "loss_weights"]
    return RowTable(pre.run(records, example_index_offset=example_index_offset, allow_empty=allow_empty,
                            num_workers=num_workers), columns)


preprocess_dataset = preprocess_records
