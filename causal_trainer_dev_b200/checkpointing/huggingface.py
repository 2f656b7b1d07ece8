"""Hugging Face checkpoint import / export for single-replica and FSDP-sharded parameters.

Formats are those of the reference (src/causal_trainer/checkpointing/huggingface.py):

* ``model.safetensors``: HF Llama key names, ``[out,in]`` layout, one dtype, tensor order =
  sorted parameter-tree order (``hf_export_order``), ``__metadata__ = {"format": "pt",
  "checkpoint_id": <32 hex>}`` (``:634-655, 1156-1213``);
* ``config.json`` rewritten with the actual parameter dtype; tokenizer files and
  ``chat_templates/*.jinja`` copied (``:676-739``);
* ``optimizer/state.safetensors`` with keys ``state/%06d`` + ``optimizer/manifest.json``
  (``format: optimizer-state-safetensors``, ``format_version: 1``) (``:1517-1646``).

Because ``nn.Linear`` already stores ``[out,in]``, no transposes happen anywhere.  Loading is
lazy: a rank maps the files and copies only the byte ranges that fall into its shard.
Export streams one tensor at a time to rank 0 in bounded rounds (64 MiB), so host memory on
every rank stays bounded by one round regardless of model size (``:787-988, 1099-1337``).
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import shutil
import uuid
from pathlib import Path
from typing import Any, Callable, Iterator

import torch

from ..models.config import ModelConfig
from ..models.params import ModelParams, hf_export_order, hf_name_map, unit_layouts
from ..parallel import runtime as rt
from . import safetensors_io as st

GATHER_ROUND_BYTES = 64 * 1024 * 1024
TOKENIZER_NAMES = {
    "added_tokens.json", "chat_template.json", "generation_config.json", "merges.txt", "preprocessor_config.json",
    "processor_config.json", "special_tokens_map.json", "tokenizer.json", "tokenizer.model", "tokenizer_config.json",
    "vocab.json",
}
TOKENIZER_SUFFIXES = (".jinja", ".model", ".tiktoken")
TORCH_DTYPE_NAMES = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}


# --------------------------------------------------------------------------------------- sources
def resolve_hf_source(repo_id_or_path: str | os.PathLike[str], *, revision: str | None = None,
                      token: str | None = None, cache_dir: str | None = None, local_files_only: bool = False) -> Path:
    """A local directory is used as is; anything else is fetched from the Hub (with retries)."""
    candidate = Path(repo_id_or_path).expanduser()
    if candidate.exists():
        if not candidate.is_dir():
            raise ValueError(f"model source must be a directory, got {candidate}")
        return candidate.resolve()
    from huggingface_hub import snapshot_download

    from ..hf_retry import retry_hf_call

    return Path(retry_hf_call(lambda: snapshot_download(
        repo_id=str(repo_id_or_path), revision=revision, token=token, cache_dir=cache_dir,
        local_files_only=local_files_only,
        allow_patterns=["*.json", "*.jinja", "chat_templates/*.jinja", "*.model", "*.safetensors", "*.tiktoken", "*.txt"],
    ), description=f"download {repo_id_or_path}"))


def load_hf_config(source: str | os.PathLike[str]) -> dict[str, Any]:
    path = Path(source) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"missing model config: {path}")
    value = json.loads(path.read_text(encoding="utf-8"))
    if not isinstance(value, dict):
        raise ValueError(f"{path} must contain a JSON object")
    return value


SafeTensorIndex = st.SafeTensorIndex          # the reader classes live in safetensors_io; these names keep
TensorInfo = st.TensorInfo                    # code written against this module's reference counterpart working


@dataclasses.dataclass(frozen=True)
class TensorMapping:
    """Where a leaf of the nested parameter tree is stored: its Hugging Face key, and whether the
    stored tensor is the transpose of the tree's ``[in, out]`` kernel."""
    parameter_path: str
    hf_key: str
    transpose: bool = False


_TREE_LEAVES = {
    ("attention", "kernel"): ("self_attn.{p}.weight", True), ("attention", "bias"): ("self_attn.{p}.bias", False),
    ("mlp", "kernel"): ("mlp.{p}.weight", True),
}
_TREE_PROJECTIONS = {"attention": ("q_proj", "k_proj", "v_proj", "o_proj"), "mlp": ("gate_proj", "up_proj", "down_proj")}
_TREE_TOP = {"embed_tokens/embedding": ("model.embed_tokens.weight", False), "norm/scale": ("model.norm.weight", False),
             "lm_head/kernel": ("lm_head.weight", True)}


def parameter_to_hf_mapping(path: str) -> TensorMapping:
    """Nested-tree path (``layers/3/attention/q_proj/kernel``, optionally under ``model/``) to its
    Hugging Face tensor (src/causal_trainer/checkpointing/huggingface.py:108-146).  Kernels are
    ``[in, out]`` in the tree and ``[out, in]`` on disk, hence ``transpose``; this framework keeps
    the on-disk orientation in memory (``ModelParams.tensor(hf_key)``)."""
    path = path.strip("/")
    path = path[len("model/"):] if path.startswith("model/") else path
    if path in _TREE_TOP:
        key, transpose = _TREE_TOP[path]
        return TensorMapping(path, key, transpose)
    parts = path.split("/")
    if len(parts) >= 4 and parts[0] == "layers" and parts[1].isdigit():
        prefix = f"model.layers.{parts[1]}."
        if len(parts) == 4 and parts[2] in ("input_layernorm", "post_attention_layernorm") and parts[3] == "scale":
            return TensorMapping(path, f"{prefix}{parts[2]}.weight")
        if len(parts) == 5 and (parts[2], parts[4]) in _TREE_LEAVES and parts[3] in _TREE_PROJECTIONS[parts[2]]:
            template, transpose = _TREE_LEAVES[(parts[2], parts[4])]
            return TensorMapping(path, prefix + template.format(p=parts[3]), transpose)
    raise KeyError(f"no Hugging Face tensor mapping for parameter path {path!r}")


def expected_model_layout(cfg: ModelConfig, dtype: torch.dtype) -> dict[str, tuple[str, tuple[int, ...]]]:
    """``{hf_key: (safetensors dtype, shape)}`` of a merged checkpoint of this architecture."""
    mapping = hf_name_map(cfg)
    layouts = {lay.name: lay for lay in unit_layouts(cfg)}
    out = {}
    for name in hf_export_order(cfg):
        unit, seg, _, rows = mapping[name]
        shape = layouts[unit].segment(seg).shape
        out[name] = (st.DTYPE_NAMES[dtype], (rows, *shape[1:]))
    return out


# --------------------------------------------------------------------------------------- loading
def _check_source(index: st.SafeTensorIndex, cfg: ModelConfig) -> None:
    want = expected_model_layout(cfg, torch.bfloat16)
    missing = sorted(k for k in want if k not in index.where)
    unexpected = sorted(k for k in index.where if k not in want)
    if missing or unexpected:
        # an extra tensor (an output-projection bias, a tied or renamed head) is a different architecture
        raise ValueError("checkpoint tensors do not exactly match the supported architecture; "
                         f"missing {missing[:4]}{'...' if len(missing) > 4 else ''}, "
                         f"unexpected {unexpected[:4]}{'...' if len(unexpected) > 4 else ''}")
    for key, (_, shape) in want.items():
        got = index.info(key).shape
        if tuple(got) != tuple(shape):
            raise ValueError(f"{key}: checkpoint shape {tuple(got)} does not match the architecture {tuple(shape)}")


def load_parameters(source: str | os.PathLike[str], params: ModelParams) -> None:
    """Fills a full replica from ``model.safetensors`` (cast to the replica's dtype)."""
    index = st.SafeTensorIndex(source)
    try:
        _check_source(index, params.config)
        with torch.no_grad():
            for name in params.hf_names():
                params.tensor(name).copy_(index.tensor(name).to(params.dtype))
    finally:
        index.close()


def tp_window(name: str, cfg: ModelConfig, tp: int, tp_rank: int) -> tuple[int, int, int, int, str]:
    """``(row0, rows, col0, cols, kind)`` of the part of Hugging Face tensor ``name`` that tensor-
    parallel rank ``tp_rank`` stores; ``kind`` is how the parts tile the tensor: ``"rows"``
    (column-parallel weights, biases, embedding, head), ``"cols"`` (row-parallel o/down weights),
    ``"rep"`` (norm scales, every rank holds all of it) or ``"heads"`` (key/value projections with
    fewer heads than ranks: row blocks, each stored by ``tp / Hkv`` consecutive ranks)."""
    d, q, kv, f, v = cfg.hidden_size, cfg.query_width, cfg.key_value_width, cfg.intermediate_size, cfg.vocab_size
    leaf = name.split(".")[-2]
    vector = name.endswith(".bias") or "norm" in name
    if "norm" in name:
        return 0, d, 0, 1, "rep"
    if leaf in ("k_proj", "v_proj") and cfg.num_key_value_heads % tp:
        # fewer key/value heads than ranks: groups of tp / Hkv ranks hold a copy of one whole head
        rep = tp // cfg.num_key_value_heads
        return (tp_rank // rep) * cfg.head_dim, cfg.head_dim, 0, (1 if vector else d), "heads"
    rows_of = {"q_proj": q, "k_proj": kv, "v_proj": kv, "gate_proj": f, "up_proj": f, "embed_tokens": v, "lm_head": v}
    if leaf in rows_of:
        n = rows_of[leaf] // tp
        return tp_rank * n, n, 0, (1 if vector else d), "rows"
    if leaf == "o_proj":
        return 0, d, tp_rank * (q // tp), q // tp, "cols"
    if leaf == "down_proj":
        return 0, d, tp_rank * (f // tp), f // tp, "cols"
    raise KeyError(name)


def _full_columns(name: str, cfg: ModelConfig) -> int:
    leaf = name.split(".")[-2]
    if name.endswith(".bias") or "norm" in name:
        return 1
    return {"o_proj": cfg.query_width, "down_proj": cfg.intermediate_size}.get(leaf, cfg.hidden_size)


def load_sharded_parameters(source: str | os.PathLike[str], runtime) -> None:
    """Fills the FSDP shards: every rank reads only the byte ranges that fall inside its slices
    (of its tensor-parallel window of each tensor, when the runtime holds a tp slice)."""
    cfg = runtime.cfg
    full_cfg = getattr(runtime, "full_cfg", cfg)
    tp, tp_rank = getattr(runtime, "tp_world", 1), getattr(runtime, "tp_rank", 0)
    index = st.SafeTensorIndex(source)
    mapping = hf_name_map(cfg)
    try:
        _check_source(index, full_cfg)
        by_unit: dict[str, list[str]] = {}
        for name in hf_export_order(cfg):
            by_unit.setdefault(mapping[name][0], []).append(name)
        with torch.no_grad():
            for unit_name, names in by_unit.items():
                u = runtime.units[unit_name]
                lo, hi = runtime.rank * u.shard_elems, (runtime.rank + 1) * u.shard_elems
                shard = runtime.shard_view(unit_name)
                shard.zero_()
                for name in names:
                    _, seg_name, r0, rows = mapping[name]
                    seg = u.layout.segment(seg_name)
                    inner = 1
                    for s in seg.shape[1:]:
                        inner *= s
                    t0 = seg.offset + r0 * inner            # flat extent of this rank's part in the unit
                    t1 = t0 + rows * inner
                    a, b = max(t0, lo), min(t1, hi)
                    if b <= a:
                        continue
                    f = index.file_of(name)
                    if tp == 1:
                        piece = f.flat_range(name, a - t0, b - t0)
                    else:
                        row0, _, col0, cols, _ = tp_window(name, full_cfg, tp, tp_rank)
                        width = _full_columns(name, full_cfg)
                        i0, i1 = (a - t0) // inner, (b - t0 - 1) // inner + 1      # local rows touched
                        block = f.flat_range(name, (row0 + i0) * width, (row0 + i1) * width).view(i1 - i0, width)
                        local = block[:, col0:col0 + cols].reshape(-1)
                        piece = local[(a - t0) - i0 * inner:(b - t0) - i0 * inner]
                    shard[a - lo:b - lo].copy_(piece.to(torch.bfloat16))
    finally:
        index.close()


# --------------------------------------------------------------------------------------- export
class TensorSource:
    """Where export reads tensors from: a local replica or the FSDP runtime (bounded gathers)."""

    def __init__(self, cfg: ModelConfig, params: ModelParams | None = None, runtime=None,
                 transform: Callable[[str, torch.Tensor], torch.Tensor] | None = None):
        if (params is None) == (runtime is None):
            raise ValueError("give exactly one of params / runtime")
        self.cfg, self.params, self.runtime, self.transform = cfg, params, runtime, transform
        # under tensor parallelism the runtime stores slices laid out by its local config
        self.mapping = hf_name_map(runtime.cfg if runtime is not None else cfg)
        self.dtype = params.dtype if params is not None else torch.bfloat16

    def chunks(self, name: str) -> Iterator[torch.Tensor]:
        """Flat CPU pieces of tensor ``name`` in order; collective under FSDP, data on rank 0 only."""
        if self.params is not None:
            t = self.params.tensor(name).detach()
            if self.transform is not None:
                t = self.transform(name, t)
            flat = t.reshape(-1)
            step = max(1, GATHER_ROUND_BYTES // flat.element_size())
            for i in range(0, flat.numel(), step):
                yield flat[i:i + step].cpu()
            return
        yield from self._sharded_chunks(name)

    def _sharded_chunks(self, name: str) -> Iterator[torch.Tensor]:
        rtm = self.runtime
        tp, tp_rank = getattr(rtm, "tp_world", 1), getattr(rtm, "tp_rank", 0)
        unit_name, seg_name, r0, rows = self.mapping[name]
        u = rtm.units[unit_name]
        seg = u.layout.segment(seg_name)
        inner = 1
        for s in seg.shape[1:]:
            inner *= s
        t0 = seg.offset + r0 * inner
        local_numel = rows * inner
        step = max(1, GATHER_ROUND_BYTES // 2)
        shard = rtm.shard_view(unit_name)
        lo, hi = rtm.rank * u.shard_elems, (rtm.rank + 1) * u.shard_elems
        me = rt.process_index()

        def gather_round(want_tp: int | None, a: int, b: int):
            """Every process sends the part of local flat range [a, b) it owns (if its tp rank is
            wanted); process 0 gets ``[(tp_rank, start, piece), ...]``."""
            x, y = max(t0 + a, lo), min(t0 + b, hi)
            mine = torch.empty(0, dtype=torch.bfloat16)
            if y > x and (want_tp is None or want_tp == tp_rank):
                mine = shard[x - lo:y - lo].detach().cpu()
            return rt.gather_object_to_zero((tp_rank, x - t0, mine))

        kind = "rows" if tp == 1 else tp_window(name, self.cfg, tp, 0)[4]
        if kind in ("rows", "rep", "heads"):
            owners = range(tp)
            if kind == "rep":
                owners = range(1)
            elif kind == "heads":
                owners = range(0, tp, tp // self.cfg.num_key_value_heads)     # first rank of every head
            for r in owners:
                for a in range(0, local_numel, step):
                    b = min(local_numel, a + step)
                    pieces = gather_round(r, a, b)
                    if me == 0:
                        out = torch.empty(b - a, dtype=torch.bfloat16)
                        for _, start, piece in pieces:
                            if piece.numel():
                                out[start - a:start - a + piece.numel()] = piece
                        yield out
                    else:
                        yield torch.empty(0, dtype=torch.bfloat16)
            return
        # row-parallel weight: every output row is the concatenation of the tp ranks' row pieces
        block_rows = max(1, step // (inner * tp))
        for i0 in range(0, rows, block_rows):
            i1 = min(rows, i0 + block_rows)
            pieces = gather_round(None, i0 * inner, i1 * inner)
            if me == 0:
                parts = [torch.empty((i1 - i0) * inner, dtype=torch.bfloat16) for _ in range(tp)]
                for r, start, piece in pieces:
                    if piece.numel():
                        parts[r][start - i0 * inner:start - i0 * inner + piece.numel()] = piece
                yield torch.cat([x.view(i1 - i0, inner) for x in parts], dim=1).reshape(-1)
            else:
                yield torch.empty(0, dtype=torch.bfloat16)


def copy_hf_assets(source: Path | None, destination: Path, cfg: ModelConfig, dtype: torch.dtype) -> None:
    """``config.json`` (normalised, actual dtype) plus tokenizer files and chat templates."""
    destination.mkdir(parents=True, exist_ok=True)
    # The source's config keeps its extra keys; every semantic field is rewritten from the model
    # configuration.  Reading accepts the Transformers 5 spellings (``dtype``, ``rope_parameters``)
    # but a full / merged checkpoint always goes back to the fixed source format
    # (src/causal_trainer/checkpointing/huggingface.py:684-718).
    config: dict[str, Any] = {}
    if source is not None and (source / "config.json").is_file():
        config = json.loads((source / "config.json").read_text(encoding="utf-8"))
    config.update(cfg.to_dict())
    config.pop("rope_parameters", None)
    config.pop("dtype", None)
    config["torch_dtype"] = TORCH_DTYPE_NAMES.get(dtype, "bfloat16")
    config.setdefault("architectures", ["LlamaForCausalLM"])
    (destination / "config.json").write_text(json.dumps(config, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    if source is None:
        return
    for item in sorted(source.iterdir()):
        if item.is_file() and (item.name in TOKENIZER_NAMES or item.name.endswith(TOKENIZER_SUFFIXES)):
            if item.resolve() != (destination / item.name).resolve():
                shutil.copy2(item, destination / item.name)
    templates = source / "chat_templates"
    if templates.is_dir():
        (destination / "chat_templates").mkdir(exist_ok=True)
        for item in sorted(templates.glob("*.jinja")):
            shutil.copy2(item, destination / "chat_templates" / item.name)


def export_plan_digest(names: list[str], layout: dict[str, tuple[str, tuple[int, ...]]]) -> bytes:
    return rt.digest_of([[n, layout[n][0], list(layout[n][1])] for n in names])


def export_hf_checkpoint(destination: str | os.PathLike[str], source: TensorSource, *, checkpoint_id: str,
                         assets_from: Path | None = None) -> None:
    """Streams ``model.safetensors`` (+ assets) into ``destination``; collective, rank 0 writes."""
    dest = Path(destination)
    cfg = source.cfg
    layout = expected_model_layout(cfg, source.dtype)
    names = hf_export_order(cfg)
    rt.assert_equal(export_plan_digest(names, layout), "checkpoint export plan")
    writer = None
    error: BaseException | None = None
    if rt.process_index() == 0:
        try:
            entries = [(n, layout[n][0], layout[n][1]) for n in names]
            writer = st.StreamingWriter(dest / "model.safetensors", entries,
                                        {"format": "pt", "checkpoint_id": checkpoint_id})
        except BaseException as exc:  # noqa: BLE001 - propagated through the error bus
            error = exc
    rt.raise_if_process_zero_error(error, "open model.safetensors")
    try:
        for name in names:
            pieces = source.chunks(name)
            if writer is not None:
                writer.write_chunks(name, pieces)
            else:
                for _ in pieces:
                    pass
    except BaseException as exc:  # noqa: BLE001
        error = exc
        if writer is not None:
            writer.abort()
            writer = None
    rt.raise_if_any_process_error(error, "stream model tensors")
    if rt.process_index() == 0:
        try:
            writer.close()
            copy_hf_assets(assets_from, dest, cfg, source.dtype)
        except BaseException as exc:  # noqa: BLE001
            error = exc
    rt.raise_if_process_zero_error(error, "finalize model.safetensors")


# --------------------------------------------------------------------------------------- optimizer state
def export_adapter_checkpoint(destination: str | os.PathLike[str], lora, *, base_model_name_or_path: str,
                              checkpoint_id: str, revision: str | None = None) -> Path:
    """PEFT adapter files of a :class:`~..models.lora.LoraState`: ``adapter_model.safetensors``
    (``lora_A`` = ``A^T``, ``lora_B`` = ``B^T``, plus the trained embedding / LM-head copies when
    present) and ``adapter_config.json`` with ``lora_alpha = r``
    (src/causal_trainer/checkpointing/huggingface.py:1420-1514).  Adapters are replicated, so rank 0
    writes and the other ranks return at once."""
    from ..models.lora import peft_adapter_config

    dest = Path(destination)
    if rt.process_index() == 0:
        dest.mkdir(parents=True, exist_ok=True)
        st.save_file(lora.peft_tensors(), dest / "adapter_model.safetensors",
                     {"format": "pt", "checkpoint_id": checkpoint_id})
        config = peft_adapter_config(base_model_name_or_path, lora.rank,
                                     train_embed_and_lm_head=lora.train_embed_and_lm_head, revision=revision)
        (dest / "adapter_config.json").write_text(json.dumps(config, indent=2, sort_keys=True) + "\n")
    return dest


def layout_fingerprint(entries: list[dict[str, Any]]) -> str:
    """SHA-256 of the compact, key-sorted JSON of the manifest's tensor entries."""
    return hashlib.sha256(json.dumps(entries, separators=(",", ":"), sort_keys=True).encode("utf-8")).hexdigest()


def export_optimizer_stream(destination: str | os.PathLike[str], layout: list[tuple[str, torch.dtype, tuple[int, ...]]],
                            pieces, *, global_step: int, checkpoint_id: str) -> None:
    """Collective.  Writes ``optimizer/state.safetensors`` + ``optimizer/manifest.json`` from a stream.

    ``layout`` names every tensor up front (``path``, dtype, shape; identical on all ranks) so the
    header can be written first.  ``pieces`` yields, in the same order, ``(path, chunks)`` where
    ``chunks`` iterates over consecutive flat pieces of the tensor.  Every rank drains both
    iterators, because producing a piece may be a collective (a shard sent to rank 0); only rank 0
    holds the piece and writes it, one piece at a time, so neither the device nor the host of any
    rank ever holds more than one shard of one tensor
    (src/causal_trainer/checkpointing/huggingface.py:787-988)."""
    out = Path(destination) / "optimizer"
    writer = None
    error: BaseException | None = None
    names = [f"state/{i:06d}" for i in range(len(layout))]
    if rt.process_index() == 0:
        try:
            out.mkdir(parents=True, exist_ok=True)
            writer = st.StreamingWriter(out / "state.safetensors",
                                        [(n, st.DTYPE_NAMES[dt], tuple(shape)) for n, (_, dt, shape) in zip(names, layout)],
                                        {"format": "pt", "checkpoint_id": checkpoint_id})
        except BaseException as exc:  # noqa: BLE001 - reported to every rank below
            error = exc
    for name, (path, _, _), (got, chunks) in zip(names, layout, pieces):
        if got != path:
            raise ValueError(f"optimizer state arrives out of order: expected {path!r}, got {got!r}")
        if writer is not None and error is None:
            try:
                writer.write_chunks(name, chunks)
                continue
            except BaseException as exc:  # noqa: BLE001
                error = exc
        for _ in chunks:               # still take part in the collectives behind the remaining pieces
            pass
    if rt.process_index() == 0 and error is None:
        try:
            writer.close()
            entries = [{"dtype": st.PLAIN_DTYPE_NAMES[st.DTYPE_NAMES[dt]], "file": "state.safetensors", "key": n,
                        "ordinal": i, "path": path, "shape": list(shape)}
                       for i, (n, (path, dt, shape)) in enumerate(zip(names, layout))]
            total = sum(int(torch.tensor([], dtype=dt).element_size()) * int(torch.Size(shape).numel())
                        for _, dt, shape in layout)
            manifest = {
                "format": "optimizer-state-safetensors", "format_version": 1, "global_step": int(global_step),
                "jax_version": f"torch-{torch.__version__}", "optax_version": "causal-trainer-b200-adamw-1",
                "layout_fingerprint": layout_fingerprint(entries), "tensor_count": len(entries), "tensors": entries,
                "total_size": int(total), "checkpoint_id": checkpoint_id,
            }
            tmp = out / "manifest.json.tmp"
            tmp.write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n", encoding="utf-8")
            os.replace(tmp, out / "manifest.json")
        except BaseException as exc:  # noqa: BLE001
            error = exc
    elif writer is not None:
        writer.abort()
    rt.raise_if_process_zero_error(error, "write optimizer state")


def export_optimizer_checkpoint(destination: str | os.PathLike[str], state: list[tuple[str, torch.Tensor]], *,
                                global_step: int, checkpoint_id: str) -> None:
    """Same files from state that is already whole on this process: an ordered list of
    ``(path, tensor)``, ``count`` first, then ``mu/...`` and ``nu/...`` buffers."""
    layout = [(path, t.dtype, tuple(t.shape)) for path, t in state]
    export_optimizer_stream(destination, layout, ((path, iter([t.reshape(-1)])) for path, t in state),
                            global_step=global_step, checkpoint_id=checkpoint_id)


class OptimizerCheckpoint:
    """Validated read access to a saved optimizer state: whole tensors or flat ranges of them (a rank
    of a sharded run pages in only the bytes of its own shards)."""

    def __init__(self, source: str | os.PathLike[str], expected_paths: list[str], *, global_step: int):
        d = Path(source) / "optimizer"
        manifest = json.loads((d / "manifest.json").read_text(encoding="utf-8"))
        if manifest.get("format") != "optimizer-state-safetensors" or manifest.get("format_version") != 1:
            raise ValueError("unsupported optimizer checkpoint format")
        if manifest.get("optax_version") != "causal-trainer-b200-adamw-1":
            raise ValueError("optimizer state was written by a different optimizer implementation")
        if manifest.get("global_step") != global_step:
            raise ValueError(f"optimizer state is for step {manifest.get('global_step')}, expected {global_step}")
        if [e["path"] for e in manifest["tensors"]] != expected_paths:
            raise ValueError("optimizer state layout does not match this run")
        if manifest.get("layout_fingerprint") != layout_fingerprint(manifest["tensors"]):
            raise ValueError("optimizer manifest fingerprint mismatch")
        self.file = st.SafeTensorsFile(d / "state.safetensors")
        if self.file.metadata.get("checkpoint_id") != manifest.get("checkpoint_id"):
            self.file.close()
            raise ValueError("optimizer state belongs to a different checkpoint")
        self.keys = {e["path"]: e["key"] for e in manifest["tensors"]}
        if "count" in self.keys and int(self.file.tensor(self.keys["count"])) != global_step:
            self.file.close()
            raise ValueError("optimizer step counter does not match the checkpoint step")

    def tensor(self, path: str) -> torch.Tensor:
        return self.file.tensor(self.keys[path]).clone()

    def flat_range(self, path: str, start: int, stop: int) -> torch.Tensor:
        return self.file.flat_range(self.keys[path], start, stop).clone()

    def close(self) -> None:
        self.file.close()

    def __enter__(self) -> "OptimizerCheckpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def load_optimizer_checkpoint(source: str | os.PathLike[str], expected_paths: list[str], *, global_step: int
                              ) -> dict[str, torch.Tensor]:
    """Reads a whole optimizer state back; refuses a foreign framework version, layout or step."""
    with OptimizerCheckpoint(source, expected_paths, global_step=global_step) as ckpt:
        return {path: ckpt.tensor(path) for path in expected_paths}


def remove_optimizer_checkpoint(destination: str | os.PathLike[str]) -> None:
    d = Path(destination) / "optimizer"
    if d.is_dir() and rt.process_index() == 0:
        shutil.rmtree(d)


def new_checkpoint_id() -> str:
    """uuid4 hex chosen on rank 0 and broadcast (paths may differ per host, the id may not)."""
    value = uuid.uuid4().hex if rt.process_index() == 0 else None
    raw = rt.host_broadcast_bytes(value.encode() if value else None, 32)
    return raw.decode("ascii")


parameter_hf_layout = expected_model_layout   # name of src/causal_trainer/checkpointing/huggingface.py:149
