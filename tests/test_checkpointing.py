import json
import struct

import pytest
import torch

from causal_trainer_dev_b200.checkpointing import bundles, huggingface as hfio, safetensors_io as st
from causal_trainer_dev_b200.models.config import preset
from causal_trainer_dev_b200.models.params import ModelParams, hf_export_order


def test_roundtrip_is_bit_exact_and_interoperates_with_the_safetensors_package(tmp_path):
    torch.manual_seed(0)
    tensors = {"b": torch.randn(3, 5).bfloat16(), "a": torch.randn(7), "i": torch.arange(6).view(2, 3),
               "s": torch.tensor(3.5)}
    st.save_file(tensors, tmp_path / "x.safetensors", {"format": "pt"})
    back = st.load_file(tmp_path / "x.safetensors")
    assert list(back) == list(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and torch.equal(back[k], tensors[k])
    raw = (tmp_path / "x.safetensors").read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert hlen % 8 == 0 and raw[8:8 + hlen].rstrip(b" ").endswith(b"}")
    from safetensors.torch import load_file, save_file

    theirs = load_file(str(tmp_path / "x.safetensors"))
    assert all(torch.equal(theirs[k], tensors[k]) for k in tensors)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "y.safetensors"))
    ours = st.load_file(tmp_path / "y.safetensors")
    assert all(torch.equal(ours[k], tensors[k]) for k in tensors)


def test_reader_slices_and_validation(tmp_path):
    t = torch.arange(40, dtype=torch.float32).view(10, 4)
    st.save_file({"w": t}, tmp_path / "w.safetensors")
    with st.SafeTensorsFile(tmp_path / "w.safetensors") as f:
        assert torch.equal(f.rows("w", 3, 6), t[3:6]) and torch.equal(f.flat_range("w", 5, 9), t.reshape(-1)[5:9])
    raw = bytearray((tmp_path / "w.safetensors").read_bytes())
    (tmp_path / "trunc.safetensors").write_bytes(raw[:-4])
    with pytest.raises(ValueError, match="payload size"):
        st.read_header(tmp_path / "trunc.safetensors")
    w = st.StreamingWriter(tmp_path / "o.safetensors", [("a", "F32", (2,)), ("b", "F32", (2,))])
    with pytest.raises(ValueError, match="header order"):
        w.write("b", torch.zeros(2))
    w.abort()
    assert not (tmp_path / "o.safetensors").exists() and not (tmp_path / "o.safetensors.tmp").exists()


def _export(tmp_path, name="out", step=3, total=10, signature="sig", seed=0, optimizer=False, **kw):
    cfg = preset("tiny", vocab_size=128, num_hidden_layers=1, hidden_size=64, intermediate_size=128,
                 num_attention_heads=1, num_key_value_heads=1)
    params = ModelParams.init_random(cfg, seed=seed, dtype=torch.bfloat16)
    dest = tmp_path / name

    from helpers import write_tokenizer

    assets = write_tokenizer(tmp_path / "assets")

    def export_model(d, cid):
        hfio.export_hf_checkpoint(d, hfio.TensorSource(cfg, params=params), checkpoint_id=cid, assets_from=assets)

    export_opt = None
    if optimizer:
        state = [("count", torch.tensor(step)), ("mu/0", torch.zeros(4).bfloat16()), ("nu/0", torch.ones(4).bfloat16())]

        def export_opt(d, cid):
            hfio.export_optimizer_checkpoint(d, state, global_step=step, checkpoint_id=cid)
    bundles.save_checkpoint_bundle(dest, export_model=export_model, export_optimizer=export_opt, global_step=step,
                                   total_steps=total, signature=signature, **kw)
    return cfg, params, dest


def test_export_order_metadata_and_reload_bit_exact(tmp_path):
    cfg, params, dest = _export(tmp_path)
    tensors, meta, _ = st.read_header(dest / "model.safetensors")
    assert list(tensors) == hf_export_order(cfg) and meta["format"] == "pt" and len(meta["checkpoint_id"]) == 32
    assert list(tensors)[:2] == ["model.embed_tokens.weight", "model.layers.0.self_attn.k_proj.weight"]
    assert list(tensors)[-2:] == ["lm_head.weight", "model.norm.weight"]
    again = ModelParams(cfg, torch.bfloat16)
    hfio.load_parameters(dest, again)
    for name in params.hf_names():
        assert torch.equal(again.tensor(name), params.tensor(name))
    assert json.loads((dest / "config.json").read_text())["torch_dtype"] == "bfloat16"


def test_discovery_prefers_highest_step_and_root_at_equal_step(tmp_path):
    out = tmp_path / "run"
    _export(out, "checkpoint-3", step=3)
    _export(out, "checkpoint-6", step=6)
    found = bundles.find_latest_checkpoint(out, "sig")
    assert found.global_step == 6 and found.path.name == "checkpoint-6"
    _export(tmp_path, "run", step=6)
    assert bundles.find_latest_checkpoint(out, "sig").path == out
    assert bundles.find_latest_checkpoint(tmp_path / "nothing", "sig") is None


def test_incompatible_and_corrupt_bundles_are_hard_errors(tmp_path):
    out = tmp_path / "run"
    _, _, d = _export(out, "checkpoint-3", step=3)
    with pytest.raises(ValueError, match="incompatible"):
        bundles.find_latest_checkpoint(out, "other-signature")
    blob = bytearray((d / "model.safetensors").read_bytes())
    blob[-1] ^= 0xFF                                     # same size, different payload
    (d / "model.safetensors").write_bytes(blob)
    with pytest.raises(ValueError, match="corrupt"):
        bundles.find_latest_checkpoint(out, "sig")
    assert bundles.find_latest_checkpoint(out, "sig", verify_artifact_digests=False) is not None


def test_model_file_from_another_bundle_is_caught_by_checkpoint_id(tmp_path):
    out = tmp_path / "run"
    _, _, a = _export(out, "checkpoint-3", step=3)
    _, _, b = _export(tmp_path, "other", step=3)
    m = json.loads((a / bundles.MANIFEST_NAME).read_text())
    (a / "model.safetensors").write_bytes((b / "model.safetensors").read_bytes())
    m["artifact_digests"]["model.safetensors"] = bundles.file_sha256(a / "model.safetensors")
    (a / bundles.MANIFEST_NAME).write_text(json.dumps(m))
    with pytest.raises(ValueError, match="corrupt"):
        bundles.find_latest_checkpoint(out, "sig")


def test_resume_action_table(tmp_path):
    out = tmp_path / "run"
    mk = lambda **k: bundles.ResumeCheckpoint(**{**dict(path=out / "checkpoint-5", global_step=5, total_steps=10,
                                                        has_optimizer_state=True, checkpoint_id="0" * 32,
                                                        manifest_digest="d"), **k})
    ra = lambda c: bundles.resume_action(c, output_dir=out, total_steps=10)
    assert ra(None) == "start" and ra(mk()) == "continue"
    assert ra(mk(global_step=10, path=out / "checkpoint-10")) == "finalize" and ra(mk(global_step=10, path=out)) == "complete"
    with pytest.raises(ValueError, match="optimizer state"):
        ra(mk(has_optimizer_state=False))
    with pytest.raises(ValueError, match="total_steps"):
        ra(mk(total_steps=11))
    assert ra(mk(training_complete=True, path=out, global_step=10, streaming_data_digest="0" * 64)) == "complete"


def test_optimizer_state_roundtrip_and_pruning(tmp_path):
    out = tmp_path / "run"
    _, _, d = _export(out, "checkpoint-3", step=3, optimizer=True)
    found = bundles.find_latest_checkpoint(out, "sig")
    assert found.has_optimizer_state
    state = hfio.load_optimizer_checkpoint(d, ["count", "mu/0", "nu/0"], global_step=3)
    assert int(state["count"]) == 3 and state["nu/0"].dtype == torch.bfloat16
    with pytest.raises(ValueError, match="layout"):
        hfio.load_optimizer_checkpoint(d, ["count", "mu/1", "nu/1"], global_step=3)
    _export(out, "checkpoint-6", step=6)
    _export(out, "checkpoint-9", step=9)
    removed = bundles.prune_periodic_exports(out, 2, "sig")
    assert [p.name for p in removed] == ["checkpoint-3"] and (out / "checkpoint-9").is_dir()


def _refresh_inventory(path, optimizer):
    mpath = path / bundles.MANIFEST_NAME
    m = json.loads(mpath.read_text(encoding="utf-8"))
    files = bundles.artifact_files(path, m["artifact_kind"], optimizer)
    m["artifact_sizes"] = {str(f.relative_to(path)): f.stat().st_size for f in files}
    m["artifact_digests"] = {str(f.relative_to(path)): bundles.file_sha256(f) for f in files}
    mpath.write_text(json.dumps(m), encoding="utf-8")


def test_optimizer_manifest_conventions_and_tampering(tmp_path):
    """The optimizer manifest spells dtypes the numpy way and carries a fingerprint of its entries; a
    manifest whose fingerprint does not match, or a model header with a malformed dtype, makes the
    bundle corrupt rather than silently usable (also when the artifact inventory was refreshed)."""
    out = tmp_path / "run"
    _, _, d = _export(out, "checkpoint-4", step=4, optimizer=True)
    mpath = d / "optimizer" / "manifest.json"
    manifest = json.loads(mpath.read_text(encoding="utf-8"))
    assert [e["dtype"] for e in manifest["tensors"]] == ["int64", "bfloat16", "bfloat16"]
    assert manifest["layout_fingerprint"] == hfio.layout_fingerprint(manifest["tensors"])
    assert bundles.find_latest_checkpoint(out, "sig").global_step == 4
    manifest["layout_fingerprint"] = "0" * 64
    mpath.write_text(json.dumps(manifest), encoding="utf-8")
    _refresh_inventory(d, True)
    with pytest.raises(ValueError, match="corrupt completed checkpoints"):
        bundles.find_latest_checkpoint(out, "sig")
    # a header whose dtype is not even a string
    out2 = tmp_path / "run2"
    _, _, d2 = _export(out2, "checkpoint-4", step=4)
    model = d2 / "model.safetensors"
    payload = model.read_bytes()
    hlen = int.from_bytes(payload[:8], "little")
    header = json.loads(payload[8:8 + hlen].decode("utf-8").rstrip(" "))
    header["model.norm.weight"]["dtype"] = []
    enc = json.dumps(header, separators=(",", ":")).encode("utf-8")
    assert len(enc) <= hlen
    model.write_bytes(payload[:8] + enc + b" " * (hlen - len(enc)) + payload[8 + hlen:])
    _refresh_inventory(d2, False)
    with pytest.raises(ValueError, match="corrupt completed checkpoints"):
        bundles.find_latest_checkpoint(out2, "sig")


def test_export_normalises_a_v5_config_and_copies_named_chat_templates(tmp_path):
    """Reading accepts the Transformers 5 spellings; a merged checkpoint returns to the fixed source format."""
    import json

    import torch

    from causal_trainer_dev_b200.checkpointing import huggingface as hfio
    from causal_trainer_dev_b200.models.config import ModelConfig, preset

    source, destination = tmp_path / "source", tmp_path / "destination"
    (source / "chat_templates").mkdir(parents=True)
    (source / "tokenizer.json").write_text("{}", encoding="utf-8")
    (source / "chat_templates" / "tool_use.jinja").write_text("tool template", encoding="utf-8")
    raw = {**preset("tiny").to_dict(), "custom_note": "kept"}
    for key in ("torch_dtype", "rope_theta", "partial_rotary_factor", "rope_scaling"):
        raw.pop(key)
    raw["dtype"] = "float32"
    raw["rope_parameters"] = {"rope_type": "default", "rope_theta": 1_000_000.0, "partial_rotary_factor": 0.5}
    (source / "config.json").write_text(json.dumps(raw), encoding="utf-8")
    cfg = ModelConfig.from_dict(raw)
    assert cfg.rope_theta == 1_000_000.0 and cfg.partial_rotary_factor == 0.5 and cfg.torch_dtype == "float32"
    hfio.copy_hf_assets(source, destination, cfg, torch.bfloat16)
    written = json.loads((destination / "config.json").read_text(encoding="utf-8"))
    assert "dtype" not in written and "rope_parameters" not in written
    assert written["torch_dtype"] == "bfloat16"                      # the dtype of the tensors actually written
    assert written["rope_scaling"] is None and written["rope_theta"] == 1_000_000.0
    assert written["partial_rotary_factor"] == 0.5 and written["custom_note"] == "kept"
    assert (destination / "tokenizer.json").is_file()
    assert (destination / "chat_templates" / "tool_use.jinja").read_text(encoding="utf-8") == "tool template"


def test_model_load_rejects_tensors_outside_the_architecture(tmp_path):
    import torch

    from causal_trainer_dev_b200.checkpointing import huggingface as hfio
    from causal_trainer_dev_b200.checkpointing import safetensors_io as st
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.params import ModelParams

    cfg = preset("tiny", num_hidden_layers=1)
    params = ModelParams.init_random(cfg, seed=0, dtype=torch.float32)
    tensors = {name: params.tensor(name).clone() for name in params.hf_names()}
    tensors["model.layers.0.self_attn.o_proj.bias"] = torch.zeros(cfg.hidden_size)
    st.save_file(tensors, tmp_path / "model.safetensors")
    with pytest.raises(ValueError, match="do not exactly match.*unexpected.*o_proj.bias"):
        hfio.load_parameters(tmp_path, ModelParams(cfg, torch.float32, "cpu"))
    del tensors["model.layers.0.self_attn.o_proj.bias"], tensors["model.norm.weight"]
    st.save_file(tensors, tmp_path / "model.safetensors")
    with pytest.raises(ValueError, match="do not exactly match.*missing.*model.norm.weight"):
        hfio.load_parameters(tmp_path, ModelParams(cfg, torch.float32, "cpu"))


def test_rope_pairing_default_follows_the_model_family():
    from causal_trainer_dev_b200.models.config import ModelConfig, preset

    raw = preset("tiny").to_dict()
    del raw["rope_style"]
    assert ModelConfig.from_dict({**raw, "model_type": "llama"}).rope_style == "gpt-neox"
    assert ModelConfig.from_dict({**raw, "model_type": "opaque-metadata"}).rope_style == "gpt-j"
    assert ModelConfig.from_dict({**raw, "model_type": "opaque-metadata", "rope_style": "gpt-neox"}).rope_style == "gpt-neox"
    with pytest.raises(ValueError, match="rope_style"):
        ModelConfig.from_dict({**raw, "rope_style": "llama"})


def test_adapter_bundle_is_discoverable_and_reloads_bit_exact(tmp_path):
    from causal_trainer_dev_b200.models.lora import LoraState

    cfg = preset("tiny")
    lora = LoraState.init(cfg, 4, seed=1, dtype=torch.float32)
    for b in lora.b.values():
        torch.nn.init.normal_(b.data)
    sig = bundles.training_signature({"run": "adapter"})
    dest = tmp_path / "out" / "checkpoint-3"
    cid = bundles.save_adapter_checkpoint_bundle(lora, dest, base_model_name_or_path="org/base", global_step=3,
                                                 total_steps=10, signature=sig, revision="abc")
    config = json.loads((dest / "adapter_config.json").read_text())
    assert config["r"] == config["lora_alpha"] == 4 and config["base_model_name_or_path"] == "org/base"
    assert config["revision"] == "abc" and config["modules_to_save"] is None
    found = bundles.find_latest_checkpoint(tmp_path / "out", sig, expected_artifact_kind="peft-adapter")
    assert found is not None and found.global_step == 3 and found.checkpoint_id == cid
    assert not found.has_optimizer_state
    again = LoraState.init(cfg, 4, seed=2, dtype=torch.float32)
    again.load_peft_tensors(st.load_file(dest / "adapter_model.safetensors"))
    for key in lora.a:
        assert torch.equal(again.a[key], lora.a[key]) and torch.equal(again.b[key], lora.b[key])


def test_tree_paths_map_onto_every_exported_tensor():
    cfg = preset("tiny", attention_bias=True)
    keys = set()
    for i in range(cfg.num_hidden_layers):
        for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
            keys.add(hfio.parameter_to_hf_mapping(f"layers/{i}/attention/{proj}/kernel"))
        for proj in ("q_proj", "k_proj", "v_proj"):
            keys.add(hfio.parameter_to_hf_mapping(f"model/layers/{i}/attention/{proj}/bias"))
        for proj in ("gate_proj", "up_proj", "down_proj"):
            keys.add(hfio.parameter_to_hf_mapping(f"layers/{i}/mlp/{proj}/kernel"))
        for norm in ("input_layernorm", "post_attention_layernorm"):
            keys.add(hfio.parameter_to_hf_mapping(f"layers/{i}/{norm}/scale"))
    for top in ("embed_tokens/embedding", "norm/scale", "lm_head/kernel"):
        keys.add(hfio.parameter_to_hf_mapping(top))
    assert {m.hf_key for m in keys} == set(hf_export_order(cfg))
    assert all(m.transpose == (m.parameter_path.endswith("kernel")) for m in keys)
    assert set(hfio.parameter_hf_layout(cfg, torch.bfloat16)) == set(hf_export_order(cfg))
    for bad in ("layers/0/mlp/q_proj/kernel", "layers/0/mlp/up_proj/bias", "layers/x/mlp/up_proj/kernel", "router/kernel"):
        with pytest.raises(KeyError):
            hfio.parameter_to_hf_mapping(bad)
    assert hfio.SafeTensorIndex is st.SafeTensorIndex and hfio.TensorInfo is st.TensorInfo


def test_stray_files_do_not_invalidate_a_bundle_but_stale_weights_do(tmp_path):
    _, _, dest = _export(tmp_path, name="out", step=10, total=10)
    (dest / "train.log").write_text("noise")
    (dest / "profile_steps.json").write_text("{}")
    (dest / ".cache").mkdir()
    (dest / ".cache" / "blob").write_text("x")
    found = bundles.find_latest_checkpoint(dest, "sig")
    assert found is not None and found.global_step == 10
    manifest = json.loads((dest / bundles.MANIFEST_NAME).read_text())
    assert "train.log" not in manifest["artifact_sizes"] and "model.safetensors" in manifest["artifact_sizes"]
    assert "tokenizer.json" in manifest["artifact_sizes"] and "training_args.json" not in manifest["artifact_sizes"]
    # adapter weights beside merged weights: the bundle cannot be trusted
    (dest / "adapter_model.safetensors").write_bytes(b"\0" * 16)
    with pytest.raises(ValueError, match="corrupt"):
        bundles.find_latest_checkpoint(dest, "sig")
    (dest / "adapter_model.safetensors").unlink()
    # an optimizer directory the manifest does not announce
    (dest / "optimizer").mkdir()
    with pytest.raises(ValueError, match="corrupt"):
        bundles.find_latest_checkpoint(dest, "sig")
    with pytest.raises(RuntimeError, match="stale optimizer"):
        bundles.artifact_files(dest, "merged", False)
