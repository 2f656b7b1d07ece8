"""The layerwise sm_100a engine against autograd through the PyTorch oracle decoder."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def _batch(cfg, b, s, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(3, cfg.vocab_size, (b, s), generator=g)
    mask = torch.ones(b, s, dtype=torch.int32)
    seg = torch.ones(b, s, dtype=torch.int32)
    seg[:, s // 3:] = 2
    seg[0, (2 * s) // 3:] = 3
    mask[1, :17] = 0
    seg[1, :17] = 0
    ids[1, :17] = cfg.pad_token_id
    return {k: v.cuda() for k, v in dict(input_ids=ids, attention_mask=mask, segment_ids=seg).items()}


@pytest.mark.parametrize("bias", [False, True])
def test_engine_matches_oracle_gradients(cuda_lib, bias):
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.decoder import ForwardOptions
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import LayerwiseEngine, LocalProvider
    from causal_trainer_dev_b200.training.steps import AutogradProducer

    cfg = preset("tiny", vocab_size=4096, attention_bias=bias)
    base = ModelParams.init_random(cfg, seed=1, dtype=torch.bfloat16)
    if bias:
        for i in range(cfg.num_hidden_layers):
            base.layer(i).view("qkv_b").normal_(0, 0.02)
    batch = _batch(cfg, 2, 256)
    # oracle in fp32 on the same bf16-rounded weights
    ref = ModelParams(cfg, dtype=torch.float32, device="cuda")
    ref.load_state_dict({k: v.float() for k, v in base.state_dict().items()})
    nll_ref, w_ref = AutogradProducer(ref, ForwardOptions(attn_mechanism="vanilla"))(batch, 1.0 / 400, True)
    eng_params = ModelParams(cfg, dtype=torch.bfloat16, device="cuda")
    eng_params.load_state_dict(base.state_dict())
    engine = LayerwiseEngine(cfg, LocalProvider(eng_params, torch.float32))
    nll, wsum = engine(batch, 1.0 / 400, True)
    assert abs(nll.item() - nll_ref.item()) / nll_ref.item() < 5e-3
    assert abs(wsum.item() - w_ref.item()) < 1e-3
    for name in eng_params.hf_names():
        g, r = eng_params.grad_tensor(name), ref.grad_tensor(name)
        assert _rel(g, r) < 0.06, name
    # accumulation: a second micro-batch with first=False doubles the gradient
    engine(batch, 1.0 / 400, False)
    for name in ("model.layers.0.self_attn.q_proj.weight", "model.layers.1.mlp.down_proj.weight",
                 "lm_head.weight", "model.norm.weight", "model.embed_tokens.weight"):
        assert _rel(eng_params.grad_tensor(name), 2 * ref.grad_tensor(name)) < 0.06, name
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_engine_training_reduces_loss(cuda_lib):
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import LayerwiseEngine, LocalProvider
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig
    from causal_trainer_dev_b200.training.steps import TrainStep

    cfg = preset("tiny", vocab_size=4096)
    params = ModelParams.init_random(cfg, seed=0, dtype=torch.bfloat16).to("cuda")
    engine = LayerwiseEngine(cfg, LocalProvider(params, torch.bfloat16))
    step = TrainStep(params, engine, AdamWConfig(weight_decay=0.1), ScheduleConfig(1e-3, 0.0, "constant", 0, 10))
    batch = _batch(cfg, 2, 256)
    first = step.run([batch]).to_floats()
    for _ in range(6):
        last = step.run([batch]).to_floats()
    assert abs(first["loss"] - 8.3178) < 0.1  # ln(4096)
    assert last["loss"] < first["loss"] - 1.0
    assert engine.launches > 0
    # one AdamW launch per unit; the per-tensor moments are views into the units' flat moment buffers
    arenas = step.optimizer.arenas
    assert len(arenas) == len(params.units)
    assert all(m.data_ptr() >= a["m"].data_ptr() for a in arenas for m in (step.optimizer.m[i] for i in a["regions"]))
    assert float(sum(a["m"].float().abs().sum() for a in arenas)) > 0


def test_unit_wide_adamw_matches_the_per_tensor_update(cuda_lib):
    """The same three steps with one AdamW launch per unit and with one per tensor."""
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import LayerwiseEngine, LocalProvider
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig
    from causal_trainer_dev_b200.training.steps import TrainStep

    cfg = preset("tiny", vocab_size=4096)
    batch = _batch(cfg, 2, 256)
    results = []
    for whole_units in (True, False):
        params = ModelParams.init_random(cfg, seed=0, dtype=torch.bfloat16).to("cuda")
        engine = LayerwiseEngine(cfg, LocalProvider(params, torch.bfloat16))
        step = TrainStep(params, engine, AdamWConfig(weight_decay=0.1), ScheduleConfig(1e-3, 0.0, "constant", 0, 10),
                         frozen=("norm",))
        if not whole_units:
            step.optimizer.arenas = None
        history = [step.run([batch]).to_floats() for _ in range(3)]
        results.append((history, params))
    (ha, pa), (hb, pb) = results
    for x, y in zip(ha, hb):
        assert abs(x["loss"] - y["loss"]) < 2e-3 and abs(x["grad_norm"] - y["grad_norm"]) < 2e-3 * y["grad_norm"]
    for name in pa.hf_names():
        assert _rel(pa.tensor(name), pb.tensor(name)) < 2e-3, name


def test_engine_with_moba_layers_matches_oracle(cuda_lib):
    """MoBA layers in the engine (native routing + block-sparse kernels) against autograd through the
    oracle decoder with the reference MoBA operator; routing near-ties may differ, so the bound is loose."""
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.decoder import ForwardOptions
    from causal_trainer_dev_b200.models.moba import AttentionOptions
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import EngineOptions, LayerwiseEngine, LocalProvider
    from causal_trainer_dev_b200.training.steps import AutogradProducer

    cfg = preset("tiny", vocab_size=4096)
    ao = AttentionOptions(method="moba", moba_block_size=128, moba_top_k=2, dense_prefix_layers=1)
    base = ModelParams.init_random(cfg, seed=2, dtype=torch.bfloat16)
    batch = _batch(cfg, 2, 1024)
    ref = ModelParams(cfg, dtype=torch.float32, device="cuda")
    ref.load_state_dict({k: v.float() for k, v in base.state_dict().items()})
    opts = ForwardOptions(attn_mechanism="vanilla", attention_options=AttentionOptions(
        method="moba", backend="reference", moba_block_size=128, moba_top_k=2, dense_prefix_layers=1))
    nll_ref, _ = AutogradProducer(ref, opts)(batch, 1.0 / 1500, True)
    eng_params = ModelParams(cfg, dtype=torch.bfloat16, device="cuda")
    eng_params.load_state_dict(base.state_dict())
    engine = LayerwiseEngine(cfg, LocalProvider(eng_params, torch.float32), EngineOptions(attention_options=ao))
    nll, _ = engine(batch, 1.0 / 1500, True)
    assert engine._uses_moba(1, 1024) and not engine._uses_moba(0, 1024)
    assert abs(nll.item() - nll_ref.item()) / nll_ref.item() < 5e-3
    for name in ("model.layers.1.self_attn.q_proj.weight", "model.layers.1.self_attn.v_proj.weight",
                 "model.layers.0.mlp.down_proj.weight", "lm_head.weight"):
        assert _rel(eng_params.grad_tensor(name), ref.grad_tensor(name)) < 0.1, name
    assert cuda_lib.device_status() == (0, 0, 0, 0)


@pytest.mark.parametrize("backend", ["cut", "logits"])
def test_engine_sparse_supervision_compacts_rows(cuda_lib, backend):
    """Assistant-only style loss weights: the LM head runs on the supervised rows only (row
    compaction) and both loss backends agree with the oracle."""
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.decoder import ForwardOptions
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import EngineOptions, LayerwiseEngine, LocalProvider
    from causal_trainer_dev_b200.training.steps import AutogradProducer

    cfg = preset("tiny", vocab_size=4096)
    base = ModelParams.init_random(cfg, seed=4, dtype=torch.bfloat16)
    batch = _batch(cfg, 2, 256)
    g = torch.Generator().manual_seed(9)
    batch["loss_weights"] = (torch.rand(2, 256, generator=g) < 0.3).float().cuda()
    ref = ModelParams(cfg, dtype=torch.float32, device="cuda")
    ref.load_state_dict({k: v.float() for k, v in base.state_dict().items()})
    nll_ref, w_ref = AutogradProducer(ref, ForwardOptions(attn_mechanism="vanilla"))(batch, 1.0 / 150, True)
    eng_params = ModelParams(cfg, dtype=torch.bfloat16, device="cuda")
    eng_params.load_state_dict(base.state_dict())
    engine = LayerwiseEngine(cfg, LocalProvider(eng_params, torch.float32), EngineOptions(loss_backend=backend))
    nll, wsum = engine(batch, 1.0 / 150, True)
    assert abs(wsum.item() - w_ref.item()) < 1e-3 and w_ref.item() < 0.5 * 512
    assert abs(nll.item() - nll_ref.item()) / nll_ref.item() < 5e-3
    for name in ("lm_head.weight", "model.norm.weight", "model.layers.1.mlp.down_proj.weight",
                 "model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight"):
        assert _rel(eng_params.grad_tensor(name), ref.grad_tensor(name)) < 0.06, name


def test_lora_engine_matches_oracle_adapter_gradients(cuda_lib):
    """Frozen base on the tcgen05 GEMMs + rank-r adapter paths against autograd through the oracle decoder."""
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.decoder import ForwardOptions
    from causal_trainer_dev_b200.models.lora import LoraState
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import LocalProvider
    from causal_trainer_dev_b200.training.lora_engine import LoraLayerwiseEngine
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig
    from causal_trainer_dev_b200.training.steps import AutogradProducer, TrainStep

    cfg = preset("tiny", vocab_size=4096)
    base = ModelParams.init_random(cfg, seed=1, dtype=torch.bfloat16)
    batch = _batch(cfg, 2, 256)
    lora = LoraState.init(cfg, 16, seed=4, dtype=torch.bfloat16, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(9)
    with torch.no_grad():
        for key, b in lora.b.items():                # a trained adapter: B is no longer zero
            b.copy_(torch.randn(b.shape, generator=gen, device="cuda") * 0.02)
    # oracle: fp32 autograd on the same bf16-rounded base weights and adapters
    ref = ModelParams(cfg, dtype=torch.float32, device="cuda")
    ref.load_state_dict({k: v.float() for k, v in base.state_dict().items()})
    ref_lora = LoraState(cfg, 16)
    for key in lora.a:
        ref_lora.a[key] = lora.a[key].detach().float().requires_grad_()
        ref_lora.b[key] = lora.b[key].detach().float().requires_grad_()
    nll_ref, _ = AutogradProducer(ref, ForwardOptions(attn_mechanism="vanilla", lora=ref_lora), lora=ref_lora)(
        batch, 1.0 / 400, True)
    params = ModelParams(cfg, dtype=torch.bfloat16, device="cuda")
    params.load_state_dict(base.state_dict())
    engine = LoraLayerwiseEngine(cfg, LocalProvider(params, torch.bfloat16), lora)
    nll, _ = engine(batch, 1.0 / 400, True)
    assert abs(nll.item() - nll_ref.item()) / nll_ref.item() < 5e-3
    for key in lora.a:
        ga, gb = engine.grads[key]
        assert _rel(ga, ref_lora.a[key].grad) < 0.08, key
        assert _rel(gb, ref_lora.b[key].grad) < 0.08, key
    assert all(u.grad is None for u in params.units.values())          # no gradient memory for the frozen base
    engine(batch, 1.0 / 400, False)                                     # accumulation over micro-batches
    key = (1, "gate_proj")
    assert _rel(engine.grads[key][0], 2 * ref_lora.a[key].grad) < 0.08
    # adapters train, the base stays bit-identical
    before = {k: v.clone() for k, v in params.state_dict().items()}
    step = TrainStep(params, engine, AdamWConfig(weight_decay=0.0), ScheduleConfig(2e-3, 0.0, "constant", 0, 10),
                     extra_regions=engine.extra_regions(), train_base=False)
    first = step.run([batch]).to_floats()
    for _ in range(6):
        last = step.run([batch]).to_floats()
    assert last["loss"] < first["loss"] - 0.05
    assert all(torch.equal(v, before[k]) for k, v in params.state_dict().items())
    assert cuda_lib.device_status() == (0, 0, 0, 0)


@pytest.mark.parametrize("remat,group,chunk", [("full", 2, 0), ("full", 3, 0), ("full", 3, 128), ("none", 1, 128),
                                               ("none", 1, 0)])
def test_memory_options_do_not_change_the_gradients(cuda_lib, remat, group, chunk):
    """Recompute in groups of layers, tile the MLP, keep everything: the same gradients as
    recomputing layer by layer.  Grouping only changes when a layer's input is rebuilt, so it is
    bit-exact; the tiled MLP sums its weight gradients tile by tile and kept activations are
    re-normalised from their rounded copies, so those agree to rounding."""
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.training.engine import EngineOptions, LayerwiseEngine, LocalProvider

    cfg = preset("tiny", vocab_size=4096, num_hidden_layers=5)
    base = ModelParams.init_random(cfg, seed=2, dtype=torch.bfloat16)
    batch = _batch(cfg, 2, 256)

    def run(options):
        params = ModelParams(cfg, dtype=torch.bfloat16, device="cuda")
        params.load_state_dict(base.state_dict())
        engine = LayerwiseEngine(cfg, LocalProvider(params, torch.float32), options)
        nll, _ = engine(batch, 1.0 / 400, True)
        return nll, params, engine

    nll_0, p_0, _ = run(EngineOptions(remat="full"))
    nll_1, p_1, engine = run(EngineOptions(remat=remat, remat_group_size=group, mlp_chunk_rows=chunk))
    assert engine.kept_layers == (0 if remat == "full" else cfg.num_hidden_layers)
    exact = remat == "full" and chunk == 0
    assert torch.equal(nll_0, nll_1) if exact else abs(nll_0.item() - nll_1.item()) < 1e-3 * abs(nll_0.item())
    for name in p_0.hf_names():
        a, b = p_0.grad_tensor(name), p_1.grad_tensor(name)
        if exact:
            assert torch.equal(a, b), name
        else:
            assert _rel(b, a) < 2e-2, name
