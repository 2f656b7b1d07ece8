import math

import pytest
import torch

from causal_trainer_dev_b200.models import decoder as D
from causal_trainer_dev_b200.models.config import ModelConfig, preset, validate_splash_block_size
from causal_trainer_dev_b200.models.decoder import ForwardOptions
from causal_trainer_dev_b200.models.params import ModelParams
from causal_trainer_dev_b200.ops import attention as A
from causal_trainer_dev_b200.ops import elementwise as E
from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig, learning_rate_at
from causal_trainer_dev_b200.training.steps import AutogradProducer, TrainStep


def test_config_reads_v4_and_v5_spellings():
    base = dict(vocab_size=100, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                num_key_value_heads=1)
    c = ModelConfig.from_dict({**base, "dtype": "float32", "rope_parameters": {"rope_type": "default", "rope_theta": 5e5}})
    assert c.torch_dtype == "float32" and c.rope_theta == 5e5 and c.head_dim == 64 and c.rope_style == "gpt-neox"
    assert ModelConfig.from_dict({**base, "model_type": "qwen2"}).attention_bias is True
    with pytest.raises(ValueError, match="unscaled"):
        ModelConfig.from_dict({**base, "rope_scaling": {"rope_type": "yarn"}})
    with pytest.raises(ValueError):
        ModelConfig(**{**base, "head_dim": 64, "num_key_value_heads": 3})
    assert validate_splash_block_size(4096, 512, "q") == 512
    with pytest.raises(ValueError):
        validate_splash_block_size(4096, 100, "q")


def test_segment_canonicalisation_and_positions():
    mask = torch.tensor([[0, 1, 1, 1, 1, 1, 0, 1]])
    seg = torch.tensor([[5, 0, 0, 7, 7, 0, 0, 0]])
    assert D.canonicalize_segment_ids(mask, seg).tolist() == [[0, 1, 1, 2, 2, 3, 0, 4]]
    assert D.make_position_ids(mask, seg).tolist() == [[0, 0, 1, 0, 1, 0, 0, 0]]


@pytest.mark.parametrize("style", ["gpt-j", "gpt-neox"])
def test_rope_is_a_rotation_and_partial(style):
    torch.manual_seed(0)
    x = torch.randn(5, 2, 8)
    inv = E.inverse_frequencies(4, 10000.0)
    cos, sin = E.rope_table_reference(torch.arange(5), inv, torch.float32)
    y = E.rope_reference(x, cos, sin, 4, style)
    assert torch.equal(y[..., 4:], x[..., 4:]) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.allclose(E.rope_reference(y, cos, sin, 4, style, inverse=True), x, atol=1e-5)
    assert torch.allclose(y[0], x[0])   # position 0 is the identity


def test_vanilla_attention_masks_and_zero_rows():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 6, 2, 4), torch.randn(1, 6, 1, 4), torch.randn(1, 6, 1, 4)
    seg = torch.tensor([[0, 1, 1, 2, 2, 2]])
    out = A.vanilla_attention(q, k, v, seg)
    assert torch.all(out[0, 0] == 0) and torch.allclose(out[0, 1], v[0, 1].expand(2, 4), atol=1e-6)
    assert torch.allclose(out[0, 3], v[0, 3].expand(2, 4), atol=1e-6)  # first token of document 2 sees only itself
    end = torch.tensor([[0, 1, 2, 5, 5, 5]])                           # document 2 bidirectional
    both = A.vanilla_attention(q, k, v, seg, end)
    assert not torch.allclose(both[0, 3], out[0, 3]) and torch.allclose(both[0, 1:3], out[0, 1:3])


def test_perturbing_one_document_does_not_change_another_bit_for_bit():
    cfg = preset("tiny", vocab_size=200)
    p = ModelParams.init_random(cfg, 0, torch.float32)
    ids = torch.randint(3, 200, (1, 24))
    seg = torch.tensor([[1] * 10 + [2] * 14])
    mask = torch.ones(1, 24, dtype=torch.long)
    a = D.decoder_forward(p, ids, mask, seg)
    ids2 = ids.clone()
    ids2[0, :10] = torch.randint(3, 200, (10,))
    b = D.decoder_forward(p, ids2, mask, seg)
    assert torch.equal(a[0, 10:], b[0, 10:]) and not torch.equal(a[0, :10], b[0, :10])


def test_checkpointed_and_tiled_mlp_match_plain_forward():
    cfg = preset("tiny", vocab_size=200)
    p = ModelParams.init_random(cfg, 0, torch.float32).requires_grad_()
    ids = torch.randint(3, 200, (2, 16))
    mask = torch.ones(2, 16, dtype=torch.long)
    plain = D.decoder_forward(p, ids, mask)
    tiled = D.decoder_forward(p, ids, mask, options=ForwardOptions(mlp_chunk_size=4, gradient_checkpointing=True))
    assert torch.allclose(plain, tiled, atol=1e-5)


def test_schedules():
    cos = ScheduleConfig(1.0, 0.1, "cosine", 2, 12)
    assert learning_rate_at(cos, 0) == 0.0 and learning_rate_at(cos, 1) == 0.5 and learning_rate_at(cos, 2) == 1.0
    assert abs(learning_rate_at(cos, 7) - (0.1 + 0.9 * 0.5)) < 1e-9 and abs(learning_rate_at(cos, 12) - 0.1) < 1e-9
    lin = ScheduleConfig(1.0, 0.0, "linear", 0, 10)
    assert abs(learning_rate_at(lin, 5) - 0.5) < 1e-9 and learning_rate_at(ScheduleConfig(2.0, 0, "constant", 0, 5), 4) == 2.0


def test_adamw_matches_torch_and_masks_decay():
    torch.manual_seed(0)
    w = torch.randn(4, 3)
    g = torch.randn(4, 3)
    ref = torch.nn.Parameter(w.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1)
    ref.grad = g.clone()
    opt.step()
    p, m, v = w.clone(), torch.zeros_like(w), torch.zeros_like(w)
    E.adamw_reference(p, g, m, v, lr=1e-2, b1=0.9, b2=0.999, eps=1e-8, decay=0.1, step=1)
    assert torch.allclose(p, ref.detach(), atol=1e-6)


def test_global_normalisation_over_microbatches_equals_one_big_batch():
    cfg = preset("tiny", vocab_size=300)
    torch.manual_seed(1)
    ids = torch.randint(3, 300, (4, 32))
    mask = torch.ones(4, 32, dtype=torch.long)
    mask[1, :20] = 0                                    # very different token counts per row
    batch = dict(input_ids=ids, attention_mask=mask)
    halves = [{k: v[:2] for k, v in batch.items()}, {k: v[2:] for k, v in batch.items()}]
    outs = []
    for micro in ([batch], halves):
        p = ModelParams.init_random(cfg, 0, torch.float32)
        step = TrainStep(p, AutogradProducer(p, ForwardOptions()), AdamWConfig(0.1), ScheduleConfig(1e-2, 0, "constant", 0, 4))
        m = step.run(micro).to_floats()
        outs.append((m, p.grad_tensor("model.layers.0.mlp.down_proj.weight").clone()))
    assert abs(outs[0][0]["loss"] - outs[1][0]["loss"]) < 1e-5 and outs[0][0]["token_count"] == outs[1][0]["token_count"]
    assert torch.allclose(outs[0][1], outs[1][1], atol=1e-7, rtol=1e-4)   # same normalised gradient


def test_tiny_training_run_then_export_and_reload(tmp_path):
    """Config 1 of the benchmark list, shortened: packed rows, shifted loss, AdamW, export, bit-exact reload."""
    from causal_trainer_dev_b200.checkpointing import huggingface as hfio
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows

    cfg = preset("tiny", vocab_size=1000)
    data = pretraining_rows(4, 128, 1000, eos_token_id=2, pad_token_id=0, median_len=40, min_len=8, seed=0)
    batch = {k: torch.from_numpy(v) for k, v in data.items()}
    p = ModelParams.init_random(cfg, 0, torch.float32)
    step = TrainStep(p, AutogradProducer(p, ForwardOptions()), AdamWConfig(0.1), ScheduleConfig(1e-3, 0, "constant", 0, 10))
    losses = [step.run([batch]).to_floats()["loss"] for _ in range(4)]
    assert abs(losses[0] - math.log(1000)) < 0.2 and losses[-1] < losses[0]
    hfio.export_hf_checkpoint(tmp_path / "m", hfio.TensorSource(cfg, params=p), checkpoint_id="0" * 32)
    q = ModelParams(cfg, torch.float32)
    hfio.load_parameters(tmp_path / "m", q)
    assert all(torch.equal(q.tensor(n), p.tensor(n)) for n in p.hf_names())


def test_frozen_components_and_lora_keep_the_base_untouched():
    from causal_trainer_dev_b200.models.lora import LoraState

    cfg = preset("tiny", vocab_size=300)
    ids = torch.randint(3, 300, (2, 16))
    batch = dict(input_ids=ids, attention_mask=torch.ones(2, 16, dtype=torch.long))
    p = ModelParams.init_random(cfg, 0, torch.float32)
    before = {n: p.tensor(n).clone() for n in p.hf_names()}
    step = TrainStep(p, AutogradProducer(p, ForwardOptions()), AdamWConfig(), ScheduleConfig(1e-2, 0, "constant", 0, 4),
                     frozen=("embed", "norm"))
    step.run([batch])
    changed = {n for n in p.hf_names() if not torch.equal(before[n], p.tensor(n))}
    assert "model.embed_tokens.weight" not in changed and not any("norm" in n for n in changed)
    assert "lm_head.weight" in changed and "model.layers.0.mlp.up_proj.weight" in changed
    # LoRA: step 0 equals the base model; only adapters move; merge equals the adapted forward
    p = ModelParams.init_random(cfg, 0, torch.float32)
    lora = LoraState.init(cfg, 4, seed=1, dtype=torch.float32)
    opts = ForwardOptions(lora=lora)
    mask = batch["attention_mask"]
    assert torch.allclose(D.decoder_forward(p, ids, mask, options=opts), D.decoder_forward(p, ids, mask), atol=1e-6)
    extra = [(t.detach(), t.dim() > 1, (lambda t=t: t.grad)) for _, t in lora.trainable()]
    step = TrainStep(p, AutogradProducer(p, opts, lora=lora), AdamWConfig(), ScheduleConfig(1e-2, 0, "constant", 0, 4),
                     extra_regions=extra, train_base=False)
    base = {n: p.tensor(n).clone() for n in p.hf_names()}
    step.run([batch]); step.run([batch])
    assert all(torch.equal(base[n], p.tensor(n)) for n in p.hf_names())
    assert lora.b[(0, "q_proj")].abs().sum() > 0
    adapted = D.decoder_forward(p, ids, mask, options=opts)
    merged = ModelParams(cfg, torch.float32)
    tf = lora.export_transform()
    merged.load_state_dict({n: tf(n, p.tensor(n).detach()) for n in p.hf_names()})
    assert torch.allclose(D.decoder_forward(merged, ids, mask), adapted, atol=1e-4)
    peft = lora.peft_tensors()
    assert peft["base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight"].shape == (4, cfg.hidden_size)


def test_lora_function_level_helpers_agree_with_the_adapter_state():
    import pytest
    import torch

    from causal_trainer_dev_b200.models import lora as L
    from causal_trainer_dev_b200.models.config import preset

    cfg = preset("tiny")
    state = L.LoraState.init(cfg, 4, seed=3, dtype=torch.float32)
    for b in state.b.values():
        torch.nn.init.normal_(b.data)
    shapes = L.lora_parameter_shapes(cfg, 4)
    named = dict(state.named_tensors())
    assert list(shapes) == list(named) and all(tuple(named[k].shape) == v for k, v in shapes.items())
    peft = state.peft_tensors()
    for path, tensor in named.items():
        key, transposed = L.lora_parameter_to_peft_key(path)
        assert transposed and torch.equal(peft[key], tensor.detach().t())
    assert L.lora_parameter_to_peft_key("adapters/lm_head/kernel") == ("base_model.model.lm_head.weight", False)
    with pytest.raises(KeyError):
        L.lora_parameter_to_peft_key("layers/0/router/lora_a")
    a, b = (t.detach() for t in state.pair(0, "q_proj"))
    x = torch.randn(3, 5, a.shape[0])
    kernel = torch.randn(a.shape[0], b.shape[1])
    merged = L.merge_lora_kernel(kernel, a, b)
    assert torch.allclose(x @ merged, x @ kernel + L.lora_linear_delta(x, a, b), atol=1e-4)
    assert torch.allclose(merged.t(), kernel.t() + state.merged_delta("model.layers.0.self_attn.q_proj.weight"), atol=1e-6)
    assert L.merge_lora_kernel(kernel.bfloat16(), a, b).dtype == torch.bfloat16
    with pytest.raises(ValueError, match="incompatible"):
        L.merge_lora_kernel(kernel.t().contiguous()[:, :3], a, b)
    with pytest.raises(ValueError, match="input width"):
        L.lora_linear_delta(x[..., :-1], a, b)


def test_step_builder_functions_equal_the_hand_wired_steps():
    import pytest

    from causal_trainer_dev_b200.models.lora import LoraState
    from causal_trainer_dev_b200.training.steps import (make_frozen_full_train_step, make_lora_train_step,
                                                        make_train_step)

    cfg = preset("tiny", vocab_size=300)
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(3, 300, (2, 16), generator=gen)
    batch = dict(input_ids=ids, attention_mask=torch.ones(2, 16, dtype=torch.long))
    kw = dict(adamw=AdamWConfig(0.1), schedule=ScheduleConfig(1e-2, 0, "constant", 0, 4))

    built, wired = ModelParams.init_random(cfg, 0, torch.float32), ModelParams.init_random(cfg, 0, torch.float32)
    a = make_train_step(built, ForwardOptions(), **kw).run([batch]).to_floats()
    b = TrainStep(wired, AutogradProducer(wired, ForwardOptions()), kw["adamw"], kw["schedule"]).run([batch]).to_floats()
    assert a == b and all(torch.equal(built.tensor(n), wired.tensor(n)) for n in built.hf_names())

    p = ModelParams.init_random(cfg, 0, torch.float32)
    before = {n: p.tensor(n).clone() for n in p.hf_names()}
    make_frozen_full_train_step(p, ForwardOptions(), ("lm_head",), **kw).run([batch])
    assert torch.equal(before["lm_head.weight"], p.tensor("lm_head.weight"))
    assert not torch.equal(before["model.embed_tokens.weight"], p.tensor("model.embed_tokens.weight"))
    with pytest.raises(ValueError, match="must not be empty"):
        make_frozen_full_train_step(p, ForwardOptions(), (), **kw)

    p = ModelParams.init_random(cfg, 0, torch.float32)
    before = {n: p.tensor(n).clone() for n in p.hf_names()}
    lora = LoraState.init(cfg, 4, seed=1, dtype=torch.float32)
    step = make_lora_train_step(p, lora, ForwardOptions(), **kw)
    first = step.run([batch]).to_floats()["loss"]
    for _ in range(3):
        last = step.run([batch]).to_floats()["loss"]
    assert last < first and all(torch.equal(before[n], p.tensor(n)) for n in p.hf_names())
    assert len(step.optimizer.m) == 2 * 7 * cfg.num_hidden_layers


def test_lora_gradients_do_not_leak_from_one_step_into_the_next():
    """With lr = 0 and the same batch every step, the adapter gradient norm must not grow: each
    optimizer step starts from empty adapter gradients.  Two micro-batches still accumulate."""
    from causal_trainer_dev_b200.models.lora import LoraState
    from causal_trainer_dev_b200.training.steps import make_lora_train_step

    cfg = preset("tiny", vocab_size=300)
    gen = torch.Generator().manual_seed(7)
    ids = torch.randint(3, 300, (2, 16), generator=gen)
    batch = dict(input_ids=ids, attention_mask=torch.ones(2, 16, dtype=torch.long))
    p = ModelParams.init_random(cfg, 0, torch.float32)
    lora = LoraState.init(cfg, 4, seed=1, dtype=torch.float32)
    with torch.no_grad():
        for b in lora.b.values():
            b.normal_(0, 0.02, generator=gen)
    step = make_lora_train_step(p, lora, ForwardOptions(), adamw=AdamWConfig(0.0, max_grad_norm=0.0),
                                schedule=ScheduleConfig(0.0, 0, "constant", 0, 8))
    norms = [step.run([batch]).to_floats()["grad_norm"] for _ in range(3)]
    assert norms[0] > 0 and norms[1] == norms[0] and norms[2] == norms[0]
    halves = [{k: v[i:i + 1] for k, v in batch.items()} for i in range(2)]
    assert abs(step.run(halves).to_floats()["grad_norm"] - norms[0]) < 1e-5 * norms[0]

    # a trajectory against torch.optim.AdamW on the same leaves
    lora2 = LoraState.init(cfg, 4, seed=1, dtype=torch.float32)
    ref = LoraState.init(cfg, 4, seed=1, dtype=torch.float32)
    with torch.no_grad():
        for k in lora2.b:
            lora2.b[k].normal_(0, 0.02, generator=torch.Generator().manual_seed(3))
            ref.b[k].copy_(lora2.b[k])
    ours = make_lora_train_step(p, lora2, ForwardOptions(), adamw=AdamWConfig(0.0, max_grad_norm=0.0),
                                schedule=ScheduleConfig(1e-3, 0, "constant", 0, 8))
    leaves = [t for _, t in ref.trainable()]
    opt = torch.optim.AdamW(leaves, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
    from causal_trainer_dev_b200.training import losses
    from causal_trainer_dev_b200.models.decoder import decoder_forward
    for _ in range(3):
        ours.run([batch])
        opt.zero_grad()
        hidden = decoder_forward(p, batch["input_ids"], batch["attention_mask"], None, None, None, ForwardOptions(lora=ref))
        nll, wsum = losses.causal_lm_loss(hidden, p.units["final"].view("lm_head"), batch)
        (nll / wsum).backward()
        opt.step()
    for (_, a), (_, b) in zip(lora2.trainable(), ref.trainable()):
        assert torch.allclose(a, b, atol=2e-6, rtol=1e-4)
