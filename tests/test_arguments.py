import pytest

from causal_trainer_dev_b200.training.arguments import parse_args, parse_frozen_parameter_components

BASE = ["--repo_id", "m", "--dataset_name", "d"]


def test_both_spellings_and_bool_forms():
    a = parse_args(BASE + ["--max-sequence-length", "8192", "--packing", "--no-shuffle", "--lora", "True",
                           "--track_memory", "false"])
    assert a.max_sequence_length == 8192 and a.packing is True and a.shuffle is False and a.lora is True
    assert a.track_memory is False
    b = parse_args(["--repo-id", "m", "--dataset-name", "d", "--max_sequence_length", "8192"])
    assert b.max_sequence_length == 8192


def test_mesh_starting_with_minus_one_is_a_value():
    a = parse_args(BASE + ["--sharding_axis", "-1, 1, 1, 2, 1"])
    assert a.mesh_sizes == (-1, 1, 1, 2, 1)
    assert parse_args(BASE).sharding_axis == "-1,1,1,4,1"


@pytest.mark.parametrize("s,expected", [(4096, 128), (131071, 128), (131072, 256), (262144, 512), (524288, 1024)])
def test_automatic_attention_block_sizes(s, expected):
    a = parse_args(BASE + ["--max_sequence_length", str(s)])
    assert a.block_size_q == expected and a.block_size_k == expected
    assert parse_args(BASE + ["--block_size_q", "256"]).block_size_q == 256


def test_automatic_mlp_chunk_size():
    assert parse_args(BASE).mlp_chunk_size == 1024
    assert parse_args(BASE + ["--max_sequence_length", "2048"]).mlp_chunk_size == 0
    assert parse_args(BASE + ["--max_sequence_length", "131072"]).mlp_chunk_size == 0
    assert parse_args(BASE + ["--lora"]).mlp_chunk_size == 0
    assert parse_args(BASE + ["--sharding_axis", "1,1,1,1,2"]).mlp_chunk_size == 0
    assert parse_args(BASE + ["--mlp_chunk_size", "0"]).mlp_chunk_size == 0


def test_automatic_scan_layers():
    assert parse_args(BASE).scan_layers is False
    assert parse_args(BASE + ["--max_sequence_length", "524288"]).scan_layers is True
    assert parse_args(BASE + ["--max_sequence_length", "131072", "--total_batch_size", "1"]).scan_layers is True
    assert parse_args(BASE + ["--max_sequence_length", "262144", "--total_batch_size", "1"]).scan_layers is False
    assert parse_args(BASE + ["--max_sequence_length", "262144", "--total_batch_size", "1", "--attention_method",
                              "moba"]).scan_layers is True
    assert parse_args(BASE + ["--max_sequence_length", "524288", "--lora"]).scan_layers is False
    assert parse_args(BASE + ["--scan_layers"]).scan_layers is True
    assert parse_args(BASE + ["--max_sequence_length", "524288", "--no-scan-layers"]).scan_layers is False


def test_defaults_that_matter():
    a = parse_args(BASE)
    assert a.save_optimizer_state is False and a.attn_mechanism == "efficient" and a.loss_implementation == "auto"
    assert a.moba_top_k == 12 and a.moba_block_size == 4096 and a.attention_options is None
    assert a.effective_batch_size == 32 and a.fused_collectives is True


@pytest.mark.parametrize("extra,fragment", [
    (["--assistant_only_loss", "--last_assistant_only_loss", "--dataset_text_field", "messages"], "mutually exclusive"),
    (["--assistant_only_loss"], "requires --dataset_text_field messages"),
    (["--lora_save_adapter_only"], "requires --lora"),
    (["--lora", "--save_optimizer_state"], "lora_save_adapter_only"),
    (["--learning_rate_end", "1"], "cannot exceed learning_rate"),
    (["--maskgit_probability", "0.5"], "requires --dataset_text_field messages"),
    (["--maskgit_probability", "0.5", "--dataset_text_field", "messages", "--attention_method", "moba"], "MaskGIT"),
    (["--cut_chunk_size", "64", "--loss_implementation", "xla"], "Cut loss backend"),
    (["--remat_group_size", "2"], "scan_layers=True"),
    (["--projection_chunk_size", "128"], "total_batch_size=1"),
    (["--dataset_streaming", "--num_train_epochs", "1.5"], "integer num_train_epochs"),
    (["--endprompt_enable", "--endprompt_logical_length", "100"], "at least max_sequence_length"),
    (["--hf_retry_initial_delay", "100"], "cannot exceed"),
    (["--attention_dense_prefix_layers", "1"], "require moba"),
])
def test_cross_field_validation(extra, fragment):
    with pytest.raises(ValueError, match=fragment):
        parse_args(BASE + extra)


def test_frozen_parameters_are_normalised():
    assert parse_frozen_parameter_components("norm, embed") == ("embed", "norm")
    assert parse_args(BASE + ["--frozen_parameters", "norm|lm_head"]).frozen_parameters == "lm_head|norm"
    with pytest.raises(ValueError):
        parse_frozen_parameter_components("attention")


def test_flags_of_this_framework_have_defaults_and_choices():
    a = parse_args(BASE)
    assert a.balance_rows is True and a.activation_memory == "auto" and a.fused_collectives is True
    assert a.sp_layout == "contiguous" and parse_args(BASE + ["--sp-layout", "zigzag"]).sp_layout == "zigzag"
    b = parse_args(BASE + ["--no-balance-rows", "--activation-memory", "recompute", "--fused_collectives", "false"])
    assert b.balance_rows is False and b.activation_memory == "recompute" and b.fused_collectives is False
    with pytest.raises(SystemExit):
        parse_args(BASE + ["--activation_memory", "sometimes"])
