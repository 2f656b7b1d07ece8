import pytest

from causal_trainer_dev_b200.data.preprocessing import EndPromptSettings, Preprocessor, keep_last_span
from causal_trainer_dev_b200.data.tokenizer import TrainingTokenizer
from helpers import write_tokenizer

MSGS = [{"role": "user", "content": "w1 w2"}, {"role": "assistant", "content": "w3 w4"},
        {"role": "user", "content": "w5"}, {"role": "assistant", "content": "w6"}]


@pytest.fixture()
def tok(tmp_path):
    return TrainingTokenizer.from_directory(write_tokenizer(tmp_path / "tok"))


def test_raw_tokenisation_never_adds_special_tokens(tok):
    out = tok("w1 w2 w3")
    assert out["input_ids"] == [tok.token_to_id("w1"), tok.token_to_id("w2"), tok.token_to_id("w3")]
    with pytest.raises(ValueError, match="unsupported"):
        tok("w1", add_special_tokens=True)
    assert tok.pad_token_id == 0 and tok.eos_token_id == 2


def test_assistant_mask_covers_generation_blocks_only(tok):
    out = tok.apply_chat_template(MSGS, return_assistant_tokens_mask=True)
    ids, mask = out["input_ids"], out["assistant_masks"]
    words = [tok.decode([i]) for i in ids]
    picked = [w for w, m in zip(words, mask) if m]
    assert picked == ["w3", "w4", "<|im_end|>", "w6", "<|im_end|>"]


def test_message_level_loss_false_removes_only_that_span(tok):
    off = [dict(MSGS[0]), dict(MSGS[1], loss=False), dict(MSGS[2]), dict(MSGS[3])]
    a = tok.apply_chat_template(MSGS, return_assistant_tokens_mask=True)
    b = tok.apply_chat_template(off, return_assistant_tokens_mask=True)
    assert a["input_ids"] == b["input_ids"]
    picked = [tok.decode([i]) for i, m in zip(b["input_ids"], b["assistant_masks"]) if m]
    assert picked == ["w6", "<|im_end|>"]


def test_template_files_override_config(tmp_path):
    d = write_tokenizer(tmp_path / "t")
    (d / "chat_template.jinja").write_text("{% for m in messages %}{{ m['content'] }}\n{% endfor %}")
    t = TrainingTokenizer.from_directory(d)
    assert t.apply_chat_template(MSGS[:1], tokenize=False) == "w1 w2\n"
    (d / "chat_templates").mkdir()
    (d / "chat_templates" / "tool_use.jinja").write_text("TOOLS")
    t = TrainingTokenizer.from_directory(d)
    assert t.apply_chat_template(MSGS[:1], tokenize=False, tools=[{"name": "f"}]) == "TOOLS"


def test_last_span_helper():
    assert keep_last_span([0, 1, 1, 0, 1, 1, 1, 0]) == [0, 0, 0, 0, 1, 1, 1, 0]
    assert keep_last_span([0, 0]) == [0, 0]


def test_assistant_only_trims_after_last_trainable_token(tok):
    pre = Preprocessor(tok, "messages", 64, assistant_only_loss=True)
    ex = pre({"messages": MSGS})
    assert ex["assistant_masks"][-1] == 1 and len(ex["input_ids"]) == len(ex["assistant_masks"])
    short = Preprocessor(tok, "messages", 12, assistant_only_loss=True)({"messages": MSGS})
    assert 0 < len(short["input_ids"]) <= 12 and short["assistant_masks"][-1] == 1
    last = Preprocessor(tok, "messages", 64, last_assistant_only_loss=True)({"messages": MSGS})
    assert [tok.decode([i]) for i, m in zip(last["input_ids"], last["assistant_masks"]) if m] == ["w6", "<|im_end|>"]


def test_raw_text_rejects_assistant_modes_and_filters(tok):
    with pytest.raises(ValueError, match="only for messages"):
        Preprocessor(tok, "text", 16, assistant_only_loss=True)({"text": "w1"})
    pre = Preprocessor(tok, "messages", 4, assistant_only_loss=True)
    with pytest.raises(ValueError, match="filtered out"):
        pre.run([{"messages": MSGS}])
    assert pre.run([{"messages": MSGS}], allow_empty=True) == []


def test_endprompt_logical_lengths_and_weights(tok):
    s = EndPromptSettings(16, 24, ("w9 w10",), prompt_loss_weight=0.1, context_loss_weight=1.0)
    assert s.logical_length_for_row(0) == 16 + (12345 & 0x7FFFFFFF) % 9
    assert s.logical_length_for_row(7) == 16 + ((7 * 1103515245 + 12345) & 0x7FFFFFFF) % 9
    pre = Preprocessor(tok, "text", 8, endprompt=s)
    ex = pre({"text": "w1 w2 w3 w4 w5 w6 w7 w8 w9"}, example_index=3)
    assert len(ex["input_ids"]) == 8 and ex["input_ids"][-2:] == [tok.token_to_id("w9"), tok.token_to_id("w10")]
    logical = s.logical_length_for_row(3)
    assert ex["position_ids"] == [0, 1, 2, 3, 4, 5, logical - 2, logical - 1]
    assert ex["loss_weights"] == [1.0] * 6 + [0.1, 0.1]


def test_output_schema_follows_the_options_even_when_every_row_is_filtered(tok):
    from causal_trainer_dev_b200.data.preprocessing import preprocess_records

    empty = preprocess_records([{"messages": MSGS}], tok, dataset_text_field="messages", max_sequence_length=4,
                               assistant_only_loss=True, allow_empty=True)
    assert len(empty) == 0 and empty.column_names == ["input_ids", "attention_mask", "assistant_masks"]
    s = EndPromptSettings(16, 24, ("w9 w10",))
    for kwargs in ({}, {"endprompt": s}):
        rows = preprocess_records([{"text": "w1 w2 w3 w4 w5 w6 w7"}], tok, dataset_text_field="text",
                                  max_sequence_length=8, **kwargs)
        assert sorted(rows[0]) == sorted(rows.column_names)
    rows = preprocess_records([{"messages": MSGS}], tok, dataset_text_field="messages", max_sequence_length=16,
                              assistant_only_loss=True, endprompt=s)
    assert sorted(rows[0]) == sorted(rows.column_names)


def test_function_level_tokenisation_matches_the_preprocessor(tok):
    from causal_trainer_dev_b200.data import preprocessing as pp

    s = EndPromptSettings(16, 24, ("w9 w10",))
    text = "w1 w2 w3 w4 w5 w6 w7 w8 w9"
    assert pp.tokenize_raw_text(text, tok, max_sequence_length=6) == Preprocessor(tok, "text", 6)({"text": text})
    assert (pp.tokenize_messages(MSGS, tok, max_sequence_length=64, assistant_only_loss=True)
            == Preprocessor(tok, "messages", 64, assistant_only_loss=True)({"messages": MSGS}))
    assert (pp.tokenize_endprompt_text(text, tok, max_sequence_length=8, settings=s, example_index=3)
            == Preprocessor(tok, "text", 8, endprompt=s)({"text": text}, 3))
    assert (pp.tokenize_endprompt_messages(MSGS, tok, max_sequence_length=16, assistant_only_loss=True, settings=s,
                                           example_index=2)
            == Preprocessor(tok, "messages", 16, assistant_only_loss=True, endprompt=s)({"messages": MSGS}, 2))
    assert (pp.preprocess_example({"messages": MSGS}, tok, dataset_text_field="messages", max_sequence_length=64,
                                  last_assistant_only_loss=True)
            == Preprocessor(tok, "messages", 64, last_assistant_only_loss=True)({"messages": MSGS}))
    with pytest.raises(ValueError, match="raw string"):
        pp.tokenize_endprompt_text(MSGS, tok, max_sequence_length=8, settings=s, example_index=0)
    with pytest.raises(ValueError, match="must be positive"):
        pp.tokenize_raw_text(text, tok, max_sequence_length=0)
