import json
from pathlib import Path

import numpy as np
import pytest

from causal_trainer_dev_b200 import prepare
from causal_trainer_dev_b200.data import prepared as P
from helpers import write_tokenizer


def _write_jsonl(path, n=30):
    rows = [{"text": " ".join(f"w{(i * 7 + j) % 40}" for j in range(2 + i % 9))} for i in range(n)]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    return path


def _prepare(tmp_path, shards=2, extra=()):
    tok = write_tokenizer(tmp_path / "tok")
    data = _write_jsonl(tmp_path / "d.jsonl")
    out = tmp_path / "prepared"
    args = prepare.parse_args(["--dataset_name", str(data), "--tokenizer_name_or_path", str(tok), "--output_dir", str(out),
                               "--max_sequence_length", "16", "--packing", "--num_shards", str(shards), *extra])
    return prepare.prepare_dataset(args), out


def test_prepare_cli_writes_manifest_last_and_valid_shards(tmp_path):
    manifest, out = _prepare(tmp_path)
    assert (out / P.PREPARED_MANIFEST_FILENAME).is_file() and len(manifest.shards) == 2
    assert [s.path for s in manifest.shards] == ["data/shard-00000-of-00002.parquet", "data/shard-00001-of-00002.parquet"]
    again = P.load_prepared_manifest(str(out))
    assert again.global_digest == manifest.global_digest and again.to_dict()["format"] == "causal-trainer-prepared"
    cols = P.load_prepared_dataset(str(out), again)
    assert cols["input_ids"].shape == (manifest.total_rows, 16) and cols["loss_weights"].dtype == np.float32
    assert cols["input_ids"].dtype == np.int32 and (cols["segment_ids"] > 0).sum() == (cols["attention_mask"] == 1).sum()
    # contiguous file assignment per process
    a = P.load_prepared_dataset(str(out), again, process_index=0, process_count=2)
    b = P.load_prepared_dataset(str(out), again, process_index=1, process_count=2)
    assert np.array_equal(np.concatenate([a["input_ids"], b["input_ids"]]), cols["input_ids"])


def test_output_dir_must_be_empty_and_failures_clean_up(tmp_path):
    _, out = _prepare(tmp_path)
    with pytest.raises(ValueError, match="must be empty"):
        _prepare(tmp_path)
    bad = tmp_path / "bad"
    tok = tmp_path / "tok"
    args = prepare.parse_args(["--dataset_name", str(tmp_path / "d.jsonl"), "--tokenizer_name_or_path", str(tok),
                               "--output_dir", str(bad), "--max_sequence_length", "16", "--dataset_text_field", "nope"])
    with pytest.raises(KeyError):
        prepare.prepare_dataset(args)
    assert not bad.exists()


def test_corrupt_shard_is_detected_by_digest(tmp_path):
    manifest, out = _prepare(tmp_path, shards=1)
    f = out / manifest.shards[0].path
    blob = bytearray(f.read_bytes())
    blob[len(blob) // 2] ^= 0xFF
    f.write_bytes(blob)
    with pytest.raises(RuntimeError, match="checksum mismatch"):
        P.load_prepared_dataset(str(out), manifest)


def test_manifest_validation():
    shard = P.PreparedShard("data/a.parquet", 3, "0" * 64)
    m = P.PreparedDatasetManifest(8, "train", (shard,), {}, {}, {}, 10, 7)
    d = m.to_dict()
    assert P.PreparedDatasetManifest.from_dict(d).global_digest == m.global_digest
    with pytest.raises(ValueError, match="total_rows"):
        P.PreparedDatasetManifest.from_dict({**d, "total_rows": 4})
    with pytest.raises(ValueError, match="fields mismatch"):
        P.PreparedDatasetManifest.from_dict({k: v for k, v in d.items() if k != "schema"})
    for bad in ("../x.parquet", "/abs/x.parquet", "a\\b.parquet", "x.txt"):
        with pytest.raises(ValueError):
            P.PreparedShard(bad, 1, "0" * 64)


def test_semantic_row_validation():
    ok = dict(input_ids=[[5, 6, 7, 0]], attention_mask=[[1, 1, 1, 0]], position_ids=[[0, 1, 2, 0]],
              segment_ids=[[1, 1, 1, 0]], loss_weights=[[1.0, 1.0, 1.0, 0.0]])
    kw = dict(max_sequence_length=4, max_token_id=10, max_position_id=5, uses_assistant_loss_mask=False)
    P.validate_prepared_batch(ok, **kw)
    for field, value, msg in [
        ("input_ids", [[5, 6, 11, 0]], "max_token_id"), ("attention_mask", [[1, 2, 1, 0]], "0/1"),
        ("segment_ids", [[1, 1, 0, 0]], "positive exactly"), ("position_ids", [[0, 1, 2, 3]], "zero outside"),
        ("loss_weights", [[1.0, 1.0, 1.0, 0.5]], "zero outside"), ("loss_weights", [[1.0, 0.0, 0.0, 0.0]], "no positive-weight"),
        ("segment_ids", [[1, 2, 1, 0]], "reuses segment_id=1 after its contiguous run"),
    ]:
        with pytest.raises(ValueError, match=msg):
            P.validate_prepared_batch({**ok, field: value}, **kw)
    # a run that padding interrupts has ended too; ids need not be monotonic as long as they are not reused
    gap = dict(input_ids=[[5, 6, 0, 7]], attention_mask=[[1, 1, 0, 1]], position_ids=[[0, 1, 0, 0]],
               segment_ids=[[1, 1, 0, 1]], loss_weights=[[0.0, 1.0, 0.0, 0.0]])
    with pytest.raises(ValueError, match="reuses segment_id=1 after its contiguous run"):
        P.validate_prepared_batch(gap, **kw)
    P.validate_prepared_batch({**gap, "segment_ids": [[3, 3, 0, 2]]}, **kw)


def test_prepared_streaming_envelopes(tmp_path):
    manifest, out = _prepare(tmp_path)
    env = list(P.iter_prepared_streaming_batches(str(out), manifest, num_epochs=2, window_size=3))
    assert sum(e.is_epoch_end for e in env) == 2 and sum(e.source_examples for e in env) == 2 * manifest.total_rows


def test_manifest_records_preprocessing_without_secrets_and_rejects_empty_shards(tmp_path):
    manifest, out = _prepare(tmp_path, extra=("--endprompt_enable", "--endprompt_logical_length", "16",
                                              "--endprompt_prompts", "go on", "--token", "do-not-serialize-me"))
    pre = manifest.preprocessing
    assert set(pre) == {"dataset_text_field", "packing", "packing_batch_size", "assistant_only_loss",
                        "last_assistant_only_loss", "preprocessing_num_workers", "num_shards", "endprompt"}
    assert pre["endprompt"] == {"logical_length_min": 16, "logical_length_max": 16, "prompts": ["go on"],
                                "prompt_loss_weight": 0.1, "context_loss_weight": 1.0}
    assert "do-not-serialize-me" not in (out / P.PREPARED_MANIFEST_FILENAME).read_text(encoding="utf-8")
    # more shards than source rows: the empty one is an error and nothing stays behind
    tok = tmp_path / "tok"
    one = tmp_path / "one.jsonl"
    one.write_text(json.dumps({"text": "w1 w2 w3"}))
    target = tmp_path / "too_many"
    args = prepare.parse_args(["--dataset_name", str(one), "--tokenizer_name_or_path", str(tok), "--output_dir",
                               str(target), "--max_sequence_length", "16", "--num_shards", "3"])
    with pytest.raises(ValueError, match="prepared shard 1 is empty"):
        prepare.prepare_dataset(args)
    assert not (target / P.PREPARED_MANIFEST_FILENAME).exists() and not (target / "data").exists()


def test_hub_upload_creates_repo_and_branch_before_uploading_every_shard(tmp_path, monkeypatch):
    calls = []

    class FakeApi:
        def create_repo(self, *args, **kwargs):
            calls.append(("create", args, kwargs))

        def create_branch(self, **kwargs):
            calls.append(("branch", (), kwargs))

        def upload_folder(self, **kwargs):
            folder = Path(kwargs["folder_path"])
            assert (folder / P.PREPARED_MANIFEST_FILENAME).is_file()
            assert len(list((folder / "data").glob("*.parquet"))) == 2
            calls.append(("upload", (), kwargs))

    monkeypatch.setattr(prepare, "HfApi", FakeApi)
    _prepare(tmp_path, shards=2, extra=("--hub-repo-id", "org/prepared", "--hub-revision", "data-branch", "--private",
                                        "--token", "secret"))
    assert [c[0] for c in calls] == ["create", "branch", "upload"]
    assert calls[0][1:] == (("org/prepared",), {"token": "secret", "private": True, "repo_type": "dataset",
                                                "exist_ok": True})
    assert calls[1][2] == {"repo_id": "org/prepared", "branch": "data-branch", "token": "secret",
                           "repo_type": "dataset", "exist_ok": True}
    assert calls[2][2]["revision"] == "data-branch" and calls[2][2]["repo_type"] == "dataset"


def test_remote_tokenizer_download_fetches_tokenizer_files_only(tmp_path, monkeypatch):
    tok = write_tokenizer(tmp_path / "downloaded")
    calls = []

    def fake_snapshot_download(*args, **kwargs):
        calls.append((args, kwargs))
        return str(tok)

    monkeypatch.setattr(prepare, "snapshot_download", fake_snapshot_download)
    args = prepare.parse_args(["--dataset-name", "source", "--tokenizer-name-or-path", "org/tokenizer",
                               "--tokenizer-revision", "abc123", "--token", "secret", "--output-dir",
                               str(tmp_path / "out")])
    assert str(prepare.resolve_tokenizer_directory(args)) == str(tok)
    assert calls == [(("org/tokenizer",), {"repo_type": "model", "revision": "abc123", "token": "secret",
                                           "allow_patterns": list(prepare.TOKENIZER_GLOBS)})]


def test_hub_loading_downloads_only_this_process_interval(tmp_path, monkeypatch):
    import dataclasses

    manifest, out = _prepare(tmp_path, shards=5)
    downloads = []

    def fake_download(**kwargs):
        assert kwargs["repo_id"] == "org/prepared" and kwargs["repo_type"] == "dataset"
        assert kwargs["revision"] == "prepared-commit" and kwargs["token"] == "secret"
        downloads.append(kwargs["filename"])
        return str(out / kwargs["filename"])

    monkeypatch.setattr(P, "hf_hub_download", fake_download)
    columns = P.load_prepared_dataset("org/prepared", manifest, revision="prepared-commit", token="secret",
                                      process_index=1, process_count=2)
    assert downloads == [s.path for s in manifest.shards[3:]]
    assert len(columns["input_ids"]) == sum(s.rows for s in manifest.shards[3:])
    # a process past the last file downloads nothing and gets typed empty columns
    downloads.clear()
    empty = P.load_prepared_dataset("org/prepared", manifest, process_index=7, process_count=8)
    assert downloads == [] and empty["input_ids"].shape == (0, 16) and empty["loss_weights"].dtype == np.float32
    # streaming selects every file, and checks all checksums before the first row is read
    downloads.clear()
    stream = P.load_prepared_dataset("org/prepared", manifest, streaming=True, revision="prepared-commit", token="secret")
    assert downloads == [s.path for s in manifest.shards]
    assert sum(1 for _ in stream) == manifest.total_rows == sum(1 for _ in stream)
    corrupt = dataclasses.replace(manifest, shards=(dataclasses.replace(manifest.shards[0], sha256="0" * 64),
                                                    *manifest.shards[1:]))
    for kwargs in ({"process_index": 0, "process_count": 2}, {"streaming": True}):
        with pytest.raises(RuntimeError, match="checksum mismatch"):
            P.load_prepared_dataset(str(out), corrupt, **kwargs)
    P.load_prepared_dataset(str(out), corrupt, verify_checksums=False)


def test_loading_rejects_values_above_the_manifest_maxima(tmp_path):
    import dataclasses

    manifest, out = _prepare(tmp_path, shards=1)
    for field, match in (("max_token_id", "max_token_id"), ("max_position_id", "max_position_id")):
        lowered = dataclasses.replace(manifest, **{field: 0})
        with pytest.raises(ValueError, match=match):
            P.load_prepared_dataset(str(out), lowered)
        with pytest.raises(ValueError, match=match):
            list(P.iter_prepared_streaming_batches(str(out), lowered, num_epochs=1))
    wrong_rows = dataclasses.replace(manifest, shards=(dataclasses.replace(manifest.shards[0],
                                                                           rows=manifest.shards[0].rows + 1),))
    with pytest.raises(ValueError, match="rows, manifest says"):
        list(P.iter_prepared_streaming_batches(str(out), wrong_rows, num_epochs=1))


def test_canonical_columns_have_fixed_dtypes_and_validate_semantics():
    columns = dict(input_ids=[[5, 6, 0, 0]], attention_mask=[[1, 1, 0, 0]], position_ids=[[0, 1, 0, 0]],
                   segment_ids=[[1, 1, 0, 0]], loss_weights=[[0.0, 1.0, 0.0, 0.0]])
    typed = P.canonical_prepared_dataset(columns, max_sequence_length=4)
    assert all(v.shape == (1, 4) for v in typed.values())
    assert typed["loss_weights"].dtype == np.float32 and typed["input_ids"].dtype == np.int32
    assert P.canonical_prepared_features(4) == P.schema_dict(4, False)
    assert "assistant_masks" in P.canonical_prepared_features(4, uses_assistant_loss_mask=True)
    P.validate_prepared_dataset(typed, max_sequence_length=4, expected_rows=1, max_token_id=6, max_position_id=1)
    with pytest.raises(ValueError, match="has 1 rows, expected 2"):
        P.validate_prepared_dataset(typed, max_sequence_length=4, expected_rows=2)
    with pytest.raises(ValueError, match="max_token_id=5"):
        P.validate_prepared_dataset(typed, max_sequence_length=4, max_token_id=5)
    with pytest.raises(ValueError, match="fields mismatch"):
        P.canonical_prepared_dataset(columns, max_sequence_length=4, uses_assistant_loss_mask=True)
    with pytest.raises(TypeError):
        P.canonical_prepared_features(4, uses_assistant_loss_mask=1)
