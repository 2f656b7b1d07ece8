import errno

import pytest

from causal_trainer_dev_b200.hf_retry import is_retryable_hf_error, retry_hf_call


class Http(Exception):
    def __init__(self, status):
        self.response = type("R", (), {"status_code": status})()


@pytest.mark.parametrize("status,retry", [(401, False), (403, False), (404, False), (408, True), (425, True),
                                         (429, True), (500, True), (503, True)])
def test_status_codes(status, retry):
    assert is_retryable_hf_error(Http(status)) is retry


def test_errno_chain_and_plain_errors():
    assert is_retryable_hf_error(OSError(errno.ECONNRESET, "reset"))
    assert not is_retryable_hf_error(OSError(errno.ENOENT, "missing"))
    wrapped = RuntimeError("outer")
    wrapped.__cause__ = TimeoutError()
    assert is_retryable_hf_error(wrapped) and not is_retryable_hf_error(ValueError("bad data"))


def test_backoff_doubles_up_to_the_cap(monkeypatch):
    sleeps = []
    monkeypatch.setattr("time.sleep", sleeps.append)
    calls = {"n": 0}

    def flaky():
        calls["n"] += 1
        if calls["n"] < 5:
            raise ConnectionError()
        return "ok"

    assert retry_hf_call(flaky, initial_delay=1.0, max_delay=3.0) == "ok" and sleeps == [1.0, 2.0, 3.0, 3.0]
    with pytest.raises(ValueError):
        retry_hf_call(lambda: (_ for _ in ()).throw(ValueError("x")))
