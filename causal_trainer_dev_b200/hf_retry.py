"""Retry policy for transient network failures while talking to the Hugging Face Hub.

Transient means: HTTP 408 / 425 / 429 / 5xx, connection and timeout exceptions, a small set
of socket errnos, or an exception whose class comes from a networking library and carries a
known transient name.  Authentication (401/403), missing objects (404) and application
errors fail at once.  Retries never give up: exponential backoff capped by ``max_delay``
(src/causal_trainer/hf_retry.py:103-183).
"""
from __future__ import annotations

import errno
import logging
import math
import time
from typing import Callable, Iterator, TypeVar

R = TypeVar("R")
log = logging.getLogger(__name__)

RETRYABLE_STATUS = frozenset({408, 425, 429})
RETRYABLE_ERRNO = frozenset({
    errno.ECONNABORTED, errno.ECONNREFUSED, errno.ECONNRESET, errno.EHOSTUNREACH, errno.ENETDOWN, errno.ENETRESET,
    errno.ENETUNREACH, errno.EPIPE, errno.ETIMEDOUT,
})
NETWORK_LIBRARIES = ("aiohttp", "fsspec", "httpcore", "http", "httpx", "requests", "ssl", "urllib", "urllib3")
TRANSIENT_NAMES = frozenset("""
ChunkedEncodingError ClientConnectionError ClientConnectorError ClientOSError ClientPayloadError ContentDecodingError
ConnectError ConnectTimeout ConnectionClosed ConnectionError ConnectionResetError DecodingError FSTimeoutError
IncompleteRead MaxRetryError NetworkError NewConnectionError PoolTimeout ProtocolError ProxyError ReadError ReadTimeout
ReadTimeoutError RemoteDisconnected RemoteProtocolError ServerConnectionError ServerDisconnectedError ServerTimeoutError
SSLError Timeout TimeoutError TransportError URLError WriteError WriteTimeout gaierror
""".split())


def _causes(error: BaseException) -> Iterator[BaseException]:
    seen: set[int] = set()
    cur: BaseException | None = error
    while cur is not None and id(cur) not in seen:
        seen.add(id(cur))
        yield cur
        cur = cur.__cause__ or cur.__context__


def _status(error: BaseException) -> int | None:
    response = getattr(error, "response", None)
    for holder, attr in ((response, "status_code"), (response, "status"), (error, "status_code"), (error, "status"),
                         (error, "code")):
        value = getattr(holder, attr, None)
        if value is not None:
            return value if type(value) is int else None
    return None


def _from_network_library(cls: type) -> bool:
    for base in cls.__mro__:
        mod = base.__module__ or ""
        if base.__name__ in TRANSIENT_NAMES and any(mod == r or mod.startswith(r + ".") for r in NETWORK_LIBRARIES):
            return True
    return False


def is_retryable_hf_error(error: BaseException) -> bool:
    for e in _causes(error):
        status = _status(e)
        if status is not None:
            return status in RETRYABLE_STATUS or status >= 500
        if isinstance(e, (ConnectionError, TimeoutError)):
            return True
        if isinstance(e, OSError) and getattr(e, "errno", None) in RETRYABLE_ERRNO:
            return True
        if type(e).__name__ == "gaierror" or _from_network_library(type(e)):
            return True
    return False


def retry_hf_call(call: Callable[[], R], initial_delay: float = 1.0, max_delay: float = 60.0,
                  operation: str = "Hugging Face operation", description: str | None = None) -> R:
    if not callable(call):
        raise TypeError("call must be callable")
    initial, maximum = float(initial_delay), float(max_delay)
    if not math.isfinite(initial) or not math.isfinite(maximum):
        raise ValueError("retry delays must be finite")
    if initial < 0:
        raise ValueError("initial_delay cannot be negative")
    if maximum < initial:
        raise ValueError("max_delay must be greater than or equal to initial_delay")
    what = description or operation
    delay, attempt = initial, 0
    while True:
        try:
            return call()
        except Exception as exc:  # KeyboardInterrupt and friends are never intercepted
            if not is_retryable_hf_error(exc):
                raise
            attempt += 1
            log.warning("%s failed because of a transient network error; retrying indefinitely in %.1fs "
                        "(attempt %d): %s", what, delay, attempt, exc)
            time.sleep(delay)
            delay = min(maximum, max(initial, delay * 2.0))
