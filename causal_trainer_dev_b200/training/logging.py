"""Logging, throughput / MFU accounting, device memory statistics, optional Weights & Biases.

Rank 0 logs at INFO, other ranks at WARNING (src/causal_trainer/training/logging.py:7-12).
Beyond the reference's ``steps_per_second`` this module reports tokens/s and model-FLOP
utilisation against the measured bf16 peak of the box (``MEASURED_PEAKS.json`` when present,
1400 TFLOP/s otherwise): the two figures a training run is usually compared by.
"""
from __future__ import annotations

import json
import logging
from pathlib import Path

import torch

log = logging.getLogger("causal_trainer")


def configure_logging(process_index: int) -> None:
    logging.basicConfig(level=logging.INFO if process_index == 0 else logging.WARNING,
                        format="%(asctime)s %(levelname)s %(name)s: %(message)s")


def measured_bf16_peak_tflops() -> float:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["bf16_tflops_sustained"])
    except (OSError, KeyError, ValueError):
        return 1400.0


class ThroughputTracker:
    """Host-side wall-clock throughput over the steps since the last report."""

    def __init__(self, cfg, seq_len: int, n_gpus: int):
        self.flops_per_token = cfg.flops_per_token(seq_len)
        self.seq_len, self.n_gpus = seq_len, max(1, n_gpus)
        self.peak = measured_bf16_peak_tflops() * 1e12
        self.reset()

    def reset(self) -> None:
        self.steps, self.rows, self.seconds = 0, 0, 0.0

    def step(self, rows: int, seconds: float) -> None:
        self.steps += 1
        self.rows += rows
        self.seconds += seconds

    def report(self) -> dict[str, float]:
        s = max(self.seconds, 1e-9)
        tokens_per_s = self.rows * self.seq_len / s
        out = {"steps_per_second": self.steps / s, "examples_per_second": self.rows / s, "tokens_per_second": tokens_per_s,
               "mfu": tokens_per_s * self.flops_per_token / (self.n_gpus * self.peak)}
        self.reset()
        return out


class StepProfiler:
    """``--profile_steps N``: device time of N optimizer steps, after ``skip`` untimed ones.

    On CUDA each timed step is bracketed by CUDA events on the current stream and wrapped in an
    NVTX range (``train_step/<n>``) so that a trace lines up with the numbers; on CPU the host clock
    is used.  :meth:`finish` is collective: per step it takes the maximum over ranks, then reports
    the mean step time, tokens/s of the whole job and MFU against the measured bf16 rate.
    """

    def __init__(self, count: int, device: torch.device | None, *, tokens_per_step: int, flops_per_token: float,
                 n_gpus: int, skip: int = 2):
        self.count, self.skip = max(0, int(count)), max(0, int(skip))
        self.cuda = device is not None and device.type == "cuda"
        self.device = device
        self.tokens_per_step, self.flops_per_token, self.n_gpus = tokens_per_step, flops_per_token, max(1, n_gpus)
        self.seen = 0
        self._open = None
        self._spans: list[tuple] = []

    @property
    def timing(self) -> bool:
        return self.count > 0 and self.skip <= self.seen < self.skip + self.count

    def begin(self) -> None:
        if not self.timing:
            return
        if self.cuda:
            torch.cuda.nvtx.range_push(f"train_step/{self.seen}")
            start = torch.cuda.Event(enable_timing=True)
            start.record()
            self._open = start
        else:
            import time

            self._open = time.perf_counter()

    def end(self) -> None:
        if self._open is not None:
            if self.cuda:
                stop = torch.cuda.Event(enable_timing=True)
                stop.record()
                torch.cuda.nvtx.range_pop()
                self._spans.append((self._open, stop))
            else:
                import time

                self._spans.append((self._open, time.perf_counter()))
            self._open = None
        self.seen += 1

    def finish(self) -> dict | None:
        """Collective when ``count > 0``; the report (same on every rank) or None when nothing was timed."""
        if self.count <= 0:
            return None
        from ..parallel import runtime as rt

        if self.cuda:
            torch.cuda.synchronize(self.device)
            local = [a.elapsed_time(b) for a, b in self._spans]
        else:
            local = [(b - a) * 1e3 for a, b in self._spans]
        per_rank = rt.allgather_object(local)
        steps = min(len(x) for x in per_rank)
        if steps == 0:
            return None
        ms = [max(x[i] for x in per_rank) for i in range(steps)]
        mean = sum(ms) / steps
        tokens_per_s = self.tokens_per_step / (mean * 1e-3)
        return {"profiled_steps": steps, "skipped_steps": self.skip, "ms_per_step": mean, "ms_per_step_min": min(ms),
                "ms_per_step_max": max(ms), "tokens_per_second": tokens_per_s,
                "mfu": tokens_per_s * self.flops_per_token / (self.n_gpus * measured_bf16_peak_tflops() * 1e12),
                "clock": "cuda events, max over ranks" if self.cuda else "host clock, max over ranks"}


def device_memory_stats(device: torch.device | None) -> dict[str, float]:
    if device is None or device.type != "cuda":
        return {}
    gib = float(1 << 30)
    return {"bytes_in_use_gib": torch.cuda.memory_allocated(device) / gib,
            "peak_bytes_in_use_gib": torch.cuda.max_memory_allocated(device) / gib}


class ExperimentLogger:
    """Weights & Biases run when ``enabled`` (naming the flag without the package installed is an
    error, src/causal_trainer/training/logging.py:30-46); a no-op otherwise."""

    def __init__(self, enabled: bool, project: str, run_name: str | None, config: dict | None):
        self._run = None
        if enabled:
            try:
                import wandb
            except ImportError as error:
                raise RuntimeError("--use_wandb requires the wandb package") from error
            self._run = wandb.init(project=project, name=run_name, config=config)

    @property
    def active(self) -> bool:
        return self._run is not None

    def log(self, values: dict, step: int) -> None:
        if self._run is not None:
            self._run.log(values, step=step)

    def finish(self) -> None:
        if self._run is not None:
            self._run.finish()


def memory_metrics(devices=None) -> dict[str, float]:
    """``device_<i>/bytes_in_use_gib`` and ``device_<i>/peak_bytes_in_use_gib`` for the given CUDA
    devices (this process's current device by default); empty without CUDA."""
    if not torch.cuda.is_available():
        return {}
    devices = [torch.cuda.current_device()] if devices is None else list(devices)
    out: dict[str, float] = {}
    for device in devices:
        index = torch.device("cuda", device).index if isinstance(device, int) else torch.device(device).index
        for key, value in device_memory_stats(torch.device("cuda", index)).items():
            out[f"device_{index}/{key}"] = value
    return out


def init_wandb(args):
    """The run's :class:`ExperimentLogger` (rank 0 only calls this), or None when not asked for."""
    if not args.use_wandb:
        return None
    config = {k: str(v) for k, v in vars(args).items()} if hasattr(args, "__dict__") else None
    return ExperimentLogger(True, args.wandb_project, args.wandb_run_name, config)


def log_step(latest: dict[str, float] | None, tracker: ThroughputTracker, device, wandb_run) -> None:
    if latest is None:
        return
    record = {**latest, **tracker.report(), **device_memory_stats(device)}
    log.info("step %(step)d loss %(loss).4f grad_norm %(grad_norm).3f lr %(learning_rate).3e "
             "tok/s %(tokens_per_second).0f mfu %(mfu).3f", record)
    if wandb_run is not None:
        wandb_run.log({k: v for k, v in record.items() if k != "step"}, step=int(record["step"]))
