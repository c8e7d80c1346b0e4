"""Host-side mirror of the reference's evaluation harness and experiment driver.

  load_tokens      harness.go:17-32      little-endian uint16 token file
  eval_loss        harness.go:46-89      validation loss over the last 10 000 tokens in windows that
                                         overlap by one token; the per-window sum runs on the device
                                         (Engine.eval_loss), no logits come back to the host
  val_bpb          bench_test.go:147-158 loss / ln 2 / 3.7
  lr_schedule      experiment.go:69-75   5 % linear warm-up, cosine decay to 10 % of the peak
  train            README.md:17, program.md:31: steps for a fixed wall-clock budget that starts after
                   the first three steps, learning rate set from the schedule before every step.  The
                   reference describes this loop but ships an empty main.go; this is the loop as described.
  benchmark_step / benchmark_eval_logits / benchmark_eval_loss
                   bench_test.go:75-158  the three benchmarks with the reference's metric names

The reference's evalLoss slices the [vocab][seq] logits as if they were [seq][vocab] (harness.go:62); the
device path scores position t with the logits of position t, i.e. the indexing the harness intends.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field

import numpy as np

EVAL_TOKENS = 10_000        # harness.go:36
EVAL_SEQ_LEN = 256          # harness.go:37
AVG_BYTES_PER_TOKEN = 3.7   # harness.go:43
WARMUP_FRACTION = 0.05      # experiment.go:41
WARMUP_STEPS = 3            # program.md:31: the budget excludes the first three steps
LR_FLOOR_FRACTION = 1e-3    # SetLR rejects lr <= 0 (ane/engine.go:370-372): the ramp starts at peak/1000


def load_tokens(path: str) -> np.ndarray:
    """harness.go:17-32: the file is a flat array of little-endian uint16; an odd size is an error."""
    data = np.fromfile(path, dtype=np.uint8)
    if data.size % 2 != 0:
        raise ValueError(f"read tokens: file size {data.size} is not even")
    return data.view("<u2").astype(np.uint16)


def eval_windows(tokens: np.ndarray, eval_tokens: int = EVAL_TOKENS, seq: int = EVAL_SEQ_LEN) -> np.ndarray:
    """The windows harness.go:46-57 visits: start every seq-1 tokens inside the last `eval_tokens` tokens
    while a full window still fits (pos + seq < len, strictly)."""
    if tokens.size < eval_tokens + seq:
        raise ValueError(f"eval: need at least {eval_tokens + seq} tokens, got {tokens.size}")
    val = tokens[tokens.size - eval_tokens:]
    starts = range(0, val.size - seq, seq - 1)
    return np.stack([val[p:p + seq] for p in starts]) if len(starts) else np.zeros((0, seq), np.uint16)


def _eval_loss_reference_indexing(engine, windows: np.ndarray) -> float:
    """harness.go:58-84 as written: EvalLogits returns [vocab][seq] (logits[v*seq+t]) but the loop slices it as
    logits[t*vocab:(t+1)*vocab], and the running maximum starts at the smallest positive float64
    (math.SmallestNonzeroFloat64), so a row of negative values keeps that start value.  Reproduces the reference's
    val_loss / val_bpb for regression comparisons with numbers from its own harness."""
    total, positions = 0.0, 0
    seq, vocab = engine.seq, engine.vocab
    tiny = np.float64(5e-324)
    for w in windows:
        flat = engine.eval_logits(w, layout=0).reshape(-1).astype(np.float64)
        rows = flat.reshape(seq, vocab)[:seq - 1]          # the reference's slicing of the flat buffer
        targets = w[1:seq].astype(np.int64)
        mx = np.maximum(rows.max(axis=1), tiny)
        lse = mx + np.log(np.exp(rows - mx[:, None]).sum(axis=1))
        total += float((lse - rows[np.arange(seq - 1), targets]).sum())
        positions += seq - 1
    if positions == 0:
        raise ValueError("eval: no positions evaluated")
    return total / positions


def eval_loss(engine, tokens: np.ndarray, eval_tokens: int = EVAL_TOKENS, reference_indexing: bool = False) -> float:
    """Mean next-token cross-entropy in nats over the validation windows (harness.go:46-89).
    reference_indexing=True walks the downloaded logits exactly like the reference's loop does (see
    _eval_loss_reference_indexing); the default scores position t with the logits of position t on the device."""
    windows = eval_windows(np.asarray(tokens, dtype=np.uint16), eval_tokens, engine.seq)
    if reference_indexing:
        return _eval_loss_reference_indexing(engine, windows)
    total, positions = 0.0, 0
    batch = max(1, engine.opts.batch)
    for i in range(0, len(windows), batch):
        s, n = engine.eval_loss(windows[i:i + batch])
        total += s
        positions += n
    if positions == 0:
        raise ValueError("eval: no positions evaluated")
    return total / positions


def val_bpb(loss: float) -> float:
    return loss / math.log(2.0) / AVG_BYTES_PER_TOKEN


def lr_schedule(progress: float, peak_lr: float = 3e-4) -> float:
    """experiment.go:69-75."""
    if progress < WARMUP_FRACTION:
        return peak_lr * progress / WARMUP_FRACTION
    decay = 0.5 * (1.0 + math.cos(math.pi * (progress - WARMUP_FRACTION) / (1.0 - WARMUP_FRACTION)))
    return peak_lr * (0.1 + 0.9 * decay)


@dataclass
class TrainLog:
    steps: int = 0
    tokens: int = 0
    seconds: float = 0.0
    losses: list = field(default_factory=list)
    lrs: list = field(default_factory=list)

    @property
    def tok_per_s(self) -> float:
        return self.tokens / self.seconds if self.seconds > 0 else 0.0


def train(engine, budget_s: float | None = None, max_steps: int | None = None, peak_lr: float = 3e-4,
          clock=time.perf_counter) -> TrainLog:
    """Runs Step() until the wall-clock budget (or step count) is used up.  Progress for the schedule is
    elapsed / budget when a budget is given, else step / max_steps.  The first WARMUP_STEPS steps run at the
    start of the ramp and are not counted against the budget or in the throughput.  The schedule is 0 at
    progress 0 and SetLR refuses lr <= 0 (ane/engine.go:370-372), so values below peak_lr * LR_FLOOR_FRACTION
    are raised to that floor."""
    if budget_s is None and max_steps is None:
        raise ValueError("train: give a time budget or a step count")
    log = TrainLog()
    tokens_per_step = engine.opts.batch * engine.seq * max(1, engine.opts.world_size)
    floor = peak_lr * LR_FLOOR_FRACTION
    for _ in range(WARMUP_STEPS):
        engine.set_lr(max(lr_schedule(0.0, peak_lr), floor))
        engine.step()
    t0 = clock()
    while True:
        elapsed = clock() - t0
        if budget_s is not None:
            if elapsed >= budget_s:
                break
            progress = elapsed / budget_s
        else:
            progress = log.steps / max_steps
        if max_steps is not None and log.steps >= max_steps:
            break
        lr = max(lr_schedule(progress, peak_lr), floor)
        engine.set_lr(lr)
        r = engine.step()
        log.steps += 1
        log.tokens += tokens_per_step
        log.losses.append(r.loss)
        log.lrs.append(lr)
    engine.flush()
    log.seconds = clock() - t0
    return log


def benchmark_step(engine, n: int = 10, accum_steps: int | None = None) -> dict:
    """BenchmarkStep (bench_test.go:75-119): three untimed steps, then n steps; metrics taken from the last
    StepResult as the reference does.  `tok/s` follows the reference's formula, seq * AccumSteps / StepDuration
    (bench_test.go:92,107-110), although one Step() handles `batch` sequences and no accumulation loop - with
    the reference's own engine (batch 1) that over-reports by AccumSteps; `tok/s_processed` counts the tokens
    the step really pushed through.  `ane_ms` is the device time of the step (the reference's ANE evaluation
    time), `adam_ms` the optimizer's, as ane.StepResult reports them."""
    for _ in range(3):
        engine.step()
    accum = accum_steps if accum_steps is not None else max(1, int(getattr(engine.opts, "accum_steps", 1)))
    last = None
    t0 = time.perf_counter()
    for _ in range(n):
        last = engine.step()
    wall = time.perf_counter() - t0
    out = {"loss": float(last.loss), "step_ms": last.step_duration * 1e3,
           "ane_ms": last.device_eval_duration * 1e3, "adam_ms": last.adam_duration * 1e3,
           "ns/op": wall / n * 1e9}
    if last.step_duration > 0:
        out["tok/s"] = engine.seq * accum / last.step_duration
        out["tok/s_processed"] = engine.opts.batch * engine.seq / last.step_duration
    return out


def benchmark_eval_logits(engine, tokens: np.ndarray, n: int = 10, seq: int = EVAL_SEQ_LEN) -> dict:
    """BenchmarkEvalLogits (bench_test.go:121-139): one window of `seq` tokens per call, logits returned."""
    window = np.ascontiguousarray(tokens[:seq])
    engine.eval_logits(window)
    t0 = time.perf_counter()
    for _ in range(n):
        engine.eval_logits(window)
    dt = (time.perf_counter() - t0) / n
    return {"ns/op": dt * 1e9, "tok/s": seq / dt}


def benchmark_eval_loss(engine, tokens: np.ndarray, n: int = 1, eval_tokens: int = EVAL_TOKENS,
                        reference_indexing: bool = False) -> dict:
    """BenchmarkEvalLoss (bench_test.go:141-158): the full validation pass; val_loss in nats, val_bpb = loss /
    ln 2 / 3.7."""
    loss = 0.0
    t0 = time.perf_counter()
    for _ in range(n):
        loss = eval_loss(engine, tokens, eval_tokens=eval_tokens, reference_indexing=reference_indexing)
    dt = (time.perf_counter() - t0) / n
    return {"val_loss": loss, "val_bpb": val_bpb(loss), "ns/op": dt * 1e9}
