#!/usr/bin/env python
"""Benchmark of the training-step hot path.

  python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

One "step" = forward + backward + AdamW over one micro-batch of the 110M Llama2-style config
(dim 768, 12 layers, 12 heads, SwiGLU hidden 2048, vocab 32000, seq 256, micro-batch 32 per GPU,
bf16 GEMM operands, fp32 master weights and optimizer).  Synthetic data: seeded Zipf(1.1) token
stream and N(0, 0.02) weights stand in for TinyStories and the stories110M checkpoint.

`value` is tokens/s with the token stream resident in HBM (Engine.Step samples windows on the
device): the timed region of exactly `--steps` steps is repeated (`--repeats`, default 5) and the median
repeat is reported, with the spread beside it.  `e2e` is the same metric through ane_step_tokens with host
batches copied H2D and the loss read back every step.  `c4` is the fixed-global-batch form of the
data-parallel configuration: 256 sequences per optimizer update, gradient accumulation 256 / (32 N) on
N GPUs.  At one GPU the line also carries `extras`: batch-64 evaluation, the GQA seq-1024 step and its
KV-cached decode, and the reference architecture's step, each with its fraction of the step roofline.
`--impl reference` times the CPU restatement of the reference's Go step (the reference itself cannot be
built here) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
import zlib

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "autoresearch-go-ane_b200"))

import numpy as np  # noqa: E402

WORKLOADS = {
    # the configuration the headline metric is quoted on
    "110m": dict(cfg=dict(dim=768, hidden=2048, n_layers=12, n_heads=12, n_kv_heads=12, vocab=32000, seq=256),
                 batch=32, arch="llama",
                 name="110M Llama2-style train step: dim 768, 12 layers, 12 heads, SwiGLU 2048, vocab 32000, seq 256, "
                      "micro-batch 32 per GPU; Zipf(1.1) tokens, N(0,0.02) weights"),
    # GQA long-context variant (12 query heads / 4 KV heads, seq 1024, micro-batch 8)
    "gqa1024": dict(cfg=dict(dim=768, hidden=2048, n_layers=12, n_heads=12, n_kv_heads=4, vocab=32000, seq=1024),
                    batch=8, arch="llama",
                    name="GQA variant: dim 768, 12 layers, 12 query / 4 KV heads, SwiGLU 2048, vocab 32000, seq 1024, "
                         "micro-batch 8 per GPU"),
    # the network the reference itself trains, at the benchmark's micro-batch
    "reference": dict(cfg=dict(dim=768, hidden=2048, n_layers=12, n_heads=12, n_kv_heads=12, vocab=32000, seq=256),
                      batch=32, arch="reference",
                      name="reference architecture (ReLU^2 FFN, QK-norm, value embeddings, smear, backout, softcap): "
                           "dim 768, 12 layers, seq 256, micro-batch 32 per GPU"),
}
WORKLOAD = WORKLOADS["110m"]["cfg"]
MICRO_BATCH = WORKLOADS["110m"]["batch"]
N_STREAM_TOKENS = 1 << 22


def train_flops_per_token(cfg, arch):
    """Algorithmic FLOPs per trained token: 6*N_mm + 3.5*(2*L*T*D), N_mm = matmul parameters incl. classifier."""
    D, Hd, L, H, KV, V, T = (cfg[k] for k in ("dim", "hidden", "n_layers", "n_heads", "n_kv_heads", "vocab", "seq"))
    hd = D // H
    n_mm = L * (2 * D * D + 2 * D * KV * hd + (3 if arch == "llama" else 2) * D * Hd) + V * D
    if arch == "reference":
        n_mm += D * D  # smear gate
    return 6 * n_mm + 3.5 * (2 * L * T * D)


TRAIN_FLOPS_PER_TOKEN = train_flops_per_token(WORKLOAD, "llama")

# DRAM bytes (read + write) of all gemm_tc_kernel launches of one 110M step, from an ncu capture of this
# command; bench.py cannot run ncu itself, so the figure is tagged with the commit it was taken at.
GEMM_TRAFFIC = {"dram_bytes_per_step": 12312445952,
                "source": "ncu dram__bytes_read.sum + dram__bytes_write.sum over the 169 gemm_tc_kernel launches of one step "
                          "(--cache-control none, one pass per launch), captured at commit 883cf8c; 14.42 GB with the "
                          "stored-logits head"}


def zipf_tokens(n, vocab, seed, s=1.1):
    rng = np.random.Generator(np.random.PCG64(seed))
    p = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    return np.minimum(np.searchsorted(cdf, rng.random(n), side="right"), vocab - 1).astype(np.uint16)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks, power and throttle reasons with nvidia-smi (every 50 ms) through both timed legs
    (device-resident and end-to-end), so that neither leg pays for polling that the other does not.  The
    process is started before the warm-up steps; mark() / window() bracket each timed region, and only
    samples that arrived inside one are reported."""

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.lines: list[str] = []
        self.windows: list[tuple[int, int]] = []
        self._mark = 0

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            # nvidia-smi needs 0.1-0.3 s before its first line: wait for it here, outside every timed region, so that
            # even a short timed region (ten steps are 80 ms) holds samples
            t0 = time.perf_counter()
            while not self.lines and time.perf_counter() - t0 < 3.0:
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        self._mark = len(self.lines)

    def window(self):
        self.windows.append((self._mark, len(self.lines)))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        picked = [ln for a, b in self.windows for ln in self.lines[a:b]]
        window = "timed regions of the device-resident and end-to-end legs, one sample per 50 ms"
        if not picked:  # regions shorter than one sampling period: fall back to everything since the warm-up began
            picked = list(self.lines)
            window = "warm-up and timed regions (no sample fell inside a timed region alone)"
        for ln in picked:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                pw.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w": float(np.median(pw)) if pw else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": window}


def init_weights(engine, ane, seed, cfg):
    """N(0, 0.02) for every matrix / embedding the architecture has; scalars keep the library defaults,
    except the reference architecture's lambdas which take their RandomInit values
    (ane/stories/weights.go:190-202)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    for layer in range(cfg["n_layers"]):
        for tid in (ane.T_WQ, ane.T_WK, ane.T_WV, ane.T_WO, ane.T_W1, ane.T_W2, ane.T_W3, ane.T_VE_EMBED):
            n = engine.tensor_size(tid, layer)
            if n > 0:
                engine.import_tensor(tid, layer, (0.02 * rng.standard_normal(n)).astype(np.float32))
        n = engine.tensor_size(ane.T_VE_GATE, layer)
        if n > 0:
            engine.import_tensor(ane.T_VE_GATE, layer, (0.02 * rng.random(n)).astype(np.float32))
    for tid in (ane.T_EMBED, ane.T_SMEAR_GATE):
        n = engine.tensor_size(tid, 0)
        if n > 0:
            engine.import_tensor(tid, 0, (0.02 * rng.standard_normal(n)).astype(np.float32))
    for tid, val in ((ane.T_X0_LAMBDAS, 0.1), (ane.T_SMEAR_LAMBDA, 0.01), (ane.T_BACKOUT_LAMBDA, 0.01)):
        n = engine.tensor_size(tid, 0)
        if n > 0:
            engine.import_tensor(tid, 0, np.full(n, val, dtype=np.float32))


def fwd_flops_per_token(cfg, arch):
    """Forward-only FLOPs per token (evaluation, prefill): 2*N_mm + causal attention 2*L*T*D."""
    D, Hd, L, H, KV, V, T = (cfg[k] for k in ("dim", "hidden", "n_layers", "n_heads", "n_kv_heads", "vocab", "seq"))
    hd = D // H
    n_mm = L * (2 * D * D + 2 * D * KV * hd + (3 if arch == "llama" else 2) * D * Hd) + V * D
    return 2 * n_mm + 2 * L * T * D


def open_engine(ane, wl, batch, tokens, *, accum=1, rank=0, world=1, local_rank=0, dp_id=None, ce_chunk=0, ce_cols=0):
    is_ref_arch = wl["arch"] == "reference"
    opts = ane.Options(tokens=tokens, batch=batch, arch=ane.ARCH_REFERENCE if is_ref_arch else ane.ARCH_LLAMA,
                       quirks=1 if is_ref_arch else 0, compute_dtype=ane.DTYPE_BF16,
                       accum_steps=accum, lr=3e-4, adam_beta1=0.9, adam_beta2=0.95, weight_decay=0.1, grad_clip=1.0,
                       seed=42, device=local_rank, rank=rank, world_size=world, dp_id=dp_id, ce_chunk_rows=ce_chunk, ce_chunk_cols=ce_cols,
                       **wl["cfg"])
    e = ane.open(opts)
    init_weights(e, ane, seed=1234, cfg=wl["cfg"])
    return e


def run_ours(args):
    import ane

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod

        dist = dist_mod
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))

    def new_dp_id():
        if dist is None:
            return None
        obj = [ane.dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0)
        return obj[0]

    def barrier():
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()
        ane._ffi.lib.ane_dev_sync()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_steps(engine, n):
        """Exactly n steps between a barrier + synchronize on both sides; device time, max over ranks."""
        barrier()
        engine.timer_begin()
        last = None
        for _ in range(n):
            last = engine.step()
        ms = engine.timer_end()
        barrier()
        return max_over_ranks(ms), last

    wl = WORKLOADS[args.workload]
    WORKLOAD, MICRO_BATCH = wl["cfg"], wl["batch"]
    if args.batch > 0:  # another micro-batch than the workload's own (the workload name then says so)
        wl = dict(wl, name=wl["name"].replace(f"micro-batch {MICRO_BATCH} per GPU", f"micro-batch {args.batch} per GPU"))
        MICRO_BATCH = args.batch
    flops_per_token = train_flops_per_token(WORKLOAD, wl["arch"])
    hbm, tf_burst, tf_sust, src = measured_peaks()
    tokens = zipf_tokens(N_STREAM_TOKENS, WORKLOAD["vocab"], seed=0)
    e = open_engine(ane, wl, MICRO_BATCH, tokens, rank=rank, world=world, local_rank=local_rank, dp_id=new_dp_id(),
                    ce_chunk=args.ce_chunk, ce_cols=args.ce_cols)
    T = WORKLOAD["seq"]
    tokens_per_step = MICRO_BATCH * T * world

    # ---- device-resident leg ("value"): `repeats` timed regions of exactly `steps` steps, median reported
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        e.step()
    launches0 = e.launch_count()
    region_ms, last = [], None
    t0 = time.perf_counter()
    for _ in range(max(1, args.repeats)):
        sampler.mark()
        ms, last = timed_steps(e, args.steps)
        sampler.window()
        region_ms.append(ms)
    wall_ms = (time.perf_counter() - t0) * 1e3 / max(1, args.repeats)
    launches = (e.launch_count() - launches0) // max(1, args.repeats)
    ms = float(np.median(region_ms))
    ms_per_step = ms / args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    repeats = {"n": len(region_ms), "ms_per_step_median": round(ms_per_step, 4),
               "ms_per_step_min": round(min(region_ms) / args.steps, 4),
               "ms_per_step_max": round(max(region_ms) / args.steps, 4)}

    # ---- end-to-end leg: host batches in, loss out, every step (clock sampling continues)
    rng = np.random.default_rng(7 + rank)
    pos = rng.integers(0, tokens.size - T - 1, size=(args.steps + 1, MICRO_BATCH))
    batches = []
    for s in range(args.steps + 1):
        inp = np.stack([tokens[p:p + T] for p in pos[s]])
        tgt = np.stack([tokens[p + 1:p + 1 + T] for p in pos[s]])
        batches.append((inp, tgt))
    e.step_tokens(*batches[-1])
    e2e_runs = []
    for _ in range(max(1, args.repeats)):
        barrier()
        sampler.mark()
        t0 = time.perf_counter()
        for s in range(args.steps):
            e.step_tokens(*batches[s])
        ane._ffi.lib.ane_dev_sync()
        e2e_runs.append(max_over_ranks(time.perf_counter() - t0))
        sampler.window()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    e2e_value = tokens_per_step * args.steps / float(np.median(e2e_runs))
    h2d = 2 * MICRO_BATCH * T * 2
    d2h = 8

    # ---- replicas must stay identical under data parallelism: checksums of two weight tensors per rank
    dp_check = None
    if dist is not None:
        import torch
        sums = [zlib.crc32(e.export_tensor(ane.T_WQ, 1).tobytes()), zlib.crc32(e.export_tensor(ane.T_EMBED, 0).tobytes())]
        mine = torch.tensor(sums + [0], dtype=torch.int64, device="cuda")
        loss_t = torch.tensor([float(last.loss)], dtype=torch.float64, device="cuda")
        all_sums = [torch.zeros_like(mine) for _ in range(world)]
        all_loss = [torch.zeros_like(loss_t) for _ in range(world)]
        dist.all_gather(all_sums, mine)
        dist.all_gather(all_loss, loss_t)
        same = all(bool(torch.equal(t, all_sums[0])) for t in all_sums)
        losses = [float(t.item()) for t in all_loss]
        dp_check = {"replicas_identical": same, "tensors": ["wq[1]", "embed"], "checksum": "crc32 of the fp32 bytes",
                    "loss_spread": round(max(losses) - min(losses), 5),
                    "note": "ranks train on different windows, so their last losses differ; weights must not"}

    # ---- dominant-kernel roofline: every GEMM launch timed with CUDA events over a profiled step
    # (three profiled steps, the median taken: one step's sum moves by several per cent with the clocks)
    prof = []
    for _ in range(3):
        e.profile_gemm(True)
        e.step()
        prof.append(e.profile_read())
        e.profile_gemm(False)
    gemm_ms, gemm_flops, gemm_launches = sorted(prof, key=lambda t: t[0])[1]
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    step_tflops = flops_per_token * tokens_per_step / world / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": round(achieved, 1), "peak": tf_burst, "unit": "TFLOP/s",
                "frac": round(achieved / tf_burst, 4), "traffic": GEMM_TRAFFIC["dram_bytes_per_step"],
                "traffic_source": GEMM_TRAFFIC["source"],
                "peak_source": f"bf16_tflops burst ({src}); a step is 8 ms of mixed kernels, not the seconds-long GEMM loop "
                               "of the sustained figure",
                "frac_of_sustained_peak": round(achieved / tf_sust, 4),
                "kernel": "gemm_tc_kernel (tcgen05 GEMM, all shapes of one step)", "gemm_launches_per_step": gemm_launches,
                "gemm_ms_per_step": round(gemm_ms, 3),
                "gemm_ms_per_step_profiled": [round(t[0], 3) for t in prof],
                "algorithmic_flops_per_step": gemm_flops,
                "step_tflops": round(step_tflops, 1),
                "step_frac_of_burst_peak": round(step_tflops / tf_burst, 4)}

    # ---- EvalLogits latency (the second half of the headline metric): one 256-token window per call,
    # full 32000 x 256 fp32 logits returned to the host in the reference's [vocab][seq] order.
    window = np.ascontiguousarray(tokens[:T])
    for _ in range(3):
        e.eval_logits(window)
    n_eval = 10
    t0 = time.perf_counter()
    for _ in range(n_eval):
        e.eval_logits(window)
    eval_ns = (time.perf_counter() - t0) / n_eval * 1e9
    logits_out = np.empty((1, WORKLOAD["vocab"], T), dtype=np.float32)
    e.eval_logits(window, out=logits_out)
    t0 = time.perf_counter()
    for _ in range(n_eval):
        e.eval_logits(window, out=logits_out)
    eval_reuse_ns = (time.perf_counter() - t0) / n_eval * 1e9
    pinned_out = ane.pinned_empty((1, WORKLOAD["vocab"], T))
    e.eval_logits(window, out=pinned_out)
    t0 = time.perf_counter()
    for _ in range(n_eval):
        e.eval_logits(window, out=pinned_out)
    eval_pinned_ns = (time.perf_counter() - t0) / n_eval * 1e9
    del pinned_out
    t0 = time.perf_counter()
    for _ in range(n_eval):
        e.eval_loss(window)
    eval_loss_ns = (time.perf_counter() - t0) / n_eval * 1e9
    eval_logits = {"ns_per_op": round(eval_ns), "ns_per_op_reused_output": round(eval_reuse_ns),
                   "ns_per_op_page_locked_output": round(eval_pinned_ns),
                   "eval_loss_ns_per_op": round(eval_loss_ns),
                   "d2h_bytes_per_op": WORKLOAD["vocab"] * T * 4,
                   "note": "host-visible latency of one EvalLogits call (batch 1): into a fresh array as the reference returns "
                           "one, into a reused array, and into page-locked memory of the caller (no staging copy); "
                           "EvalLoss keeps logits on the device"}

    # ---- extra legs (one GPU): the other configurations, each with its fraction of the step roofline
    extras = None
    if args.extras and world == 1 and args.workload == "110m":
        extras = {}
        nb = 64
        batch_tokens = np.ascontiguousarray(tokens[:nb * T])
        fwd_fl = fwd_flops_per_token(WORKLOAD, wl["arch"]) * nb * T
        e.eval_loss(batch_tokens)
        t0 = time.perf_counter()
        for _ in range(5):
            e.eval_loss(batch_tokens)
        dt = (time.perf_counter() - t0) / 5
        extras["eval_loss_batch64"] = {"ms_per_op": round(dt * 1e3, 3), "tok_per_s": round(nb * T / dt, 1),
                                       "frac_of_burst_peak": round(fwd_fl / dt / 1e12 / tf_burst, 4),
                                       "note": "64 windows of 256 tokens, fused device loss, host-visible"}
        e.eval_logits(batch_tokens, layout=1)
        t0 = time.perf_counter()
        for _ in range(3):
            e.eval_logits(batch_tokens, layout=1)
        dt = (time.perf_counter() - t0) / 3
        extras["eval_logits_batch64"] = {"ms_per_op": round(dt * 1e3, 3), "tok_per_s": round(nb * T / dt, 1),
                                         "d2h_bytes_per_op": nb * T * WORKLOAD["vocab"] * 4,
                                         "d2h_gb_per_s": round(nb * T * WORKLOAD["vocab"] * 4 / dt / 1e9, 1),
                                         "note": "host-visible, fp32 logits for 64 x seq tokens copied to the host: bound "
                                                 "by the 2.1 GB download, not by the device"}
        e.close()
        e = None
        for key in ("gqa1024", "reference"):
            w2 = WORKLOADS[key]
            toks2 = tokens
            e2 = open_engine(ane, w2, w2["batch"], toks2)
            for _ in range(3):
                e2.step()
            ms2, last2 = timed_steps(e2, 10)
            tps = w2["batch"] * w2["cfg"]["seq"]
            fl2 = train_flops_per_token(w2["cfg"], w2["arch"]) * tps
            extras[f"train_step_{key}"] = {"workload": w2["name"], "ms_per_step": round(ms2 / 10, 4),
                                           "tok_per_s": round(tps / (ms2 / 10 * 1e-3), 1),
                                           "step_frac_of_burst_peak": round(fl2 / (ms2 / 10 * 1e-3) / 1e12 / tf_burst, 4),
                                           "loss": round(float(last2.loss), 4)}
            e2.close()
        # KV-cached greedy decoding of the GQA variant: 32 sequences, 512-token prompts, 256 new tokens
        w2 = WORKLOADS["gqa1024"]
        e2 = open_engine(ane, w2, 32, tokens)
        prompts = np.ascontiguousarray(tokens[:32 * 512].reshape(32, 512))
        e2.decode_greedy(prompts[:, :64], 4)
        t0 = time.perf_counter()
        e2.decode_greedy(prompts, 256)
        dt = time.perf_counter() - t0
        # per decode step every weight (bf16) and the KV cache up to the current position are read once
        n_w = (train_flops_per_token(w2["cfg"], "llama") - 3.5 * 2 * 12 * 1024 * 768) / 6
        kvd = w2["cfg"]["dim"] // w2["cfg"]["n_heads"] * w2["cfg"]["n_kv_heads"]
        kv_bytes = sum(32 * (512 + i) * kvd * 2 * 2 * 12 for i in range(256))
        dec_bytes = 256 * n_w * 2 + kv_bytes
        extras["decode_greedy_gqa1024"] = {"batch": 32, "prompt": 512, "new_tokens": 256, "seconds": round(dt, 4),
                                           "generated_tok_per_s": round(32 * 256 / dt, 1),
                                           "hbm_frac_lower_bound": round(dec_bytes / dt / 1e9 / hbm, 4),
                                           "note": "prefill + 256 KV-cached greedy steps, host-visible; the fraction sets "
                                                   "weight + KV-cache bytes of the decode steps against the measured copy "
                                                   "bandwidth over the whole call (prefill included in the time)"}
        e2.close()
    if e is not None:
        e.close()

    # ---- configuration with a fixed global batch: 256 sequences per optimizer update on every N
    c4 = None
    if args.workload == "110m" and args.batch <= 0 and 256 % (MICRO_BATCH * world) == 0:
        accum = 256 // (MICRO_BATCH * world)
        e4 = open_engine(ane, wl, MICRO_BATCH, tokens, accum=accum, rank=rank, world=world, local_rank=local_rank,
                         dp_id=new_dp_id(), ce_chunk=args.ce_chunk, ce_cols=args.ce_cols)
        for _ in range(accum):          # one optimizer step of warm-up
            e4.step()
        n_opt = 3
        ms4, last4 = timed_steps(e4, n_opt * accum)
        e4.close()
        c4 = {"global_batch": 256, "accum_steps": accum, "micro_batch_per_gpu": MICRO_BATCH,
              "ms_per_optimizer_step": round(ms4 / n_opt, 4), "tok_per_s": round(256 * T * n_opt / (ms4 * 1e-3), 1),
              "optimizer_steps_timed": n_opt, "flushed_last": bool(last4.flushed), "scaling": "strong"}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload == "110m":
        cpu_baseline = cpu_reference_leg(steps=8, warmup=1)
    if rank == 0:
        line = {
            "metric": "train tok/s (110M, seq 256)", "value": round(value, 1), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl["name"],
                       "global_batch": MICRO_BATCH * world, "seq_len": T, "parallelism": f"dp{world}",
                       "l2_policy": "inputs larger than L2 (GBs of activations per step)"},
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "loss": round(float(last.loss), 4),
            "repeats": repeats, "wall_ms_per_step": round(wall_ms / args.steps, 4), "eval_logits": eval_logits,
        }
        if c4 is not None:
            line["c4"] = c4
        if dp_check is not None:
            line["dp_check"] = dp_check
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        if extras is not None:
            line["extras"] = extras
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    if dp_check is not None and not dp_check["replicas_identical"]:
        sys.exit(3)


def cpu_reference_leg(steps: int, warmup: int):
    """Times the CPU restatement of the reference step (oracle port) on the host cores: one sequence
    of 256 tokens through forward + backward + gradient accumulation per sample."""
    from oracle import oracle as O

    m = O.Model(dim=768, hidden=2048, heads=12, kv_heads=12, layers=12, vocab=32000, seq=256, arch=O.ARCH_L, quirks=0,
                accum_steps=1 << 30, lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1, grad_clip=1.0)
    O.init_weights(m, 1234)
    toks = zipf_tokens(4096, 32000, seed=0)
    for _ in range(warmup):
        m.accumulate(toks[:256].copy(), toks[1:257].copy())
    t0 = time.perf_counter()
    for s in range(steps):
        o = 257 * (s % 8)
        m.accumulate(toks[o:o + 256].copy(), toks[o + 1:o + 257].copy())
    dt = time.perf_counter() - t0
    cores = int(O.lib().orc_num_threads())
    m.close()
    return {"value": round(256 * steps / dt, 2), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{steps} sequence(s) of 256 tokens (1/32 of one GPU micro-batch), fwd+bwd+grad accumulation, "
                      f"{dt:.1f} s of CPU work"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 4))
    base = cpu_reference_leg(steps=steps, warmup=1 if args.warmup > 0 else 0)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": "train tok/s (110M, seq 256)", "value": base["value"], "unit": "tok/s",
        "n_gpus": world, "steps": steps, "warmup": 1 if args.warmup > 0 else 0,
        "ms_per_step": round(256 / base["value"] * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "110M Llama2-style train step on host cores (CPU restatement of the reference's Go step; "
                               "each step = 1 sequence of 256 tokens)", "global_batch": 1, "seq_len": 256,
                   "parallelism": "cpu"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


KERNEL_CASES = {
    # name: (M, N, K, a_mn, b_mn, out_mode)  -- shapes of the 110M step at micro-batch 32
    "classifier_fwd": (8192, 32000, 768, 0, 0, 0),   # logits = x_norm . Embed^T, bf16 out (524 MB written)
    "qkv_fwd": (8192, 2304, 768, 0, 0, 0),
    "w2_dx": (8192, 768, 4096, 0, 1, 1),
    "w13_dw": (4096, 768, 8192, 1, 1, 2),
    "wo_fwd": (8192, 768, 768, 0, 0, 1, 1),          # fp32 out + fp32 residual (x2 = x + att . Wo^T)
    "w2_fwd": (8192, 768, 2048, 0, 0, 1, 1),
    "wo_dx": (8192, 768, 768, 0, 1, 0),
    "w13_fwd_swiglu": (8192, 4096, 768, 0, 0, 3),    # h1|h3 interleaved in bf16 plus gate = silu(h1) * h3 [M, N/2]
    "w2_dx_plain": (8192, 2048, 768, 0, 1, 0),       # d gate = dOut . W2, bf16 out (the SwiGLU backward then a kernel of its own)
    "w2_dx_dswiglu": (8192, 2048, 768, 0, 1, 7),     # the same product with the SwiGLU backward in its epilogue
}


def run_kernel_case(args):
    """One GEMM shape of the step in isolation on seeded random operands (zeros would draw less power and run at
    higher clocks than the step does), for ncu captures and per-shape roofline numbers:
    python bench.py --kernel-case classifier_fwd --steps 3 --warmup 2"""
    import ctypes

    import ane
    from ane import _ffi

    lib = _ffi.lib
    M, N, K, a_mn, b_mn, out_mode = KERNEL_CASES[args.kernel_case][:6]
    with_res = len(KERNEL_CASES[args.kernel_case]) > 6
    c_bytes = M * N * (2 if out_mode == 0 else 4)
    if out_mode == 7:
        c_bytes = M * 2 * N * 2   # d h13 [M, 2N] bf16
    dA, dB, dC = lib.ane_dev_malloc(M * K * 2), lib.ane_dev_malloc(N * K * 2), lib.ane_dev_malloc(c_bytes)
    lib.ane_dev_memset(dC, 0, c_bytes)
    rng = np.random.Generator(np.random.PCG64(5))

    def fill_bf16(dst, n, scale):   # N(0, scale) in bf16, uploaded in pieces through an fp32 staging buffer
        piece = 1 << 24
        stage = lib.ane_dev_malloc(piece * 4)
        for o in range(0, n, piece):
            m = min(piece, n - o)
            a = (scale * rng.standard_normal(m, dtype=np.float32)).astype(np.float32)
            lib.ane_dev_h2d(stage, a.ctypes.data, m * 4)
            lib.ane_op_cast_f32_to_bf16(stage, dst + o * 2, m)
        lib.ane_dev_sync()
        lib.ane_dev_free(stage)

    fill_bf16(dA, M * K, 1.0)
    fill_bf16(dB, N * K, 0.02)
    g = _ffi.GemmArgs()
    g.struct_size = ctypes.sizeof(_ffi.GemmArgs)
    g.dtype = ane.DTYPE_BF16
    g.d_a, g.d_b, g.d_c = dA, dB, dC
    g.m, g.n, g.k = M, N, K
    g.lda = M if a_mn else K
    g.ldb = N if b_mn else K
    g.ldc = 2 * N if out_mode == 7 else N
    g.a_mn, g.b_mn, g.out_mode, g.alpha = a_mn, b_mn, out_mode, 1.0
    if out_mode == 7:
        dH = lib.ane_dev_malloc(M * 2 * N * 2)
        fill_bf16(dH, M * 2 * N, 1.0)
        g.d_aux, g.ldaux = dH, 2 * N
    if out_mode == 3:
        dH = lib.ane_dev_malloc(M * N)
        lib.ane_dev_memset(dH, 0, M * N)
        g.d_aux, g.ldaux = dH, N // 2
    if with_res:
        dR = lib.ane_dev_malloc(c_bytes)
        lib.ane_dev_memset(dR, 0, c_bytes)
        g.d_res1, g.ldres = dR, N
    for _ in range(args.warmup):
        assert lib.ane_op_gemm(ctypes.byref(g)) == 0, lib.ane_ops_last_error()
    lib.ane_dev_sync()
    lib.ane_timer_begin()
    for _ in range(args.steps):
        assert lib.ane_op_gemm(ctypes.byref(g)) == 0, lib.ane_ops_last_error()
    ms = ctypes.c_float(0)
    lib.ane_timer_end(ctypes.byref(ms))
    per = ms.value / args.steps
    _, tf_burst, _, src = measured_peaks()
    tflops = 2.0 * M * N * K / (per * 1e-3) / 1e12
    alg_bytes = (M * K + N * K) * 2 + c_bytes * (2 if (out_mode in (2, 7) or with_res) else 1) + (M * N if out_mode == 3 else 0)
    print(json.dumps({"kernel_case": args.kernel_case, "shape": [M, N, K], "us_per_launch": round(per * 1e3, 2),
                      "achieved_tflops": round(tflops, 1), "frac_of_burst_peak": round(tflops / tf_burst, 4),
                      "peak_source": src, "algorithmic_bytes": alg_bytes}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ce-chunk", type=int, default=0, help="token rows per classifier/CE chunk (0 = library default)")
    ap.add_argument("--ce-cols", type=int, default=0,
                    help="vocabulary columns per gradient block of the logit-free head (0 = library default)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="110m")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="skip the extra one-GPU legs (batch-64 evaluation, GQA seq-1024 step and decode, reference architecture)")
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU per step (0 = the workload's own)")
    ap.add_argument("--kernel-case", choices=sorted(KERNEL_CASES), default=None)
    args = ap.parse_args()
    if args.kernel_case:
        run_kernel_case(args)
        return
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
