"""Shared helpers for the parity tests: build an oracle model and a GPU engine with identical
seeded weights and compare tensors in the reference's layouts."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    den = np.linalg.norm(b)
    if den == 0:
        return float(np.linalg.norm(a))
    return float(np.linalg.norm(a - b) / den)


def make_pair(ane, cfg: dict, *, arch: int, quirks: int, dtype: int, batch: int, seed: int = 0, std: float = 0.02,
              hyper: dict | None = None, debug_taps: bool = True, tokens=None, perturb_scalars: bool = False):
    """Returns (oracle_model, engine) holding identical weights."""
    hyper = dict(hyper or {})
    okw = dict(cfg)
    okw.update(arch=arch, quirks=quirks)
    for k_o, k_e in (("lr", "lr"), ("beta1", "adam_beta1"), ("beta2", "adam_beta2"), ("eps", "adam_eps"),
                     ("weight_decay", "weight_decay"), ("grad_clip", "grad_clip"), ("loss_scale", "loss_scale"),
                     ("accum_steps", "accum_steps")):
        if k_e in hyper:
            okw[k_o] = hyper[k_e]
    m = O.Model(**okw)
    O.init_weights(m, seed, std=std)
    if perturb_scalars and arch == O.ARCH_N:
        rng = np.random.default_rng(seed + 17)
        m.tensor(O.T_RESID_LAMBDAS)[:] = (1.0 + 0.1 * rng.standard_normal(cfg["layers"])).astype(np.float32)
        m.tensor(O.T_X0_LAMBDAS)[:] = (0.1 + 0.05 * rng.standard_normal(cfg["layers"])).astype(np.float32)
        m.tensor(O.T_SMEAR_LAMBDA)[:] = 0.2
        m.tensor(O.T_BACKOUT_LAMBDA)[:] = 0.15
    eo = ane.Options(dim=cfg["dim"], hidden=cfg["hidden"], n_layers=cfg["layers"], n_heads=cfg["heads"],
                     n_kv_heads=cfg.get("kv_heads", cfg["heads"]), vocab=cfg["vocab"], seq=cfg["seq"], batch=batch,
                     arch=arch, quirks=quirks, compute_dtype=dtype, debug_taps=debug_taps, tokens=tokens, **hyper)
    e = ane.open(eo)
    for tid, layer, a in m.tensors(O.W):
        e.import_tensor(tid, layer, a)
    return m, e


def oracle_batch_accumulate(m, inp: np.ndarray, tgt: np.ndarray, seq: int):
    """Feed a [B, seq] batch to the oracle one sequence at a time (the reference's Step is batch 1);
    returns the per-sequence losses."""
    inp = inp.reshape(-1, seq)
    tgt = tgt.reshape(-1, seq)
    return [m.accumulate(np.ascontiguousarray(inp[b]), np.ascontiguousarray(tgt[b])) for b in range(inp.shape[0])]


def compare_grads(m, e, report: list, which: int = O.G):
    worst = 0.0
    for tid, layer, g in m.tensors(which):
        ge = e.export_tensor(tid, layer, which)
        err = rel_l2(ge, g)
        report.append((O.TENSOR_NAMES[tid], layer, err, float(np.linalg.norm(g))))
        if np.linalg.norm(g) > 0:
            worst = max(worst, err)
    return worst
