"""Generates tests/golden/oracle_tiny.npz from the CPU oracle.

The reference ships no golden vectors for this path and cannot be built here (no Go toolchain),
so these vectors pin the oracle restatement against regressions and platform drift; they are not
outputs of the reference itself.  Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CFG = dict(dim=48, hidden=64, heads=4, layers=4, vocab=96, seq=16)


def run_case():
    out = {}
    for name, arch, quirks, extra in (("N", O.ARCH_N, 1, {}), ("L", O.ARCH_L, 0, {"kv_heads": 2})):
        m = O.Model(arch=arch, quirks=quirks, accum_steps=2, lr=3e-3, beta1=0.9, beta2=0.95, weight_decay=0.1,
                    grad_clip=1.0, **CFG, **extra)
        O.init_weights(m, 7, std=0.08)
        toks = O.zipf_tokens(4096, CFG["vocab"], 21)
        pos = O.drand48_positions(42, toks.size, CFG["seq"], 6)
        losses = []
        for p in pos:
            losses.append(m.step(toks[p:p + CFG["seq"]].copy(), toks[p + 1:p + 1 + CFG["seq"]].copy()))
        out[f"{name}_positions"] = np.array(pos, dtype=np.int64)
        out[f"{name}_losses"] = np.array(losses, dtype=np.float32)
        out[f"{name}_final"] = m.tap(O.TAP_FINAL).copy()
        out[f"{name}_wq0"] = m.tensor(O.T_WQ, 0).copy()
        out[f"{name}_embed_rows"] = m.tensor(O.T_EMBED).reshape(CFG["vocab"], CFG["dim"])[:4].copy()
        out[f"{name}_logits"] = m.eval_logits(toks[:CFG["seq"]].copy())[:8].copy()
        m.close()
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_tiny.npz")
    np.savez_compressed(path, **run_case())
    print("wrote", path, os.path.getsize(path), "bytes")
