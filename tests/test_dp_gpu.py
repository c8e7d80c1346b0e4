"""Data-parallel equivalence on real GPUs (needs >= 2 devices; skipped otherwise): two ranks with
micro-batch B, NCCL gradient all-reduce overlapped with backward, must end at the same weights as
one rank with micro-batch 2B on the same drand48 sample stream.  Ranks leave only between steps,
with nothing in flight."""
import multiprocessing as mp
import os
import sys

import numpy as np
import pytest

import ane
from oracle import oracle as O

pytestmark = pytest.mark.gpu

CFG = dict(dim=128, hidden=256, n_layers=3, n_heads=4, n_kv_heads=2, vocab=512, seq=64)
HYPER = dict(lr=1e-3, adam_beta1=0.9, adam_beta2=0.95, weight_decay=0.1, grad_clip=1.0, accum_steps=1, seed=42)
STEPS, B = 3, 2
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weights(seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    D, Hd, V, H, KV = CFG["dim"], CFG["hidden"], CFG["vocab"], CFG["n_heads"], CFG["n_kv_heads"]
    hd = D // H
    w = {(ane.T_EMBED, 0): 0.05 * rng.standard_normal(V * D)}
    for layer in range(CFG["n_layers"]):
        for tid, n in ((ane.T_WQ, D * D), (ane.T_WK, KV * hd * D), (ane.T_WV, KV * hd * D), (ane.T_WO, D * D),
                       (ane.T_W1, Hd * D), (ane.T_W2, D * Hd), (ane.T_W3, Hd * D)):
            w[(tid, layer)] = 0.05 * rng.standard_normal(n)
    return {k: v.astype(np.float32) for k, v in w.items()}


def _run(rank, world, batch, dp_id, tokens, dtype, out_path, accum=1):
    sys.path.insert(0, os.path.join(ROOT, "autoresearch-go-ane_b200"))
    import ane as A

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    e = A.open(A.Options(tokens=tokens, batch=batch, arch=A.ARCH_LLAMA, quirks=0, compute_dtype=dtype, device=rank,
                         rank=rank, world_size=world, dp_id=dp_id, **CFG, **dict(HYPER, accum_steps=accum)))
    for (tid, layer), v in _weights(3).items():
        e.import_tensor(tid, layer, v)
    losses = [e.step().loss for _ in range(STEPS * accum)]
    np.savez(out_path, losses=np.array(losses), wq=e.export_tensor(A.T_WQ, 1), embed=e.export_tensor(A.T_EMBED, 0),
             w2=e.export_tensor(A.T_W2, 2),
             # Adam moments of a layer matrix: each rank updates only its slice; the export gathers them (collective)
             m_w1=e.export_tensor(A.T_W1, 0, A.M), v_wq=e.export_tensor(A.T_WQ, 2, A.V))
    e.close()


def _join_or_kill(procs, timeout=300):
    """A child that does not finish in time is ended here (terminate, then kill), so that it cannot keep a GPU
    after the test has failed."""
    codes = []
    for p in procs:
        p.join(timeout=timeout)
        if p.is_alive():
            p.terminate()
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
            codes.append("timeout")
        else:
            codes.append(p.exitcode)
    assert codes == [0] * len(procs), codes


@pytest.mark.parametrize("dtype,accum", [(ane.DTYPE_F32, 1), (ane.DTYPE_BF16, 1), (ane.DTYPE_F32, 2)])
def test_two_gpu_data_parallel_matches_single_gpu(tmp_path, dtype, accum):
    if ane._ffi.lib.ane_device_count() < 2:
        pytest.skip("needs two GPUs")
    tokens = O.zipf_tokens(1 << 14, CFG["vocab"], 4)
    ctx = mp.get_context("spawn")
    dp_id = ane.dp_unique_id()
    procs = [ctx.Process(target=_run, args=(r, 2, B, dp_id, tokens, dtype, str(tmp_path / f"r{r}.npz"), accum)) for r in range(2)]
    for p in procs:
        p.start()
    _join_or_kill(procs)
    single = ctx.Process(target=_run, args=(0, 1, 2 * B, None, tokens, dtype, str(tmp_path / "single.npz"), accum))
    single.start()
    _join_or_kill([single])
    r0, r1, s = (np.load(tmp_path / f) for f in ("r0.npz", "r1.npz", "single.npz"))
    tol = 2e-5 if dtype == ane.DTYPE_F32 else 2e-3
    np.testing.assert_allclose((r0["losses"] + r1["losses"]) / 2, s["losses"], atol=1e-3 if dtype == ane.DTYPE_BF16 else 1e-5)
    for k in ("wq", "embed", "w2", "m_w1", "v_wq"):
        np.testing.assert_array_equal(r0[k], r1[k])  # replicas stay identical
        err = np.linalg.norm(r0[k] - s[k]) / np.linalg.norm(s[k])
        # (bf16: the first moment is a few gradients old, so it carries their rounding undamped)
        assert err < (3 * tol if k in ("m_w1", "v_wq") and dtype == ane.DTYPE_BF16 else tol), (k, err)
