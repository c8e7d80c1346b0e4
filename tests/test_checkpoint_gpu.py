"""Save / resume through the reference's checkpoint format against device-resident state: a run that is
saved in the middle of a gradient-accumulation window and resumed in a fresh engine continues like the
uninterrupted run (weights, Adam moments, pending gradients, counters and learning rate all travel)."""
import numpy as np
import pytest

import ane
from ane import checkpoint as C
from oracle import oracle as O
from parity_utils import make_pair, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("arch,quirks", [(O.ARCH_N, 1), (O.ARCH_L, 0)])
def test_resume_mid_accumulation_continues_the_same_trajectory(tmp_path, arch, quirks):
    cfg = dict(dim=64, hidden=96, heads=4, layers=4, vocab=256, seq=32)
    hyper = dict(lr=1e-3, adam_beta1=0.9, adam_beta2=0.95, weight_decay=0.1, grad_clip=1.0, loss_scale=256.0,
                 accum_steps=2)
    B, S = 2, cfg["seq"]
    toks = O.zipf_tokens(7 * B * (S + 1), cfg["vocab"], 3).reshape(7, B, S + 1)
    batches = [(np.ascontiguousarray(t[:, :-1]), np.ascontiguousarray(t[:, 1:])) for t in toks]

    _, full = make_pair(ane, cfg, arch=arch, quirks=quirks, dtype=ane.DTYPE_F32, batch=B, hyper=hyper, debug_taps=False)
    want = [full.step_tokens(i, t).loss for i, t in batches]

    _, first = make_pair(ane, cfg, arch=arch, quirks=quirks, dtype=ane.DTYPE_F32, batch=B, hyper=hyper, debug_taps=False)
    got = [first.step_tokens(i, t).loss for i, t in batches[:3]]         # one update + one pending micro-step
    first.set_lr(7e-4)
    st = first.state()
    assert st.pending_steps == 1 and st.adam_t == 1
    path = str(tmp_path / "run.ckpt")
    meta = C.save_checkpoint(first, path, C.TrainMeta(step=3, total_steps=7))
    assert meta.adam_t == 1 and meta.lr == pytest.approx(7e-4)
    first.close()

    _, second = make_pair(ane, cfg, arch=arch, quirks=quirks, dtype=ane.DTYPE_F32, batch=B, hyper=hyper, seed=99,
                          debug_taps=False)                               # different weights until the load
    back = C.load_checkpoint(second, path)
    assert (back.step, back.total_steps, back.adam_t) == (3, 7, 1)
    st2 = second.state()
    assert (st2.pending_steps, st2.adam_t, st2.cum_steps) == (1, 1, 3)
    assert second.lr() == pytest.approx(7e-4)
    second.set_lr(1e-3)                                                   # the uninterrupted run never changed it
    got += [second.step_tokens(i, t).loss for i, t in batches[3:]]
    # the weight-gradient GEMMs add their k-splits with atomics, so two runs agree to rounding, not bit for bit
    np.testing.assert_allclose(got, want, rtol=0, atol=2e-5)
    for tid in (ane.T_EMBED, ane.T_WQ, ane.T_W2):
        assert rel_l2(second.export_tensor(tid, 1), full.export_tensor(tid, 1)) < 1e-5
        assert rel_l2(second.export_tensor(tid, 1, ane.M), full.export_tensor(tid, 1, ane.M)) < 1e-4
    full.close()
    second.close()
