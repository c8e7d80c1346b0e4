"""GPU checks of the callers around the step: the training driver and evaluation harness on a real engine,
Open with a model path (llama2.c model file, else a checkpoint: ane/engine.go:250-257), and what
LoadCheckpoint does beyond copying tensors (sampler reseed, wall clock: ane/engine.go:559-560)."""
import struct

import numpy as np
import pytest

import ane
from ane import checkpoint as C
from ane import harness as H
from oracle import oracle as O
from parity_utils import make_pair, rel_l2

pytestmark = pytest.mark.gpu

CFG = dict(dim=64, hidden=96, heads=4, layers=3, vocab=256, seq=32)


def _options(cfg, **kw):
    return ane.Options(dim=cfg["dim"], hidden=cfg["hidden"], n_layers=cfg["layers"], n_heads=cfg["heads"],
                       n_kv_heads=cfg.get("kv_heads", cfg["heads"]), vocab=cfg["vocab"], seq=cfg["seq"], **kw)


@pytest.mark.parametrize("arch,quirks", [(O.ARCH_N, 1), (O.ARCH_L, 0)])
def test_training_driver_and_evaluation_harness_on_an_engine(arch, quirks):
    """harness.train for six counted steps (after its three warm-up steps) with the schedule's learning rates
    set before every step, then eval_loss / val_bpb over the validation windows against the oracle's
    window loss on the engine's own trained weights."""
    toks = O.zipf_tokens(4096, CFG["vocab"], 17)
    hyper = dict(lr=1e-3, adam_beta1=0.9, adam_beta2=0.95, weight_decay=0.1, grad_clip=1.0, accum_steps=2)
    m, e = make_pair(ane, CFG, arch=arch, quirks=quirks, dtype=ane.DTYPE_F32, batch=2, hyper=hyper, tokens=toks,
                     debug_taps=False, std=0.1)
    log = H.train(e, max_steps=6, peak_lr=1e-3)
    assert log.steps == 6 and log.tokens == 6 * 2 * CFG["seq"] and len(log.losses) == 6
    assert all(np.isfinite(l) for l in log.losses)
    st = e.state()
    assert st.cum_steps == 6 + H.WARMUP_STEPS and st.pending_steps == 0          # train() ends with a flush
    assert st.adam_t == 5                                                        # 9 micro-steps of 2: 4 updates + the final flush
    assert log.lrs[0] == pytest.approx(1e-6) and log.lrs[1] == pytest.approx(H.lr_schedule(1 / 6, 1e-3))
    assert e.lr() == pytest.approx(log.lrs[-1])
    # evaluation: the harness's windows over the last 600 tokens, fused device loss against the oracle on the
    # same (trained) weights
    for tid, layer, a in m.tensors(O.W):
        a[:] = e.export_tensor(tid, layer).reshape(a.shape)
    got = H.eval_loss(e, toks, eval_tokens=600)
    windows = H.eval_windows(toks, 600, CFG["seq"])
    assert len(windows) == 19                                                    # starts 0, 31, ..., 558
    tot, n = 0.0, 0
    for w in windows:
        s, k = m.eval_loss_window(np.ascontiguousarray(w))
        tot, n = tot + s, n + k
    assert got == pytest.approx(tot / n, abs=1e-4)
    assert H.val_bpb(got) == pytest.approx(got / np.log(2.0) / 3.7)
    # the reference's own (mis-indexed) walk over downloaded logits, reproduced from the oracle's logits
    ref_walk = H.eval_loss(e, toks, eval_tokens=600, reference_indexing=True)

    class OracleLogits:
        seq, vocab, opts = CFG["seq"], CFG["vocab"], e.opts

        def eval_logits(self, w, layout=0):
            return m.eval_logits(np.ascontiguousarray(w))[None]

    assert ref_walk == pytest.approx(H.eval_loss(OracleLogits(), toks, eval_tokens=600, reference_indexing=True), abs=1e-4)
    e.close()


def test_benchmarks_with_the_reference_metric_names_on_an_engine():
    """The three benchmarks of bench_test.go:75-158 through the harness twins on a real engine: metric names,
    consistency of tok/s with the step's own duration, val_bpb from val_loss."""
    toks = O.zipf_tokens(4096, CFG["vocab"], 19)
    hyper = dict(lr=1e-3, accum_steps=2)
    m, e = make_pair(ane, CFG, arch=O.ARCH_L, quirks=0, dtype=ane.DTYPE_F32, batch=2, hyper=hyper, tokens=toks,
                     debug_taps=False, std=0.1)
    b = H.benchmark_step(e, n=4)
    assert set(b) >= {"loss", "tok/s", "tok/s_processed", "step_ms", "ane_ms", "adam_ms", "ns/op"}
    assert np.isfinite(b["loss"]) and b["step_ms"] > 0 and 0 < b["ane_ms"] <= b["step_ms"] + 1e-6
    assert b["tok/s"] == pytest.approx(CFG["seq"] * 2 / (b["step_ms"] * 1e-3))
    assert b["tok/s_processed"] == pytest.approx(2 * CFG["seq"] / (b["step_ms"] * 1e-3))
    assert e.state().cum_steps == 7
    lg = H.benchmark_eval_logits(e, toks, n=3, seq=CFG["seq"])
    assert lg["ns/op"] > 0 and lg["tok/s"] == pytest.approx(CFG["seq"] / (lg["ns/op"] * 1e-9))
    ev = H.benchmark_eval_loss(e, toks, eval_tokens=600)
    assert ev["val_loss"] == pytest.approx(H.eval_loss(e, toks, eval_tokens=600), abs=1e-6)
    assert ev["val_bpb"] == pytest.approx(ev["val_loss"] / np.log(2.0) / 3.7)
    e.close()


def test_eval_logits_into_page_locked_memory_matches_the_staged_copy():
    """ane.pinned_empty gives page-locked memory; EvalLogits copies into it straight from the device and must
    return what the staged path (pageable array) returns, in both layouts and for several windows."""
    toks = O.zipf_tokens(4096, CFG["vocab"], 23)
    m, e = make_pair(ane, CFG, arch=O.ARCH_L, quirks=0, dtype=ane.DTYPE_F32, batch=2, hyper=dict(lr=1e-3), tokens=toks,
                     debug_taps=False, std=0.1)
    windows = np.ascontiguousarray(toks[:3 * CFG["seq"]])
    for layout in (0, 1):
        want = e.eval_logits(windows, layout=layout)
        out = ane.pinned_empty(want.shape)
        out[...] = -1.0
        got = e.eval_logits(windows, layout=layout, out=out)
        assert got is out
        np.testing.assert_array_equal(got, want)
    del out, got
    e.close()


def test_load_checkpoint_reseeds_the_sampler_and_keeps_the_wall_clock(tmp_path):
    toks = O.zipf_tokens(8192, CFG["vocab"], 5)
    hyper = dict(lr=1e-3, accum_steps=1, seed=7)
    _, first = make_pair(ane, CFG, arch=O.ARCH_N, quirks=1, dtype=ane.DTYPE_F32, batch=2, hyper=hyper, tokens=toks,
                         debug_taps=False)
    for _ in range(3):
        first.step()
    wall = first.state().cum_wall_ms
    path = str(tmp_path / "r.ckpt")
    C.save_checkpoint(first, path, C.TrainMeta(step=3))
    first.close()
    _, second = make_pair(ane, CFG, arch=O.ARCH_N, quirks=1, dtype=ane.DTYPE_F32, batch=2, hyper=hyper, tokens=toks,
                          debug_taps=False)
    C.load_checkpoint(second, path)
    second.step()
    # ane/engine.go:559: the resumed stream is drand48Seed(seed + meta.Step), not a replay of the first run
    want = O.drand48_positions(7 + 3, toks.size, CFG["seq"], 2)
    assert second.state().token_pos == want[1] + CFG["seq"]
    replay = O.drand48_positions(7, toks.size, CFG["seq"], 2)
    assert want[1] != replay[1]
    assert second.state().cum_wall_ms >= wall                                     # ane/engine.go:560
    second.close()


def test_open_with_a_model_path_reads_a_model_file_or_a_checkpoint(tmp_path):
    cfg = dict(CFG)
    rng = np.random.default_rng(2)
    L, V, D, Hd, H_ = cfg["layers"], cfg["vocab"], cfg["dim"], cfg["hidden"], cfg["heads"]
    parts = dict(embed=(V * D,), rms_att=(L, D), wq=(L, D * D), wk=(L, D * D), wv=(L, D * D), wo=(L, D * D),
                 rms_ffn=(L, D), w1=(L, Hd * D), w2=(L, D * Hd), w3=(L, Hd * D), rms_final=(D,))
    data = {k: (0.05 * rng.standard_normal(s)).astype(np.float32) for k, s in parts.items()}
    model = str(tmp_path / "model.bin")
    with open(model, "wb") as f:
        f.write(struct.pack("<7i", D, Hd, L, H_, H_, V, cfg["seq"]))
        for k in parts:
            data[k].tofile(f)
    e = ane.open(_options(cfg, arch=ane.ARCH_LLAMA, quirks=0, compute_dtype=ane.DTYPE_F32, batch=1, model_path=model))
    np.testing.assert_array_equal(e.export_tensor(ane.T_WK, 2), data["wk"][2])
    np.testing.assert_array_equal(e.export_tensor(ane.T_W3, 1), data["w3"][1])
    np.testing.assert_array_equal(e.export_tensor(ane.T_RMS_FINAL, 0), data["rms_final"])
    # the same weights saved as a checkpoint open again through the second branch of Open
    C.random_init(e, 4)
    ckpt = str(tmp_path / "init.ckpt")
    C.save_checkpoint(e, ckpt, C.TrainMeta(step=0, lr=3e-4))
    e2 = ane.open(_options(cfg, arch=ane.ARCH_LLAMA, quirks=0, compute_dtype=ane.DTYPE_F32, batch=1, model_path=ckpt))
    for tid in (ane.T_EMBED, ane.T_WQ, ane.T_W2, ane.T_W3):
        np.testing.assert_array_equal(e2.export_tensor(tid, 1 if tid != ane.T_EMBED else 0),
                                      e.export_tensor(tid, 1 if tid != ane.T_EMBED else 0))
    window = O.zipf_tokens(cfg["seq"], V, 3)
    assert rel_l2(e2.eval_logits(window), e.eval_logits(window)) < 1e-6
    e.close()
    e2.close()
    with pytest.raises(ane.EngineError, match="load model"):
        ane.open(_options(cfg, arch=ane.ARCH_LLAMA, compute_dtype=ane.DTYPE_F32, batch=1,
                          model_path=str(tmp_path / "missing.bin")))
    junk = tmp_path / "junk.bin"
    junk.write_bytes(b"\x01" * 64)
    with pytest.raises(ane.EngineError, match="load model"):
        ane.open(_options(cfg, arch=ane.ARCH_LLAMA, compute_dtype=ane.DTYPE_F32, batch=1, model_path=str(junk)))
