"""CPU checks of the host-side callers and data formats around the device path: the evaluation windows
and learning-rate schedule of the reference's harness / experiment files, the fixed-budget training loop,
the V5 checkpoint + "SANE" trailer and the llama2.c model file (against an in-memory engine stand-in),
and the oracle's temperature sampler."""
import math
import os
import struct

import numpy as np
import pytest

from ane import checkpoint as C
from ane import engine as E
from ane import harness as H
from oracle import oracle as O


# ------------------------------------------------------------------ harness.go / experiment.go
def test_lr_schedule_matches_experiment_go():
    peak = 3e-4
    assert H.lr_schedule(0.0, peak) == 0.0
    assert H.lr_schedule(0.025, peak) == pytest.approx(1.5e-4)
    assert H.lr_schedule(0.05, peak) == pytest.approx(peak)                       # cos(0) = 1
    assert H.lr_schedule(0.525, peak) == pytest.approx(peak * (0.1 + 0.9 * 0.5))   # half-way down the cosine
    assert H.lr_schedule(1.0, peak) == pytest.approx(0.1 * peak)
    xs = [H.lr_schedule(p / 100, peak) for p in range(5, 101)]
    assert all(a >= b for a, b in zip(xs, xs[1:]))


def test_eval_windows_are_the_39_overlapping_windows_of_harness_go():
    tokens = np.arange(20_000, dtype=np.uint16)
    w = H.eval_windows(tokens)
    assert w.shape == (39, 256)                         # pos = 0, 255, ..., 9690 (pos + 256 < 10000)
    assert w[0, 0] == 10_000 and w[1, 0] == 10_255      # the last 10 000 tokens, stride seq - 1
    assert w[-1, -1] == 10_000 + 38 * 255 + 255
    with pytest.raises(ValueError):
        H.eval_windows(tokens[:10_000])                 # needs evalTokens + evalSeqLen tokens
    assert H.val_bpb(math.log(2.0) * 3.7) == pytest.approx(1.0)


def test_load_tokens_reads_little_endian_u16(tmp_path):
    p = tmp_path / "tok.bin"
    p.write_bytes(bytes([0x01, 0x00, 0xFF, 0x7C, 0x34, 0x12]))
    assert H.load_tokens(str(p)).tolist() == [1, 0x7CFF, 0x1234]
    p.write_bytes(b"\x00\x01\x02")
    with pytest.raises(ValueError):
        H.load_tokens(str(p))


class FakeEngine:
    """Holds tensors in host memory behind the Engine methods the host-side code uses."""

    def __init__(self, arch=E.ARCH_REFERENCE, layers=4, vocab=50, dim=8, hidden=12, heads=2, seq=16, batch=2):
        self.opts = E.Options(n_layers=layers, vocab=vocab, dim=dim, hidden=hidden, n_heads=heads, seq=seq, arch=arch,
                              batch=batch)
        self.seq = seq
        self._lr = 3e-4
        self._st = E.State()
        self.lrs, self.steps = [], 0
        d = C.dims_of(self)
        rng = np.random.default_rng(5)
        sizes = {E.T_WQ: dim * dim, E.T_WK: dim * dim, E.T_WV: dim * dim, E.T_WO: dim * dim, E.T_W1: hidden * dim,
                 E.T_W2: dim * hidden}
        self.t = {}
        for l in range(layers):
            per = dict(sizes)
            if arch == E.ARCH_LLAMA:
                per.update({E.T_W3: hidden * dim, E.T_RMS_ATT: dim, E.T_RMS_FFN: dim})
            elif C.is_ve_layer(l, d):
                per.update({E.T_VE_EMBED: vocab * dim, E.T_VE_GATE: heads * 12})
            for tid, n in per.items():
                for which in range(4):
                    self.t[(tid, l, which)] = rng.standard_normal(n).astype(np.float32)
        model = {E.T_EMBED: vocab * dim}
        if arch == E.ARCH_LLAMA:
            model[E.T_RMS_FINAL] = dim
        else:
            model.update({E.T_RESID_LAMBDAS: layers, E.T_X0_LAMBDAS: layers, E.T_SMEAR_GATE: dim * dim,
                          E.T_SMEAR_LAMBDA: 1, E.T_BACKOUT_LAMBDA: 1})
        for tid, n in model.items():
            for which in range(4):
                self.t[(tid, 0, which)] = rng.standard_normal(n).astype(np.float32)

    def _alive(self, what):
        pass

    def tensor_size(self, tid, layer=0):
        a = self.t.get((tid, layer, 0))
        return 0 if a is None else a.size

    def export_tensor(self, tid, layer=0, which=0):
        a = self.t.get((tid, layer, which))
        return None if a is None else a.copy()

    def import_tensor(self, tid, layer, arr, which=0):
        assert self.t[(tid, layer, which)].size == np.asarray(arr).size
        self.t[(tid, layer, which)] = np.asarray(arr, dtype=np.float32).copy()

    def lr(self):
        return self._lr

    def set_lr(self, lr):
        if lr <= 0:  # ane/engine.go:370-372, mirrored by the library
            raise E.EngineError(-1, "storiesane set lr: lr must be > 0")
        self._lr = float(np.float32(lr))
        self.lrs.append(lr)

    def reseed(self, seed):
        self.seed_now = seed

    def state(self):
        return self._st

    def load_state(self, st):
        self._st = st

    def step(self):
        self.steps += 1
        return E.StepResult(loss=10.0 / self.steps)

    def flush(self):
        return 0.0


def test_train_loop_spends_the_budget_after_three_warmup_steps():
    e = FakeEngine()
    now = [0.0]

    def clock():
        now[0] += 0.25          # every look at the clock costs a quarter second
        return now[0]

    log = H.train(e, budget_s=10.0, peak_lr=1e-3, clock=clock)
    assert e.steps == log.steps + H.WARMUP_STEPS
    assert 35 <= log.steps <= 40 and log.tokens == log.steps * 2 * 16
    assert e.lrs[:3] == [pytest.approx(1e-6)] * 3        # warm-up steps: the ramp's floor (SetLR refuses zero)
    assert max(log.lrs) <= 1e-3 and log.lrs[-1] < 0.2e-3 and log.lrs[0] == pytest.approx(0.5e-3)  # 0.25 s of 10 s
    assert log.losses == [10.0 / (i + 4) for i in range(log.steps)]
    by_steps = H.train(FakeEngine(), max_steps=20, peak_lr=1e-3)
    assert by_steps.steps == 20 and by_steps.lrs[1] == pytest.approx(1e-3)  # progress 1/20 = end of warm-up


# ------------------------------------------------------------------ ckpt.go / engine.go trailer
def test_benchmark_step_reports_the_reference_metric_names():
    """bench_test.go:75-119: three untimed steps, then n; loss / step_ms / ane_ms / adam_ms from the last result
    and tok/s by the reference's own formula (seq * AccumSteps / StepDuration)."""
    e = FakeEngine(seq=16, batch=2)
    real_step = e.step

    def step():
        r = real_step()
        r.step_duration, r.device_eval_duration, r.adam_duration = 0.004, 0.003, 0.0005
        return r

    e.step = step
    out = H.benchmark_step(e, n=5, accum_steps=8)
    assert e.steps == 8
    assert out["loss"] == pytest.approx(10.0 / 8)
    assert out["step_ms"] == pytest.approx(4.0) and out["ane_ms"] == pytest.approx(3.0) and out["adam_ms"] == pytest.approx(0.5)
    assert out["tok/s"] == pytest.approx(16 * 8 / 0.004)               # the reference's figure
    assert out["tok/s_processed"] == pytest.approx(2 * 16 / 0.004)     # tokens the step really handled
    assert out["ns/op"] > 0


def test_header_is_96_bytes_in_the_reference_field_order():
    d = C.Dims(layers=12, vocab=32000, dim=768, hidden=2048, heads=12, seq=256, arch=E.ARCH_REFERENCE)
    meta = C.TrainMeta(step=7, total_steps=100, lr=3e-4, loss=2.5, cum_compile=1.5, cum_train=20.25, cum_wall=30.5,
                       cum_steps=9, cum_batches=4, adam_t=3)
    raw = C.pack_header(5, meta, d)
    assert len(raw) == 96
    assert raw[:8] == bytes([0x54, 0x5A, 0x4C, 0x42, 5, 0, 0, 0])              # magic 0x424C5A54, version 5
    assert struct.unpack_from("<8i", raw, 8) == (7, 100, 12, 32000, 768, 2048, 12, 256)
    assert struct.unpack_from("<2f", raw, 40) == (np.float32(3e-4), 2.5)
    assert struct.unpack_from("<3d", raw, 48) == (1.5, 20.25, 30.5)
    assert struct.unpack_from("<6i", raw, 72) == (9, 4, 3, 0, 0, 0)
    ver, back = C.unpack_header(raw, d)
    assert ver == 5 and back.step == 7 and back.adam_t == 3 and back.cum_wall == 30.5
    with pytest.raises(ValueError, match="bad checkpoint header"):
        C.unpack_header(b"\0" * 96, d)
    with pytest.raises(ValueError, match="config mismatch"):
        C.unpack_header(raw, C.Dims(layers=6, vocab=32000, dim=768, hidden=2048, heads=12, seq=256, arch=0))
    with pytest.raises(ValueError, match="unexpected EOF"):
        C.unpack_header(raw[:50], d)


def test_checkpoint_size_matches_the_reference_formula():
    e = FakeEngine(layers=4, vocab=50, dim=8, hidden=12, heads=2)
    L, V, D, Hd, H_ = 4, 50, 8, 12, 2
    wq, wo, w1, w2 = D * D, D * D, Hd * D, D * Hd
    layer_w = L * (wq * 3 + wo + w1 + w2)
    layer_o = L * (wq * 6 + wo * 2 + w1 * 2 + w2 * 2)
    n_ve = sum(1 for l in range(L) if l % 2 == (L - 1) % 2)
    layer_w += n_ve * (V * D + H_ * 12)
    layer_o += n_ve * 2 * (V * D + H_ * 12)
    model = V * D * 3 + L * 3 + L * 3 + D * D * 3 + 3 + 3
    assert C.checkpoint_size(e) == 96 + 4 * (layer_w + layer_o + model)       # storiesCheckpointSize


@pytest.mark.parametrize("arch", [E.ARCH_REFERENCE, E.ARCH_LLAMA])
def test_checkpoint_round_trip_restores_weights_moments_gradients_and_counters(tmp_path, arch):
    src = FakeEngine(arch=arch)
    src._st = E.State(token_pos=123456789012, last_loss=2.25, cum_train_ms=11.5, cum_wall_ms=12.5, cum_steps=6,
                      cum_batches=3, adam_t=3, pending_steps=1)
    src._lr = float(np.float32(1.25e-4))
    path = str(tmp_path / "sub" / "ckpt.bin")
    meta = C.save_checkpoint(src, path, C.TrainMeta(step=6, total_steps=50))
    assert not os.path.exists(path + ".tmp")
    size = os.path.getsize(path)
    n_grad = sum(a.size for (tid, l, which), a in src.t.items() if which == E.G)
    assert size == C.checkpoint_size(src) + 4 + 16 + 4 * n_grad
    with open(path, "rb") as f:
        f.seek(C.checkpoint_size(src))
        assert f.read(4) == b"SANE"
        assert struct.unpack("<IQI", f.read(16)) == (2, 123456789012, 1)
    dst = FakeEngine(arch=arch)
    for k in dst.t:
        dst.t[k] = np.zeros_like(dst.t[k])
    got = C.load_checkpoint(dst, path)
    assert (got.step, got.total_steps, got.adam_t, got.cum_steps) == (6, 50, 3, 6) and got.lr == meta.lr
    assert dst.lr() == src.lr()
    st = dst.state()
    assert (st.token_pos, st.pending_steps, st.adam_t, st.cum_batches, st.last_loss) == (123456789012, 1, 3, 3, 2.25)
    for k, a in src.t.items():
        np.testing.assert_array_equal(dst.t[k], a, err_msg=str(k))
    # the first tensor after the header is layer 0's Wq, the last before the trailer the final model tensor's v
    with open(path, "rb") as f:
        f.seek(96)
        np.testing.assert_array_equal(np.fromfile(f, "<f4", 64), src.t[(E.T_WQ, 0, E.W)])
    # without a trailer: weights load, pending gradients are cleared, the position restarts at 0
    cut = str(tmp_path / "cut.bin")
    with open(path, "rb") as f, open(cut, "wb") as g:
        g.write(f.read(C.checkpoint_size(src)))
    C.load_checkpoint(dst, cut)
    assert dst.state().pending_steps == 0 and dst.state().token_pos == 0
    assert all(not dst.t[k].any() for k in dst.t if k[2] == E.G)
    # truncated inside the tensors
    with open(cut, "r+b") as g:
        g.truncate(200)
    with pytest.raises(ValueError, match="unexpected EOF"):
        C.load_checkpoint(dst, cut)
    # a file of the other architecture is refused
    other = FakeEngine(arch=E.ARCH_LLAMA if arch == E.ARCH_REFERENCE else E.ARCH_REFERENCE)
    with pytest.raises(ValueError, match="config mismatch"):
        C.load_checkpoint(other, path)


@pytest.mark.parametrize("arch", [E.ARCH_REFERENCE, E.ARCH_LLAMA])
def test_llama2c_model_file_import(tmp_path, arch):
    e = FakeEngine(arch=arch)
    L, V, D, Hd, H_ = 4, 50, 8, 12, 2
    rng = np.random.default_rng(9)
    parts = dict(embed=(V * D,), rms_att=(L, D), wq=(L, D * D), wk=(L, D * D), wv=(L, D * D), wo=(L, D * D), rms_ffn=(L, D),
                 w1=(L, Hd * D), w2=(L, D * Hd), w3=(L, Hd * D), rms_final=(D,))
    data = {k: rng.standard_normal(s).astype(np.float32) for k, s in parts.items()}
    path = str(tmp_path / "m.bin")
    with open(path, "wb") as f:
        f.write(struct.pack("<7i", D, Hd, L, H_, H_, V, 16))
        for k in parts:
            data[k].tofile(f)
        np.zeros(2 * 16 * (D // H_) // 2, np.float32).tofile(f)      # rotary tables follow in llama2.c files; unread
    before_w3 = {k: v.copy() for k, v in e.t.items()}
    cfg = C.load_pretrained(e, path)
    assert cfg["shared_classifier"] and cfg["n_layers"] == L
    np.testing.assert_array_equal(e.t[(E.T_EMBED, 0, 0)], data["embed"])
    for l in range(L):
        np.testing.assert_array_equal(e.t[(E.T_WK, l, 0)], data["wk"][l])
        np.testing.assert_array_equal(e.t[(E.T_W2, l, 0)], data["w2"][l])
        if arch == E.ARCH_LLAMA:
            np.testing.assert_array_equal(e.t[(E.T_W3, l, 0)], data["w3"][l])
            np.testing.assert_array_equal(e.t[(E.T_RMS_FFN, l, 0)], data["rms_ffn"][l])
    if arch == E.ARCH_LLAMA:
        np.testing.assert_array_equal(e.t[(E.T_RMS_FINAL, 0, 0)], data["rms_final"])
    else:  # norm weights and W3 are skipped; the scalars of the reference model are untouched
        np.testing.assert_array_equal(e.t[(E.T_RESID_LAMBDAS, 0, 0)], before_w3[(E.T_RESID_LAMBDAS, 0, 0)])
    with open(path, "r+b") as f:
        f.write(struct.pack("<i", D + 1))
    with pytest.raises(ValueError, match="config mismatch"):
        C.load_pretrained(e, path)


def test_load_checkpoint_restarts_the_sampler_at_seed_plus_step(tmp_path):
    src = FakeEngine()
    src.opts.seed = 7
    path = str(tmp_path / "c.bin")
    C.save_checkpoint(src, path, C.TrainMeta(step=11))
    dst = FakeEngine()
    dst.opts.seed = 7
    C.load_checkpoint(dst, path)
    assert dst.seed_now == 7 + 11                         # ane/engine.go:559: drand48Seed(seed + meta.Step)
    dst.opts.seed = 0
    C.load_checkpoint(dst, path)
    assert dst.seed_now == 42 + 11                        # Open's default seed (ane/engine.go:200-202)


def test_open_style_load_takes_weights_and_moments_only(tmp_path):
    src = FakeEngine()
    src._st = E.State(token_pos=99, cum_steps=6, adam_t=3, pending_steps=1)
    path = str(tmp_path / "c.bin")
    C.save_checkpoint(src, path, C.TrainMeta(step=6))
    dst = FakeEngine()
    grads_before = {k: v.copy() for k, v in dst.t.items() if k[2] == E.G}
    C.load_weights_and_moments(dst, path)                 # what ane.Open does with a checkpoint path
    for k, a in src.t.items():
        if k[2] != E.G:
            np.testing.assert_array_equal(dst.t[k], a, err_msg=str(k))
    for k, a in grads_before.items():
        np.testing.assert_array_equal(dst.t[k], a)
    assert dst.state().token_pos == 0 and dst.state().adam_t == 0 and dst.lrs == []


def test_random_init_follows_the_distributions_of_the_reference():
    e = FakeEngine(layers=4, vocab=400, dim=32, hidden=48, heads=2)
    C.random_init(e, 3)
    s = math.sqrt(3.0) / math.sqrt(32)
    wq = e.t[(E.T_WQ, 1, 0)]
    assert abs(wq).max() <= s and abs(wq).max() > 0.9 * s and abs(float(wq.mean())) < 0.05 * s
    assert not e.t[(E.T_WO, 0, 0)].any() and not e.t[(E.T_W2, 3, 0)].any()     # output projections start at zero
    emb = e.t[(E.T_EMBED, 0, 0)]
    assert 0.95 < float(emb.std()) < 1.05
    np.testing.assert_array_equal(e.t[(E.T_RESID_LAMBDAS, 0, 0)], np.ones(4, np.float32))
    np.testing.assert_array_equal(e.t[(E.T_X0_LAMBDAS, 0, 0)], np.full(4, 0.1, np.float32))
    assert e.t[(E.T_SMEAR_LAMBDA, 0, 0)][0] == np.float32(0.01) and e.t[(E.T_BACKOUT_LAMBDA, 0, 0)][0] == np.float32(0.01)
    gate = e.t[(E.T_VE_GATE, 3, 0)]
    assert gate.min() >= 0 and gate.max() < 0.02
    again = FakeEngine(layers=4, vocab=400, dim=32, hidden=48, heads=2)
    C.random_init(again, 3)
    np.testing.assert_array_equal(again.t[(E.T_WQ, 1, 0)], wq)                   # seeded
    lm = FakeEngine(arch=E.ARCH_LLAMA, layers=2, vocab=400, dim=32, hidden=48, heads=2)
    C.random_init(lm, 1)
    assert 0.018 < float(lm.t[(E.T_W3, 1, 0)].std()) < 0.022


def test_eval_loss_with_the_reference_indexing():
    """harness.go:58-84 slices the [vocab][seq] logits as [seq][vocab]; the switch reproduces that walk."""
    seq, vocab = 16, 50

    class LogitsEngine:
        def __init__(self):
            self.seq, self.vocab = seq, vocab
            self.opts = E.Options(seq=seq, vocab=vocab, batch=1)

        def eval_logits(self, w, layout=0):
            rng = np.random.default_rng(int(w[0]))
            return rng.standard_normal((1, vocab, seq)).astype(np.float32)

    tokens = (np.arange(200) % vocab).astype(np.uint16)
    got = H.eval_loss(LogitsEngine(), tokens, eval_tokens=100, reference_indexing=True)
    total, n = 0.0, 0
    for w in H.eval_windows(tokens, 100, seq):
        flat = LogitsEngine().eval_logits(w).reshape(-1).astype(np.float64)
        for t in range(seq - 1):                                                  # the reference's loop, literally
            row = flat[t * vocab:(t + 1) * vocab]
            mx = 5e-324
            for v in row:
                mx = max(mx, v)
            total += math.log(sum(math.exp(v - mx) for v in row)) - (row[int(w[t + 1])] - mx)
            n += 1
    assert got == pytest.approx(total / n, rel=1e-12)


# ------------------------------------------------------------------ sampleFromLogits
def test_oracle_sampler_follows_the_serial_walk():
    import ctypes
    rng = np.random.default_rng(3)
    logits = (3.0 * rng.standard_normal(1000)).astype(np.float32)
    fp = logits.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
    lib = O.lib()
    assert lib.orc_sample(fp, 1000, 0.0, 0.3) == int(np.argmax(logits)) == lib.orc_argmax(fp, 1000)
    for temp in (0.5, 1.0, 2.0):
        w = np.exp((logits.astype(np.float64) - float(logits.max())) * float(np.float32(1) / np.float32(temp)))
        cum = np.cumsum(w)                                  # numpy's cumsum is the same serial double sum
        for u in (0.0, 1e-9, 0.25, 0.5, 0.999999, 1.0 - 2 ** -53):
            want = int(np.searchsorted(cum, u * cum[-1], side="left"))
            assert lib.orc_sample(fp, 1000, temp, u) == min(want, 999), (temp, u)
    counts = np.bincount([lib.orc_sample(fp, 1000, 1.0, float(u)) for u in rng.random(4000)], minlength=1000)
    p = np.exp(logits.astype(np.float64) - logits.max())
    p /= p.sum()
    top = np.argsort(p)[-5:]
    assert np.all(np.abs(counts[top] / 4000 - p[top]) < 0.03)
