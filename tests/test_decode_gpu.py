"""KV-cache greedy decoding (llama-style architecture, GQA) against full-recompute forwards.

fp32: every generated token equals the argmax of the oracle's full forward over the growing sequence
(argmax is an index path: bit-exact).  bf16: the cached path equals the engine's own full-recompute
EvalLogits argmax wherever the top-2 margin is clear."""
import numpy as np
import pytest

import ane
from oracle import oracle as O
from parity_utils import make_pair

pytestmark = pytest.mark.gpu


def test_decode_fp32_matches_oracle_full_recompute():
    cfg = dict(dim=64, hidden=96, heads=4, kv_heads=2, layers=3, vocab=256, seq=48)
    m, e = make_pair(ane, cfg, arch=O.ARCH_L, quirks=0, dtype=ane.DTYPE_F32, batch=3, std=0.3, debug_taps=False)
    prompts = O.zipf_tokens(3 * 20, cfg["vocab"], 8).reshape(3, 20)
    n_new = 12
    got = e.decode_greedy(prompts, n_new)
    for b in range(3):
        seq = list(prompts[b])
        for step in range(n_new):
            padded = np.zeros(cfg["seq"], dtype=np.uint16)
            padded[:len(seq)] = seq                      # causal: later positions do not matter
            logits = m.eval_logits(padded)               # [vocab, seq]
            want = int(O.lib().orc_argmax(np.ascontiguousarray(logits[:, len(seq) - 1]).ctypes.data_as(
                __import__("ctypes").POINTER(__import__("ctypes").c_float)), cfg["vocab"]))
            assert int(got[b, step]) == want, (b, step)
            seq.append(want)
    e.close()


def test_decode_bf16_matches_own_full_forward():
    cfg = dict(dim=256, hidden=512, heads=4, kv_heads=2, layers=3, vocab=2048, seq=128)
    _, e = make_pair(ane, cfg, arch=O.ARCH_L, quirks=0, dtype=ane.DTYPE_BF16, batch=4, std=0.08, debug_taps=False)
    prompts = O.zipf_tokens(4 * 64, cfg["vocab"], 9).reshape(4, 64)
    n_new = 24
    got = e.decode_greedy(prompts, n_new)
    agree = total = 0
    for b in range(4):
        full = np.zeros(cfg["seq"], dtype=np.uint16)
        full[:64] = prompts[b]
        full[64:64 + n_new] = got[b]
        logits = e.eval_logits(full)[0]                  # teacher-forced on the generated tokens
        for step in range(n_new):
            col = logits[:, 63 + step]
            top2 = np.sort(col)[-2:]
            if top2[1] - top2[0] > 0.05:                 # clear margin: bf16 noise cannot flip it
                total += 1
                agree += int(col.argmax() == got[b, step])
    assert total > 0 and agree == total
    with pytest.raises(ane.EngineError):
        e.decode_greedy(prompts, 100)                    # prompt_len + n_new > seq
    e.close()


def test_decode_bf16_gqa_full_size_batch_32_prompt_512():
    """The decode configuration at full size: 110M GQA model (12 query / 4 KV heads, 12 layers, vocab 32000, KV cache
    of 1024 positions), 32 sequences, 512-token prompts (prefill through the tcgen05 attention kernels, four 128-row
    tiles), then KV-cached greedy steps.  Checked against the engine's own full-recompute forward on four of the
    sequences: wherever the top-2 margin is clear the cached path picks the same token."""
    cfg = dict(dim=768, hidden=2048, heads=12, kv_heads=4, layers=12, vocab=32000, seq=1024)
    _, e = make_pair(ane, cfg, arch=O.ARCH_L, quirks=0, dtype=ane.DTYPE_BF16, batch=32, std=0.05, debug_taps=False)
    prompts = O.zipf_tokens(32 * 512, cfg["vocab"], 12).reshape(32, 512)
    n_new = 24
    got = e.decode_greedy(prompts, n_new)
    assert got.shape == (32, n_new) and got.max() < cfg["vocab"]
    agree = total = 0
    for b in (0, 7, 19, 31):
        full = np.zeros(cfg["seq"], dtype=np.uint16)
        full[:512] = prompts[b]
        full[512:512 + n_new] = got[b]
        logits = e.eval_logits(full)[0]                  # [vocab, seq], teacher-forced on the generated tokens
        for step in range(n_new):
            col = logits[:, 511 + step]
            top2 = np.sort(col)[-2:]
            if top2[1] - top2[0] > 0.05:
                total += 1
                agree += int(col.argmax() == got[b, step])
    print(f"decode agreement {agree}/{total} on clear margins")
    assert total >= 8 and agree == total
    e.close()


def test_decode_rejected_for_reference_arch():
    cfg = dict(dim=64, hidden=96, heads=4, layers=2, vocab=256, seq=32)
    _, e = make_pair(ane, cfg, arch=O.ARCH_N, quirks=1, dtype=ane.DTYPE_F32, batch=1, debug_taps=False)
    with pytest.raises(ane.EngineError):
        e.decode_greedy(np.zeros((1, 8), np.uint16), 4)
    e.close()


def _upload(lib, a):
    p = lib.ane_dev_malloc(a.nbytes)
    assert lib.ane_dev_h2d(p, a.ctypes.data, a.nbytes) == 0
    return p


def test_sampler_rows_match_oracle_serial_walk():
    """sampleFromLogits (ane/train_full.go:318-342) is an index path: the device's chunked double sums must
    land on the oracle's index for the same uniform draw (a different index needs the target within double
    rounding of a prefix boundary, which seeded draws do not hit)."""
    import ctypes
    from ane import _ffi
    lib = _ffi.lib
    rng = np.random.default_rng(11)
    rows, vocab = 16, 32000
    logits = (4.0 * rng.standard_normal((rows, vocab))).astype(np.float32)
    logits[3, :] = 0.25                       # flat row: every index equally likely
    logits[4, 100] = 60.0                     # one dominant logit
    d_logits = _upload(lib, logits)
    d_out = lib.ane_dev_malloc(4 * rows)
    fp = ctypes.POINTER(ctypes.c_float)
    for temp in (0.0, 0.7, 1.0, 1.8):
        for trial in range(3):
            u = rng.random(rows)
            if trial == 0:
                u[:3] = (0.0, 1.0 - 2.0 ** -53, 0.5)
            d_u = _upload(lib, u)
            assert lib.ane_op_sample_rows(d_logits, d_u, temp, d_out, rows, vocab) == 0, lib.ane_ops_last_error()
            got = np.zeros(rows, dtype=np.int32)
            assert lib.ane_dev_d2h(got.ctypes.data, d_out, got.nbytes) == 0
            for r in range(rows):
                want = O.lib().orc_sample(logits[r].ctypes.data_as(fp), vocab, temp, float(u[r]))
                assert int(got[r]) == want, (temp, trial, r)
            lib.ane_dev_free(d_u)
    lib.ane_dev_free(d_logits)
    lib.ane_dev_free(d_out)


def test_decode_sample_fp32_matches_oracle_full_recompute():
    import ctypes
    cfg = dict(dim=64, hidden=96, heads=4, kv_heads=2, layers=3, vocab=256, seq=48)
    m, e = make_pair(ane, cfg, arch=O.ARCH_L, quirks=0, dtype=ane.DTYPE_F32, batch=3, std=0.3, debug_taps=False)
    prompts = O.zipf_tokens(3 * 20, cfg["vocab"], 8).reshape(3, 20)
    n_new, temp = 10, 0.9
    u = np.random.default_rng(21).random((n_new, 3))
    got = e.decode_sample(prompts, n_new, temp, u)
    fp = ctypes.POINTER(ctypes.c_float)
    for b in range(3):
        seq = list(prompts[b])
        for step in range(n_new):
            padded = np.zeros(cfg["seq"], dtype=np.uint16)
            padded[:len(seq)] = seq
            col = np.ascontiguousarray(m.eval_logits(padded)[:, len(seq) - 1])
            want = O.lib().orc_sample(col.ctypes.data_as(fp), cfg["vocab"], temp, float(u[step, b]))
            if int(got[b, step]) != want:
                # fp32 GEMM summation order moves the logits by ~1e-6: accept a neighbour only when the draw sits
                # on that boundary
                w = np.exp((col.astype(np.float64) - col.max()) / temp)
                cum = np.cumsum(w) / w.sum()
                assert abs(cum[min(want, int(got[b, step]))] - u[step, b]) < 1e-5, (b, step)
            seq.append(int(got[b, step]))
    assert (e.decode_sample(prompts, n_new, 0.0, u) == e.decode_greedy(prompts, n_new)).all()
    with pytest.raises(ane.EngineError):
        e.decode_sample(prompts, n_new, temp, u[:, :2])
    e.close()
