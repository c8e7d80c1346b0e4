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


def test_decode_rejected_for_reference_arch():
    cfg = dict(dim=64, hidden=96, heads=4, layers=2, vocab=256, seq=32)
    _, e = make_pair(ane, cfg, arch=O.ARCH_N, quirks=1, dtype=ane.DTYPE_F32, batch=1, debug_taps=False)
    with pytest.raises(ane.EngineError):
        e.decode_greedy(np.zeros((1, 8), np.uint16), 4)
    e.close()
