"""CPU tests of the oracle restatement (no GPU): integer paths against an independent big-int
restatement, finite-difference checks of the exact-gradient mode, invariants, and the committed
golden vectors."""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "oracle_tiny.npz")


def test_drand48_matches_bigint_lcg():
    # ane/engine.go:873-880: X' = (0x5DEECE66D*X + 0xB) mod 2^48, seed ((s & 0xffffffff) << 16) | 0x330E
    L = O.lib()
    for seed in (42, 0, 1, 2**31 + 5, -7):
        x = ((seed & 0xFFFFFFFF) << 16) | 0x330E
        assert L.orc_drand48_seed(seed) == x
        st = ctypes.c_uint64(x)
        n_tokens, seq = 1_000_003, 256
        limit = n_tokens - seq - 1
        for _ in range(50):
            x = (0x5DEECE66D * x + 0xB) & ((1 << 48) - 1)
            want = min(int((x / float(1 << 48)) * limit), limit - 1)
            got = L.orc_sample_pos(ctypes.byref(st), n_tokens, seq)
            assert got == want
            assert st.value == x


def test_sampler_short_stream():
    L = O.lib()
    st = ctypes.c_uint64(L.orc_drand48_seed(42))
    assert L.orc_sample_pos(ctypes.byref(st), 258, 256) == 0  # limit = 1 -> only position 0


def test_argmax_first_strict_maximum():
    L = O.lib()
    v = np.array([1.0, 5.0, 5.0, -2.0, 5.0], dtype=np.float32)
    assert L.orc_argmax(v.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), v.size) == 1


def test_embed_out_of_range_token_is_zero_row():
    m = O.Model(dim=16, hidden=16, heads=2, layers=2, vocab=32, seq=8, arch=O.ARCH_L)
    O.init_weights(m, 3, std=0.2)
    toks = np.array([1, 2, 40000, 4, 5, 6, 7, 3], dtype=np.uint16)
    tgt = np.array([2, 3, 4, 5, 65535, 7, 3, 1], dtype=np.uint16)
    loss = m.accumulate(toks, tgt)
    assert np.isfinite(loss)
    x = m.tap(O.TAP_X, 0)
    assert np.all(x[:, 2] == 0.0)           # ane/stories/cpu.go:60-65
    dl = m.tap(O.TAP_DLOGITS)
    assert np.all(dl[:, 4] == 0.0)          # ane/stories/cpu.go:253-258
    assert not np.all(dl[:, 3] == 0.0)


def test_softmax_rows_sum_to_one_and_causal():
    rng = np.random.default_rng(0)
    H, hd, T = 2, 8, 16
    q, k, v = (rng.standard_normal((H * hd, T)).astype(np.float32) for _ in range(3))
    out = np.empty_like(q)
    fp = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
    O.lib().orc_attention(fp(out), fp(q), fp(k), fp(v), H, H, hd, T)
    # position 0 attends only to itself
    np.testing.assert_allclose(out[:, 0], v[:, 0], rtol=1e-6)
    # changing a future key/value must not change earlier outputs
    k2, v2 = k.copy(), v.copy()
    k2[:, 10:] += 1.0
    v2[:, 10:] -= 2.0
    out2 = np.empty_like(q)
    O.lib().orc_attention(fp(out2), fp(q), fp(k2), fp(v2), H, H, hd, T)
    np.testing.assert_array_equal(out[:, :10], out2[:, :10])


def _directional_fd(arch, **kw):
    cfg = dict(dim=32, hidden=48, heads=4, kv_heads=(2 if arch == O.ARCH_L else 4), layers=4, vocab=64, seq=12,
               arch=arch, quirks=0, loss_scale=1.0, accum_steps=1000, grad_clip=0.0)
    cfg.update(kw)
    m = O.Model(**cfg)
    O.init_weights(m, 1, std=0.3)
    for tid in (O.T_SMEAR_LAMBDA, O.T_BACKOUT_LAMBDA):
        a = m.tensor(tid)
        if a is not None:
            a[:] = 0.3
    a = m.tensor(O.T_X0_LAMBDAS)
    if a is not None:
        a[:] = np.linspace(0.1, 0.4, a.size)
    a = m.tensor(O.T_RESID_LAMBDAS)
    if a is not None:
        a[:] = np.linspace(0.8, 1.2, a.size)
    for tid, layer, a in m.tensors():
        if tid in (O.T_RMS_ATT, O.T_RMS_FFN, O.T_RMS_FINAL):
            a[:] = 1 + 0.2 * np.random.default_rng(layer + tid).standard_normal(a.size)
        if tid == O.T_VE_GATE:
            a[:] = 0.5 * np.random.default_rng(layer).standard_normal(a.size)
    toks = O.zipf_tokens(13, 64, 3)
    inp, tgt = toks[:12].copy(), toks[1:13].copy()
    m.accumulate(inp, tgt)
    rng = np.random.default_rng(0)
    worst = 0.0
    for tid, layer, w in m.tensors(O.W):
        g = m.tensor(tid, layer, O.G).copy()
        d = rng.choice([-1.0, 1.0], size=w.size).astype(np.float32)
        if tid in (O.T_EMBED, O.T_VE_EMBED):
            mask = np.zeros((cfg["vocab"], cfg["dim"]), np.float32)
            mask[np.unique(np.concatenate([inp, tgt]))] = 1
            d *= mask.ravel()
        old = w.copy()
        nums = []
        for h in (2e-3, 1e-3):
            w[:] = old + h * d
            lp = m.loss_only(inp, tgt)
            w[:] = old - h * d
            lm = m.loss_only(inp, tgt)
            nums.append((lp - lm) / (2 * h))
        w[:] = old
        num = (4 * nums[1] - nums[0]) / 3  # Richardson
        ana = float(np.dot(g.astype(np.float64), d))
        err = abs(num - ana) / max(1e-2, abs(num) + abs(ana))
        worst = max(worst, err)
        assert err < 2e-2, (O.TENSOR_NAMES[tid], layer, num, ana)
    return worst


def test_exact_gradients_reference_arch_quirks_off():
    _directional_fd(O.ARCH_N)


def test_exact_gradients_llama_arch_gqa():
    _directional_fd(O.ARCH_L)


def test_llama_arch_matches_torch_autograd_fp64():
    """An independent statement of the llama-style network in torch (fp64, autograd): weighted RMSNorm
    (eps 1e-5), rotation of interleaved pairs, causal GQA attention, SwiGLU, tied classifier, mean
    cross-entropy over the valid targets.  Loss and every parameter gradient of the oracle must agree
    with it; one target lies outside the vocabulary."""
    import torch

    D, Hd, H, KV, L, V, T = 32, 48, 4, 2, 3, 64, 12
    hd = D // H
    m = O.Model(dim=D, hidden=Hd, heads=H, kv_heads=KV, layers=L, vocab=V, seq=T, arch=O.ARCH_L, quirks=0,
                loss_scale=1.0, accum_steps=1000, grad_clip=0.0)
    O.init_weights(m, 1, std=0.3)
    for tid, layer, a in m.tensors():
        if tid in (O.T_RMS_ATT, O.T_RMS_FFN, O.T_RMS_FINAL):
            a[:] = 1 + 0.2 * np.random.default_rng(layer + tid).standard_normal(a.size)
    toks = O.zipf_tokens(T + 1, V, 3)
    inp, tgt = toks[:T].copy(), toks[1:T + 1].copy()
    tgt[4] = 65535
    loss = m.accumulate(inp, tgt)
    P = {(tid, layer): torch.tensor(a.astype(np.float64), requires_grad=True) for tid, layer, a in m.tensors(O.W)}
    theta = float(m.cfg.rope_theta)

    def rms(x, w):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w

    def rope(x, nh):
        x = x.view(T, nh, hd // 2, 2)
        pos = torch.arange(T, dtype=torch.float64)[:, None]
        i = torch.arange(hd // 2, dtype=torch.float64)[None, :]
        ang = pos / theta ** (2 * i / hd)
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        e, o = x[..., 0], x[..., 1]
        return torch.stack([e * c - o * s, o * c + e * s], -1).view(T, nh * hd)

    emb = P[(O.T_EMBED, 0)].view(V, D)
    x = emb[torch.tensor(inp.astype(np.int64))]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for l in range(L):
        xn = rms(x, P[(O.T_RMS_ATT, l)])
        q = rope(xn @ P[(O.T_WQ, l)].view(H * hd, D).T, H)
        k = rope(xn @ P[(O.T_WK, l)].view(KV * hd, D).T, KV)
        v = xn @ P[(O.T_WV, l)].view(KV * hd, D).T
        outs = []
        for h in range(H):
            g = h // (H // KV)
            sc = q[:, h * hd:(h + 1) * hd] @ k[:, g * hd:(g + 1) * hd].T / np.sqrt(hd)
            outs.append(torch.softmax(sc.masked_fill(~causal, float("-inf")), -1) @ v[:, g * hd:(g + 1) * hd])
        x2 = x + torch.cat(outs, 1) @ P[(O.T_WO, l)].view(D, H * hd).T
        x2n = rms(x2, P[(O.T_RMS_FFN, l)])
        h1 = x2n @ P[(O.T_W1, l)].view(Hd, D).T
        h3 = x2n @ P[(O.T_W3, l)].view(Hd, D).T
        x = x2 + (torch.nn.functional.silu(h1) * h3) @ P[(O.T_W2, l)].view(D, Hd).T
    logits = rms(x, P[(O.T_RMS_FINAL, 0)]) @ emb.T
    valid = torch.tensor(tgt < V)
    lt = torch.nn.functional.cross_entropy(logits[valid], torch.tensor(tgt.astype(np.int64))[valid])
    lt.backward()
    assert abs(loss - float(lt.detach())) < 1e-5
    for (tid, layer), p in P.items():
        g = m.tensor(tid, layer, O.G)
        ref = p.grad.numpy().ravel()
        err = np.linalg.norm(g - ref) / np.linalg.norm(ref)
        assert err < 1e-4, (O.TENSOR_NAMES[tid], layer, err)


def test_reference_arch_matches_torch_autograd_fp64():
    """The same for the network the reference trains, with its backward quirks off (exact gradients):
    embedding norm, smear, parameterless RMSNorm, rotation then 1.2 x per-head norm of q and k, value
    embeddings on odd layers, lambda-weighted residuals with the x0 skip, ReLU^2, backout of the middle
    layer's output, soft-capped logits (ane/train_full.go:383-453,480-558)."""
    import torch

    D, Hd, H, L, V, T = 32, 48, 4, 4, 64, 12
    hd = D // H
    m = O.Model(dim=D, hidden=Hd, heads=H, kv_heads=H, layers=L, vocab=V, seq=T, arch=O.ARCH_N, quirks=0,
                loss_scale=1.0, accum_steps=1000, grad_clip=0.0)
    O.init_weights(m, 1, std=0.3)
    m.tensor(O.T_SMEAR_LAMBDA)[:] = 0.3
    m.tensor(O.T_BACKOUT_LAMBDA)[:] = 0.3
    a = m.tensor(O.T_X0_LAMBDAS)
    a[:] = np.linspace(0.1, 0.4, a.size)
    a = m.tensor(O.T_RESID_LAMBDAS)
    a[:] = np.linspace(0.8, 1.2, a.size)
    for tid, layer, a in m.tensors():
        if tid == O.T_VE_GATE:
            a[:] = 0.5 * np.random.default_rng(layer).standard_normal(a.size)
    toks = O.zipf_tokens(T + 1, V, 3)
    inp, tgt = toks[:T].copy(), toks[1:T + 1].copy()
    tgt[4] = 65535
    loss = m.accumulate(inp, tgt)
    P = {(tid, layer): torch.tensor(a.astype(np.float64), requires_grad=True) for tid, layer, a in m.tensors(O.W)}
    theta = float(m.cfg.rope_theta)

    def rms(x):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5)

    def rope(x):
        x = x.view(T, H, hd // 2, 2)
        pos = torch.arange(T, dtype=torch.float64)[:, None]
        i = torch.arange(hd // 2, dtype=torch.float64)[None, :]
        ang = pos / theta ** (2 * i / hd)
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        e, o = x[..., 0], x[..., 1]
        return torch.stack([e * c - o * s, o * c + e * s], -1)

    def qknorm(x):
        x = x.reshape(T, H, hd)
        return (1.2 * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5)).reshape(T, H * hd)

    emb = P[(O.T_EMBED, 0)].view(V, D)
    tok = torch.tensor(inp.astype(np.int64))
    x0 = rms(emb[tok])
    gp = x0 @ P[(O.T_SMEAR_GATE, 0)].view(D, D).T
    shifted = torch.cat([torch.zeros(1, D, dtype=torch.float64), x0[:-1]], 0)
    x = x0 + P[(O.T_SMEAR_LAMBDA, 0)] * torch.sigmoid(gp) * shifted   # position 0 has no predecessor
    rl, xl = P[(O.T_RESID_LAMBDAS, 0)], P[(O.T_X0_LAMBDAS, 0)]
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    xmid = None
    for l in range(L):
        xn = rms(x)
        q = qknorm(rope(xn @ P[(O.T_WQ, l)].view(D, D).T))
        k = qknorm(rope(xn @ P[(O.T_WK, l)].view(D, D).T))
        v = xn @ P[(O.T_WV, l)].view(D, D).T
        if (O.T_VE_EMBED, l) in P:
            g = torch.sigmoid(x[:, :12] @ P[(O.T_VE_GATE, l)].view(H, 12).T)
            ve = P[(O.T_VE_EMBED, l)].view(V, D)[tok].view(T, H, hd)
            v = (v.view(T, H, hd) + 3 * g[:, :, None] * ve).reshape(T, D)
        outs = []
        for h in range(H):
            sc = q[:, h * hd:(h + 1) * hd] @ k[:, h * hd:(h + 1) * hd].T / np.sqrt(hd)
            outs.append(torch.softmax(sc.masked_fill(~causal, float("-inf")), -1) @ v[:, h * hd:(h + 1) * hd])
        x2 = rl[l] * x + torch.cat(outs, 1) @ P[(O.T_WO, l)].view(D, D).T + xl[l] * x0
        h1 = rms(x2) @ P[(O.T_W1, l)].view(Hd, D).T
        x = rl[l] * x2 + (torch.relu(h1) ** 2) @ P[(O.T_W2, l)].view(D, Hd).T + xl[l] * x0
        if l == L // 2 - 1:
            xmid = x
    x = x - P[(O.T_BACKOUT_LAMBDA, 0)] * xmid
    logits = 15 * torch.tanh((rms(x) @ emb.T) / 15)
    valid = torch.tensor(tgt < V)
    lt = torch.nn.functional.cross_entropy(logits[valid], torch.tensor(tgt.astype(np.int64))[valid])
    lt.backward()
    assert abs(loss - float(lt.detach())) < 1e-5
    assert any(tid == O.T_VE_EMBED for tid, _ in P)
    for (tid, layer), p in P.items():
        g = m.tensor(tid, layer, O.G)
        ref = p.grad.numpy().ravel()
        err = np.linalg.norm(g - ref) / np.linalg.norm(ref)
        assert err < 1e-4, (O.TENSOR_NAMES[tid], layer, err)


def test_quirks_change_only_the_backward():
    cfg = dict(dim=32, hidden=48, heads=4, layers=2, vocab=64, seq=12, arch=O.ARCH_N, loss_scale=1.0, accum_steps=100)
    toks = O.zipf_tokens(13, 64, 3)
    inp, tgt = toks[:12].copy(), toks[1:13].copy()
    res = []
    for q in (0, 1):
        m = O.Model(quirks=q, **cfg)
        O.init_weights(m, 1, std=0.3)
        res.append((m.accumulate(inp, tgt), m.tensor(O.T_WQ, 0, O.G).copy(), m.tap(O.TAP_FINAL).copy()))
    assert res[0][0] == res[1][0]
    np.testing.assert_array_equal(res[0][2], res[1][2])
    assert not np.allclose(res[0][1], res[1][1])


def test_adam_matches_closed_form_first_step():
    # ane/train_full.go:1113-1150 with t = 1: m = (1-b1) g, v = (1-b2) g^2, mh = g, vh = g^2
    n = 64
    rng = np.random.default_rng(4)
    w = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    w0 = w.copy()
    fp = lambda a: a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
    O.lib().orc_adam(fp(w), fp(g), fp(m), fp(v), n, 1, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    want = w0 - 1e-2 * (np.sign(g) + 0.1 * w0)
    np.testing.assert_allclose(w, want, rtol=2e-4, atol=2e-6)


def test_accumulate_then_flush_equals_mean_gradient_step():
    cfg = dict(dim=32, hidden=48, heads=4, layers=2, vocab=64, seq=12, arch=O.ARCH_L, accum_steps=2, lr=1e-2,
               grad_clip=0.0)
    m = O.Model(**cfg)
    O.init_weights(m, 1, std=0.1)
    toks = O.zipf_tokens(26, 64, 9)
    m.step(toks[0:12].copy(), toks[1:13].copy())
    assert m.pending == 1 and m.adam_t == 0
    m.step(toks[13:25].copy(), toks[14:26].copy())
    assert m.pending == 0 and m.adam_t == 1


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden vectors not generated")
def test_golden_vectors():
    from golden.make_golden import run_case

    want = np.load(GOLDEN)
    got = run_case()
    for k in want.files:
        np.testing.assert_allclose(got[k], want[k], rtol=2e-5, atol=1e-7, err_msg=k)
