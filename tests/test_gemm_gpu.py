"""tcgen05 GEMM (and the fp32 SIMT GEMM) against the oracle's naive loops, through the C ABI.
Shapes cover the step's three operand layouts, ragged edges and split-K accumulation."""
import ctypes

import numpy as np
import pytest

import ane
from ane import _ffi
from oracle import oracle as O
from parity_utils import rel_l2

pytestmark = pytest.mark.gpu
lib = _ffi.lib


def _ck(rc):
    assert rc == 0, lib.ane_ops_last_error().decode()


def _up(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    p = lib.ane_dev_malloc(a.nbytes)
    _ck(lib.ane_dev_h2d(p, a.ctypes.data, a.nbytes))
    return p


def _up_bf16(a):
    p = _up(a)
    q = lib.ane_dev_malloc(a.size * 2)
    _ck(lib.ane_op_cast_f32_to_bf16(p, q, a.size))
    lib.ane_dev_free(p)
    return q


def _down(p, shape):
    a = np.empty(shape, dtype=np.float32)
    _ck(lib.ane_dev_d2h(a.ctypes.data, p, a.nbytes))
    return a


def _bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(a.shape)


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _gemm(dtype, A_store, B_store, C_init, M, N, K, a_mn, b_mn, out_mode, split_k=0, res=None):
    upf = _up_bf16 if dtype == ane.DTYPE_BF16 else _up
    dA, dB, dC = upf(A_store), upf(B_store), _up(C_init)
    dR = _up(res) if res is not None else None
    g = _ffi.GemmArgs()
    g.struct_size = ctypes.sizeof(_ffi.GemmArgs)
    g.dtype = dtype
    g.d_a, g.d_b, g.d_c = dA, dB, dC
    g.m, g.n, g.k = M, N, K
    g.lda, g.ldb, g.ldc = A_store.shape[1], B_store.shape[1], N
    g.a_mn, g.b_mn, g.out_mode, g.alpha, g.split_k = a_mn, b_mn, out_mode, 1.0, split_k
    if dR is not None:
        g.d_res1, g.ldres = dR, N
    _ck(lib.ane_op_gemm(ctypes.byref(g)))
    _ck(lib.ane_dev_sync())
    st = ctypes.c_int32(0)
    _ck(lib.ane_ops_device_status(ctypes.byref(st)))
    assert st.value == 0
    out = _down(dC, (M, N))
    for p in (dA, dB, dC) + ((dR,) if dR is not None else ()):
        lib.ane_dev_free(p)
    return out


def test_step_sized_shapes_take_the_wide_tile_and_tma_residual_paths():
    """Shapes of the 110M step that select the 256-row tiles (long K, enough tiles), the stream-K weight
    gradient on 256-row tiles and the TMA-fed residual epilogue; checked against numpy on the same
    bf16-rounded operands (fp32 accumulation order differs, hence 1e-4)."""
    rng = np.random.default_rng(3)
    # dx form: C[M,N] = A[M,K] . B[K,N]
    M, N, K = 8192, 768, 2304
    A = _bf16_round(rng.standard_normal((M, K)).astype(np.float32) * 0.1)
    B = _bf16_round(rng.standard_normal((K, N)).astype(np.float32) * 0.1)
    got = _gemm(ane.DTYPE_BF16, A, B, np.zeros((M, N), np.float32), M, N, K, 0, 1, 1)
    assert rel_l2(got, A @ B) < 1e-4
    # dW form with accumulation: C[M,N] += A^T[M,K] . B[K,N], A stored [K, M]
    M, N, K = 2304, 768, 8192
    At = _bf16_round(rng.standard_normal((K, M)).astype(np.float32) * 0.1)
    B = _bf16_round(rng.standard_normal((K, N)).astype(np.float32) * 0.1)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    got = _gemm(ane.DTYPE_BF16, At, B, C0, M, N, K, 1, 1, 2)
    assert rel_l2(got, C0 + At.T @ B) < 1e-4
    # forward form with a residual: C = A . W^T + R
    M, N, K = 8192, 768, 768
    A = _bf16_round(rng.standard_normal((M, K)).astype(np.float32) * 0.1)
    W = _bf16_round(rng.standard_normal((N, K)).astype(np.float32) * 0.1)
    R = rng.standard_normal((M, N)).astype(np.float32)
    got = _gemm(ane.DTYPE_BF16, A, W, np.zeros((M, N), np.float32), M, N, K, 0, 0, 1, res=R)
    assert rel_l2(got, A @ W.T + R) < 1e-4
    # ragged rows and columns through the same residual path (TMA clips the residual pieces)
    M, N, K = 8100, 760, 768
    got = _gemm(ane.DTYPE_BF16, A[:M], W[:N], np.zeros((M, N), np.float32), M, N, K, 0, 0, 1, res=np.ascontiguousarray(R[:M, :N]))
    assert rel_l2(got, A[:M] @ W[:N].T + R[:M, :N]) < 1e-4


def test_short_k_wide_n_shapes_take_the_cta_pair_tiles():
    """K = 768 with enough 256 x 256 tiles to fill the CTA pairs: the planner picks the two-CTA kernel
    (tcgen05.mma.cta_group::2, half of the B tile per CTA).  Both B layouts, a residual, and ragged M and N
    (the second CTA's rows / B columns then start or end outside the tensors)."""
    rng = np.random.default_rng(5)
    for (M, N, K, b_mn, res) in [(8192, 2304, 768, 0, False), (4000, 2300, 768, 1, False), (3900, 2304, 704, 0, True),
                                 (8192, 2048, 768, 1, False)]:
        A = _bf16_round(rng.standard_normal((M, K)).astype(np.float32) * 0.1)
        if b_mn:
            B = _bf16_round(rng.standard_normal((K, N + (-N) % 8)).astype(np.float32) * 0.1)   # 16-byte row pitch
            want = A @ B[:, :N]
        else:
            B = _bf16_round(rng.standard_normal((N, K)).astype(np.float32) * 0.1)
            want = A @ B.T
        R = rng.standard_normal((M, N)).astype(np.float32) if res else None
        got = _gemm(ane.DTYPE_BF16, A, B, np.zeros((M, N), np.float32), M, N, K, 0, b_mn, 1, res=R)
        assert rel_l2(got, want + (R if res else 0)) < 1e-4, (M, N, K, b_mn, res)


def test_split_precision_gemm_carries_fp32_operands_through_the_tensor_cores():
    """ANE_DTYPE_BF16X3: fp32 operands cut into bf16 (hi, lo) pairs, three tcgen05 products.  Against float64
    on the unrounded operands the result must be fp32-like (a single bf16 product is ~3e-3 off); the three
    operand layouts of the step, a residual, an accumulating output and ragged sizes."""
    rng = np.random.default_rng(8)
    M, N, K = 1024, 768, 2304
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    got = _gemm(ane.DTYPE_BF16X3, A, B, np.zeros((M, N), np.float32), M, N, K, 0, 1, 1)
    want = A.astype(np.float64) @ B.astype(np.float64)
    assert rel_l2(got, want) < 2e-5
    one = _gemm(ane.DTYPE_BF16, A, B, np.zeros((M, N), np.float32), M, N, K, 0, 1, 1)
    assert rel_l2(one, want) > 1e-3                                     # the single bf16 product, for scale
    M, N, K = 1000, 760, 776                                            # forward form, ragged, with a residual
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = rng.standard_normal((N, K)).astype(np.float32)
    R = rng.standard_normal((M, N)).astype(np.float32)
    got = _gemm(ane.DTYPE_BF16X3, A, W, np.zeros((M, N), np.float32), M, N, K, 0, 0, 1, res=R)
    assert rel_l2(got, A.astype(np.float64) @ W.astype(np.float64).T + R) < 2e-5
    M, N, K = 2304, 768, 2048                                           # weight-gradient form, accumulating
    At = rng.standard_normal((K, M)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    got = _gemm(ane.DTYPE_BF16X3, At, B, C0, M, N, K, 1, 1, 2)
    assert rel_l2(got, C0 + At.astype(np.float64).T @ B.astype(np.float64)) < 2e-5


@pytest.mark.parametrize("dtype", [ane.DTYPE_BF16, ane.DTYPE_F32, ane.DTYPE_BF16X3])
@pytest.mark.parametrize("oc,ic,seq", [(96, 64, 40), (256, 136, 300), (768, 256, 128)])
def test_linear_forward_dx_dw_match_oracle(dtype, oc, ic, seq):
    """linearCF / linearBackwardDXCF / accumLinearGradCF (ane/common.go:91, ane/train_full.go:213,242)."""
    rng = np.random.default_rng(oc + seq)
    rnd = _bf16_round if dtype == ane.DTYPE_BF16 else (lambda a: a)
    W = rnd(rng.standard_normal((oc, ic)).astype(np.float32) * 0.1)
    x_cf = rnd(rng.standard_normal((ic, seq)).astype(np.float32))          # reference layout [C][seq]
    dy_cf = rnd(rng.standard_normal((oc, seq)).astype(np.float32))
    tol = 2e-5
    # forward: y[t,o] = x[t,:] . W[o,:]
    want = np.empty((oc, seq), np.float32)
    O.lib().orc_linear(_fp(want), _fp(W), _fp(x_cf), oc, ic, seq)
    got = _gemm(dtype, np.ascontiguousarray(x_cf.T), W, np.zeros((seq, oc), np.float32), seq, oc, ic, 0, 0, 1)
    assert rel_l2(got.T, want) < tol
    # dx[t,i] = dy[t,:] . W[:,i]   (B stored [K=oc, N=ic])
    want = np.empty((ic, seq), np.float32)
    O.lib().orc_linear_dx(_fp(want), _fp(W), _fp(dy_cf), oc, ic, seq)
    got = _gemm(dtype, np.ascontiguousarray(dy_cf.T), W, np.zeros((seq, ic), np.float32), seq, ic, oc, 0, 1, 1)
    assert rel_l2(got.T, want) < tol
    # dW[o,i] += sum_t dy[t,o] x[t,i]   (both operands stored [K=seq, .]); beta = 1
    dw0 = rng.standard_normal((oc, ic)).astype(np.float32)
    want = dw0.copy()
    O.lib().orc_linear_dw(_fp(want), _fp(dy_cf), _fp(x_cf), oc, ic, seq)
    for split in (1, 2):
        got = _gemm(dtype, np.ascontiguousarray(dy_cf.T), np.ascontiguousarray(x_cf.T), dw0, oc, ic, seq, 1, 1, 2, split)
        assert rel_l2(got, want) < tol


def _down_bf16(p, shape):
    n = int(np.prod(shape))
    q = lib.ane_dev_malloc(n * 4)
    _ck(lib.ane_op_cast_bf16_to_f32(p, q, n))
    out = _down(q, shape)
    lib.ane_dev_free(q)
    return out


@pytest.mark.parametrize("M,Hd,K", [(8192, 2048, 768), (300, 96, 136), (1000, 2048, 768)])
def test_swiglu_backward_fused_into_the_dx_product(M, Hd, K):
    """out_mode 7: d gate = dOut . W2 stays in the accumulators; the epilogue reads h1 | h3 (interleaved in blocks
    of 32 columns) and writes d h1 = d gate * h3 * silu'(h1), d h3 = d gate * silu(h1) in the same layout.  Against
    float64 on the same bf16 operands; the step's shape (CTA-pair tiles) and ragged ones (single-CTA tiles)."""
    rng = np.random.default_rng(M + Hd)
    dOut = _bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    W2 = _bf16_round((rng.standard_normal((K, Hd)) / np.sqrt(K)).astype(np.float32))       # stored [K, N]: MN-major B
    h1 = _bf16_round(rng.standard_normal((M, Hd)).astype(np.float32) * 2.0)
    h3 = _bf16_round(rng.standard_normal((M, Hd)).astype(np.float32))
    h13 = np.empty((M, 2 * Hd), np.float32)
    blk = h13.reshape(M, Hd // 32, 2, 32)
    blk[:, :, 0, :] = h1.reshape(M, Hd // 32, 32)
    blk[:, :, 1, :] = h3.reshape(M, Hd // 32, 32)
    dA, dB, dH = _up_bf16(dOut), _up_bf16(W2), _up_bf16(h13)
    dC = lib.ane_dev_malloc(M * 2 * Hd * 2)
    _ck(lib.ane_dev_memset(dC, 0xFF, M * 2 * Hd * 2))
    g = _ffi.GemmArgs()
    g.struct_size = ctypes.sizeof(_ffi.GemmArgs)
    g.dtype = ane.DTYPE_BF16
    g.d_a, g.d_b, g.d_c, g.d_aux = dA, dB, dC, dH
    g.m, g.n, g.k = M, Hd, K
    g.lda, g.ldb, g.ldc, g.ldaux = K, Hd, 2 * Hd, 2 * Hd
    g.a_mn, g.b_mn, g.out_mode, g.alpha = 0, 1, 7, 1.0
    _ck(lib.ane_op_gemm(ctypes.byref(g)))
    _ck(lib.ane_dev_sync())
    st = ctypes.c_int32(0)
    _ck(lib.ane_ops_device_status(ctypes.byref(st)))
    assert st.value == 0
    got = _down_bf16(dC, (M, 2 * Hd)).reshape(M, Hd // 32, 2, 32)
    dg = dOut.astype(np.float64) @ W2.astype(np.float64)
    x = h1.astype(np.float64)
    sg = 1.0 / (1.0 + np.exp(-x))
    want1 = dg * h3 * sg * (1.0 + x * (1.0 - sg))
    want3 = dg * x * sg
    assert np.isfinite(got).all()
    assert rel_l2(got[:, :, 0, :].reshape(M, Hd), want1) < 4e-3          # one bf16 rounding of the output
    assert rel_l2(got[:, :, 1, :].reshape(M, Hd), want3) < 4e-3
    for p in (dA, dB, dH, dC):
        lib.ane_dev_free(p)


@pytest.mark.parametrize("M,Hd,K", [(8192, 2048, 768), (320, 192, 128), (100, 64, 72)])
def test_relu2_backward_fused_into_the_dx_product(M, Hd, K):
    """out_mode 10: d gate = dOut . W2 stays in the accumulators; the epilogue reads h and writes
    d h = d gate * 2 max(h, 0) (the reference's ReLU^2 activation, ane/common.go:146, differentiated).  Against
    float64 on the same bf16 operands; the step's shape (CTA-pair tiles) and ragged ones (single-CTA tiles)."""
    rng = np.random.default_rng(M + Hd + 1)
    dOut = _bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    W2 = _bf16_round((rng.standard_normal((K, Hd)) / np.sqrt(K)).astype(np.float32))       # stored [K, N]: MN-major B
    h = _bf16_round(rng.standard_normal((M, Hd)).astype(np.float32) * 2.0)
    dA, dB, dH = _up_bf16(dOut), _up_bf16(W2), _up_bf16(h)
    dC = lib.ane_dev_malloc(M * Hd * 2)
    _ck(lib.ane_dev_memset(dC, 0xFF, M * Hd * 2))
    g = _ffi.GemmArgs()
    g.struct_size = ctypes.sizeof(_ffi.GemmArgs)
    g.dtype = ane.DTYPE_BF16
    g.d_a, g.d_b, g.d_c, g.d_aux = dA, dB, dC, dH
    g.m, g.n, g.k = M, Hd, K
    g.lda, g.ldb, g.ldc, g.ldaux = K, Hd, Hd, Hd
    g.a_mn, g.b_mn, g.out_mode, g.alpha = 0, 1, 10, 1.0
    _ck(lib.ane_op_gemm(ctypes.byref(g)))
    _ck(lib.ane_dev_sync())
    st = ctypes.c_int32(0)
    _ck(lib.ane_ops_device_status(ctypes.byref(st)))
    assert st.value == 0
    got = _down_bf16(dC, (M, Hd))
    want = (dOut.astype(np.float64) @ W2.astype(np.float64)) * 2.0 * np.maximum(h.astype(np.float64), 0.0)
    assert np.isfinite(got).all()
    assert rel_l2(got, want) < 4e-3          # one bf16 rounding of the output
    assert np.all(got[h <= 0] == 0)          # exact zeros where the activation was off
    for p in (dA, dB, dH, dC):
        lib.ane_dev_free(p)


def test_gemm_rejects_misaligned_pitch():
    A = np.zeros((16, 20), np.float32)  # 20 bf16 = 40 bytes per row: not a 16-byte multiple
    dA, dB, dC = _up_bf16(A), _up_bf16(A), _up(np.zeros((16, 16), np.float32))
    g = _ffi.GemmArgs()
    g.struct_size = ctypes.sizeof(_ffi.GemmArgs)
    g.dtype = ane.DTYPE_BF16
    g.d_a, g.d_b, g.d_c = dA, dB, dC
    g.m, g.n, g.k, g.lda, g.ldb, g.ldc, g.out_mode, g.alpha = 16, 16, 20, 20, 20, 16, 1, 1.0
    assert lib.ane_op_gemm(ctypes.byref(g)) != 0
    assert b"16-byte" in lib.ane_ops_last_error()
    for p in (dA, dB, dC):
        lib.ane_dev_free(p)
