"""ctypes binding of the CPU oracle (oracle/oracle.cpp) -- TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the cpu_baseline / reference legs of bench.py
import this module.  The product library never does.

PARITY UNPINNED: the reference has no golden vectors for this path (see oracle.h).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int32, c_int64, c_uint16, c_uint32, c_uint64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")

ARCH_N, ARCH_L = 0, 1
W, G, M, V = 0, 1, 2, 3

# tensor ids (oracle.h)
T_EMBED, T_WQ, T_WK, T_WV, T_WO, T_W1, T_W2, T_W3 = range(8)
T_RMS_ATT, T_RMS_FFN, T_RMS_FINAL, T_VE_EMBED, T_VE_GATE = 8, 9, 10, 11, 12
T_RESID_LAMBDAS, T_X0_LAMBDAS, T_SMEAR_GATE, T_SMEAR_LAMBDA, T_BACKOUT_LAMBDA = 13, 14, 15, 16, 17
T_COUNT = 18
LAYER_TENSORS = (T_WQ, T_WK, T_WV, T_WO, T_W1, T_W2, T_W3, T_RMS_ATT, T_RMS_FFN, T_VE_EMBED, T_VE_GATE)
GLOBAL_TENSORS = (T_EMBED, T_RMS_FINAL, T_RESID_LAMBDAS, T_X0_LAMBDAS, T_SMEAR_GATE, T_SMEAR_LAMBDA, T_BACKOUT_LAMBDA)
TENSOR_NAMES = {
    T_EMBED: "embed", T_WQ: "wq", T_WK: "wk", T_WV: "wv", T_WO: "wo", T_W1: "w1", T_W2: "w2", T_W3: "w3",
    T_RMS_ATT: "rms_att", T_RMS_FFN: "rms_ffn", T_RMS_FINAL: "rms_final", T_VE_EMBED: "ve_embed",
    T_VE_GATE: "ve_gate", T_RESID_LAMBDAS: "resid_lambdas", T_X0_LAMBDAS: "x0_lambdas",
    T_SMEAR_GATE: "smear_gate", T_SMEAR_LAMBDA: "smear_lambda", T_BACKOUT_LAMBDA: "backout_lambda",
}

# taps (oracle.h)
(TAP_X, TAP_XNORM, TAP_Q, TAP_K, TAP_V, TAP_ATT, TAP_X2, TAP_X2NORM, TAP_H1, TAP_GATE, TAP_FFN_OUT, TAP_QPRE,
 TAP_KPRE, TAP_H3, TAP_DOUT, TAP_DH1, TAP_DX2, TAP_DQ, TAP_DK, TAP_DV, TAP_DH3) = range(21)
(TAP_X0, TAP_XMID, TAP_FINAL, TAP_FINAL_NORM, TAP_LOGITS_PRE, TAP_LOGITS, TAP_DLOGITS, TAP_DFINAL) = range(32, 40)


class Config(ctypes.Structure):
    _fields_ = [
        ("dim", c_int32), ("hidden", c_int32), ("heads", c_int32), ("kv_heads", c_int32), ("layers", c_int32),
        ("vocab", c_int32), ("seq", c_int32), ("arch", c_int32), ("quirks", c_int32), ("rope_theta", c_float),
        ("accum_steps", c_int32), ("lr", c_float), ("beta1", c_float), ("beta2", c_float), ("eps", c_float),
        ("weight_decay", c_float), ("grad_clip", c_float), ("loss_scale", c_float), ("embed_lr_mult", c_float),
        ("scalar_lr_mult", c_float), ("lambda_lr_mult", c_float), ("lambda_beta1", c_float),
        ("lambda_beta2", c_float),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only, no GPU needed)."""
    if force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH) for f in ("oracle.cpp", "oracle.h")
    ):
        subprocess.check_call(["make", "-C", _HERE], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def usable_cpus() -> int:
    """CPUs this process may really use: the affinity mask capped by the cgroup CPU quota.  OpenMP
    sizing from the raw core count oversubscribes a quota-limited container badly."""
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        n = os.cpu_count() or 1
    for path in ("/sys/fs/cgroup/cpu.max", "/sys/fs/cgroup/cpu/cpu.cfs_quota_us"):
        try:
            with open(path) as f:
                parts = f.read().split()
            if path.endswith("cpu.max"):
                if parts[0] != "max":
                    n = min(n, max(1, int(float(parts[0]) / float(parts[1]))))
            else:
                q = int(parts[0])
                if q > 0:
                    with open("/sys/fs/cgroup/cpu/cpu.cfs_period_us") as g:
                        n = min(n, max(1, q // int(g.read().split()[0])))
            break
        except Exception:
            continue
    env = os.environ.get("ANE_ORACLE_THREADS")
    if env:
        n = max(1, int(env))
    return max(1, min(n, 64))


def lib():
    global _lib
    if _lib is not None:
        return _lib
    build()
    os.environ.setdefault("OMP_WAIT_POLICY", "PASSIVE")
    L = ctypes.CDLL(_LIB_PATH)
    fp = POINTER(c_float)
    u16p = POINTER(c_uint16)
    L.orc_create.restype = c_void_p
    L.orc_create.argtypes = [POINTER(Config)]
    L.orc_destroy.argtypes = [c_void_p]
    L.orc_get_config.argtypes = [c_void_p, POINTER(Config)]
    L.orc_tensor.restype = fp
    L.orc_tensor.argtypes = [c_void_p, c_int32, c_int32, c_int32, POINTER(c_uint64)]
    L.orc_tap.restype = fp
    L.orc_tap.argtypes = [c_void_p, c_int32, c_int32, POINTER(c_uint64)]
    for name in ("orc_step", "orc_accumulate"):
        f = getattr(L, name)
        f.restype = c_float
        f.argtypes = [c_void_p, u16p, u16p]
    L.orc_flush.argtypes = [c_void_p]
    L.orc_pending.restype = c_uint32
    L.orc_pending.argtypes = [c_void_p]
    L.orc_adam_t.restype = c_uint32
    L.orc_adam_t.argtypes = [c_void_p]
    L.orc_set_lr.argtypes = [c_void_p, c_float]
    L.orc_eval_logits.argtypes = [c_void_p, u16p, fp]
    L.orc_eval_loss_window.restype = c_double
    L.orc_eval_loss_window.argtypes = [c_void_p, u16p, POINTER(c_int32)]
    L.orc_loss_only.restype = c_double
    L.orc_loss_only.argtypes = [c_void_p, u16p, u16p]
    L.orc_drand48_seed.restype = c_uint64
    L.orc_drand48_seed.argtypes = [c_int64]
    L.orc_sample_pos.restype = c_uint64
    L.orc_sample_pos.argtypes = [POINTER(c_uint64), c_uint64, c_uint32]
    L.orc_rmsnorm.argtypes = [fp, fp, fp, c_int32, c_int32]
    L.orc_rmsnorm_final.argtypes = [fp, fp, fp, c_int32, c_int32]
    L.orc_rmsnorm_bwd.argtypes = [fp, fp, fp, fp, fp, c_int32, c_int32]
    L.orc_linear.argtypes = [fp, fp, fp, c_int32, c_int32, c_int32]
    L.orc_linear_dx.argtypes = [fp, fp, fp, c_int32, c_int32, c_int32]
    L.orc_linear_dw.argtypes = [fp, fp, fp, c_int32, c_int32, c_int32]
    L.orc_rope.argtypes = [fp, c_int32, c_int32, c_int32, c_float, c_int32]
    L.orc_qknorm.argtypes = [fp, fp, c_int32, c_int32, c_int32]
    L.orc_attention.argtypes = [fp, fp, fp, fp, c_int32, c_int32, c_int32, c_int32]
    L.orc_attention_bwd.argtypes = [fp, fp, fp, fp, fp, fp, fp, c_int32, c_int32, c_int32, c_int32, c_float]
    L.orc_cross_entropy.restype = c_float
    L.orc_cross_entropy.argtypes = [fp, fp, u16p, c_int32, c_int32]
    L.orc_softcap.argtypes = [fp, c_uint64]
    L.orc_adam.argtypes = [fp, fp, fp, fp, c_uint64, c_int32, c_float, c_float, c_float, c_float, c_float]
    L.orc_argmax.restype = c_int32
    L.orc_argmax.argtypes = [fp, c_int32]
    L.orc_sample.restype = c_int32
    L.orc_sample.argtypes = [fp, c_int32, c_float, c_double]
    L.orc_set_reference_threading.argtypes = [c_int32]
    L.orc_num_threads.restype = c_int32
    L.orc_set_num_threads.argtypes = [c_int32]
    L.orc_set_num_threads(usable_cpus())
    _lib = L
    return L


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(POINTER(c_float))


def _u16(a: np.ndarray):
    assert a.dtype == np.uint16 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(POINTER(c_uint16))


class Model:
    """One oracle model instance; tensors and taps are numpy views into its storage."""

    def __init__(self, **kw):
        cfg = Config()
        for k, v in kw.items():
            if not hasattr(cfg, k):
                raise TypeError(f"unknown config field {k}")
            setattr(cfg, k, v)
        self._lib = lib()
        self._h = self._lib.orc_create(ctypes.byref(cfg))
        if not self._h:
            raise ValueError("orc_create rejected the configuration")
        self.cfg = Config()
        self._lib.orc_get_config(self._h, ctypes.byref(self.cfg))

    def close(self):
        if self._h:
            self._lib.orc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor(self, tid: int, layer: int = 0, which: int = W):
        n = c_uint64(0)
        p = self._lib.orc_tensor(self._h, tid, layer, which, ctypes.byref(n))
        if not p or n.value == 0:
            return None
        return np.ctypeslib.as_array(p, shape=(n.value,))

    def tap(self, tap_id: int, layer: int = 0):
        n = c_uint64(0)
        p = self._lib.orc_tap(self._h, tap_id, layer, ctypes.byref(n))
        if not p or n.value == 0:
            return None
        a = np.ctypeslib.as_array(p, shape=(n.value,))
        return a.reshape(-1, self.cfg.seq)

    def tensors(self, which: int = W):
        """Yield (tensor_id, layer, array) for every parameter tensor that exists."""
        for tid in GLOBAL_TENSORS:
            a = self.tensor(tid, 0, which)
            if a is not None:
                yield tid, 0, a
        for layer in range(self.cfg.layers):
            for tid in LAYER_TENSORS:
                a = self.tensor(tid, layer, which)
                if a is not None:
                    yield tid, layer, a

    def step(self, inp, tgt) -> float:
        return float(self._lib.orc_step(self._h, _u16(inp), _u16(tgt)))

    def accumulate(self, inp, tgt) -> float:
        return float(self._lib.orc_accumulate(self._h, _u16(inp), _u16(tgt)))

    def flush(self):
        self._lib.orc_flush(self._h)

    @property
    def pending(self):
        return int(self._lib.orc_pending(self._h))

    @property
    def adam_t(self):
        return int(self._lib.orc_adam_t(self._h))

    def set_lr(self, lr):
        self._lib.orc_set_lr(self._h, lr)

    def eval_logits(self, tokens):
        out = np.empty((self.cfg.vocab, self.cfg.seq), dtype=np.float32)
        self._lib.orc_eval_logits(self._h, _u16(tokens), _fp(out))
        return out

    def eval_loss_window(self, tokens):
        n = c_int32(0)
        total = self._lib.orc_eval_loss_window(self._h, _u16(tokens), ctypes.byref(n))
        return float(total), int(n.value)

    def loss_only(self, inp, tgt) -> float:
        return float(self._lib.orc_loss_only(self._h, _u16(inp), _u16(tgt)))


# ---- seeded synthetic inputs shared by the oracle and GPU tests -----------------------------

def zipf_tokens(n: int, vocab: int, seed: int, s: float = 1.1) -> np.ndarray:
    """i.i.d. Zipf(s) token ids over [0, vocab): p(k) ~ (k+1)^-s, inverse-CDF sampling."""
    rng = np.random.Generator(np.random.PCG64(seed))
    p = (np.arange(1, vocab + 1, dtype=np.float64)) ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = rng.random(n)
    return np.minimum(np.searchsorted(cdf, u, side="right"), vocab - 1).astype(np.uint16)


def init_weights(model: Model, seed: int, std: float = 0.02, reference_scalars: bool = True):
    """N(0, std) matrices / embeddings from one seeded generator; norm weights 1; the
    reference-architecture scalars at their RandomInit values (ane/stories/weights.go:190-202)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    for tid, layer, a in model.tensors(W):
        if tid in (T_RMS_ATT, T_RMS_FFN, T_RMS_FINAL):
            a[:] = 1.0
        elif tid == T_RESID_LAMBDAS:
            a[:] = 1.0
        elif tid == T_X0_LAMBDAS:
            a[:] = 0.1 if reference_scalars else 0.0
        elif tid in (T_SMEAR_LAMBDA, T_BACKOUT_LAMBDA):
            a[:] = 0.01 if reference_scalars else 0.0
        elif tid == T_VE_GATE:
            a[:] = (0.02 * rng.random(a.size)).astype(np.float32)
        else:
            a[:] = (std * rng.standard_normal(a.size)).astype(np.float32)


def drand48_positions(seed: int, n_tokens: int, seq: int, count: int) -> list[int]:
    L = lib()
    st = c_uint64(L.orc_drand48_seed(seed))
    return [int(L.orc_sample_pos(ctypes.byref(st), n_tokens, seq)) for _ in range(count)]
