"""Python mirror of the reference's `ane` package surface (ane/engine.go): Options, Open,
Engine.Step / EvalLogits / EvalLoss / Flush / LR / SetLR / State / LoadState / Close, with the
same argument meaning and error behaviour (errors carry the reference's "storiesane <op>:" text).
Everything is executed by libane_b200.so on the GPU."""
from __future__ import annotations

import ctypes
import weakref
from ctypes import POINTER, byref, c_double, c_float, c_uint8, c_uint16, c_uint64, c_void_p
from dataclasses import dataclass, field

import numpy as np

from . import _ffi
from ._ffi import ARCH_LLAMA, ARCH_REFERENCE, DTYPE_BF16, DTYPE_BF16X3, DTYPE_F32, lib

# tensor ids (include/ane_b200.h)
T_EMBED, T_WQ, T_WK, T_WV, T_WO, T_W1, T_W2, T_W3 = range(8)
T_RMS_ATT, T_RMS_FFN, T_RMS_FINAL, T_VE_EMBED, T_VE_GATE = 8, 9, 10, 11, 12
T_RESID_LAMBDAS, T_X0_LAMBDAS, T_SMEAR_GATE, T_SMEAR_LAMBDA, T_BACKOUT_LAMBDA = 13, 14, 15, 16, 17
W, G, M, V = 0, 1, 2, 3


class EngineError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{msg} (status {code})")
        self.code = code


@dataclass
class Options:
    """ane.Options (ane/engine.go:14-40) plus the runtime model dimensions.  `model_path` is the
    reference's ModelPath: a llama2.c model file or a checkpoint, loaded by open() (ane/engine.go:250-257);
    left empty, the engine starts from zero weights and the caller imports tensors (tests do)."""
    model_path: str = ""
    tokens: np.ndarray | None = None
    seq: int = 0
    accum_steps: int = 0
    lr: float = 0.0
    seed: int = 0
    adam_beta1: float = 0.0
    adam_beta2: float = 0.0
    adam_eps: float = 0.0
    weight_decay: float = 0.0
    grad_clip: float = 0.0
    loss_scale: float = 0.0
    use_ane: bool = False
    hybrid_backward: bool = False
    embed_lr_mult: float = 0.0
    scalar_lr_mult: float = 0.0
    lambda_lr_mult: float = 0.0
    lambda_beta1: float = 0.0
    lambda_beta2: float = 0.0
    # additive fields (zero = reference value)
    dim: int = 0
    hidden: int = 0
    n_layers: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    vocab: int = 0
    batch: int = 0
    arch: int = ARCH_REFERENCE
    quirks: int = 1
    compute_dtype: int = DTYPE_BF16
    rope_theta: float = 0.0
    device: int = 0
    rank: int = 0
    world_size: int = 1
    dp_id: bytes | None = None
    debug_taps: bool = False
    ce_chunk_rows: int = 0
    ce_chunk_cols: int = 0


@dataclass
class StepResult:
    """ane.StepResult (ane/engine.go:55-69); durations in seconds."""
    loss: float = 0.0
    step_duration: float = 0.0
    device_eval_duration: float = 0.0
    cpu_work_duration: float = 0.0
    adam_duration: float = 0.0
    flushed: bool = False
    device_status: int = 0


@dataclass
class State:
    """ane.State (ane/engine.go:43-52)."""
    token_pos: int = 0
    last_loss: float = 0.0
    cum_train_ms: float = 0.0
    cum_wall_ms: float = 0.0
    cum_steps: int = 0
    cum_batches: int = 0
    adam_t: int = 0
    pending_steps: int = 0


def dp_unique_id() -> bytes:
    buf = (c_uint8 * 128)()
    rc = lib.ane_dp_unique_id(buf)
    if rc != 0:
        raise EngineError(rc, lib.ane_last_error(None).decode())
    return bytes(buf)


def _u16p(a: np.ndarray):
    return a.ctypes.data_as(POINTER(c_uint16))


class Engine:
    def __init__(self, handle: c_void_p, opts: Options):
        self._h = handle
        self.opts = opts

    # -- ane.Open (ane/engine.go:184)
    @staticmethod
    def open(opts: Options) -> "Engine":
        o = _ffi.Options()
        o.struct_size = ctypes.sizeof(_ffi.Options)
        for name in ("dim", "hidden", "n_layers", "n_heads", "n_kv_heads", "vocab", "seq", "batch", "arch", "quirks",
                     "compute_dtype", "rope_theta", "accum_steps", "lr", "seed", "adam_beta1", "adam_beta2", "adam_eps",
                     "weight_decay", "grad_clip", "loss_scale", "embed_lr_mult", "scalar_lr_mult", "lambda_lr_mult",
                     "lambda_beta1", "lambda_beta2", "device", "rank", "world_size", "ce_chunk_rows", "ce_chunk_cols"):
            setattr(o, name, getattr(opts, name))
        o.use_ane = int(opts.use_ane)
        o.hybrid_backward = int(opts.hybrid_backward)
        o.debug_taps = int(opts.debug_taps)
        tok_ptr, n_tok = None, 0
        if opts.tokens is not None and len(opts.tokens) > 0:
            toks = np.ascontiguousarray(opts.tokens, dtype=np.uint16)
            tok_ptr, n_tok = _u16p(toks), toks.size
        dp = None
        if opts.dp_id is not None:
            dp = (c_uint8 * 128).from_buffer_copy(opts.dp_id)
        h = c_void_p()
        rc = lib.ane_open(byref(o), tok_ptr, n_tok, dp, byref(h))
        if rc != 0:
            raise EngineError(rc, lib.ane_last_error(None).decode())
        eng = Engine(h, opts)
        if opts.model_path:
            # ane/engine.go:250-257: a llama2.c model file first, else a training checkpoint (weights and
            # optimizer state only: Open does not restore counters, the trailer or the learning rate)
            from . import checkpoint
            try:
                try:
                    checkpoint.load_pretrained(eng, opts.model_path)
                except (ValueError, OSError) as first:
                    try:
                        checkpoint.load_weights_and_moments(eng, opts.model_path)
                    except (ValueError, OSError):
                        raise EngineError(-1, f"storiesane open: load model: {first}") from first
            except Exception:
                eng.close()
                raise
        return eng

    def _check(self, rc: int):
        if rc != 0:
            raise EngineError(rc, lib.ane_last_error(self._h).decode())

    def _alive(self, what: str):
        if not self._h:
            raise EngineError(-1, f"storiesane {what}: engine is closed")

    def close(self):  # ane/engine.go:567
        if self._h:
            lib.ane_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _result(r: _ffi.StepResult) -> StepResult:
        return StepResult(loss=r.loss, step_duration=r.step_ns * 1e-9, device_eval_duration=r.device_eval_ns * 1e-9,
                          cpu_work_duration=r.cpu_work_ns * 1e-9, adam_duration=r.adam_ns * 1e-9,
                          flushed=bool(r.flushed), device_status=r.device_status)

    def step(self) -> StepResult:  # ane/engine.go:381
        self._alive("step")
        r = _ffi.StepResult()
        r.struct_size = ctypes.sizeof(_ffi.StepResult)
        self._check(lib.ane_step(self._h, byref(r)))
        return self._result(r)

    def step_tokens(self, inp: np.ndarray, tgt: np.ndarray) -> StepResult:
        self._alive("step")
        inp = np.ascontiguousarray(inp, dtype=np.uint16)
        tgt = np.ascontiguousarray(tgt, dtype=np.uint16)
        n_seq = inp.size // self.seq
        r = _ffi.StepResult()
        r.struct_size = ctypes.sizeof(_ffi.StepResult)
        self._check(lib.ane_step_tokens(self._h, _u16p(inp), _u16p(tgt), n_seq, byref(r)))
        return self._result(r)

    def flush(self) -> float:  # ane/engine.go:484
        self._alive("flush")
        ms = c_double(0)
        self._check(lib.ane_flush(self._h, byref(ms)))
        return ms.value

    @property
    def seq(self) -> int:
        return self.opts.seq if self.opts.seq > 0 else 256

    @property
    def vocab(self) -> int:
        return self.opts.vocab if self.opts.vocab > 0 else 32000

    def eval_logits(self, tokens: np.ndarray, layout: int = 0, out: np.ndarray | None = None) -> np.ndarray:
        """ane/engine.go:449.  Returns a fresh array like the reference does; `out` lets a caller that
        evaluates many windows reuse one (a fresh 32 MB array costs page faults on every call)."""
        self._alive("eval logits")
        tokens = np.ascontiguousarray(tokens, dtype=np.uint16)
        if tokens.size % self.seq != 0 or tokens.size == 0:
            raise EngineError(-1, f"storiesane eval logits: token len={tokens.size} want={self.seq}")
        n_seq = tokens.size // self.seq
        shape = (n_seq, self.vocab, self.seq) if layout == 0 else (n_seq * self.seq, self.vocab)
        if out is None:
            out = np.empty(shape, dtype=np.float32)
        elif out.dtype != np.float32 or not out.flags.c_contiguous or out.size != int(np.prod(shape)):
            raise EngineError(-1, "storiesane eval logits: out must be a C-contiguous float32 array of the result's size")
        self._check(lib.ane_eval_logits(self._h, _u16p(tokens), n_seq, out.ctypes.data_as(POINTER(c_float)), out.size,
                                        layout))
        return out

    def eval_loss(self, tokens: np.ndarray) -> tuple[float, int]:
        self._alive("eval loss")
        tokens = np.ascontiguousarray(tokens, dtype=np.uint16)
        n_seq = tokens.size // self.seq
        s, n = c_double(0), c_uint64(0)
        self._check(lib.ane_eval_loss(self._h, _u16p(tokens), n_seq, byref(s), byref(n)))
        return s.value, int(n.value)

    def decode_greedy(self, prompts: np.ndarray, n_new: int) -> np.ndarray:
        """prompts [n_seq, prompt_len] -> generated tokens [n_seq, n_new] (KV-cached greedy decoding)."""
        self._alive("decode")
        prompts = np.ascontiguousarray(prompts, dtype=np.uint16)
        n_seq, plen = prompts.shape
        out = np.empty((n_seq, n_new), dtype=np.uint16)
        self._check(lib.ane_decode_greedy(self._h, _u16p(prompts), n_seq, plen, n_new, _u16p(out)))
        return out

    def decode_sample(self, prompts: np.ndarray, n_new: int, temperature: float, uniforms: np.ndarray) -> np.ndarray:
        """decode_greedy with the reference's temperature sampler (ane/train_full.go:318-342); `uniforms`
        [n_new, n_seq] holds the caller's draws in [0, 1), one per generated token."""
        self._alive("decode")
        prompts = np.ascontiguousarray(prompts, dtype=np.uint16)
        n_seq, plen = prompts.shape
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
        if uniforms.shape != (n_new, n_seq):
            raise EngineError(-1, f"storiesane decode: uniforms shape={uniforms.shape} want={(n_new, n_seq)}")
        out = np.empty((n_seq, n_new), dtype=np.uint16)
        self._check(lib.ane_decode_sample(self._h, _u16p(prompts), n_seq, plen, n_new, temperature,
                                          uniforms.ctypes.data_as(POINTER(c_double)), _u16p(out)))
        return out

    def lr(self) -> float:  # ane/engine.go:358
        return float(lib.ane_get_lr(self._h)) if self._h else 0.0

    def set_lr(self, lr: float):  # ane/engine.go:366
        self._alive("set lr")
        self._check(lib.ane_set_lr(self._h, lr))

    def state(self) -> State:  # ane/engine.go:498
        if not self._h:
            return State()
        s = _ffi.State()
        s.struct_size = ctypes.sizeof(_ffi.State)
        self._check(lib.ane_get_state(self._h, byref(s)))
        return State(token_pos=s.token_pos, last_loss=s.last_loss, cum_train_ms=s.cum_train_ms,
                     cum_wall_ms=s.cum_wall_ms, cum_steps=s.cum_steps, cum_batches=s.cum_batches, adam_t=s.adam_t,
                     pending_steps=s.pending_steps)

    def load_state(self, st: State):  # ane/engine.go:506
        self._alive("load state")
        s = _ffi.State()
        s.struct_size = ctypes.sizeof(_ffi.State)
        for k in ("token_pos", "last_loss", "cum_train_ms", "cum_wall_ms", "cum_steps", "cum_batches", "adam_t",
                  "pending_steps"):
            setattr(s, k, getattr(st, k))
        self._check(lib.ane_set_state(self._h, byref(s)))

    def reseed(self, seed: int):
        """Restart the window sampler from drand48Seed(seed) (ane/engine.go:559, :873)."""
        self._alive("reseed")
        self._check(lib.ane_reseed(self._h, int(seed)))

    # -- tensors and taps
    def tensor_size(self, tid: int, layer: int = 0) -> int:
        return int(lib.ane_tensor_size(self._h, tid, layer))

    def import_tensor(self, tid: int, layer: int, arr: np.ndarray, which: int = W):
        a = np.ascontiguousarray(arr, dtype=np.float32).ravel()
        self._check(lib.ane_import_tensor(self._h, tid, layer, which, a.ctypes.data_as(POINTER(c_float)), a.size))

    def export_tensor(self, tid: int, layer: int = 0, which: int = W) -> np.ndarray | None:
        n = self.tensor_size(tid, layer)
        if n <= 0:
            return None
        out = np.empty(n, dtype=np.float32)
        self._check(lib.ane_export_tensor(self._h, tid, layer, which, out.ctypes.data_as(POINTER(c_float)), n))
        return out

    def tap(self, tap_id: int, layer: int = 0, max_floats: int | None = None) -> np.ndarray | None:
        cap = max_floats or (self.opts.batch or 1) * self.seq * max(
            self.opts.hidden or 2048, (self.opts.dim or 768) * 3, 1) * 2
        buf = np.empty(cap, dtype=np.float32)
        n = lib.ane_get_tap(self._h, tap_id, layer, buf.ctypes.data_as(POINTER(c_float)), cap)
        if n < 0:
            raise EngineError(int(n), lib.ane_last_error(self._h).decode())
        if n == 0:
            return None
        return buf[:n].reshape(-1, self.seq)

    def timer_begin(self):
        self._check(lib.ane_engine_timer_begin(self._h))

    def timer_end(self) -> float:
        ms = c_float(0)
        self._check(lib.ane_engine_timer_end(self._h, byref(ms)))
        return float(ms.value)

    def profile_gemm(self, enable: bool):
        self._check(lib.ane_profile_gemm(self._h, int(enable)))

    def profile_read(self) -> tuple[float, float, int]:
        ms, fl, n = c_double(0), c_double(0), c_uint64(0)
        self._check(lib.ane_profile_read(self._h, byref(ms), byref(fl), byref(n)))
        return ms.value, fl.value, int(n.value)

    def launch_count(self) -> int:
        return int(lib.ane_launch_count(self._h))


def pinned_empty(shape, dtype=np.float32) -> np.ndarray:
    """An uninitialised array in page-locked host memory (ane_host_malloc), freed when the array and its views are
    gone.  Engine.eval_logits(out=...) writes such an array straight from the device, without the staging copy an
    ordinary array needs."""
    dt = np.dtype(dtype)
    count = int(np.prod(shape))
    nbytes = max(1, count * dt.itemsize)
    p = lib.ane_host_malloc(nbytes)
    if not p:
        raise MemoryError(lib.ane_ops_last_error().decode())
    buf = (ctypes.c_byte * nbytes).from_address(p)
    weakref.finalize(buf, lib.ane_host_free, p)
    return np.frombuffer(buf, dtype=dt, count=count).reshape(shape)


def open(opts: Options) -> Engine:  # noqa: A001 - mirrors ane.Open
    return Engine.open(opts)
