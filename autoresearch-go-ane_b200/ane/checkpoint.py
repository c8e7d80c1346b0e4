"""Checkpoint files of the reference, read and written against device-resident state.

  V5 training checkpoint   ane/stories/ckpt.go:77-269 (writer), :271-405 + :421-579 (reader)
  "SANE" trailer           ane/engine.go:684-791 (token position, pending micro-steps, accumulated gradients)
  Engine.SaveCheckpoint / LoadCheckpoint   ane/engine.go:515-565
  llama2.c model file      ane/stories/weights.go:73-153 (LoadPretrained)

Every tensor goes through Engine.export_tensor / import_tensor, so the file layout lives here and the
library never sees a path.  All numbers are little-endian; tensors are flat fp32 in the reference's
row-major [out, in] order, which is also the order of the tensor import/export calls.

The V5 layout has no slot for RMSNorm weights or W3, so it describes the reference architecture only;
the llama-style architecture is saved with the same header and trailer under version 105 (V5 sections
plus W3 after W2 and the norm weights after the per-layer matrices), a format of this library.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass

import numpy as np

from . import engine as E
from ._ffi import ARCH_LLAMA, ARCH_REFERENCE

CKPT_MAGIC = 0x424C5A54          # ane/stories/ckpt.go:12
CKPT_VERSION_V5 = 5              # ane/stories/ckpt.go:16
CKPT_VERSION_LLAMA = 105         # this library: V5 layout + W3 + RMSNorm weights
HEADER_BYTES = 96                # ane/engine.go:768
TRAILER_MAGIC = b"SANE"          # ane/engine.go:685
TRAILER_V1, TRAILER_V2 = 1, 2    # ane/engine.go:686-687
_HEADER = struct.Struct("<10i2f3d3i3i")


@dataclass
class TrainMeta:
    """stories.TrainMeta (ane/stories/ckpt.go:26-37)."""
    step: int = 0
    total_steps: int = 0
    lr: float = 0.0
    loss: float = 0.0
    cum_compile: float = 0.0
    cum_train: float = 0.0
    cum_wall: float = 0.0
    cum_steps: int = 0
    cum_batches: int = 0
    adam_t: int = 0


@dataclass
class Dims:
    layers: int
    vocab: int
    dim: int
    hidden: int
    heads: int
    seq: int
    arch: int


def dims_of(engine) -> Dims:
    """The engine's effective sizes (zero option fields mean the reference's 110M values,
    ane/stories/config.go:3-18)."""
    o = engine.opts
    return Dims(layers=o.n_layers or 12, vocab=o.vocab or 32000, dim=o.dim or 768, hidden=o.hidden or 2048,
                heads=o.n_heads or 12, seq=o.seq or 256, arch=o.arch)


def pack_header(version: int, meta: TrainMeta, d: Dims) -> bytes:
    """ane/stories/ckpt.go:103-160: ten int32, lr and loss, three float64 clocks, three counters, three
    zero words."""
    return _HEADER.pack(CKPT_MAGIC, version, meta.step, meta.total_steps, d.layers, d.vocab, d.dim, d.hidden, d.heads,
                        d.seq, meta.lr, meta.loss, meta.cum_compile, meta.cum_train, meta.cum_wall, meta.cum_steps,
                        meta.cum_batches, meta.adam_t, 0, 0, 0)


def unpack_header(raw: bytes, d: Dims) -> tuple[int, TrainMeta]:
    """ane/stories/ckpt.go:299-395.  The stored sequence length is read and ignored, like the reference does."""
    if len(raw) < HEADER_BYTES:
        raise ValueError("unexpected EOF")
    f = _HEADER.unpack(raw[:HEADER_BYTES])
    magic, ver = f[0], f[1]
    if magic != CKPT_MAGIC or ver not in (2, 3, 4, CKPT_VERSION_V5, CKPT_VERSION_LLAMA):
        raise ValueError(f"bad checkpoint header magic={magic & 0xffffffff:x} version={ver}")
    if (f[4], f[5], f[6], f[7], f[8]) != (d.layers, d.vocab, d.dim, d.hidden, d.heads):
        raise ValueError("checkpoint config mismatch")
    if ver in (2, 3, 4):
        raise ValueError(f"checkpoint version {ver}: only V5 files are read (older layouts carry tensors "
                         "the current model no longer has)")
    meta = TrainMeta(step=f[2], total_steps=f[3], lr=f[10], loss=f[11], cum_compile=f[12], cum_train=f[13],
                     cum_wall=f[14], cum_steps=f[15], cum_batches=f[16], adam_t=f[17])
    return ver, meta


def is_ve_layer(layer: int, d: Dims) -> bool:
    """ane/stories/weights.go:22."""
    return d.arch == ARCH_REFERENCE and layer % 2 == (d.layers - 1) % 2


def _layer_weight_ids(d: Dims) -> list[int]:
    ids = [E.T_WQ, E.T_WK, E.T_WV, E.T_WO, E.T_W1, E.T_W2]
    if d.arch == ARCH_LLAMA:
        ids += [E.T_W3, E.T_RMS_ATT, E.T_RMS_FFN]
    return ids + [E.T_VE_EMBED, E.T_VE_GATE]


def _model_ids(d: Dims) -> list[int]:
    if d.arch == ARCH_LLAMA:
        return [E.T_EMBED, E.T_RMS_FINAL]
    return [E.T_EMBED, E.T_RESID_LAMBDAS, E.T_X0_LAMBDAS, E.T_SMEAR_GATE, E.T_SMEAR_LAMBDA, E.T_BACKOUT_LAMBDA]


def sections(d: Dims) -> list[tuple[int, int, int]]:
    """(tensor id, layer, which) in file order, ane/stories/ckpt.go:162-262: every layer's weights, then
    every layer's Adam moments (m, v per tensor), then each model-level tensor followed by its m and v.
    Tensors a layer does not have (value embeddings on non-VE layers) have size 0 and take no bytes."""
    out = []
    for l in range(d.layers):
        out += [(t, l, E.W) for t in _layer_weight_ids(d)]
    for l in range(d.layers):
        for t in _layer_weight_ids(d):
            out += [(t, l, E.M), (t, l, E.V)]
    for t in _model_ids(d):
        out += [(t, 0, E.W), (t, 0, E.M), (t, 0, E.V)]
    return out


def grad_sections(d: Dims) -> list[tuple[int, int, int]]:
    """Accumulated gradients in trailer order (writeModelGrad, ane/engine.go:811-840)."""
    out = []
    for l in range(d.layers):
        out += [(t, l, E.G) for t in _layer_weight_ids(d)]
    return out + [(t, 0, E.G) for t in _model_ids(d)]


def checkpoint_size(engine) -> int:
    """storiesCheckpointSize (ane/engine.go:767-791): bytes before the trailer."""
    d = dims_of(engine)
    return HEADER_BYTES + 4 * sum(max(0, engine.tensor_size(t, l)) for t, l, _ in sections(d))


def save_checkpoint(engine, path: str, meta: TrainMeta | None = None) -> TrainMeta:
    """Engine.SaveCheckpoint (ane/engine.go:515-531): the meta's lr, loss, clocks and counters are taken
    from the engine; written to path.tmp and renamed (ane/stories/ckpt.go:88-90,258-266)."""
    engine._alive("save checkpoint")
    d = dims_of(engine)
    st = engine.state()
    meta = meta or TrainMeta()
    meta.lr, meta.loss = engine.lr(), st.last_loss
    meta.cum_train, meta.cum_wall = st.cum_train_ms, st.cum_wall_ms
    meta.cum_steps, meta.cum_batches, meta.adam_t = st.cum_steps, st.cum_batches, st.adam_t
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(pack_header(CKPT_VERSION_V5 if d.arch == ARCH_REFERENCE else CKPT_VERSION_LLAMA, meta, d))
        for t, l, which in sections(d):
            a = engine.export_tensor(t, l, which)
            if a is not None:
                a.astype("<f4", copy=False).tofile(f)
        # trailer, version 2 (ane/engine.go:690-716): the engine always holds accumulation buffers
        f.write(TRAILER_MAGIC)
        f.write(struct.pack("<IQI", TRAILER_V2, st.token_pos, st.pending_steps))
        for t, l, which in grad_sections(d):
            a = engine.export_tensor(t, l, which)
            if a is not None:
                a.astype("<f4", copy=False).tofile(f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return meta


def _read_into(f, n: int) -> np.ndarray:
    a = np.fromfile(f, dtype="<f4", count=n)
    if a.size != n:
        raise ValueError("unexpected EOF")
    return a


def load_weights_and_moments(engine, path: str) -> TrainMeta:
    """stories.LoadCheckpoint as ane.Open uses it on a ModelPath that is not a llama2.c file
    (ane/engine.go:252): weights and Adam moments only; counters, learning rate and trailer stay untouched."""
    engine._alive("open")
    d = dims_of(engine)
    with open(path, "rb") as f:
        ver, meta = unpack_header(f.read(HEADER_BYTES), d)
        if (ver == CKPT_VERSION_V5) != (d.arch == ARCH_REFERENCE):
            raise ValueError("checkpoint config mismatch")
        for t, l, which in sections(d):
            n = engine.tensor_size(t, l)
            if n > 0:
                engine.import_tensor(t, l, _read_into(f, n), which)
    return meta


def random_init(engine, seed: int) -> None:
    """Fresh weights with the distributions of stories.RandomInit (ane/stories/weights.go:165-210) for the
    reference architecture: Wq/Wk/Wv/W1/value embeddings uniform in +-sqrt(3/dim), Wo and W2 zero, value-embedding
    gates uniform in [0, 0.02), embedding standard normal, residual lambdas 1, x0 lambdas 0.1, smear gate
    uniform in +-1/sqrt(dim), smear and backout lambdas 0.01.  Go's math/rand stream is not
    restated, so the values are statistically, not bitwise, those of the reference for the same seed.  The
    llama-style architecture gets N(0, 0.02) matrices and unit norm weights."""
    engine._alive("random init")
    d = dims_of(engine)
    rng = np.random.default_rng(seed)
    hd = d.dim // d.heads
    kvd = (engine.opts.n_kv_heads or d.heads) * hd
    if d.arch == ARCH_REFERENCE:
        s = float(np.sqrt(3.0) / np.sqrt(d.dim))
        uni = lambda n, a: (a * (2.0 * rng.random(n, dtype=np.float32) - 1.0)).astype(np.float32)  # noqa: E731
        for l in range(d.layers):
            engine.import_tensor(E.T_WQ, l, uni(d.dim * d.dim, s))
            engine.import_tensor(E.T_WK, l, uni(kvd * d.dim, s))
            engine.import_tensor(E.T_WV, l, uni(kvd * d.dim, s))
            engine.import_tensor(E.T_WO, l, np.zeros(d.dim * d.dim, np.float32))
            engine.import_tensor(E.T_W1, l, uni(d.hidden * d.dim, s))
            engine.import_tensor(E.T_W2, l, np.zeros(d.dim * d.hidden, np.float32))
            if is_ve_layer(l, d):
                engine.import_tensor(E.T_VE_EMBED, l, uni(d.vocab * d.dim, s))
                engine.import_tensor(E.T_VE_GATE, l, (0.02 * rng.random(d.heads * 12, dtype=np.float32)))
        engine.import_tensor(E.T_EMBED, 0, rng.standard_normal(d.vocab * d.dim, dtype=np.float32))
        engine.import_tensor(E.T_RESID_LAMBDAS, 0, np.ones(d.layers, np.float32))
        engine.import_tensor(E.T_X0_LAMBDAS, 0, np.full(d.layers, 0.1, np.float32))
        engine.import_tensor(E.T_SMEAR_GATE, 0, uni(d.dim * d.dim, float(1.0 / np.sqrt(d.dim))))
        engine.import_tensor(E.T_SMEAR_LAMBDA, 0, np.full(1, 0.01, np.float32))
        engine.import_tensor(E.T_BACKOUT_LAMBDA, 0, np.full(1, 0.01, np.float32))
        return
    nrm = lambda n: (0.02 * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)  # noqa: E731
    for l in range(d.layers):
        engine.import_tensor(E.T_WQ, l, nrm(d.dim * d.dim))
        engine.import_tensor(E.T_WK, l, nrm(kvd * d.dim))
        engine.import_tensor(E.T_WV, l, nrm(kvd * d.dim))
        engine.import_tensor(E.T_WO, l, nrm(d.dim * d.dim))
        engine.import_tensor(E.T_W1, l, nrm(d.hidden * d.dim))
        engine.import_tensor(E.T_W3, l, nrm(d.hidden * d.dim))
        engine.import_tensor(E.T_W2, l, nrm(d.dim * d.hidden))
    engine.import_tensor(E.T_EMBED, 0, nrm(d.vocab * d.dim))


def load_checkpoint(engine, path: str) -> TrainMeta:
    """Engine.LoadCheckpoint (ane/engine.go:534-565): weights, Adam moments, lr and counters from the file;
    pending gradients are cleared and then restored from a version-2 trailer when one follows; a missing
    trailer or a foreign magic is not an error (ane/engine.go:726-735).  The window sampler restarts from
    drand48Seed(seed + meta.step) and the wall clock continues from the stored total (ane/engine.go:559-560)."""
    engine._alive("load checkpoint")
    d = dims_of(engine)
    with open(path, "rb") as f:
        ver, meta = unpack_header(f.read(HEADER_BYTES), d)
        if (ver == CKPT_VERSION_V5) != (d.arch == ARCH_REFERENCE):
            raise ValueError("checkpoint config mismatch")
        for t, l, which in sections(d):
            n = engine.tensor_size(t, l)
            if n > 0:
                engine.import_tensor(t, l, _read_into(f, n), which)
        st = E.State(last_loss=meta.loss, cum_train_ms=meta.cum_train, cum_wall_ms=meta.cum_wall,
                     cum_steps=meta.cum_steps, cum_batches=meta.cum_batches, adam_t=meta.adam_t)
        grads = None
        magic = f.read(4)
        if magic == TRAILER_MAGIC:
            raw = f.read(16)
            if len(raw) != 16:
                raise ValueError("storiesane load trailer: read version: unexpected EOF")
            tver, st.token_pos, st.pending_steps = struct.unpack("<IQI", raw)
            if tver == TRAILER_V2:
                grads = f
            elif tver != TRAILER_V1:  # V1 carries two buffers that no longer exist; they are skipped
                raise ValueError(f"storiesane load trailer: unsupported version {tver}")
        for t, l, which in grad_sections(d):
            n = engine.tensor_size(t, l)
            if n > 0:
                engine.import_tensor(t, l, _read_into(f, n) if grads is not None else np.zeros(n, np.float32), which)
    engine.set_lr(meta.lr)
    engine.load_state(st)
    engine.reseed((engine.opts.seed or 42) + meta.step)
    return meta


LLAMA2C_HEADER = struct.Struct("<7i")  # dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len


def load_pretrained(engine, path: str) -> dict:
    """stories.LoadPretrained (ane/stories/weights.go:73-153) for a llama2.c model file: header of seven
    int32, then embedding, rms_att, wq, wk, wv, wo, rms_ffn, w1, w2, w3, rms_final, each stacked over
    layers.  The reference architecture has no norm weights and no W3 and skips them, as the reference
    does; the llama-style architecture imports them.  A negative vocab_size marks an untied classifier,
    which neither model has: its absolute value is used, like the reference."""
    engine._alive("load pretrained")
    d = dims_of(engine)
    with open(path, "rb") as f:
        raw = f.read(LLAMA2C_HEADER.size)
        if len(raw) != LLAMA2C_HEADER.size:
            raise ValueError("read config: unexpected EOF")
        dim, hidden, layers, heads, kv_heads, vocab, seq = LLAMA2C_HEADER.unpack(raw)
        if (dim, hidden, layers) != (d.dim, d.hidden, d.layers):
            raise ValueError(f"config mismatch: got dim={dim} hidden={hidden} layers={layers}")
        if abs(vocab) != d.vocab:
            raise ValueError(f"config mismatch: got vocab={abs(vocab)}")
        llama = d.arch == ARCH_LLAMA
        kv_dim = dim // heads * kv_heads

        def stacked(tid, per_layer, keep=True):
            for l in range(layers):
                a = _read_into(f, per_layer)
                if keep:
                    engine.import_tensor(tid, l, a)

        engine.import_tensor(E.T_EMBED, 0, _read_into(f, d.vocab * dim))
        stacked(E.T_RMS_ATT, dim, keep=llama)
        stacked(E.T_WQ, dim * dim)
        stacked(E.T_WK, kv_dim * dim)
        stacked(E.T_WV, kv_dim * dim)
        stacked(E.T_WO, dim * dim)
        stacked(E.T_RMS_FFN, dim, keep=llama)
        stacked(E.T_W1, hidden * dim)
        stacked(E.T_W2, dim * hidden)
        stacked(E.T_W3, hidden * dim, keep=llama)
        rms_final = _read_into(f, dim)
        if llama:
            engine.import_tensor(E.T_RMS_FINAL, 0, rms_final)
    return dict(dim=dim, hidden_dim=hidden, n_layers=layers, n_heads=heads, n_kv_heads=kv_heads, vocab_size=vocab,
                seq_len=seq, shared_classifier=vocab > 0)
