"""Data-parallel host logic on CPU with world_size-2 gloo ranks (no GPU):
 * the window sampler shards one drand48 stream round-robin over ranks;
 * summing per-rank gradients with an all-reduce and dividing by the global sequence count is the
   reference's accumulate-then-flush (ane/train_full.go:811-818, ane/engine.go:650-654): two ranks with
   half the sequences each end at the same weights as one process with all of them."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(dim=32, hidden=48, heads=4, layers=2, vocab=64, seq=12)
HYPER = dict(lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1, grad_clip=1.0, loss_scale=256.0)
N_TOK, BATCH, SEED = 4096, 2, 42


def _paths():
    for p in (ROOT, os.path.join(ROOT, "autoresearch-go-ane_b200"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)


def _worker(rank, world, port, out_dir):
    _paths()
    import ctypes

    from ane import _ffi
    from oracle import oracle as O

    os.environ["ANE_ORACLE_THREADS"] = "2"
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    toks = O.zipf_tokens(N_TOK, CFG["vocab"], 3)
    m = O.Model(arch=O.ARCH_N, quirks=1, accum_steps=1 << 20, **CFG, **HYPER)
    O.init_weights(m, 5, std=0.2)
    rng = ctypes.c_uint64(_ffi.lib.ane_sampler_seed(SEED))
    all_pos = []
    for step in range(3):
        pos = (ctypes.c_uint64 * BATCH)()
        assert _ffi.lib.ane_sample_windows(ctypes.byref(rng), N_TOK, CFG["seq"], BATCH, rank, world, pos) == 0
        all_pos.append(list(pos))
        for p in pos:
            m.accumulate(toks[p:p + CFG["seq"]].copy(), toks[p + 1:p + 1 + CFG["seq"]].copy())
        # gradient all-reduce (sum) over the flat set of tensors, then the reference flush with the
        # global number of pending sequences
        for _, _, g in m.tensors(O.G):
            t = torch.from_numpy(g)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        # orc_flush divides by its own pending count (local); rescale so the division is by the global one
        for _, _, g in m.tensors(O.G):
            g /= world
        m.flush()
    gathered = [None] * world
    dist.all_gather_object(gathered, all_pos)
    if rank == 0:
        np.save(os.path.join(out_dir, "positions.npy"), np.array(gathered))
        np.save(os.path.join(out_dir, "wq0.npy"), m.tensor(O.T_WQ, 0).copy())
        np.save(os.path.join(out_dir, "embed.npy"), m.tensor(O.T_EMBED).copy())
    dist.destroy_process_group()


def test_two_rank_data_parallel_matches_single_process(tmp_path):
    _paths()
    from oracle import oracle as O

    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    pos = np.load(tmp_path / "positions.npy")          # [rank][step][batch]
    ref = O.drand48_positions(SEED, N_TOK, CFG["seq"], 3 * BATCH * world)
    # interleaving the ranks' draws reproduces the single reference stream exactly
    got = []
    for step in range(3):
        for b in range(BATCH):
            for r in range(world):
                got.append(int(pos[r][step][b]))
    assert got == ref
    # single-process run over the same global batches
    toks = O.zipf_tokens(N_TOK, CFG["vocab"], 3)
    m = O.Model(arch=O.ARCH_N, quirks=1, accum_steps=BATCH * world, **CFG, **HYPER)
    O.init_weights(m, 5, std=0.2)
    for p in ref:
        m.step(toks[p:p + CFG["seq"]].copy(), toks[p + 1:p + 1 + CFG["seq"]].copy())
    assert m.adam_t == 3
    np.testing.assert_allclose(np.load(tmp_path / "wq0.npy"), m.tensor(O.T_WQ, 0), rtol=2e-4, atol=2e-6)
    np.testing.assert_allclose(np.load(tmp_path / "embed.npy"), m.tensor(O.T_EMBED), rtol=2e-4, atol=2e-6)
