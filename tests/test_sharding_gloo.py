"""CPU: the multi-GPU host logic with world_size=2 over gloo -- row-range partitioning, per-rank mask
slices, K/V replication -- and that per-shard results stitched together equal the unsharded result
(the checker stands in for the kernels here; the kernels themselves only run in the gpu tests)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, random_csr, seeded_qkv


def test_equal_and_balanced_ranges(pkg):
    sh = pkg.sharding
    assert sh.equal_row_ranges(10, 3) == [(0, 3), (3, 6), (6, 10)]
    assert sh.equal_row_ranges(1000, 4, multiple=128) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert sh.equal_row_ranges(5, 8)[-1][1] == 5
    # heavy rows up front: balanced ranges give the first rank fewer rows
    counts = np.array([100] * 10 + [1] * 990)
    off = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]))
    r = sh.nnz_balanced_row_ranges(off, 2)
    assert r[0][0] == 0 and r[-1][1] == 1000 and r[0][1] == r[1][0]
    nnz = [int(off[e] - off[b]) for b, e in r]
    assert max(nnz) / (sum(nnz) / 2) < 1.06
    rows = torch.from_numpy(np.repeat(np.arange(1000), counts))
    r2 = sh.coo_nnz_balanced_row_ranges(rows, 1000, 2)
    assert abs(r2[0][1] - r[0][1]) <= 1


def test_mask_shards(pkg):
    sh = pkg.sharding
    mask, row_off, col = random_csr(64, 64, 0.2, 4, empty_rows=(0, 31, 32, 63))
    off_t, col_t = torch.from_numpy(row_off.astype(np.int64)), torch.from_numpy(col.astype(np.int32))
    o2, c2 = sh.csr_shard(off_t, col_t, 20, 40)
    assert o2[0] == 0 and o2.numel() == 21
    for r in range(20):
        assert np.array_equal(c2[o2[r]:o2[r + 1]].numpy(), np.nonzero(mask[20 + r])[0])
    rows = torch.from_numpy(np.repeat(np.arange(64), mask.sum(1)))
    r3, c3 = sh.coo_shard(rows, col_t, 32, 64)
    assert r3.min() >= 32 and r3.numel() == mask[32:].sum() and np.array_equal(c3.numpy(), col[-r3.numel():])


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry

    pkg, orc = entry.load(), entry.load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, d, w = 96, 16, 5
        Q, K, V = seeded_qkv(L, d, 77)
        ranges = pkg.sharding.equal_row_ranges(L, world)
        b, e = ranges[rank]
        # each rank starts with its own rows of K/V only
        Kf, Vf = pkg.sharding.replicate_kv(torch.from_numpy(K[b:e].copy()), torch.from_numpy(V[b:e].copy()), ranges)
        assert torch.equal(Kf, torch.from_numpy(K)) and torch.equal(Vf, torch.from_numpy(V))
        # ragged shards take the broadcast path
        ragged = [(0, 10), (10, L)]
        rb, re = ragged[rank]
        Kr, _ = pkg.sharding.replicate_kv(torch.from_numpy(K[rb:re].copy()), torch.from_numpy(V[rb:re].copy()), ragged)
        assert torch.equal(Kr, torch.from_numpy(K))
        # this rank's rows, absolute row numbers passed through
        G = np.array([2, 50, 95], dtype=np.int32)
        out = {}
        out["local"] = orc.implicit_forward("local", Q[b:e], Kf.numpy(), Vf.numpy(), w, row_begin=b, row_end=e)[2]
        out["l1d"] = orc.implicit_forward("local_1d_dilated", Q[b:e], Kf.numpy(), Vf.numpy(), w, 2, row_begin=b, row_end=e)[2]
        out["gnl"] = orc.implicit_forward("global_no_local", Q[b:e], Kf.numpy(), Vf.numpy(), w, G=G, row_begin=b, row_end=e)[2]
        np.savez(os.path.join(tmp, f"rank{rank}.npz"), b=b, e=e, **out)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_row_sharding_matches_unsharded(pkg, orc, tmp_path):
    world, port = 2, 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    L, d, w = 96, 16, 5
    Q, K, V = seeded_qkv(L, d, 77)
    G = np.array([2, 50, 95], dtype=np.int32)
    full = {"local": orc.implicit_forward("local", Q, K, V, w)[2],
            "l1d": orc.implicit_forward("local_1d_dilated", Q, K, V, w, 2)[2],
            "gnl": orc.implicit_forward("global_no_local", Q, K, V, w, G=G)[2]}
    for key, want in full.items():
        parts = [np.load(os.path.join(tmp_path, f"rank{r}.npz")) for r in range(world)]
        got = np.concatenate([p[key] for p in parts])
        np.testing.assert_array_equal(got, want)
