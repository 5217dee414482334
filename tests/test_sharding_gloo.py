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


def _exchange_case(world):
    """(L, d): every rank owns at least one 64-key tile of K/V."""
    return (192 if world <= 3 else 64 * world), 16


def _exchange_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry

    pkg, orc = entry.load(), entry.load_oracle()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, d = _exchange_case(world)
        Q, K, V = seeded_qkv(L, d, 31)
        _, row_off, col = random_csr(L, L, 0.15, 8, empty_rows=(7,))
        off_t, col_t = torch.from_numpy(row_off.astype(np.int64)), torch.from_numpy(col.astype(np.int32))
        q_ranges = pkg.sharding.nnz_balanced_row_ranges(off_t, world)   # query rows: balanced by mask entries
        kv_ranges = pkg.sharding.equal_row_ranges(L, world, multiple=64)  # K/V: equal chunks on key-tile multiples
        rb, re = q_ranges[rank]
        my_off, my_col = pkg.sharding.csr_shard(off_t, col_t, rb, re)
        my_off, my_col = my_off.numpy(), my_col.numpy()
        ex = pkg.sharding.KeyChunkExchange(L, d, kv_ranges, rank, world, "cpu")
        ex.K.fill_(float("nan"))
        ex.V.fill_(float("nan"))
        kb, ke = kv_ranges[rank]
        Ko, Vo = ex.own()
        Ko.copy_(torch.from_numpy(K[kb:ke]))
        Vo.copy_(torch.from_numpy(V[kb:ke]))
        state = orc.new_state(re - rb, d)
        seen, log = [], []

        def before():
            log.append("before")

        def on_chunk(a, b, i):
            log.append(i)
            # the chunk has landed; chunks not yet received are still poison
            assert not torch.isnan(ex.K[a:b]).any() and not torch.isnan(ex.V[a:b]).any()
            seen.append((a, b))
            have = np.zeros(L, dtype=bool)
            for x, y in seen:
                have[x:y] = True
            assert np.array_equal(~np.isnan(ex.K.numpy()).any(axis=1), have)
            # this pass: the mask entries of my rows whose key lies in [a, b)
            keep = (my_col >= a) & (my_col < b)
            rows = np.repeat(np.arange(re - rb), np.diff(my_off))
            cnt = np.bincount(rows[keep], minlength=re - rb)
            off2 = np.concatenate([[0], np.cumsum(cnt)]).astype(np.uint64)
            Kc, Vc = np.nan_to_num(ex.K.numpy()), np.nan_to_num(ex.V.numpy())
            orc.csr_forward(Q[rb:re], Kc, Vc, off2, my_col[keep], state=state)

        ex.run(on_chunk, before)
        assert log[0] == "before" and log[1:] == list(range(world))
        assert sorted(seen) == sorted(kv_ranges) and seen[0] == kv_ranges[rank]
        assert torch.equal(ex.K, torch.from_numpy(K)) and torch.equal(ex.V, torch.from_numpy(V))
        # the same forward in two passes: keys landed after the first round(s), then the rest (cyclic key ranges)
        state2 = orc.new_state(re - rb, d)
        for t in (ex.K, ex.V):
            t[:kb].fill_(float("nan"))
            t[ke:].fill_(float("nan"))
        calls = []

        def on_keys(a, b, i):
            inside = np.zeros(L, dtype=bool)
            if a < b:
                inside[a:b] = True
            else:
                inside[a:] = True
                inside[:b] = True
            assert not np.isnan(ex.K.numpy()[inside]).any()  # everything this pass may read has landed
            calls.append((a, b, i))
            keep = inside[my_col]
            rows = np.repeat(np.arange(re - rb), np.diff(my_off))
            cnt = np.bincount(rows[keep], minlength=re - rb)
            off2 = np.concatenate([[0], np.cumsum(cnt)]).astype(np.uint64)
            orc.csr_forward(Q[rb:re], np.nan_to_num(ex.K.numpy()), np.nan_to_num(ex.V.numpy()), off2, my_col[keep],
                            state=state2)

        ex.run_two_phase(on_keys, rounds_in_phase1=1 if world > 2 else 0)
        assert [c[2] for c in calls] == [0, 1]
        np.testing.assert_allclose(state2[2], state[2], rtol=0, atol=1e-12)
        # dense tiles of the own chunk first, the other tiles and the residual pass after the last round
        for t in (ex.K, ex.V):
            t[:kb].fill_(float("nan"))
            t[ke:].fill_(float("nan"))
        order = []

        def on_tiles(a, b):
            inside = np.zeros(L, dtype=bool)
            if a < b:
                inside[a:b] = True
            else:
                inside[a:] = True
                inside[:b] = True
            assert not np.isnan(ex.K.numpy()[inside]).any()
            order.append(("tiles", a, b, bool(np.isnan(ex.K.numpy()).any())))

        def on_rest():
            assert not np.isnan(ex.K.numpy()).any() and not np.isnan(ex.V.numpy()).any()
            order.append(("rest",))

        ex.run_tiles_first(on_tiles, on_rest, before=lambda: order.append(("before",)))
        assert [o[0] for o in order] == ["before", "tiles", "tiles", "rest"]
        assert (order[1][1], order[1][2]) == (kb, ke) and order[1][3]  # own chunk, while other chunks are still poison
        covered = np.zeros(L, dtype=int)
        for _, a, b, _ in order[1:3]:
            if a < b:
                covered[a:b] += 1
            else:
                covered[a:] += 1
                covered[:b] += 1
        assert (covered == 1).all()  # the two tile passes partition the keys
        np.savez(os.path.join(tmp, f"ex{rank}.npz"), rb=rb, re=re, O=state[2], l=state[1])
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3, 8])
def test_key_chunk_exchange_orders_passes_behind_arrivals(pkg, orc, tmp_path, world):
    """The overlapped K/V replication: every pass runs only after its chunk has landed (the rest of the buffers is
    still poison), the own chunk comes first, all chunks are seen exactly once, and the passes chained through the
    softmax state give the unsplit result."""
    assert pkg.sharding.exchange_offsets(8) == [1, 7, 2, 6, 3, 5, 4] and pkg.sharding.exchange_offsets(2) == [1]
    assert pkg.sharding.exchange_offsets(1) == [] and sorted(pkg.sharding.exchange_offsets(5)) == [1, 2, 3, 4]
    port = 31500 + (os.getpid() % 2000) + world
    mp.spawn(_exchange_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    L, d = _exchange_case(world)
    Q, K, V = seeded_qkv(L, d, 31)
    _, row_off, col = random_csr(L, L, 0.15, 8, empty_rows=(7,))
    want = orc.csr_forward(Q, K, V, row_off, col)
    parts = sorted((np.load(os.path.join(tmp_path, f"ex{r}.npz")) for r in range(world)), key=lambda p: int(p["rb"]))
    np.testing.assert_allclose(np.concatenate([p["O"] for p in parts]), want[2], rtol=0, atol=1e-12)
    np.testing.assert_allclose(np.concatenate([p["l"] for p in parts]), want[1], rtol=1e-12)


def test_two_phase_ranges_partition_the_keys_even_with_empty_chunks(pkg):
    """Whatever the chunks are (more ranks than key tiles leave some ranks an empty chunk), the two passes of every rank
    cover every key exactly once, for every number of rounds in pass 1."""
    Ex = pkg.sharding.KeyChunkExchange
    for L, world in ((192, 8), (512, 8), (192, 3), (128, 2), (64, 4), (1024, 5)):
        kv = pkg.sharding.equal_row_ranges(L, world, multiple=64)
        for rank in range(world):
            for rounds in range(world + 1):
                ex = object.__new__(Ex)
                ex.L, ex.world, ex.rank, ex.kv_ranges = L, world, rank, kv
                p1, p2 = ex.two_phase_ranges(rounds)
                covered = np.zeros(L, dtype=int)
                for rng in (p1, p2):
                    if rng is None or rng[0] == rng[1]:
                        continue
                    a, b = rng
                    assert a % 64 == 0 and (b % 64 == 0 or b == L)
                    if a < b:
                        covered[a:b] += 1
                    else:
                        covered[a:] += 1
                        covered[:b] += 1
                assert (covered == 1).all(), (L, world, rank, rounds, p1, p2)
                # pass 1 reads only chunks that have arrived after `rounds` rounds
                offs = pkg.sharding.exchange_offsets(world)[:min(rounds, world - 1)]
                have = np.zeros(L, dtype=bool)
                for r in [rank] + [(rank - o) % world for o in offs]:
                    have[kv[r][0]:kv[r][1]] = True
                if p1[0] != p1[1]:
                    a, b = p1
                    inside = np.zeros(L, dtype=bool)
                    if a < b:
                        inside[a:b] = True
                    else:
                        inside[a:] = True
                        inside[:b] = True
                    assert have[inside].all(), (L, world, rank, rounds, p1)


def test_default_schedule_of_the_sharded_forward(pkg):
    """One pass after the exchange up to four ranks; from eight ranks on a first pass after about 4/7 of the rounds."""
    f = pkg.sharding.default_rounds_in_phase1
    assert [f(w) for w in (1, 2, 3, 4)] == [0, 1, 2, 3]  # world - 1: everything in the first pass
    assert f(8) == 4 and 0 < f(16) < 15
