"""Query-row-range sharding of one attention forward across the GPUs of a node.

Every query row is independent: its output depends on its own q_i, on the K/V rows its mask selects
and on its own (m_i, l_i, O_i) (the reference runs one CTA per row with no inter-CTA traffic,
Sparse_FlashAttention_CSR/sp_flatt_csr_kernel.cu:29-33,208-218). So the path shards by contiguous row
ranges with NO reduction and no softmax-state exchange; the only data every rank needs in full is K
and V. The reference itself is single-GPU (README.md:10); this module is the one multi-GPU piece added.

Host-side pieces (pure index arithmetic + torch.distributed, usable with the gloo backend on CPU):
  equal_row_ranges / nnz_balanced_row_ranges / coo_nnz_balanced_row_ranges   who owns which rows
  csr_shard / coo_shard                                                      a rank's slice of an explicit mask
  replicate_kv                                                               K/V row shards -> full K/V on every rank
  KeyChunkExchange                                                           the same replication as world-1 rounds of
                                                                             point-to-point sends, with the compute on
                                                                             the chunks that have arrived overlapped
The compute itself is `capi.*_forward(..., row_begin, row_end)` on each rank's rows.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def equal_row_ranges(L: int, world: int, multiple: int = 1) -> list[tuple[int, int]]:
    """Contiguous ranges of (almost) equal row counts; interior boundaries rounded to `multiple`."""
    bounds = [0]
    for r in range(1, world):
        b = (L * r) // world
        b = min(L, (b + multiple - 1) // multiple * multiple)
        bounds.append(max(b, bounds[-1]))
    bounds.append(L)
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def nnz_balanced_row_ranges(row_off: torch.Tensor, world: int) -> list[tuple[int, int]]:
    """Row ranges holding ~nnz/world mask non-zeros each, from CSR row offsets (length L+1).

    Boundary r is the first row whose offset reaches r*nnz/world (rows are not split)."""
    off = row_off.to(torch.int64) if row_off.dtype != torch.int64 else row_off
    L = off.numel() - 1
    nnz = int(off[-1].item()) - int(off[0].item())
    targets = torch.tensor([int(off[0].item()) + (nnz * r) // world for r in range(1, world)], dtype=torch.int64,
                           device=off.device)
    cut = torch.searchsorted(off, targets, right=False).clamp_(0, L).tolist() if world > 1 else []
    bounds = [0]
    for c in cut:
        bounds.append(max(int(c), bounds[-1]))
    bounds.append(L)
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def coo_nnz_balanced_row_ranges(row_ind: torch.Tensor, L: int, world: int) -> list[tuple[int, int]]:
    """Same balance for a row-sorted COO mask: the entry at position r*nnz/world decides boundary r."""
    rows = row_ind.view(torch.int64) if row_ind.dtype == torch.uint64 else row_ind.to(torch.int64)
    nnz = rows.numel()
    bounds = [0]
    for r in range(1, world):
        b = int(rows[(nnz * r) // world].item()) if nnz else (L * r) // world
        bounds.append(min(L, max(b, bounds[-1])))
    bounds.append(L)
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def csr_shard(row_off: torch.Tensor, col_ind: torch.Tensor, row_begin: int, row_end: int):
    """(row_off', col') of rows [row_begin, row_end) with offsets rebased to the sliced column array."""
    off = row_off.view(torch.int64) if row_off.dtype == torch.uint64 else row_off.to(torch.int64)
    lo, hi = int(off[row_begin].item()), int(off[row_end].item())
    return (off[row_begin:row_end + 1] - lo).contiguous(), col_ind[lo:hi].contiguous()


def coo_shard(row_ind: torch.Tensor, col_ind: torch.Tensor, row_begin: int, row_end: int):
    """Entries of rows [row_begin, row_end) of a row-sorted COO mask (row numbers stay absolute)."""
    rows = row_ind.view(torch.int64) if row_ind.dtype == torch.uint64 else row_ind.to(torch.int64)
    edges = torch.searchsorted(rows, torch.tensor([row_begin, row_end], dtype=torch.int64, device=rows.device))
    lo, hi = int(edges[0].item()), int(edges[1].item())
    return rows[lo:hi].contiguous(), col_ind[lo:hi].contiguous()


def replicate_kv(K_shard: torch.Tensor, V_shard: torch.Tensor, ranges: list[tuple[int, int]], group=None):
    """All ranks contribute their K/V row shard and end with the full [L, d] K and V.

    One collective per tensor, no reduction. Equal shards use all_gather_into_tensor (NCCL: a single
    ring/NVLS all-gather over NVLink); ragged shards fall back to per-rank broadcasts into row slices."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    L = ranges[-1][1]
    d = K_shard.shape[1]
    sizes = [e - b for b, e in ranges]
    assert K_shard.shape[0] == sizes[rank] and V_shard.shape[0] == sizes[rank]
    K = torch.empty(L, d, dtype=K_shard.dtype, device=K_shard.device)
    V = torch.empty(L, d, dtype=V_shard.dtype, device=V_shard.device)
    if world == 1:
        K.copy_(K_shard)
        V.copy_(V_shard)
    elif len(set(sizes)) == 1:
        dist.all_gather_into_tensor(K, K_shard.contiguous(), group=group)
        dist.all_gather_into_tensor(V, V_shard.contiguous(), group=group)
    else:
        for r, (b, e) in enumerate(ranges):
            if r == rank:
                K[b:e].copy_(K_shard)
                V[b:e].copy_(V_shard)
            if e > b:
                dist.broadcast(K[b:e], src=dist.get_global_rank(group, r) if group is not None else r, group=group)
                dist.broadcast(V[b:e], src=dist.get_global_rank(group, r) if group is not None else r, group=group)
    return K, V


def exchange_offsets(world: int) -> list[int]:
    """Order in which a rank receives the other ranks' K/V chunks: in round t it receives from rank - o_t and sends
    to rank + o_t (mod world). Neighbours first (1, world-1, 2, world-2, ...): the keys nearest to a rank's own rows,
    where banded structure lives, arrive before the far ones."""
    out = []
    for k in range(1, world // 2 + 1):
        out.append(k)
        if world - k != k:
            out.append(world - k)
    return out


def default_rounds_in_phase1(world: int) -> int:
    """Rounds of the K/V exchange before the first pass of a forward cut in two along the key axis. Up to 4 ranks: all of
    them, i.e. ONE pass after the exchange (measured best on 2 and 4 GPUs: an extra pass revisits every row of a large
    shard). From 8 ranks on a shard is small enough for two passes to pay: about 4/7 of the rounds, then the rest
    (8 GPUs: 1.22 against 1.28 ms)."""
    return world - 1 if world <= 4 else (4 * (world - 1) + 6) // 7


class KeyChunkExchange:
    """K/V replication overlapped with the forward, for operators that can work on one range of keys at a time.

    K and V start row-sharded in equal chunks `kv_ranges` (rank r owns chunk r, already stored at its place inside
    the full-size buffers `self.K`, `self.V`). `run()` fetches the other ranks' chunks in world-1 rounds and calls
    back on the compute stream:

        before()                       work that needs no K/V at all (mask inspection), overlaps the first rounds
        on_chunk(key_begin, key_end, i)  once for the own chunk (i = 0), then once per received chunk as soon as it has
                                       landed (i = 1 .. world-1); the callee may read only K/V rows in that range

    Transport on GPUs (`transport="peer_copy"`, the default where it can be set up): every rank maps the other ranks'
    buffers into its address space once (CUDA IPC handles exchanged through the process group) and PULLS chunk
    rank - o in round o with a device-to-device copy over NVLink. Those copies run on the copy engines, so they take
    no SM away from the forward passes they overlap. Two one-element all-reduces on the communication stream fence
    the rounds: the first says "every rank's own chunk is final", the second "every rank has finished reading".
    `transport="nccl"`: the rounds are NCCL send/recv pairs (also what CPU ranks use, over gloo).

    No reduction and no softmax-state exchange are involved: every pass chains into the rank's own (m, l, O).
    """

    def __init__(self, L: int, d: int, kv_ranges, rank: int, world: int, device, dtype=torch.float32, group=None,
                 transport: str | None = None):
        self.L, self.d, self.rank, self.world, self.group = L, d, rank, world, group
        self.kv_ranges = list(kv_ranges)
        self.dev = torch.device(device)
        self.K = torch.empty(L, d, dtype=dtype, device=self.dev)
        self.V = torch.empty(L, d, dtype=dtype, device=self.dev)
        self.cuda = self.dev.type == "cuda"
        self.s_comm = torch.cuda.Stream(device=self.dev) if self.cuda else None
        self.s_comm2 = torch.cuda.Stream(device=self.dev) if self.cuda else None  # V travels beside K (peer copies)
        self.offsets = exchange_offsets(world)
        self.transport = "nccl"
        self.peer_K, self.peer_V = {}, {}
        if self.cuda and world > 1 and transport in (None, "peer_copy"):
            try:
                self._map_peers()
                self.transport = "peer_copy"
            except Exception:  # no IPC on this allocator / platform: the NCCL rounds do the same job
                if transport == "peer_copy":
                    raise
        self._fence = torch.zeros(1, dtype=torch.float32, device=self.dev) if self.cuda else None

    def _map_peers(self):
        """Exchange CUDA IPC handles of self.K / self.V and open every other rank's buffers."""
        from torch.multiprocessing.reductions import reduce_tensor

        mine = (reduce_tensor(self.K), reduce_tensor(self.V))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=self.group)
        ok = torch.ones(1, dtype=torch.int32, device=self.dev)
        try:
            for r, ((fk, ak), (fv, av)) in enumerate(everyone):
                if r != self.rank:
                    # Open the handle in THIS rank's device context (argument 6 of the rebuild call is the device the
                    # storage is opened under; CUDA enables peer access lazily for it). The mapped tensor then counts
                    # as local, so a copy from it is issued on this device's stream and copy engine and reads the
                    # peer over NVLink -- no context of this process runs on the peer GPU, where it would have to
                    # time-slice with the peer rank's own kernels.
                    ak, av = list(ak), list(av)
                    ak[6] = av[6] = self.dev.index
                    self.peer_K[r], self.peer_V[r] = fk(*ak), fv(*av)
        except Exception:
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)  # all ranks take the same transport
        if int(ok.item()) != 1:
            self.peer_K, self.peer_V = {}, {}
            raise RuntimeError("peer mapping failed on some rank")

    def own(self):
        b, e = self.kv_ranges[self.rank]
        return self.K[b:e], self.V[b:e]

    def _peer(self, r):
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _round(self, o):
        """One round: chunk of rank - o into its place (and, with send/recv transport, the own chunk to rank + o)."""
        dst, src = (self.rank + o) % self.world, (self.rank - o) % self.world
        sb, se = self.kv_ranges[src]
        if self.transport == "peer_copy":  # called with s_comm current: K on it, V on the second stream, joined here
            self.s_comm2.wait_stream(self.s_comm)
            self.K[sb:se].copy_(self.peer_K[src][sb:se], non_blocking=True)
            with torch.cuda.stream(self.s_comm2):
                self.V[sb:se].copy_(self.peer_V[src][sb:se], non_blocking=True)
            self.s_comm.wait_stream(self.s_comm2)
            return sb, se
        Ko, Vo = self.own()
        ops = [dist.P2POp(dist.isend, Ko, self._peer(dst), self.group), dist.P2POp(dist.isend, Vo, self._peer(dst), self.group),
               dist.P2POp(dist.irecv, self.K[sb:se], self._peer(src), self.group),
               dist.P2POp(dist.irecv, self.V[sb:se], self._peer(src), self.group)]
        for req in dist.batch_isend_irecv(ops):
            req.wait()  # NCCL: makes the communication stream wait; gloo: blocks the host until the round is done
        return sb, se

    def _fence_ranks(self):
        """On the communication stream: passes once every rank's communication stream has reached this point."""
        if self.transport == "peer_copy":
            dist.all_reduce(self._fence, group=self.group)

    def exchange_only(self):
        """The replication alone (for timing it): all rounds, then the current stream waits for the last."""
        if self.world == 1:
            return
        if not self.cuda:
            for o in self.offsets:
                self._round(o)
            return
        cur = torch.cuda.current_stream(self.dev)
        self.s_comm.wait_stream(cur)
        with torch.cuda.stream(self.s_comm):
            self._fence_ranks()
            for o in self.offsets:
                self._round(o)
            self._fence_ranks()
        cur.wait_stream(self.s_comm)

    def run(self, on_chunk, before=None, own_ready=None):
        """`own_ready`: a CUDA event after which the own chunk is final (e.g. its host->device copy on another
        stream); the rounds and the own-chunk pass wait for it, `before()` does not."""
        b, e = self.kv_ranges[self.rank]
        if not self.cuda:  # host ranks (tests): rounds and passes alternate
            if before is not None:
                before()
            on_chunk(b, e, 0)
            for i, o in enumerate(self.offsets):
                sb, se = self._round(o)
                on_chunk(sb, se, i + 1)
            return
        cur = torch.cuda.current_stream(self.dev)
        arrived = []
        if self.world > 1:
            self.s_comm.wait_stream(cur)  # the own chunk is final once the caller's earlier work is done
            if own_ready is not None:
                self.s_comm.wait_event(own_ready)
            with torch.cuda.stream(self.s_comm):
                self._fence_ranks()
                for o in self.offsets:
                    sb, se = self._round(o)
                    ev = torch.cuda.Event()
                    ev.record(self.s_comm)
                    arrived.append((sb, se, ev))
                self._fence_ranks()
        if before is not None:
            before()
        if own_ready is not None:
            cur.wait_event(own_ready)
        on_chunk(b, e, 0)
        for i, (sb, se, ev) in enumerate(arrived):
            cur.wait_event(ev)
            on_chunk(sb, se, i + 1)
        if self.world > 1:
            cur.wait_stream(self.s_comm)  # other ranks read the own chunk: nothing later may overwrite it before they end

    def two_phase_ranges(self, rounds_in_phase1: int):
        """Key ranges of a forward in two passes: what has landed after `rounds_in_phase1` rounds (the own chunk and
        the chunks on both sides of it: one cyclic interval of keys), and everything else (its complement, also one
        cyclic interval). Ranges are (key_begin, key_end) with key_begin > key_end meaning [key_begin, L) + [0, key_end)."""
        k = max(0, min(rounds_in_phase1, self.world - 1))
        before, after = (k + 1) // 2, k // 2  # chunks rank-1, rank+1, rank-2, ... arrive in that order
        if k >= self.world - 1:
            return (0, self.L), None
        first = (self.rank - before) % self.world
        last = (self.rank + after) % self.world
        a, b = self.kv_ranges[first][0], self.kv_ranges[last][1]
        covered = sum(self.kv_ranges[(first + i) % self.world][1] - self.kv_ranges[(first + i) % self.world][0]
                      for i in range(k + 1))
        if covered == 0:  # empty chunks only (more ranks than key tiles): nothing in pass 1, everything in pass 2
            return (a, a), (0, self.L)
        if covered >= self.L or (b == self.L and a == 0):
            return (0, self.L), None
        b_wrapped = 0 if b == self.L else b
        phase1 = (a, b) if a < b else (a, b_wrapped)
        phase2 = (b_wrapped, a) if b_wrapped != a else None
        if phase2 is not None and phase2[0] < phase2[1] and phase2[1] == 0:
            phase2 = (phase2[0], self.L)
        return phase1, phase2

    def run_tiles_first(self, on_tiles, on_rest, before=None, own_ready=None):
        """The schedule for a graph mask with a band: on_tiles(key_begin, key_end) for the own key chunk as soon as the
        mask inspection (`before`) is done -- the dense tiles of a band read keys near the diagonal, i.e. mostly the own
        chunk, and their pass costs nothing per row -- then, after the last round, on_tiles(the other keys: one cyclic
        range) and on_rest() (everything that visits every row: the residual entries of ALL keys, once). With one rank
        the three run back to back."""
        p1, p2 = self.two_phase_ranges(0)

        def on_keys(a, b, i):
            on_tiles(a, b)
            if p2 is None or i == 1:
                on_rest()
        self.run_two_phase(on_keys, before, own_ready, rounds_in_phase1=0)

    def run_two_phase(self, on_keys, before=None, own_ready=None, rounds_in_phase1=None):
        """Like run(), with the forward cut into at most two passes instead of one per chunk: pass 1 over the keys that
        have landed after `rounds_in_phase1` rounds, pass 2 over the rest once every round is done. Short per-row key
        lists make a pass cost far more than its share of the keys (every pass revisits every row: its offsets, its Q
        row, its running state), so few large passes beat many small ones, and on 4 GPUs one pass after the last round
        (with the mask inspection overlapping the rounds) beat every two-pass split measured, while on 8 GPUs four rounds
        before the first pass won by 4 %; `rounds_in_phase1 = None` picks accordingly (default_rounds_in_phase1).
        0 rounds means "own chunk first", world-1 or more a single pass.
        on_keys(key_begin, key_end, i)."""
        if rounds_in_phase1 is None:
            rounds_in_phase1 = default_rounds_in_phase1(self.world)
        p1, p2 = self.two_phase_ranges(rounds_in_phase1)
        k = min(rounds_in_phase1, self.world - 1) if p2 is not None else self.world - 1
        if not self.cuda:
            if before is not None:
                before()
            for i, o in enumerate(self.offsets):
                if i == k:
                    on_keys(p1[0], p1[1], 0)
                self._round(o)
            if k >= len(self.offsets):
                on_keys(p1[0], p1[1], 0)
            if p2 is not None:
                on_keys(p2[0], p2[1], 1)
            return
        cur = torch.cuda.current_stream(self.dev)
        ev1, ev2 = torch.cuda.Event(), torch.cuda.Event()
        if self.world > 1:
            self.s_comm.wait_stream(cur)
            if own_ready is not None:
                self.s_comm.wait_event(own_ready)
            with torch.cuda.stream(self.s_comm):
                self._fence_ranks()
                for i, o in enumerate(self.offsets):
                    if i == k:
                        ev1.record(self.s_comm)
                    self._round(o)
                if k >= len(self.offsets):
                    ev1.record(self.s_comm)
                ev2.record(self.s_comm)
                self._fence_ranks()
        if before is not None:
            before()
        if own_ready is not None:
            cur.wait_event(own_ready)
        if self.world > 1:
            cur.wait_event(ev1)
        on_keys(p1[0], p1[1], 0)
        if p2 is not None:
            cur.wait_event(ev2)
            on_keys(p2[0], p2[1], 1)
        if self.world > 1:
            cur.wait_stream(self.s_comm)
