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


class KeyChunkExchange:
    """K/V replication overlapped with the forward, for operators that can work on one range of keys at a time.

    K and V start row-sharded in equal chunks `kv_ranges` (rank r owns chunk r, already stored at its place inside
    the full-size buffers `self.K`, `self.V`). `run()` sends the own chunk to every other rank and receives theirs in
    world-1 rounds of point-to-point transfers (NCCL send/recv over NVLink on a communication stream; gloo on CPU),
    and calls back on the compute stream:

        before()                       work that needs no K/V at all (mask inspection), overlaps the first rounds
        on_chunk(key_begin, key_end, i)  once for the own chunk (i = 0), then once per received chunk as soon as it has
                                       landed (i = 1 .. world-1); the callee may read only K/V rows in that range

    No reduction and no softmax-state exchange are involved: every pass chains into the rank's own (m, l, O).
    """

    def __init__(self, L: int, d: int, kv_ranges, rank: int, world: int, device, dtype=torch.float32, group=None):
        self.L, self.d, self.rank, self.world, self.group = L, d, rank, world, group
        self.kv_ranges = list(kv_ranges)
        self.dev = torch.device(device)
        self.K = torch.empty(L, d, dtype=dtype, device=self.dev)
        self.V = torch.empty(L, d, dtype=dtype, device=self.dev)
        self.cuda = self.dev.type == "cuda"
        self.s_comm = torch.cuda.Stream(device=self.dev) if self.cuda else None
        self.offsets = exchange_offsets(world)

    def own(self):
        b, e = self.kv_ranges[self.rank]
        return self.K[b:e], self.V[b:e]

    def _peer(self, r):
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _round(self, o):
        """One round: own chunk to rank + o, chunk of rank - o into its place."""
        dst, src = (self.rank + o) % self.world, (self.rank - o) % self.world
        sb, se = self.kv_ranges[src]
        Ko, Vo = self.own()
        ops = [dist.P2POp(dist.isend, Ko, self._peer(dst), self.group), dist.P2POp(dist.isend, Vo, self._peer(dst), self.group),
               dist.P2POp(dist.irecv, self.K[sb:se], self._peer(src), self.group),
               dist.P2POp(dist.irecv, self.V[sb:se], self._peer(src), self.group)]
        for req in dist.batch_isend_irecv(ops):
            req.wait()  # NCCL: makes the communication stream wait; gloo: blocks the host until the round is done
        return sb, se

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
            for o in self.offsets:
                self._round(o)
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
                for o in self.offsets:
                    sb, se = self._round(o)
                    ev = torch.cuda.Event()
                    ev.record(self.s_comm)
                    arrived.append((sb, se, ev))
        if before is not None:
            before()
        if own_ready is not None:
            cur.wait_event(own_ready)
        on_chunk(b, e, 0)
        for i, (sb, se, ev) in enumerate(arrived):
            cur.wait_event(ev)
            on_chunk(sb, se, i + 1)
        if self.world > 1:
            cur.wait_stream(self.s_comm)  # the sends read the own chunk: nothing later may overwrite it before they end
