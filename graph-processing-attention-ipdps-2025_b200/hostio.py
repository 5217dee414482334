"""Forward calls on HOST buffers, with the PCIe copies and the kernels overlapped.

For Local, Local-1D-dilated and Local-2D-dilated masks a query row attends to keys within a fixed distance
(w, w*(dil+1), or its own block), so a row range can be computed as soon as the K/V rows up to its far edge are
on the device. `BandedHostPipeline` cuts the rows into chunks and overlaps three things on three streams:
host->device copies of Q/K/V chunks, row-range forward calls through the C ABI (`row_begin/row_end`), and
device->host copies of finished O chunks. PCIe is full duplex, so the O traffic hides behind the Q/K/V traffic
and the kernels hide behind both; what remains is the time of the host->device copies.

Masks whose rows may attend to any key (CSR, COO, Global-no-local) cannot start before all of K and V have
arrived; `FullKeyHostPipeline` still overlaps the Q chunks coming in, the row-range calls and the O chunks going out.
"""
from __future__ import annotations

import torch

from . import capi

_KINDS = ("local", "local_1d_dilated", "local_2d_dilated")


def chunk_edges(n_rows: int, n_chunks: int, unit: int = 256) -> list[int]:
    """Row boundaries of at most n_chunks chunks whose sizes are multiples of `unit` (the last one may be ragged)."""
    rows = max(unit, -(-n_rows // max(1, n_chunks)))
    rows = -(-rows // unit) * unit
    return list(range(0, n_rows, rows)) + [n_rows]


def chunk_needed_last(edges: list[int], c: int, halo: int, n_keys: int) -> int:
    """Index of the last chunk whose K/V rows chunk c reads when a row looks `halo` rows past its own."""
    need = min(n_keys, edges[c + 1] + halo) - 1
    return next(i for i in range(len(edges) - 1) if edges[i + 1] > need)


class BandedHostPipeline:
    """Device buffers, streams and the chunk plan for repeated calls on one shape.

    kind: "local" (p0 = window half-width), "local_1d_dilated" (p0 = half-width, p1 = dil_factor) or
    "local_2d_dilated" (p0 = block size, p1 = dil_factor). Host tensors must be pinned for the copies to overlap.
    """

    def __init__(self, kind: str, L: int, d: int, p0: int, p1: int = 0, n_chunks: int = 8, device=None):
        if kind not in _KINDS:
            raise ValueError(f"kind must be one of {_KINDS}")
        self.kind, self.L, self.d, self.p0, self.p1 = kind, L, d, p0, p1
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        unit = 256                       # chunk edges on multiples of the tiled kernel's CTA rows ...
        if kind == "local_2d_dilated":
            unit = p0                    # ... or on mask-block edges (a block never looks outside itself)
            self.halo = 0
        else:
            self.halo = p0 * (p1 + 1)
        self.edges = chunk_edges(L, n_chunks, unit)
        with torch.cuda.device(self.dev):
            f = dict(device=self.dev, dtype=torch.float32)
            self.Q, self.K, self.V, self.O = (torch.empty(L, d, **f) for _ in range(4))
            self.m, self.l = torch.empty(L, **f), torch.empty(L, **f)
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=self.dev) for _ in range(3))

    def _forward_rows(self, a: int, b: int, use_nan: bool):
        st = (self.m[a:b], self.l[a:b], self.O[a:b])
        q = self.Q[a:b]
        if self.kind == "local":
            capi.local_forward(q, self.K, self.V, *st, self.p0, a, b)
        elif self.kind == "local_1d_dilated":
            capi.local_1d_dilated_forward(q, self.K, self.V, *st, self.p0, self.p1, a, b)
        else:
            capi.local_2d_dilated_forward(q, self.K, self.V, *st, self.p0, self.p1, use_nan, a, b)

    def forward(self, hQ, hK, hV, hO, use_nan: bool = False):
        """softmax(mask(Q K^T / sqrt(d))) V from a fresh state, host in, host out (hO). Asynchronous: the
        caller's current stream waits for the last device->host copy; synchronise it before reading hO."""
        cur = torch.cuda.current_stream(self.dev)
        n = len(self.edges) - 1
        copied = [torch.cuda.Event() for _ in range(n)]
        done = [torch.cuda.Event() for _ in range(n)]
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_run):
            self.m.fill_(float("-inf"))
            self.l.zero_()
            self.O.zero_()
        with torch.cuda.stream(self.s_in):
            for c in range(n):
                a, b = self.edges[c], self.edges[c + 1]
                self.K[a:b].copy_(hK[a:b], non_blocking=True)
                self.V[a:b].copy_(hV[a:b], non_blocking=True)
                self.Q[a:b].copy_(hQ[a:b], non_blocking=True)
                copied[c].record(self.s_in)
        for c in range(n):
            a, b = self.edges[c], self.edges[c + 1]
            last = chunk_needed_last(self.edges, c, self.halo, self.L)  # chunk holding the last key row it reads
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(copied[last])
                self._forward_rows(a, b, use_nan)
                done[c].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done[c])
                hO[a:b].copy_(self.O[a:b], non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)
        return hO


class FullKeyHostPipeline:
    """Host buffers for the masks whose rows may attend to ANY key (CSR, COO, Global-no-local).

    Nothing can be computed before all of K and V are on the device, but the query side still pipelines: K and
    V go first, then Q arrives in row chunks while the previous chunk is computed (row-range call through the C
    ABI) and the chunk before that travels back. The device->host traffic and the kernels hide behind the
    host->device traffic; what remains is the time of the host->device copies plus the last chunk.

    `call(a, b, Q_ab, K, V, m_ab, l_ab, O_ab)` must enqueue the forward of rows [a, b) on the current stream, e.g.
    `capi.coo_forward(Q_ab, K, V, rows[lo:hi], cols[lo:hi], m_ab, l_ab, O_ab, row_begin=a)`.
    """

    def __init__(self, n_rows: int, n_keys: int, d: int, n_chunks: int = 8, device=None):
        self.n_rows, self.n_keys, self.d = n_rows, n_keys, d
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.edges = chunk_edges(n_rows, n_chunks, 256)
        with torch.cuda.device(self.dev):
            f = dict(device=self.dev, dtype=torch.float32)
            self.Q, self.O = torch.empty(n_rows, d, **f), torch.empty(n_rows, d, **f)
            self.K, self.V = torch.empty(n_keys, d, **f), torch.empty(n_keys, d, **f)
            self.m, self.l = torch.empty(n_rows, **f), torch.empty(n_rows, **f)
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=self.dev) for _ in range(3))

    def forward(self, call, hQ, hK, hV, hO):
        """Fresh state, host in, host out (hO). Asynchronous like BandedHostPipeline.forward."""
        cur = torch.cuda.current_stream(self.dev)
        n = len(self.edges) - 1
        copied = [torch.cuda.Event() for _ in range(n)]
        done = [torch.cuda.Event() for _ in range(n)]
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_run):
            self.m.fill_(float("-inf"))
            self.l.zero_()
            self.O.zero_()
        with torch.cuda.stream(self.s_in):
            self.K.copy_(hK, non_blocking=True)
            self.V.copy_(hV, non_blocking=True)
            for c in range(n):
                a, b = self.edges[c], self.edges[c + 1]
                self.Q[a:b].copy_(hQ[a:b], non_blocking=True)
                copied[c].record(self.s_in)
        for c in range(n):
            a, b = self.edges[c], self.edges[c + 1]
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(copied[c])
                call(a, b, self.Q[a:b], self.K, self.V, self.m[a:b], self.l[a:b], self.O[a:b])
                done[c].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done[c])
                hO[a:b].copy_(self.O[a:b], non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)
        return hO
