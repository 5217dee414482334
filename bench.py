#!/usr/bin/env python
"""Benchmark of the sparse FlashAttention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--path auto|gather|tiled]
                    [--weak] [--planned] [--no-overlap] [--rows L] [--no-cpu-baseline] [--no-per-workload]

One "step" = one forward of one mask family over one batch of seeded synthetic input. The default workload
is the COO graph configuration: L=1048576, d=64, fp32 Q/K/V ~ N(0,1), power-law row degrees plus a band
(1.6e8 mask entries), the largest configuration and the one that is split over GPUs. The other workloads
(--workload local|l1d|gnl|l2d|csr) are the remaining benchmark shapes; `blocks` is the block-level dilation
pattern as an explicit CSR mask (not expressible through the reference's own 2D operator). With the default
workload on one GPU the line also carries `per_workload`: a short measurement of every mask family.
--planned times explicit-mask calls from a dense-tile plan built once outside the timed region.

Multi-GPU (launched by torch.distributed.run, one rank per GPU): STRONG scaling. The workload's rows are split
into one contiguous query-row range per rank (balanced by mask entries for CSR/COO), K and V start row-sharded
in equal chunks, and every timed step contains the replication of K/V to all ranks: for explicit masks as world-1
rounds of point-to-point transfers with the forward of each arrived key chunk overlapped (sharding.KeyChunkExchange;
--no-overlap: all-gather first, then one forward), for implicit masks as an all-gather followed by the forward.
`compute_only_ms` (K/V already replicated) and `replicate_ms` (the exchange alone) are printed beside `value`.
--weak restores weak scaling (L rows per GPU) for the implicit masks.

`e2e` is the same step from pinned HOST buffers: host->device copies of Q/K/V (per rank: its shards), the forward,
the device->host copy of O, overlapped where the data dependencies allow (hostio.py); `e2e_plugin` is the plain
drop-in call `spfa_<mask>.forward` between whole-tensor copies (one GPU).

Prints ONE JSON line (rank 0). Timing: CUDA events on the launching stream around each step, L2 flushed
(256 MiB memset) and the (m, l, O) state re-initialised before each step outside the timed span; per-rank
total = sum of step times; reported time = max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

WORKLOADS = {
    # name: kind, L, d, p0, p1, description
    "local": dict(kind="local", L=65536, d=64, p0=256, p1=0,
                  desc="Local sliding window, L=65536, d=64, fp32, |i-j|<=256 (width 513)"),
    "csr": dict(kind="csr", L=4096, d=64, p0=0, p1=0,
                desc="CSR explicit mask, L=4096, d=64, fp32, diagonal + Bernoulli(0.01)"),
    "l1d": dict(kind="local_1d_dilated", L=131072, d=128, p0=512, p1=1,
                desc="Local 1D dilated, L=131072, d=128, fp32, 512 each side, every 2nd key (1025 keys/row)"),
    "gnl": dict(kind="global_no_local", L=131072, d=128, p0=256, p1=0,
                desc="Global-no-local, L=131072, d=128, fp32, 64 global tokens, local window 256 excluded"),
    "l2d": dict(kind="local_2d_dilated", L=262144, d=64, p0=256, p1=4,
                desc="Local 2D dilated (reference semantics), L=262144, d=64, fp32, block 256, dil_factor 4, use_nan"),
    "blocks": dict(kind="csr", L=262144, d=64, p0=256, p1=4, gen="block_dilated",
                   desc="NON-REFERENCE pattern: block-level dilation as an explicit CSR mask, L=262144, d=64, fp32, "
                        "256-row blocks, block b attends to blocks b, b+-4, b+-8 (3.3e8 entries)"),
    "bigbird": dict(kind="bigbird", L=131072, d=64, p0=256, p1=32,
                    desc="NON-REFERENCE fusion: Local(256) + Global-no-local(64 tokens) + random CSR part (~32 keys/row) in "
                         "one call, L=131072, d=64, fp32; the reference composes it from three chained calls"),
    "coo": dict(kind="coo", L=1048576, d=64, p0=64, p1=0,
                desc="COO explicit graph mask, L=1048576, d=64, fp32, Zipf(2.1) mean-32 max-8192 random cols + band 64"),
}
DEFAULT_WORKLOAD = "coo"
FULL_SIZE_L = {k: v["L"] for k, v in WORKLOADS.items()}  # --rows shrinks WORKLOADS; recorded ncu traffic is full-size
PER_WORKLOAD = ("local", "l1d", "gnl", "l2d", "csr", "coo")

# ---------------------------------------------------------------------------------------------------------
# mask sizes (closed forms) and algorithmic bytes
# ---------------------------------------------------------------------------------------------------------
def implicit_nnz(kind, L, p0, p1, G, rb, re):
    i = torch.arange(rb, re, dtype=torch.int64)
    if kind == "local":
        return int((torch.clamp(i + p0 + 1, max=L) - torch.clamp(i - p0, min=0)).sum())
    if kind == "local_1d_dilated":
        s = p1 + 1
        lo = torch.maximum(i - p0 * s, i % s)
        hi = torch.clamp(i + p0 * s, max=L - 1)
        return int(((hi - lo) // s + 1).sum())
    if kind == "local_2d_dilated":
        s, B = p1 + 1, p0
        live = ((i % B) % s == 0).sum()
        return int(live) * min(B, (B - 1) // s + 1)
    if kind == "global_no_local":
        g = torch.as_tensor(G, dtype=torch.int64)
        isg = torch.zeros(L, dtype=torch.bool)
        isg[g] = True
        lo, hi = torch.clamp(i - p0, min=0), torch.clamp(i + p0 + 1, max=L)
        n_glob_rows = L - (hi - lo)
        gs = torch.sort(g).values
        inside = torch.searchsorted(gs, hi) - torch.searchsorted(gs, lo)
        n_other = g.numel() - inside
        return int(torch.where(isg[rb:re], n_glob_rows, n_other).sum())
    raise ValueError(kind)


def algorithmic_bytes(kind, L_keys, n_rows, d, nnz, n_live_rows):
    """Explicit masks: gather-counted nnz*(2*d*4+4) + rows*(2*d*4+16) + 8*(rows+1).
    Implicit masks: compulsory traffic (Q read, K and V read once, O written) + 16 B/row of (m, l)."""
    if kind in ("csr", "coo"):
        extra = 8 * nnz if kind == "coo" else 0
        return nnz * (2 * d * 4 + 4) + n_live_rows * (2 * d * 4 + 16) + 8 * (n_rows + 1) + extra
    if kind == "local_2d_dilated":
        # only live rows are read (Q, incoming O) and only the live key rows of K, V (the same row set);
        # every row is written once (result or NaN fill)
        return (2 * n_live_rows * d + 2 * n_live_rows * d + n_rows * d) * 4 + 16 * n_live_rows
    return (2 * n_rows * d + 2 * L_keys * d) * 4 + 16 * n_live_rows


# ---------------------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------------------
def make_qkv(L, d, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return tuple(torch.randn(L, d, device=dev, generator=g, dtype=torch.float32) for _ in range(3))


def make_csr_mask(L, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    mask = torch.rand(L, L, device=dev, generator=g) < 0.01
    mask |= torch.eye(L, dtype=torch.bool, device=dev)
    counts = mask.sum(1)
    row_off = torch.zeros(L + 1, dtype=torch.int64, device=dev)
    row_off[1:] = torch.cumsum(counts, 0)
    col = mask.nonzero()[:, 1].to(torch.int32).contiguous()
    return row_off, col


def make_block_dilated_csr(L, B, step, dev, reach=2):
    """Every row of block b attends to all keys of blocks b + step*k, |k| <= reach, inside the sequence
    (columns ascending). The reference's own 2D-dilated operator cannot express this; it runs as a CSR mask."""
    nb = L // B
    blk = torch.arange(nb, device=dev).unsqueeze(1) + step * torch.arange(-reach, reach + 1, device=dev).unsqueeze(0)
    ok = (blk >= 0) & (blk < nb)                                   # [nb, 2 reach + 1]
    counts = (ok.sum(1) * B).repeat_interleave(B)                  # entries per row
    row_off = torch.zeros(L + 1, dtype=torch.int64, device=dev)
    row_off[1:] = torch.cumsum(counts, 0)
    cols_blk = (blk.unsqueeze(2) * B + torch.arange(B, device=dev).view(1, 1, B))   # [nb, 2 reach + 1, B]
    per_block = [cols_blk[b][ok[b]].reshape(-1).to(torch.int32) for b in range(nb)]  # keys of one row of block b
    col = torch.cat([c.repeat(B) for c in per_block]).contiguous()
    return row_off, col


def make_random_part(L, w, G, per_row, seed, dev):
    """Random CSR part of a BigBird mask: about per_row uniform columns per row, without the band |i-j| <= w, without
    global rows and global columns (those are covered by the other two parts), duplicates removed, columns ascending."""
    g = torch.Generator(device=dev).manual_seed(seed)
    rows = torch.arange(L, device=dev).repeat_interleave(per_row)
    cols = torch.randint(0, L, (L * per_row,), device=dev, generator=g)
    isg = torch.zeros(L, dtype=torch.bool, device=dev)
    isg[G.to(dev).long()] = True
    keep = ((rows - cols).abs() > w) & ~isg[rows] & ~isg[cols]
    keys = torch.unique(rows[keep] * L + cols[keep])
    r, c = keys // L, (keys % L).to(torch.int32)
    row_off = torch.zeros(L + 1, dtype=torch.int64, device=dev)
    row_off[1:] = torch.cumsum(torch.bincount(r, minlength=L), 0)
    return row_off, c.contiguous()


def make_coo_graph(L, band, seed, dev, mean_deg=32, max_deg=8192, alpha=2.1):
    """Row-sorted COO: power-law out-degrees (Zipf alpha, rescaled to the mean, clipped) with uniform random
    columns, united with the band |i-j| <= band; duplicates removed."""
    rng = np.random.default_rng(seed)
    z = rng.zipf(alpha, L).astype(np.float64)
    deg = np.minimum(max_deg, np.maximum(0, np.rint(z * (mean_deg / z.mean())))).astype(np.int64)
    deg_t = torch.from_numpy(deg).to(dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    r_rows = torch.repeat_interleave(torch.arange(L, device=dev), deg_t)
    r_cols = torch.randint(0, L, (int(deg.sum()),), device=dev, generator=g)
    key_r = r_rows * L + r_cols
    del r_rows, r_cols
    i = torch.arange(L, device=dev).unsqueeze(1)
    j = i + torch.arange(-band, band + 1, device=dev).unsqueeze(0)
    ok = (j >= 0) & (j < L)
    key_b = (i * L + j)[ok]
    del i, j, ok
    keys = torch.unique(torch.cat([key_r, key_b]))  # sorted ascending = (row, col) order
    del key_r, key_b
    rows = (keys // L).contiguous()
    cols = (keys % L).to(torch.int32).contiguous()
    return rows, cols


# ---------------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        try:  # address the GPU by UUID: nvidia-smi's numbering ignores CUDA_VISIBLE_DEVICES
            self.gpu = "GPU-" + str(torch.cuda.get_device_properties(gpu_index).uuid)
        except Exception:
            self.gpu = str(gpu_index)
        self.proc, self.lines, self.thread = None, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: [self.lines.append(x) for x in self.proc.stdout], daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "sm_mhz_max_seen": max(sm) if sm else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def recorded_traffic(kernel_key):
    """DRAM bytes per launch from the committed ncu summary (profiles/dram_traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get(kernel_key)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "gather", "tiled"])
    ap.add_argument("--rows", type=int, default=0, help="override the workload's L (smaller cases for profiling)")
    ap.add_argument("--weak", action="store_true",
                    help="N>1, implicit masks: L rows per GPU (sequence of N*L rows) instead of splitting L rows")
    ap.add_argument("--planned", action="store_true",
                    help="csr/coo/blocks: build the dense-tile plan once outside the timed region and time forward calls "
                         "from the stored plan (a caller that applies one mask many times); default: one-shot calls")
    ap.add_argument("--no-overlap", action="store_true",
                    help="N>1, explicit masks: all-gather K/V first, then one forward (default: forward of each key chunk "
                         "overlapped with the arrival of the next)")
    ap.add_argument("--transport", default=None, choices=["peer_copy", "nccl"],
                    help="N>1, explicit masks: how K/V chunks travel (default: peer copies where CUDA IPC works, else NCCL)")
    ap.add_argument("--phase1-rounds", type=int, default=None,
                    help="N>1, explicit masks: exchange rounds after which the first of the two forward passes starts "
                         "(default: N-1 up to 4 GPUs = a single pass after the exchange, with the mask inspection overlapping it; "
                         "about 4/7 of the rounds from 8 GPUs on)")
    ap.add_argument("--e2e-chunks", type=int, default=8,
                    help="row chunks of the host pipeline for masks whose rows may need any key (end-to-end leg, 1 GPU)")
    ap.add_argument("--tiles-first", action="store_true",
                    help="N>1, explicit masks: also run the dense tiles of the own key chunk during the exchange "
                         "(sharding.KeyChunkExchange.run_tiles_first); measured equal to or slightly behind the default")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="one process, one GPU: time only the first rank's share of an N-way strong-scaling split with K/V "
                         "resident (profiling the per-rank kernels without N GPUs); implies --no-e2e --no-cpu-baseline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-per-workload", action="store_true", help="skip the short measurement of every mask family")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer legs (profiling runs)")
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work for the cpu_baseline sample")
    return ap.parse_args()


class Job:
    """One rank's share of a workload, resident on its GPU: its query rows, the mask slice of those rows, all of K/V."""

    def __init__(self, workload, rank, world, dev, whole_on_one_gpu=False, weak=False):
        w = WORKLOADS[workload]
        self.name, self.w, self.kind, self.d = workload, w, w["kind"], w["d"]
        weak = weak and self.kind not in ("csr", "coo")
        self.weak = weak
        # strong scaling: L rows split over the GPUs; weak scaling: N*L rows in the sequence, L per GPU
        self.L = w["L"] * world if weak else w["L"]
        self.rank, self.world, self.dev = rank, world, dev
        self.p0, self.p1 = w["p0"], w["p1"]
        seed = 1000 + sorted(WORKLOADS).index(workload)
        self.seed = seed
        sh = entry.load().sharding
        full_mask = None
        if self.kind == "csr":
            full_mask = (make_block_dilated_csr(self.L, self.p0, self.p1, dev) if w.get("gen") == "block_dilated"
                         else make_csr_mask(self.L, seed, dev))
        elif self.kind == "coo":
            full_mask = make_coo_graph(self.L, self.p0, seed, dev)
        if whole_on_one_gpu:  # a single-GPU implementation given the whole job
            self.ranges = [(0, self.L)]
            rank = 0
        elif weak or self.kind == "bigbird":
            self.ranges = ([(r * w["L"], (r + 1) * w["L"]) for r in range(world)] if weak
                           else sh.equal_row_ranges(self.L, world, multiple=256))
        elif self.kind == "csr":
            self.ranges = sh.nnz_balanced_row_ranges(full_mask[0], world)
        elif self.kind == "coo":
            self.ranges = sh.coo_nnz_balanced_row_ranges(full_mask[0], self.L, world)
        else:
            self.ranges = sh.equal_row_ranges(self.L, world, multiple=256)
        # K/V start row-sharded in equal chunks on key-tile multiples, whatever the query split is
        self.kv_ranges = sh.equal_row_ranges(self.L, 1 if whole_on_one_gpu else world, multiple=64)
        self.rb, self.re = self.ranges[rank]
        self.L_local = self.re - self.rb
        Q, self.K, self.V = make_qkv(self.L, self.d, seed, dev)
        self.Q = Q[self.rb:self.re].contiguous()
        del Q
        self.G = None
        self.mask = None
        self.plan = None
        n_live = self.L_local
        if self.kind == "bigbird":
            g = torch.Generator().manual_seed(seed)
            Gc = torch.sort(torch.randperm(self.L, generator=g)[:64]).values.to(torch.int32)
            self.G_cpu, self.G = Gc, Gc.to(dev)
            row_off, col = make_random_part(self.L, self.p0, Gc, self.p1, seed, dev)
            lo, hi = int(row_off[self.rb]), int(row_off[self.re])
            self.mask = ((row_off[self.rb:self.re + 1] - lo).contiguous(), col[lo:hi].contiguous())
            self.nnz_csr = hi - lo
            self.nnz = (implicit_nnz("local", self.L, self.p0, 0, None, self.rb, self.re)
                        + implicit_nnz("global_no_local", self.L, self.p0, 0, Gc, self.rb, self.re) + self.nnz_csr)
        elif self.kind == "global_no_local":
            g = torch.Generator().manual_seed(seed)
            Gc = torch.sort(torch.randperm(self.L, generator=g)[:64]).values.to(torch.int32)
            self.G_cpu, self.G = Gc, Gc.to(dev)
            self.nnz = implicit_nnz(self.kind, self.L, self.p0, self.p1, Gc, self.rb, self.re)
        elif self.kind == "csr":
            row_off, col = full_mask
            lo, hi = int(row_off[self.rb]), int(row_off[self.re])
            self.mask = ((row_off[self.rb:self.re + 1] - lo).contiguous(), col[lo:hi].contiguous())
            self.nnz = hi - lo
        elif self.kind == "coo":
            rows, cols = full_mask
            edges = torch.searchsorted(rows, torch.tensor([self.rb, self.re], device=dev))
            lo, hi = int(edges[0]), int(edges[1])
            self.mask = (rows[lo:hi].contiguous(), cols[lo:hi].contiguous())
            self.nnz = hi - lo
        else:
            self.nnz = implicit_nnz(self.kind, self.L, self.p0, self.p1, None, self.rb, self.re)
            if self.kind == "local_2d_dilated":
                i = torch.arange(self.rb, self.re)
                n_live = int(((i % self.p0) % (self.p1 + 1) == 0).sum())
        del full_mask
        self.n_live = n_live
        self.flops = 4.0 * self.nnz * self.d
        if self.kind == "bigbird":  # compulsory bytes of the implicit parts + gather-counted bytes of the CSR part
            self.bytes = (algorithmic_bytes("local", self.L, self.L_local, self.d, 0, n_live)
                          + self.nnz_csr * (2 * self.d * 4 + 4) + 8 * (self.L_local + 1))
        else:
            self.bytes = algorithmic_bytes(self.kind, self.L, self.L_local, self.d, self.nnz, n_live)
        self.m = torch.empty(self.L_local, device=dev)
        self.l = torch.empty(self.L_local, device=dev)
        self.O = torch.empty(self.L_local, self.d, device=dev)
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def reset_state(self):
        self.m.fill_(float("-inf"))
        self.l.zero_()
        self.O.zero_()

    def flush_l2(self):
        self.flush_buf.zero_()

    def build_plan(self, capi, out=None):
        if self.kind == "csr":
            return capi.csr_plan(self.mask[0], self.mask[1], self.L, self.d, out=out)
        if self.kind == "coo":
            return capi.coo_plan(self.mask[0], self.mask[1], self.L_local, self.L, self.d, row_begin=self.rb, out=out)
        raise SystemExit("--planned applies to the explicit masks only")

    def forward(self, capi, Q=None, K=None, V=None):
        Q = self.Q if Q is None else Q
        K = self.K if K is None else K
        V = self.V if V is None else V
        k, st = self.kind, (self.m, self.l, self.O)
        if self.plan is not None:
            capi.planned_forward(Q, K, V, *st, self.plan, use_nan=False)
            return
        if k == "local":
            capi.local_forward(Q, K, V, *st, self.p0, self.rb, self.re)
        elif k == "local_1d_dilated":
            capi.local_1d_dilated_forward(Q, K, V, *st, self.p0, self.p1, self.rb, self.re)
        elif k == "local_2d_dilated":
            capi.local_2d_dilated_forward(Q, K, V, *st, self.p0, self.p1, True, self.rb, self.re)
        elif k == "global_no_local":
            capi.global_no_local_forward(Q, K, V, *st, self.G, self.p0, self.rb, self.re)
        elif k == "bigbird":
            capi.bigbird_forward(Q, K, V, *st, self.G, self.p0, self.mask[0], self.mask[1], self.rb, self.re)
        elif k == "csr":
            capi.csr_forward(Q, K, V, self.mask[0], self.mask[1], *st, use_nan=False)
        else:
            capi.coo_forward(Q, K, V, self.mask[0], self.mask[1], *st, use_nan=False, row_begin=self.rb)

    def plugin_forward(self, binding, Q, K, V, w_val):
        """The drop-in call of the reference's API (one GPU, whole tensors)."""
        st, k = (self.m, self.l, self.O), self.kind
        if k == "local":
            binding.forward(Q, K, V, *st, self.p0)
        elif k == "local_1d_dilated":
            binding.forward(Q, K, V, *st, self.p0, self.p1)
        elif k == "local_2d_dilated":
            binding.forward(Q, K, V, *st, self.p0, self.p1, True)
        elif k == "global_no_local":
            binding.forward(Q, K, V, *st, self.G, self.p0)
        elif k == "bigbird":
            binding.forward(Q, K, V, *st, self.G, self.p0, self.mask[0], self.mask[1])
        else:
            binding.forward(Q, K, V, self.mask[0], self.mask[1], w_val, *st, False)

    def chained_forward(self, capi):
        """BigBird as the reference composes it: three operator calls on one state (verification/verify.py:337-352)."""
        st = (self.m, self.l, self.O)
        capi.local_forward(self.Q, self.K, self.V, *st, self.p0, self.rb, self.re)
        capi.global_no_local_forward(self.Q, self.K, self.V, *st, self.G, self.p0, self.rb, self.re)
        capi.csr_forward(self.Q, self.K, self.V, self.mask[0], self.mask[1], *st, use_nan=False)


def dist_max(x: float, world: int, dev) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def dist_sum(x: float, world: int, dev) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def barrier(world):
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        torch.cuda.synchronize()


def timed_steps(job, fn, steps, warmup, world, counter=None, before_each=None):
    """warmup untimed calls, then `steps` calls each bracketed by CUDA events (flush + reset outside).
    Returns (per-step ms, kernels launched by the library inside the timed loop)."""
    for _ in range(warmup):
        job.reset_state()
        if before_each:
            before_each()
        fn()
    barrier(world)
    n0 = counter() if counter else 0
    evs = []
    for _ in range(steps):
        job.reset_state()
        if before_each:
            before_each()
        job.flush_l2()
        if world > 1:  # every rank enters the step together: a step contains an exchange between the ranks
            barrier(world)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        evs.append((a, b))
    barrier(world)
    n1 = counter() if counter else 0
    return [a.elapsed_time(b) for a, b in evs], n1 - n0


def roofline_of(job, workload, kernel_ms, tiled, peaks, peak_src, full_size):
    """Roofline object of one workload from its mean step time on one GPU.
    Banded masks on the tiled path (and the all-dense block pattern): tensor pipe, useful flops 4*nnz*d.
    Implicit HBM-bound masks: compulsory bytes. Explicit masks: the DRAM traffic recorded by ncu for the same
    call decides the fraction (their gather-counted bytes assume no cache reuse and exceed what DRAM moves; that
    figure is kept as `effective_gbs`)."""
    tensor_bound = tiled and (job.kind in ("local", "local_1d_dilated") or job.w.get("gen") == "block_dilated")
    if tensor_bound:
        peak = peaks["bf16_tflops"] / 2.0
        achieved = job.flops / (kernel_ms * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": recorded_traffic(f"tiled_{workload}") if full_size else None,
                "note": f"useful flops 4*nnz*d per step / mean step time; peak = {peak_src} bf16 matmul / 2 taken as TF32"}
    peak = peaks["hbm_gbs"]
    algorithmic = job.bytes / (kernel_ms * 1e-3) / 1e9
    traffic = recorded_traffic(f"gather_{workload}") if full_size else None
    if job.kind in ("csr", "coo", "bigbird"):
        real = (traffic / (kernel_ms * 1e-3) / 1e9) if traffic else None
        return {"bound": "hbm", "achieved": real, "peak": peak, "unit": "GB/s", "frac": (real / peak) if real else None,
                "traffic": traffic, "effective_gbs": algorithmic,
                "note": "achieved = DRAM bytes of one step as recorded by ncu (profiles/) / mean step time here; "
                        "effective_gbs = gather-counted bytes nnz*(2*d*4+4)+... / time (no credit for cache reuse taken "
                        f"out, so it may exceed the peak); peak = {peak_src} copy bandwidth"}
    return {"bound": "hbm", "achieved": algorithmic, "peak": peak, "unit": "GB/s", "frac": algorithmic / peak,
            "traffic": traffic,
            "note": f"compulsory bytes per step / mean step time; peak = {peak_src} copy bandwidth"}


def measure_one_gpu(workload, capi, dev, steps, warmup, peaks, peak_src, path, planned=False, job=None):
    """Short device-timed measurement of one workload on one GPU (inputs resident): the per_workload entries."""
    own = job is None
    if own:
        job = Job(workload, 0, 1, dev)
    job.plan = job.build_plan(capi) if planned else None
    times, launches = timed_steps(job, lambda: job.forward(capi), steps, warmup, 1, capi.launch_count)
    tiled = capi.last_path() == capi.PATH_TILED
    ms = statistics.mean(times)
    full = WORKLOADS[workload]["L"] == FULL_SIZE_L.get(workload)
    out = {"workload": job.w["desc"], "fwd_ms": ms, "fwd_ms_median": statistics.median(times), "steps": steps,
           "tflops": job.flops / (ms * 1e-3) / 1e12, "nnz": int(job.nnz), "dtype": "tf32" if tiled else "f32",
           "path": "tiled" if tiled else "gather", "launches_per_step": launches / max(1, steps),
           "roofline": roofline_of(job, workload, ms, tiled, peaks, peak_src, full)}
    if planned:
        out["plan"] = "dense-tile plan built once outside the timed region"
    job.plan = None
    if own:
        del job
        torch.cuda.empty_cache()
    return out


def run_ours(args, rank, world, dev):
    pkg = entry.load()
    capi = pkg.capi
    capi.lib()
    capi.set_path({"auto": capi.PATH_AUTO, "gather": capi.PATH_GATHER, "tiled": capi.PATH_TILED}[args.path])
    if args.shard_of > 1 and world == 1:  # the first rank's rows of an N-way split, on this one GPU
        job = Job(args.workload, 0, args.shard_of, dev, weak=args.weak)
        job.w = dict(job.w, desc=job.w["desc"] + f" [rows {job.rb}..{job.re}: rank 0 of a {args.shard_of}-way split]")
        args.no_e2e = args.no_cpu_baseline = args.no_per_workload = True
    else:
        job = Job(args.workload, rank, world, dev, weak=args.weak)
    explicit = job.kind in ("csr", "coo")
    peaks, peak_src = load_peaks()
    nan = float("nan")
    if args.planned:
        job.plan = job.build_plan(capi)

    # ---- compute only: inputs (all of K/V included) resident in HBM ----
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    if sampler:
        sampler.start()
    times_c, launches = timed_steps(job, lambda: job.forward(capi), args.steps, args.warmup, world, capi.launch_count)
    tiled = capi.last_path() == capi.PATH_TILED
    O_compute = job.O.clone() if world > 1 else None

    # ---- N > 1: the step that is reported contains the replication of K/V ----
    times, times_x, ex, step, poison, exchange_note = times_c, None, None, None, None, None
    if world > 1:
        sh = pkg.sharding
        ex = sh.KeyChunkExchange(job.L, job.d, job.kv_ranges, rank, world, dev, transport=args.transport)
        how = ("device-to-device peer copies over NVLink (copy engines; each rank pulls one chunk per round)"
               if ex.transport == "peer_copy" else "NCCL send/recv (own K/V chunk out, one chunk in)")
        kb, ke = job.kv_ranges[rank]
        Ko, Vo = ex.own()
        Ko.copy_(job.K[kb:ke])
        Vo.copy_(job.V[kb:ke])
        job.K = job.V = None  # from here on K/V exist only as this rank's chunk plus what the exchange delivers
        torch.cuda.empty_cache()

        def poison():  # outside the timed span: a step must not live on the chunks the previous step received
            for t in (ex.K, ex.V):
                t[:kb].fill_(nan)
                t[ke:].fill_(nan)

        overlap = (explicit and not args.no_overlap and args.path != "gather" and job.nnz >= (1 << 20)
                   and capi.lib().spfa_explicit_plan_bytes(job.L_local, job.nnz, job.L, job.d) > 0)
        if overlap:
            plan_buf = job.plan if job.plan is not None else job.build_plan(capi)
            before = None if args.planned else (lambda: job.build_plan(capi, out=plan_buf))

            if args.tiles_first:  # dense tiles of the own chunk while the other chunks travel
                def step():
                    ex.run_tiles_first(
                        lambda a, b: capi.planned_forward_parts(job.Q, ex.K, ex.V, job.m, job.l, job.O, plan_buf, a, b,
                                                                capi.PLAN_DENSE_TILES),
                        lambda: capi.planned_forward_parts(job.Q, ex.K, ex.V, job.m, job.l, job.O, plan_buf, 0, job.L,
                                                           capi.PLAN_RESIDUAL), before)
                exchange_note = ("%d rounds of %s; the mask inspection and the dense tiles of the own key chunk overlap them; "
                                 "the other dense tiles and the residual entries of all keys follow the last round"
                                 % (world - 1, how))
            else:
                rounds = sh.default_rounds_in_phase1(world) if args.phase1_rounds is None else args.phase1_rounds

                def step():
                    ex.run_two_phase(lambda a, b, i: capi.planned_forward_keys(job.Q, ex.K, ex.V, job.m, job.l, job.O,
                                                                               plan_buf, a, b),
                                     before, rounds_in_phase1=rounds)
                p1, p2 = ex.two_phase_ranges(rounds)
                exchange_note = ("%d rounds of %s; the mask inspection overlaps them, and the forward runs as %s" %
                                 (world - 1, how, "one pass after the last round" if p2 is None else
                                  "two passes: one over the keys that have landed after %d round(s) while the other chunks "
                                  "travel, one over the rest after the last round" % rounds))
        elif explicit:
            def step():
                ex.exchange_only()
                job.forward(capi, job.Q, ex.K, ex.V)
            exchange_note = "%d rounds of %s, then one forward over all keys" % (world - 1, how)
        else:
            def step():
                Kf, Vf = sh.replicate_kv(Ko, Vo, job.kv_ranges)
                job.forward(capi, job.Q, Kf, Vf)
            exchange_note = "NCCL all-gather of K and of V, then the forward"
        times, launches = timed_steps(job, step, args.steps, args.warmup, world, capi.launch_count, before_each=poison)
        torch.cuda.synchronize()
        check = float((job.O - O_compute).abs().nan_to_num(nan=1e30).max().item())  # both paths, same rows
        check = dist_max(check, world, dev)
        xfn = ex.exchange_only if explicit else (lambda: sh.replicate_kv(Ko, Vo, job.kv_ranges))
        times_x, _ = timed_steps(job, xfn, args.steps, args.warmup, world, before_each=poison)
    clocks = sampler.stop() if sampler else None
    total_ms = dist_max(sum(times), world, dev)
    total_flops = dist_sum(job.flops, world, dev)
    total_nnz = dist_sum(float(job.nnz), world, dev)
    nnz_imbalance = dist_max(float(job.nnz), world, dev) / max(total_nnz / world, 1.0)
    value = total_flops * args.steps / (total_ms * 1e-3) / 1e12
    compute_ms = dist_max(sum(times_c), world, dev) / args.steps
    replicate_ms = dist_max(sum(times_x), world, dev) / args.steps if times_x else 0.0
    median_ms = dist_max(statistics.median(times), world, dev)

    e2e = None if args.no_e2e else run_e2e(args, pkg, capi, job, ex, rank, world, dev, total_flops)

    if rank != 0:
        return None
    kernel_ms = statistics.mean(times_c)
    full = WORKLOADS[args.workload]["L"] == FULL_SIZE_L[args.workload] and world == 1 and args.shard_of <= 1
    roof = roofline_of(job, args.workload, kernel_ms, tiled, peaks, peak_src, full)
    scaling = "weak" if job.weak else "strong"
    desc = job.w["desc"]
    if world > 1:
        desc += ("; sequence of %dx%d rows, one row range per GPU" % (world, job.L_local) if job.weak else
                 "; %d rows split into %d %s query-row ranges" % (job.L, world, "nnz-balanced" if explicit else "equal"))
    line = {
        "metric": "effective_nnz_tflops_fwd", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "ms_per_step_median": median_ms,
        "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "tf32" if tiled else "f32", "data": "synthetic",
        "config": {"workload": desc, "mask": job.kind, "L": job.L, "rows_per_gpu": job.L_local, "d": job.d,
                   "nnz": int(total_nnz), "nnz_imbalance_max_over_mean": round(nnz_imbalance, 4),
                   "flops_per_step": total_flops, "path": args.path,
                   "plan": "dense-tile plan built once outside the timed region" if args.planned
                   else "none stored: every call is one-shot (mask inspection inside the timed step)",
                   "l2": "flushed (256 MiB memset) before every timed step",
                   "state": "m=-inf,l=0,O=0 re-initialised before every step outside the timed span"},
        "fwd_ms": total_ms / args.steps,
        "compute_only_ms": compute_ms,
        "replicate_ms": replicate_ms,
        "nnz_imbalance_max_over_mean": round(nnz_imbalance, 4),
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roof,
    }
    if world > 1:
        line["config"]["kv"] = ("K and V start row-sharded in %d equal chunks; every timed step replicates them: %s; chunks "
                                "received by the previous step are overwritten with NaN before each step" % (world, exchange_note))
        line["config"]["exchange_vs_resident_max_abs_diff"] = check
    if job.kind == "bigbird" and world == 1:
        t_ch, _ = timed_steps(job, lambda: job.chained_forward(capi), args.steps, args.warmup, 1)
        line["chained_three_calls_ms"] = statistics.mean(t_ch)
    if e2e:
        line.update(e2e)
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline(job, args.cpu_budget)
    if world == 1 and args.workload == DEFAULT_WORKLOAD and not args.no_per_workload and args.rows == 0:
        per = {}
        for name in PER_WORKLOAD:
            per[name] = measure_one_gpu(name, capi, dev, 6, 3, peaks, peak_src, args.path,
                                        job=job if name == args.workload else None)
        per["coo_planned"] = measure_one_gpu("coo", capi, dev, 6, 3, peaks, peak_src, args.path, planned=True, job=job)
        line["per_workload"] = per
    return line


def run_e2e(args, pkg, capi, job, ex, rank, world, dev, total_flops):
    """The step from pinned host buffers: host->device copies of this rank's Q/K/V rows, the forward (with the K/V
    exchange at N > 1), the device->host copy of its O rows -- all inside the timed span."""
    explicit = job.kind in ("csr", "coo")
    banded = job.kind in ("local", "local_1d_dilated", "local_2d_dilated")
    nan = float("nan")
    hQ = job.Q.cpu().pin_memory()
    hO = torch.empty_like(job.O, device="cpu").pin_memory()
    out = {}
    if world == 1:
        hK, hV = job.K.cpu().pin_memory(), job.V.cpu().pin_memory()
        big = job.L * job.d * 4 >= (48 << 20)
        pipe = full_pipe = chunk_call = None
        # chunking pays once a chunk's copies are large (8 chunks of 3 x 2 MB gain nothing on the 65536-row Local
        # workload: the host->device stream slows down by as much as the overlapped device->host copies save)
        if banded and big and not args.planned:
            pipe = pkg.hostio.BandedHostPipeline(job.kind, job.L, job.d, job.p0, job.p1, n_chunks=8, device=dev)
        elif not args.planned and ((banded and job.L * job.d * 4 >= (8 << 20)) or (not banded and big)):
            full_pipe = pkg.hostio.FullKeyHostPipeline(job.L, job.L, job.d, n_chunks=3 if banded else args.e2e_chunks,
                                                       device=dev)
            if banded:
                def chunk_call(a, b, q, k, v, m_, l_, o_):
                    if job.kind == "local":
                        capi.local_forward(q, k, v, m_, l_, o_, job.p0, a, b)
                    elif job.kind == "local_1d_dilated":
                        capi.local_1d_dilated_forward(q, k, v, m_, l_, o_, job.p0, job.p1, a, b)
                    else:
                        capi.local_2d_dilated_forward(q, k, v, m_, l_, o_, job.p0, job.p1, True, a, b)
            elif job.kind == "global_no_local":
                def chunk_call(a, b, q, k, v, m_, l_, o_):
                    capi.global_no_local_forward(q, k, v, m_, l_, o_, job.G, job.p0, a, b)
            elif job.kind == "bigbird":
                def chunk_call(a, b, q, k, v, m_, l_, o_):
                    ro = job.mask[0][a:b + 1]
                    lo, hi = int(cut_bb[a]), int(cut_bb[b])
                    capi.bigbird_forward(q, k, v, m_, l_, o_, job.G, job.p0, (ro - lo).contiguous(), job.mask[1][lo:hi], a, b)
                cut_bb = {e: int(job.mask[0][e]) for e in full_pipe.edges}
            elif job.kind == "coo":
                cut = torch.searchsorted(job.mask[0], torch.tensor(full_pipe.edges, device=dev)).cpu().tolist()

                def chunk_call(a, b, q, k, v, m_, l_, o_):
                    lo, hi = cut[full_pipe.edges.index(a)], cut[full_pipe.edges.index(b)]
                    capi.coo_forward(q, k, v, job.mask[0][lo:hi], job.mask[1][lo:hi], m_, l_, o_, use_nan=False, row_begin=a)
            else:
                def chunk_call(a, b, q, k, v, m_, l_, o_):  # offsets index the full column array
                    capi.csr_forward(q, k, v, job.mask[0][a:b + 1], job.mask[1], m_, l_, o_, use_nan=False)

        binding = pkg.binding("spfa_" + job.kind)
        w_val = torch.ones(1, device=dev)
        dQ, dK, dV = torch.empty_like(job.Q), torch.empty_like(job.K), torch.empty_like(job.V)
        plan_t = None
        if args.planned:
            plan_t = (binding.plan(job.mask[0], job.mask[1], job.L, job.d) if job.kind == "csr"
                      else binding.plan(job.mask[0], job.mask[1], job.L_local, job.L, job.d))

        def plugin_step():
            dQ.copy_(hQ, non_blocking=True)
            dK.copy_(hK, non_blocking=True)
            dV.copy_(hV, non_blocking=True)
            job.reset_state()
            if args.planned:
                binding.forward_planned(dQ, dK, dV, plan_t, int(job.mask[1].numel()), job.m, job.l, job.O, False)
            else:
                job.plugin_forward(binding, dQ, dK, dV, w_val)
            hO.copy_(job.O, non_blocking=True)

        def pipe_step():
            if pipe is not None:
                pipe.forward(hQ, hK, hV, hO, use_nan=True)
            else:
                full_pipe.forward(chunk_call, hQ, hK, hV, hO)

        t_plugin, _ = timed_steps(job, plugin_step, args.steps, args.warmup, 1)
        plugin_ms = statistics.mean(t_plugin)
        h2d, d2h = 3 * job.L * job.d * 4, job.L * job.d * 4
        plugin = {"value": total_flops / (plugin_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": plugin_ms,
                  "ms_per_step_median": statistics.median(t_plugin), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                  "api": "spfa_%s.%s (torch extension, the reference's module name), whole-tensor copies around one call"
                         % (job.kind, "forward_planned" if args.planned else "forward")}
        out["e2e_plugin"] = plugin
        if pipe is None and full_pipe is None:
            out["e2e"] = plugin
            return out
        t_pipe, _ = timed_steps(job, pipe_step, args.steps, args.warmup, 1)
        pipe_ms = statistics.mean(t_pipe)
        out["e2e"] = {"value": total_flops / (pipe_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": pipe_ms,
                      "ms_per_step_median": statistics.median(t_pipe), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "api": ("hostio.BandedHostPipeline.forward: 8 row chunks, host->device copies, row-range C-ABI calls "
                              "and device->host copies overlapped on three streams" if pipe is not None else
                              "hostio.FullKeyHostPipeline.forward: K and V first, then %d row chunks of Q in, row-range "
                              "C-ABI calls and O chunks out overlapped on three streams" % (len(full_pipe.edges) - 1))}
        return out

    # ---- N > 1: this rank's Q rows and its K/V chunk come from the host; the other chunks over NVLink ----
    sh = pkg.sharding
    kb, ke = job.kv_ranges[rank]
    Ko, Vo = ex.own()
    hK, hV = Ko.cpu().pin_memory(), Vo.cpu().pin_memory()
    dQ = torch.empty_like(job.Q)
    s_in = torch.cuda.Stream(device=dev)
    overlap = (explicit and not args.no_overlap and args.path != "gather" and job.nnz >= (1 << 20)
               and capi.lib().spfa_explicit_plan_bytes(job.L_local, job.nnz, job.L, job.d) > 0)
    plan_buf = (job.plan if job.plan is not None else job.build_plan(capi)) if overlap else None

    def poison():
        for t in (ex.K, ex.V):
            t.fill_(nan)
        dQ.fill_(nan)

    def step():
        cur = torch.cuda.current_stream(dev)
        kv_up, q_up = torch.cuda.Event(), torch.cuda.Event()
        s_in.wait_stream(cur)
        with torch.cuda.stream(s_in):
            Ko.copy_(hK, non_blocking=True)
            Vo.copy_(hV, non_blocking=True)
            kv_up.record(s_in)
            dQ.copy_(hQ, non_blocking=True)
            q_up.record(s_in)
        job.reset_state()
        if overlap:
            inspect = None if args.planned else (lambda: job.build_plan(capi, out=plan_buf))
            if args.tiles_first:
                first = [True]

                def on_tiles(a, b):
                    if first[0]:
                        cur.wait_event(q_up)
                        first[0] = False
                    capi.planned_forward_parts(dQ, ex.K, ex.V, job.m, job.l, job.O, plan_buf, a, b, capi.PLAN_DENSE_TILES)
                ex.run_tiles_first(on_tiles, lambda: capi.planned_forward_parts(dQ, ex.K, ex.V, job.m, job.l, job.O, plan_buf,
                                                                                0, job.L, capi.PLAN_RESIDUAL),
                                   inspect, own_ready=kv_up)
            else:
                def on_chunk(a, b, i):
                    if i == 0:
                        cur.wait_event(q_up)
                    capi.planned_forward_keys(dQ, ex.K, ex.V, job.m, job.l, job.O, plan_buf, a, b)
                ex.run_two_phase(on_chunk, inspect, own_ready=kv_up, rounds_in_phase1=args.phase1_rounds)
        else:
            cur.wait_event(q_up)
            if explicit:
                ex.exchange_only()
                job.forward(capi, dQ, ex.K, ex.V)
            else:
                Kf, Vf = sh.replicate_kv(Ko, Vo, job.kv_ranges)
                job.forward(capi, dQ, Kf, Vf)
        hO.copy_(job.O, non_blocking=True)

    t_e2e, _ = timed_steps(job, step, args.steps, args.warmup, world, before_each=poison)
    e2e_ms = dist_max(sum(t_e2e), world, dev) / args.steps
    h2d = dist_sum(float(job.L_local + 2 * (ke - kb)) * job.d * 4, world, dev)
    d2h = dist_sum(float(job.L_local) * job.d * 4, world, dev)
    out["e2e"] = {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                  "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                  "api": "per rank: K/V chunk and Q rows host->device on a copy stream, " +
                         ("sharding.KeyChunkExchange (exchange rounds start when the chunk is up; the mask inspection "
                          "meanwhile, the forward from the stored plan after the last round)"
                          if overlap else
                          "K/V replication, capi.*_forward(row range)") + ", O rows device->host; bytes are the sum over ranks"}
    return out


def cpu_baseline(job, budget):
    """The reference's dense PyTorch CPU path (SDPA-MATH on a boolean mask), row-chunked, bounded sample."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("spfa_dense_sdpa", os.path.join(ROOT, "oracle", "dense_sdpa.py"))
    ds = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ds)
    q, k, v = job.Q.cpu(), job.K.cpu(), job.V.cpu()
    G = job.G_cpu if job.kind in ("global_no_local", "bigbird") else None
    chunk = 1024 if job.L <= 65536 else (512 if job.L <= 262144 else 128)
    mask_fn = None
    if job.kind in ("csr", "coo"):  # explicit masks: scatter the chunk's entries into a dense boolean chunk
        if job.kind == "csr":
            row_off, cols = job.mask[0].cpu(), job.mask[1].cpu().long()
        else:
            row_off = torch.searchsorted(job.mask[0], torch.arange(job.L + 1, device=job.mask[0].device)).cpu()
            cols = job.mask[1].cpu().long()

        def mask_fn(r0, r1):
            lo, hi = int(row_off[r0]), int(row_off[r1])
            m = torch.zeros(r1 - r0, job.L, dtype=torch.bool)
            rr = torch.repeat_interleave(torch.arange(r1 - r0), (row_off[r0 + 1:r1 + 1] - row_off[r0:r1]))
            m[rr, cols[lo:hi]] = True
            return m
    if job.kind == "bigbird":  # union of the two closed-form masks and the scattered CSR part
        row_off, cols = job.mask[0].cpu(), job.mask[1].cpu().long()

        def mask_fn(r0, r1):
            m = ds.mask_chunk("local", job.L, r0, r1, job.p0) | ds.mask_chunk("global_no_local", job.L, r0, r1, job.p0, 0, job.G_cpu)
            lo, hi = int(row_off[r0]), int(row_off[r1])
            rr = torch.repeat_interleave(torch.arange(r1 - r0), (row_off[r0 + 1:r1 + 1] - row_off[r0:r1]))
            m[rr, cols[lo:hi]] = True
            return m
    r = ds.time_dense_cpu(job.kind, q, k, v, job.p0, job.p1, G, chunk_rows=chunk, budget_s=budget, max_chunks=64,
                          mask_fn=mask_fn)
    val = 4.0 * r["nnz"] * job.d / r["seconds"] / 1e12
    return {"value": val, "unit": "TFLOP/s", "cores": r["threads"], "kind": "port",
            "sample": f"{r['chunks']} evenly spaced chunks of {chunk} rows x all {job.L} keys ({r['rows']} of {job.L} rows), "
                      f"dense scaled_dot_product_attention under SDPBackend.MATH on CPU, {r['seconds']:.1f} s, "
                      f"{r['threads']} torch threads on {r['cores']} logical cores; useful flops 4*nnz*d of the sampled rows"}


def reference_step_fn(job, mods, dev):
    """(step function, note) running the reference's own kernel for this job's mask on the whole job.
    COO above 32768 rows: the reference COO kernel scans the row-index array once per row (O(L*nnz): 12.4 s per call
    at 16384 rows of this graph, 51.1 s at 32768, i.e. about 14 hours at 2^20) and does not complete; its CSR kernel on
    the identical mask (row offsets derived from the sorted row indices) stands in."""
    w_val = torch.ones(1, device=dev)
    st = (job.m, job.l, job.O)
    k, note = job.kind, None
    if k == "coo" and job.L > 32768:
        row_off = torch.searchsorted(job.mask[0], torch.arange(job.L + 1, device=dev)).contiguous()
        mod = mods("csr")
        if mod is None:
            return None, None
        note = ("reference CSR kernel on the identical mask: the reference COO kernel re-scans the row-index array for "
                "every row (O(L*nnz)) and does not complete at this size")
        return (lambda: mod.forward(job.Q, job.K, job.V, row_off.view(torch.uint64), job.mask[1].view(torch.uint32), w_val,
                                    *st, False)), note
    if k == "bigbird":  # the reference's own composition: three chained calls (verification/verify.py:337-352)
        ml, mg, mc = mods("local"), mods("global_no_local"), mods("csr")
        if ml is None or mg is None or mc is None:
            return None, None

        def chain():
            ml.forward(job.Q, job.K, job.V, *st, job.p0)
            mg.forward(job.Q, job.K, job.V, *st, job.G, job.p0)
            mc.forward(job.Q, job.K, job.V, job.mask[0].view(torch.uint64), job.mask[1].view(torch.uint32), w_val, *st, False)
        return chain, "the reference's chained composition: spfa_local, spfa_global_no_local, spfa_csr on one state"
    mod = mods(k)
    if mod is None:
        return None, None
    if k == "local":
        return (lambda: mod.forward(job.Q, job.K, job.V, *st, job.p0)), note
    if k == "local_1d_dilated":
        return (lambda: mod.forward(job.Q, job.K, job.V, *st, job.p0, job.p1)), note
    if k == "local_2d_dilated":
        return (lambda: mod.forward(job.Q, job.K, job.V, *st, job.p0, job.p1, True)), note
    if k == "global_no_local":
        return (lambda: mod.forward(job.Q, job.K, job.V, *st, job.G, job.p0)), note
    return (lambda: mod.forward(job.Q, job.K, job.V, job.mask[0].view(torch.uint64), job.mask[1].view(torch.uint32), w_val,
                                *st, False)), note


def run_reference(args, rank, world, dev):
    """The reference's own CUDA kernels (compiled unmodified into oracle/_ref/) on the same workload, one GPU."""
    if rank != 0:
        return None
    import importlib.util

    spec = importlib.util.spec_from_file_location("spfa_build_ref", os.path.join(ROOT, "oracle", "build_ref.py"))
    br = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(br)
    job = Job(args.workload, 0, world, dev, whole_on_one_gpu=True, weak=args.weak)  # the reference is single-GPU
    base = {"impl": "reference", "metric": "effective_nnz_tflops_fwd", "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "weak" if job.weak else "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": job.w["desc"], "mask": job.kind, "L": job.L, "d": job.d, "nnz": int(job.nnz)}}
    step, note = reference_step_fn(job, br.load, dev)
    if step is None:
        # no rebuilt reference kernels on this box: time the reference's dense CPU path instead
        cb = cpu_baseline(job, max(args.cpu_budget, 10.0))
        base.update({"value": cb["value"], "ms_per_step": None, "cpu_baseline": cb,
                     "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                     "gpu_launches": 0, "config": {**base["config"], "arm": "dense SDPA-MATH on CPU (oracle/_ref not built)"}})
        return base
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    # the reference launches on the legacy default stream; events are recorded there too
    with torch.cuda.stream(torch.cuda.default_stream(dev)):
        times, _ = timed_steps(job, step, args.steps, args.warmup, 1)
    clocks = sampler.stop()
    total_ms = sum(times)
    value = job.flops * args.steps / (total_ms * 1e-3) / 1e12
    cb = {"value": None, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "reference",
          "sample": "this arm runs the reference's CUDA kernels on the GPU (the reference has no CPU implementation); "
                    "the dense CPU path is timed in the other arm's cpu_baseline"}
    arm = ("reference CUDA kernels compiled unmodified for sm_100a (oracle/_ref), device-resident inputs, legacy default "
           "stream, the whole workload on one GPU (the reference is single-GPU)")
    base.update({"value": value, "ms_per_step": total_ms / args.steps, "ms_per_step_median": statistics.median(times),
                 "fwd_ms": total_ms / args.steps, "clocks": clocks,
                 "cpu_baseline": cb, "gpu_launches": args.steps,
                 "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                 "config": {**base["config"], "arm": arm + ("; " + note if note else ""),
                            "l2": "flushed (256 MiB memset) before every timed step"}})
    if world == 1 and args.workload == DEFAULT_WORKLOAD and not args.no_per_workload and args.rows == 0:
        per = {}
        for name in PER_WORKLOAD:
            j = job if name == args.workload else Job(name, 0, 1, dev, whole_on_one_gpu=True)
            fn, nt = reference_step_fn(j, br.load, dev)
            if fn is None:
                continue
            with torch.cuda.stream(torch.cuda.default_stream(dev)):
                t, _ = timed_steps(j, fn, 3, 1, 1)
            ms = statistics.mean(t)
            per[name] = {"workload": j.w["desc"], "fwd_ms": ms, "tflops": j.flops / (ms * 1e-3) / 1e12, "steps": 3}
            if nt:
                per[name]["note"] = nt
            if j is not job:
                del j
                torch.cuda.empty_cache()
        base["per_workload"] = per
    return base


def main():
    args = parse_args()
    if args.rows > 0:
        w = dict(WORKLOADS[args.workload])
        w["desc"] = w["desc"].replace(f"L={w['L']}", f"L={args.rows}") + " [reduced size]"
        w["L"] = args.rows
        WORKLOADS[args.workload] = w
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    if args.impl == "reference" and rank != 0:
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device: this benchmark has no CPU path"}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and args.impl == "ours":
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    try:
        line = run_ours(args, rank, world, dev) if args.impl == "ours" else run_reference(args, rank, world, dev)
        if line is not None:
            print(json.dumps(line))
    finally:
        if world > 1 and args.impl == "ours":
            import torch.distributed as dist

            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
