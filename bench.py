#!/usr/bin/env python
"""KV handoff benchmark: GB/s of prefill->decode KV movement, device-timed, max over ranks.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one handoff of the whole batch.  The default workload is the benchmark's scaling configuration
(Llama-3.1-70B shape, 80 layers, 32 prompts of 4096 tokens, 42.9 GB of F16 K/V) at every N: N = 1 moves it
between a prefill pool and a decode pool on the same GPU (HBM-bound); N = 2, 4, 8 is one process per GPU,
ranks [0, N/2) prefill and ranks [N/2, N) decode, the batch's KV heads split evenly over the pairs
(tkv_pairing_make) and every pair moving its share over NVLink -- pulled by the decode GPU's kernel (loads from the
mapped prefill pool, local stores) or, with --push, stored into the peer pool by the prefill GPU's kernel -- (strong
scaling: the batch is fixed).  The block tables of the side that does not run the kernel reach the other rank as
tkv_session_pack messages.  --workload cfg1..cfg4 select the other configurations (at N > 1 every pair then moves its
own batch: weak scaling).  Every run ends with a parity step outside the timed region: every moved row of every
layer on the destination against the source, bit for bit, or the run exits non-zero.  Prints ONE JSON line on rank 0.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np

METRIC = "kv_handoff_GBps"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum per launch divided by the algorithmic bytes of
# the same launch, from the ncu captures summarised under profiles/ (None until captured).
NCU_TRAFFIC_RATIO = {"handoff_copy_bulk": 0.979, "handoff_copy_vec": 0.954, "handoff_f16_e4m3_warp": 0.942,
                     "handoff_f16_e4m3_staged": 0.964}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ----------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index, also=()):
        """Samples `gpu_index` (whose clock is reported) and the GPUs in `also` (whose throttle reasons count as well:
        across GPUs the kernel may run on the partner)."""
        self.gpu = gpu_index
        self.gpus = [gpu_index] + [g for g in also if g != gpu_index]
        self.rows = []
        self.proc = None
        self.marks = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", ",".join(str(g) for g in self.gpus)], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
            return
        self.t = threading.Thread(target=self._read, daemon=True)
        self.t.start()
        t0 = time.perf_counter()                      # the tool takes a moment to come up: the timed region must not beat it
        while not self.rows and time.perf_counter() - t0 < 8.0:
            time.sleep(0.02)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def mark(self):
        self.marks.append(time.perf_counter())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        lo = self.marks[0] if self.marks else 0.0
        hi = self.marks[-1] if len(self.marks) > 1 else float("inf")
        sm, mx, reasons, n, others = [], [], set(), 0, {}
        for t, line in self.rows:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                idx, clk, cmax = int(parts[0]), float(parts[1]), float(parts[2])
            except ValueError:
                continue
            inside = lo - 0.05 <= t <= hi + 0.05
            if inside:
                if idx == self.gpu:
                    sm.append(clk)
                    n += 1
                else:
                    others.setdefault(idx, []).append(clk)
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            mx.append(cmax)
        if not sm:   # region shorter than the sampling period: use everything seen
            sm = [float(r[1].split(",")[1]) for r in self.rows if len(r[1].split(",")) >= 9] or [0.0]
        out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx) if mx else None,
               "reasons": sorted(reasons), "samples": n}
        if others:
            out["partner_sm_mhz"] = {str(k): statistics.median(v) for k, v in others.items()}
        return out


class NullSampler:
    def start(self): pass
    def mark(self): pass
    def stop(self): return {}


# ----------------------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------------------
def pick_workload(name: str, n_gpus: int, pool_blocks: int | None, heads: int | None = None, layers: int | None = None,
                  single_tokens: int | None = None):
    if single_tokens:               # latency probe: ONE prompt of that many tokens on the config-2/3 shape
        from tempura_b200 import workloads as W
        fn = W.llama8b_fp8 if name == "cfg3" else W.llama8b_f16
        w = fn(pool_blocks=pool_blocks or 8192, n_seqs=1, lo=single_tokens, hi=single_tokens)
        w.name += f"-1x{single_tokens}tok"
        return w
    w = _pick_workload(name, n_gpus, pool_blocks, heads)
    if layers:                      # profiling aid: same batch and tables, fewer layers
        w.n_layers = layers
        w.name += f"-{layers}layers"
    return w


def _pick_workload(name: str, n_gpus: int, pool_blocks: int | None, heads: int | None = None):
    from tempura_b200 import workloads as W
    if name == "cfg1":
        return W.tinyllama_cpu()
    if name in ("cfg2", "cfg3", "cfg4"):
        if pool_blocks is None:
            pool_blocks = 32768 if n_gpus == 1 else 65536      # two pools share one GPU at N = 1
        fn = {"cfg2": W.llama8b_f16, "cfg3": W.llama8b_fp8, "cfg4": W.llama8b_prefix}[name]
        return fn(pool_blocks=pool_blocks)
    if name == "cfg5":
        pairs = max(1, n_gpus // 2)
        return W.llama70b_f16(n_kv_heads=heads or 8 // pairs)
    raise SystemExit(f"unknown workload {name}")


def fill_source(pool, w, seed: int):
    """Seeded N(0, sigma) F16 values in every block a table names; the 0xA5 pattern stays
    elsewhere.  Outlier channels (config 3) are scaled by the workload's gain."""
    import torch
    g = torch.Generator(device=f"cuda:{pool.device}")
    g.manual_seed(seed)
    bs = w.block_size
    used = np.unique(np.concatenate([w.src_tables[q, : (int(w.seq_lens[q]) + bs - 1) // bs] for q in range(len(w.seq_lens))]))
    idx = torch.from_numpy(used.astype(np.int64)).to(f"cuda:{pool.device}")
    for l in range(pool.n_layers):
        for is_v in (False, True):
            vals = torch.randn((len(used), bs, pool.n_kv_heads, pool.head_dim), generator=g,
                               device=idx.device, dtype=torch.float32) * w.sigma
            for c in w.outlier_channels:
                vals[..., c] *= w.outlier_gain
            pool.blocks(l, is_v).index_copy_(0, idx, vals.to(pool.blocks(l, is_v).dtype))
    torch.cuda.synchronize()


# ----------------------------------------------------------------------------------------
# parity inside the run (not timed)
# ----------------------------------------------------------------------------------------
def _moved_block_ids(w, tables):
    """Block ids of every moved block, in work-list order (sequence by sequence, past the shared prefix)."""
    bs, out = w.block_size, []
    for q in range(len(w.seq_lens)):
        pre = int(w.prefix_lens[q]) // bs if w.prefix_lens is not None else 0
        nb = (int(w.seq_lens[q]) + bs - 1) // bs
        out.append(tables[q, pre:nb])
    return np.concatenate(out).astype(np.int64)


def _compact_batch(w):
    """The same moved blocks described against a transfer buffer: identity tables in work-list order, no prefix."""
    bs = w.block_size
    pre = w.prefix_lens.astype(np.int64) if w.prefix_lens is not None else np.zeros(len(w.seq_lens), dtype=np.int64)
    lens = w.seq_lens.astype(np.int64) - pre
    nb = (lens + bs - 1) // bs
    stride = int(max(1, nb.max()))
    tab = np.zeros((len(lens), stride), dtype=np.uint32)
    off = 0
    for q, k in enumerate(nb):
        tab[q, :k] = np.arange(off, off + k, dtype=np.uint32)
        off += int(k)
    return lens.astype(np.uint32), tab, stride, off


def parity_step(H, w, batch, src, dst, is_prefill, partner, multi, local, scales):
    """Not timed.  Every moved row of every layer, destination against source, bit for bit.

    Both sides gather their rows of a few layers at a time into a contiguous buffer (source pool through the
    source tables, cast as the handoff casts; destination pool through the destination tables) and the buffers
    must be byte-equal, scales included.  For same-dtype moves the reference's bits checksum (wrapping sum of
    the f32 bit patterns, engine/src/cutile_kv_cache.rs:1274-1368) of each side is reported as well, and one
    layer is also compared through torch indexing, which shares no code with the library.  For an E4M3
    destination the first and the last layer are compared with the CPU oracle's bytes and scales.  With two
    or more GPUs the decode rank sends its gathered rows to the prefill rank of its pair over NCCL.
    Returns a dict for the JSON line, or raises SystemExit."""
    import torch
    import torch.distributed as dist
    L, bs = w.n_layers, w.block_size
    n_blocks = H.batch_blocks(batch, bs)
    if n_blocks == 0:
        return {"parity": "bit-exact", "layers": 0, "bytes_compared_per_pair": 0}
    es_dst = {"f32": 4, "f16": 2, "e4m3": 1}[w.dst_dtype]
    half = n_blocks * bs * w.n_kv_heads * w.head_dim          # elements of one K or V plane
    per_layer = 2 * half * es_dst
    chunk = int(max(1, min(L, (3 << 29) // per_layer)))
    same = w.src_dtype == w.dst_dtype
    fp8_cast = w.src_dtype == "f16" and w.dst_dtype == "e4m3"
    own_dst = H.Batch(batch.seq_lens, batch.dst_tables, batch.dst_tables, batch.table_stride, batch.prefix_lens)
    have_src = is_prefill
    have_dst = (not multi) or (not is_prefill)
    dev = torch.device("cuda", local)
    M64 = (1 << 64) - 1
    ok, compared, sum_src, sum_dst = True, 0, 0, 0
    mk = lambda fill: H.Transfer.allocate(chunk, w.n_kv_heads, w.head_dim, bs, n_blocks, w.dst_dtype, device=local, scales=scales, fill_byte=fill)
    xa = mk(0x5A) if have_src else None
    xb = mk(0x5A) if have_dst else None
    xr = mk(None) if (multi and have_src) else None
    n_sc = lambda nl: 2 * nl * n_blocks * w.n_kv_heads       # scales of nl layers: K of every layer, then V

    def gather_both(l0, nl):
        """Rows of layers [l0, l0 + nl): the source's in xa, the destination's in the returned buffer (on the prefill rank)."""
        shard = H.Shard(0, 0, w.n_kv_heads, l0, 0, nl)
        pa = pb = None
        if have_src:
            xa.data.fill_(0x5A)
            pa = H.Plan.to_transfer(src, xa, batch, shard)
            pa.enqueue()
        if have_dst:
            xb.data.fill_(0x5A)
            pb = H.Plan.to_transfer(dst, xb, own_dst, shard)
            pb.enqueue()
        torch.cuda.synchronize()
        del pa, pb
        if not multi:
            return xb
        if have_dst:
            dist.send(xb.data[:nl * per_layer], partner)
            if scales:
                dist.send(xb.scales, partner)
            return xb
        dist.recv(xr.data[:nl * per_layer], partner)
        if scales:
            dist.recv(xr.scales, partner)
        return xr

    for l0 in range(0, L, chunk):
        nl = min(chunk, L - l0)
        used = nl * per_layer
        got = gather_both(l0, nl)
        if have_src:
            ok = ok and torch.equal(xa.data[:used], got.data[:used])
            if scales:
                ok = ok and torch.equal(xa.scales.view(-1)[:n_sc(nl)].view(torch.int32), got.scales.view(-1)[:n_sc(nl)].view(torch.int32))
            compared += used
        if same and w.dst_dtype in ("f16", "f32"):
            view = torch.float16 if w.dst_dtype == "f16" else torch.float32
            if have_src:
                sum_src = (sum_src + H.bits_checksum(xa.data[:used].view(view), w.dst_dtype)) & M64
            if have_dst:
                sum_dst = (sum_dst + H.bits_checksum(xb.data[:used].view(view), w.dst_dtype)) & M64

    # ---- an E4M3 destination against the oracle's own bytes and scales, first and last layer ----
    oracle_checked = []
    for layer in (sorted({0, L - 1}) if fp8_cast else []):
        got = gather_both(layer, 1)
        if have_src:
            import oracle
            xf = H.Transfer.allocate(1, w.n_kv_heads, w.head_dim, bs, n_blocks, "f16", device=local, fill_byte=0xA5)
            pf = H.Plan.to_transfer(src, xf, batch, H.Shard(0, 0, w.n_kv_heads, layer, 0, 1))
            pf.enqueue()
            torch.cuda.synchronize()
            rows = xf.data[:4 * half].cpu().numpy().view(np.uint16)
            hs = oracle.HostPool(1, w.n_kv_heads, w.head_dim, bs, n_blocks, np.dtype(np.uint16), [rows[:half]], [rows[half:2 * half]])
            hd = oracle.HostPool.filled(1, w.n_kv_heads, w.head_dim, bs, n_blocks, np.uint8, 0x5A, with_scales=True)
            lens, tab, stride, _ = _compact_batch(w)
            oracle.handoff(hs, hd, oracle.make_batch(lens, tab, tab, stride), None, "f16_e4m3", n_threads=os.cpu_count() or 1)
            dev_bytes = got.data[:2 * half].cpu().numpy()
            dev_scales = got.scales.view(-1)[:n_sc(1)].cpu().numpy().view(np.uint32)
            ok = ok and np.array_equal(dev_bytes[:half], hd.k[0]) and np.array_equal(dev_bytes[half:], hd.v[0])
            ok = ok and np.array_equal(dev_scales[:n_sc(1) // 2], hd.k_scales.view(np.uint32).reshape(-1))
            ok = ok and np.array_equal(dev_scales[n_sc(1) // 2:], hd.v_scales.view(np.uint32).reshape(-1))
            del xf, pf
        oracle_checked.append(layer)

    # ---- one layer through torch indexing (no library code on either side): the whole blocks of every sequence ----
    indep = None
    if same:
        layer = L - 1
        s_ids, d_ids = _moved_block_ids(w, w.src_tables), _moved_block_ids(w, w.dst_tables)
        whole = []
        for q in range(len(w.seq_lens)):                       # a ragged last block keeps the destination's fill in its tail rows
            pre = int(w.prefix_lens[q]) // bs if w.prefix_lens is not None else 0
            nb = (int(w.seq_lens[q]) + bs - 1) // bs
            whole += [True] * (nb - pre)
            if int(w.seq_lens[q]) % bs and nb > pre:
                whole[-1] = False
        whole = np.asarray(whole, dtype=bool)
        for is_v in (False, True):
            b = None
            if have_dst:
                b = dst.blocks(layer, is_v).index_select(0, torch.from_numpy(d_ids[whole]).to(dev)).contiguous()
                if multi:
                    dist.send(b.view(torch.uint8).reshape(-1), partner)
            if have_src:
                a = src.blocks(layer, is_v).index_select(0, torch.from_numpy(s_ids[whole]).to(dev)).contiguous()
                if multi:
                    b = torch.empty_like(a)
                    dist.recv(b.view(torch.uint8).reshape(-1), partner)
                ok = ok and torch.equal(a.view(torch.uint8), b.view(torch.uint8))
        indep = layer
    del xa, xb, xr
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    if multi:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        sums = torch.tensor([sum_src >> 32, sum_src & 0xFFFFFFFF, sum_dst >> 32, sum_dst & 0xFFFFFFFF], dtype=torch.int64, device=dev)
        gathered = [torch.zeros_like(sums) for _ in range(dist.get_world_size())]
        dist.all_gather(gathered, sums)
        pairs = dist.get_world_size() // 2
        sum_src = sum((int(g[0]) << 32) | int(g[1]) for g in gathered[:pairs]) & M64
        sum_dst = sum((int(g[2]) << 32) | int(g[3]) for g in gathered[pairs:]) & M64
    if not bool(flag.item()) or sum_src != sum_dst:
        raise SystemExit(f"PARITY FAILED: destination rows differ from source rows (bits checksum {sum_src:#x} vs {sum_dst:#x})")
    out = {"parity": "bit-exact", "layers": L, "bytes_compared_per_pair": int(compared),
           "how": "destination rows gathered through the destination tables == source rows gathered through the source tables"
                  + ("" if same else " and cast as the handoff casts") + ", every layer, bytes" + (" and scales" if scales else "")}
    if same and w.dst_dtype in ("f16", "f32"):
        out["bits_checksum"] = f"{sum_src:#018x}"
    if oracle_checked:
        out["oracle_layers"] = oracle_checked
    if indep is not None:
        out["torch_indexing_layer"] = indep
    return out


# ----------------------------------------------------------------------------------------
# CPU baseline (oracle) on a bounded sample
# ----------------------------------------------------------------------------------------
def cpu_sample_workload(w, layers: int, pool_blocks: int):
    from tempura_b200 import workloads as W
    s = W.Workload(w.name + "-cpu-sample", layers, w.n_kv_heads, w.head_dim, w.block_size, pool_blocks, pool_blocks,
                   w.seq_lens.copy(), src_dtype=w.src_dtype, dst_dtype=w.dst_dtype, prefix_lens=w.prefix_lens,
                   outlier_channels=w.outlier_channels, outlier_gain=w.outlier_gain, seed=w.seed)
    return s.build_tables()


class CpuSample:
    """The oracle's handoff (the reference's CPU path restated) on `layers` layers of the workload with all its
    sequences and full tables; pools shrunk to the next power of two above the batch so two of them fit host RAM."""

    def __init__(self, w, layers: int):
        import oracle
        self.oracle = oracle
        need = int(((w.seq_lens.astype(np.int64) + w.block_size - 1) // w.block_size).sum()) + 256
        pool_blocks = 1 << int(np.ceil(np.log2(need)))
        s = self.s = cpu_sample_workload(w, layers, pool_blocks)
        npdt = {"f16": np.uint16, "e4m3": np.uint8, "f32": np.float32}
        self.src = oracle.HostPool.filled(layers, s.n_kv_heads, s.head_dim, s.block_size, pool_blocks, npdt[s.src_dtype], 0xA5)
        self.dst = oracle.HostPool.filled(layers, s.n_kv_heads, s.head_dim, s.block_size, pool_blocks, npdt[s.dst_dtype], 0x5A,
                                          with_scales=(s.dst_dtype == "e4m3"))
        for l in range(layers if s.dst_dtype == "e4m3" else 0):   # values only matter to the FP8 path
            for kv, arrs in enumerate((self.src.k, self.src.v)):
                arrs[l][:] = oracle.gen_normal_f16(arrs[l].size, s.seed, 2 * l + kv, s.sigma, s.head_dim,
                                                   s.outlier_channels, s.outlier_gain)
        self.batch = oracle.make_batch(s.seq_lens, s.src_tables, s.dst_tables, s.table_stride, s.prefix_lens)
        self.mode = "copy" if s.src_dtype == s.dst_dtype else "f16_e4m3"
        self.payload = s.payload_bytes
        self.what = (f"{layers} of {w.n_layers} layers, all {len(w.seq_lens)} sequences ({self.payload / 1e6:.0f} MB payload per step), "
                     f"pools shrunk to {pool_blocks} blocks")

    def step(self, threads: int) -> float:
        t0 = time.perf_counter()
        self.oracle.handoff(self.src, self.dst, self.batch, None, self.mode, n_threads=threads)
        return time.perf_counter() - t0


def time_cpu(w, threads: int, layers: int, reps: int):
    c = CpuSample(w, layers)
    c.step(threads)                    # warm-up: page faults of the pools
    best = min(c.step(threads) for _ in range(reps))
    return c.payload / best / 1e9, c.what + f"; best of {reps}"


def sample_layers(w) -> int:
    """Layers of the CPU sample: about 2 GB of payload per step for a copy, about 0.3 GB for the FP8 cast."""
    per_layer = max(1, w.payload_bytes // w.n_layers)
    budget = 300_000_000 if w.dst_dtype == "e4m3" else 2_200_000_000
    return int(max(1, min(w.n_layers, budget // per_layer)))


def describe(w, world: int, small: bool, push: bool = False, gpu_order: str = "interleaved") -> dict:
    """The `config` object, the same in both arms."""
    pairs = max(1, world // 2)
    strong = w.name.startswith("llama3.1-70b")
    pulled = w.src_dtype == w.dst_dtype and not push
    return {"workload": w.name, "layers": w.n_layers, "kv_heads": w.n_kv_heads * (pairs if strong else 1),
            "kv_heads_per_pair": w.n_kv_heads, "head_dim": w.head_dim, "block_size": w.block_size, "n_seqs": len(w.seq_lens),
            "tokens_moved": w.tokens_moved, "payload_bytes": int(w.payload_bytes) * pairs, "pool_blocks": [w.src_blocks, w.dst_blocks],
            "pairs": pairs,
            "placement": ("intra-device: prefill pool -> decode pool on one GPU" if world == 1 else
                          ("one batch, KV heads split over the pairs; " if strong else "every pair its own batch; ") +
                          "prefill rank i -> decode rank i+N/2" + (" (GPUs 2i -> 2i+1), " if world > 2 and gpu_order == "interleaved" else ", ") +
                          ("the decode GPU's kernel loads from the prefill pool over NVLink and stores into its own pool" if pulled else
                           "the prefill GPU's kernel stores into the decode pool over NVLink")),
            "l2": ("256 MB written between timed launches (batch fits L2)" if small else "inputs larger than L2 (no flush needed)")}


def is_small(w) -> bool:
    return w.payload_bytes * 2 < 4 * 126_000_000


def default_workload(args) -> str:
    return args.workload or "cfg5"


def run_reference(args):
    """The reference's CPU handoff (its Rust cannot be built here: the oracle port stands in), on all host cores.
    A step is one handoff of a bounded sample of the workload (some of its layers, every sequence, full tables);
    K steps are timed after W warm-up steps, and `ms_per_step` is the measured time of such a step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(1, args.gpus)
    w = pick_workload(default_workload(args), world, 4096 if default_workload(args) != "cfg5" else None)
    pairs = max(1, world // 2)
    strong = w.name.startswith("llama3.1-70b")
    # the CPU moves the whole batch (every kv head): the unsharded workload is what it is timed on
    w_cpu = pick_workload(default_workload(args), 1, 4096 if default_workload(args) != "cfg5" else None) if strong else w
    cores = os.cpu_count() or 1
    c = CpuSample(w_cpu, sample_layers(w_cpu))
    for _ in range(max(1, args.warmup)):
        c.step(cores)
    steps, t_total, t0 = 0, 0.0, time.perf_counter()
    for _ in range(max(1, args.steps)):
        t_total += c.step(cores)
        steps += 1
        if time.perf_counter() - t0 > 150:            # bounded: a slow host stops early and says so
            break
    ms = t_total / steps * 1e3
    v = c.payload / (ms * 1e-3) / 1e9
    sample = c.what + f"; {steps} timed steps after {max(1, args.warmup)} warm-up"
    full_ms = w_cpu.payload_bytes / (v * 1e9) * 1e3
    cfg = describe(pick_workload(default_workload(args), world, None), world, is_small(w), getattr(args, "push", False), args.gpu_order)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(v, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": max(1, args.warmup), "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "strong" if strong else "weak",
        "vs_baseline": None, "dtype": "u16" if w.dst_dtype != "e4m3" else "f16->e4m3", "data": "synthetic",
        "config": cfg,
        "note": "reference CPU handoff restated in C (oracle port; the Rust reference has no toolchain here), OpenMP over (sequence, layer, K|V); "
                "a step moves the sample, not the whole batch",
        "ms_per_whole_batch_at_this_rate": round(full_ms, 2),
        "cpu_baseline": {"value": round(v, 3), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(v, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------
# comparison baseline for N > 1: staged copy through NCCL
# ----------------------------------------------------------------------------------------
def nccl_baseline(H, w, batch, src, dst, is_prefill, partner, local, scales, steps, barrier):
    """The conventional route the peer-store kernel replaces: gather the prompts' blocks into a
    contiguous staging buffer (cast before the wire for an E4M3 pool), ncclSend it, ncclRecv
    it on the decode GPU, scatter it into the decode pool.  Device-timed per rank, max over ranks."""
    import torch
    import torch.distributed as dist
    n_blocks = H.batch_blocks(batch, w.block_size)
    wire = "e4m3" if scales else "f16"
    x = H.Transfer.allocate(w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, n_blocks, wire, device=local, scales=scales)
    if is_prefill:
        plan = H.Plan.to_transfer(src, x, batch)
    else:
        own = H.Batch(batch.seq_lens, batch.dst_tables, batch.dst_tables, batch.table_stride, batch.prefix_lens)
        plan = H.Plan.from_transfer(x, dst, own)
    used = x.data                                   # whole planes travel, padding rows included
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def step():
        if is_prefill:
            plan.enqueue()
            dist.send(used, partner)
            if scales:
                dist.send(x.scales, partner)
        else:
            dist.recv(used, partner)
            if scales:
                dist.recv(x.scales, partner)
            plan.enqueue()

    for _ in range(2):
        step()
    barrier()
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    barrier()
    ms = float(t.item()) / steps
    pairs = dist.get_world_size() // 2
    payload = w.payload_bytes * pairs
    return {"value": round(payload / (ms * 1e-3) / 1e9, 2), "unit": UNIT, "ms_per_step": round(ms, 5), "steps": steps,
            "wire_bytes_per_pair": int(used.numel()) + (int(x.scales.numel()) * 4 if scales else 0),
            "what": "tkv to_transfer kernel -> ncclSend/ncclRecv (torch.distributed) -> tkv from_transfer kernel, the three stages "
                    "strictly one after another per step (not pipelined across layers): the plain library route, for comparison only"}


# ----------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------
KERNEL_NAMES = {1: "handoff_copy_vec", 2: "handoff_copy_bulk", 3: "handoff_f16_e4m3_warp", 4: "handoff_f16_e4m3_generic",
                5: "handoff_f32_cast_generic", 6: "handoff_f16_e4m3_staged", 7: "handoff_e4m3_dequant", 8: "handoff_f32_cast_vec", 9: "handoff_copy_wide"}


FLUSH_THEN_READ = False


def time_handoffs(H, plan, w, steps, stream, done_flag, gen):
    """K handoffs, inputs resident in HBM, device-timed on the launching stream.  A batch whose bytes would fit L2
    (126 MB) is timed launch by launch with a 256 MB write in between, so every timed launch starts with a cold
    L2; larger batches run back to back.  Returns (total ms, next flag generation)."""
    import torch
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if is_small(w):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        clean = torch.zeros(64 << 20, dtype=torch.int32, device="cuda") if FLUSH_THEN_READ else None
        ms = 0.0
        for i in range(steps):
            gen += 1
            flush.fill_(i & 0xFF)
            if clean is not None:
                clean.sum()                 # probe: leave L2 full of clean lines, so the timed kernel evicts nothing dirty
            ev0.record(stream)
            plan.enqueue(stream, done_flag, gen)
            ev1.record(stream)
            torch.cuda.synchronize()
            ms += ev0.elapsed_time(ev1)
        return ms, gen
    ev0.record(stream)
    for _ in range(steps):
        gen += 1
        plan.enqueue(stream, done_flag, gen)
    ev1.record(stream)
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1), gen


def quick_config(H, name, steps, peak):
    """One of the other benchmark configurations on one GPU, device-timed the same way (no end-to-end legs):
    extra keys of the line, not the line's value."""
    import torch
    w = pick_workload(name, 1, None)
    scales = w.dst_dtype == "e4m3"
    src = H.Pool.allocate(0, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.src_blocks, w.src_dtype)
    dst = H.Pool.allocate(0, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.dst_blocks, w.dst_dtype,
                          scales=scales, refcounts=w.prefix_lens is not None, fill_byte=0x5A)
    fill_source(src, w, 4321)
    batch = H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens)
    plan = H.Plan(src, dst, batch)
    stream = torch.cuda.current_stream()
    for _ in range(3):
        plan.enqueue(stream)
    torch.cuda.synchronize()
    ms, _ = time_handoffs(H, plan, w, steps, stream, 0, 0)
    par = parity_step(H, w, batch, src, dst, True, 0, False, 0, scales)
    st = plan.stats()
    per = ms / steps
    out = {"workload": w.name, "value": round(st.payload_bytes / (per * 1e-3) / 1e9, 2), "unit": UNIT, "ms_per_step": round(per, 5),
           "steps": steps, "frac": round((st.bytes_read + st.bytes_written) / (per * 1e-3) / 1e9 / peak, 4),
           "kernel": KERNEL_NAMES.get(st.kernel_variant, "?"), "pool_blocks": [w.src_blocks, w.dst_blocks], "parity": par["parity"],
           "l2": "flushed between launches" if is_small(w) else "inputs larger than L2"}
    if "oracle_layers" in par:
        out["oracle_layers"] = par["oracle_layers"]
    plan.destroy()
    del src, dst, plan
    torch.cuda.empty_cache()
    return out


def exchange_tables(w, is_prefill: bool, mover: bool, partner: int, dst_dtype: str) -> dict:
    """The handoff's metadata crosses the process boundary as the library's checksummed session messages
    (tkv_session_pack / tkv_session_unpack; SessionTransfer's field set, engine/src/session.rs:194-200): the rank whose GPU
    does not run the kernel announces, for every prompt, the pages it holds in ITS pool -- two page-granular pieces per
    prompt, sent in reverse order -- and the rank that runs the kernel builds that side of its block tables from the
    messages alone (its own seeded copy of the far side's table is wiped first).  The K/V bytes do not travel in the
    messages: the kernel moves them."""
    import torch
    import torch.distributed as dist
    from tempura_b200 import _native as N
    from tempura_b200 import session as S
    code = {"f32": N.DTYPE_F32, "f16": N.DTYPE_F16, "e4m3": N.DTYPE_E4M3}
    mine_dtype = code["f16"] if is_prefill else code[dst_dtype]
    far_dtype = code[dst_dtype] if is_prefill else code["f16"]
    n_msgs = 0
    if not mover:
        tables = w.src_tables if is_prefill else w.dst_tables
        msgs = S.pack_batch(w.seq_lens, tables, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, mine_dtype, pieces=2)[::-1]
        blob = S.frame(msgs)
        dist.send(torch.tensor([len(blob), len(msgs)], dtype=torch.int64, device="cuda"), partner)
        dist.send(torch.frombuffer(bytearray(blob), dtype=torch.uint8).cuda(), partner)
        n_msgs, n_bytes = len(msgs), len(blob)
    else:
        far = w.dst_tables if is_prefill else w.src_tables
        seeded = far.copy()
        far.fill(0xFFFFFFFF)
        head = torch.zeros(2, dtype=torch.int64, device="cuda")
        dist.recv(head, partner)
        n_bytes, n_msgs = int(head[0]), int(head[1])
        buf = torch.zeros(n_bytes, dtype=torch.uint8, device="cuda")
        dist.recv(buf, partner)
        got = S.unframe(buf.cpu().numpy().tobytes())
        assert len(got) == n_msgs
        seen = {}
        for m in got:
            h, blocks, _ = S.unpack(m)                       # refuses a damaged or truncated message
            q = int(h.seed)
            if (h.n_layers, h.n_kv_heads, h.head_dim, h.block_size, h.kv_dtype) != (w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, far_dtype) \
                    or h.seq_len != int(w.seq_lens[q]):
                raise SystemExit(f"session message for prompt {q} does not match this pool's geometry")
            far[q, h.block_begin:h.block_begin + h.n_blocks] = blocks
            seen[q] = seen.get(q, 0) + 1
            assert seen[q] <= h.piece_count
        bs = w.block_size
        for q, n in enumerate(w.seq_lens):
            nb = (int(n) + bs - 1) // bs
            if not np.array_equal(far[q, :nb], seeded[q, :nb]):
                raise SystemExit(f"block table of prompt {q} differs from what its owner holds")
    return {"messages": n_msgs, "bytes": n_bytes, "pieces_per_prompt": 2, "order": "reversed",
            "direction": "prefill rank -> decode rank" if is_prefill != mover else "decode rank -> prefill rank",
            "what": "tkv_session_pack messages (header + the sender's block table, checksummed) over torch.distributed; the "
                    "rank whose GPU runs the kernel builds the far side's block table from them alone"}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from tempura_b200 import handoff as H

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N > 1 with torch.distributed.run, one rank per GPU")
        args.gpus = world
    if world > 1 and world % 2:
        raise SystemExit("N > 1 must be even: ranks [0, N/2) prefill, [N/2, N) decode")
    from tempura_b200 import disagg
    gpu_of = lambda r: disagg.gpu_of_rank(r, world, args.gpu_order)     # N > 2: prefill rank i on GPU 2i, its decode rank on GPU 2i + 1
    local = gpu_of(local)
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    wname = default_workload(args)
    w = pick_workload(wname, world, args.pool_blocks, heads=args.heads_per_pair, layers=args.layers, single_tokens=args.single_tokens)
    if args.src_f32:                # the reference's own transfer dtype: F32 rows into the F16 cache (one GPU only)
        if world != 1 or w.dst_dtype != "f16":
            raise SystemExit("--src-f32 is a one-GPU probe of the F32 -> F16 cast")
        w.src_dtype = "f32"
        w.name += "-f32src"
    role = disagg.role_of(rank, world, 80, 8)        # rank i (prefill) <-> rank i + N/2 (decode); heads split by tkv_pairing_make
    pairs = max(1, world // 2)
    strong = wname == "cfg5"                         # one batch, its KV heads split over the pairs
    if strong and multi and not args.single_tokens and not args.heads_per_pair:
        assert w.n_kv_heads == role.n_heads, "the pools hold exactly the pair's share of the KV heads"
    is_prefill, partner = role.is_prefill, role.partner
    dst_dtype = w.dst_dtype
    scales = dst_dtype == "e4m3"
    flags = 0
    if args.variant == "vector":
        flags |= H.N.PLAN_FORCE_VECTOR
    elif args.variant == "bulk":
        flags |= H.N.PLAN_FORCE_BULK
    if args.peer_bulk:
        flags |= H.N.PLAN_PEER_BULK_STORES

    # rank 0 samples its own GPU and its partner's (the pulled handoff's kernel runs there); one nvidia-smi for the whole job
    sampler = ClockSampler(local, also=[gpu_of(partner)] if multi else []) if rank == 0 else NullSampler()
    src = dst = None
    remote_base = 0
    # Across GPUs a same-dtype batch is PULLED: the kernel runs on the decode GPU, fetches the prefill pool's blocks with
    # ordinary loads over NVLink and stores into its own pool (measured 786 GB/s per pair against 718 GB/s for stores pushed
    # from the prefill GPU, whatever their shape).  A cast to E4M3 is PUSHED: the prefill GPU encodes first, so half the
    # bytes cross the link.  --push forces the store form for the same-dtype case as well.
    pull = multi and w.src_dtype == dst_dtype and not args.push
    mover = (not is_prefill) if pull else is_prefill          # the rank whose GPU runs the handoff kernel
    # completion flag: page-locked host memory on one GPU (the kernel's release store lands where the
    # host polls it, no copy per poll); device memory of the decode GPU when two ranks are involved
    flag = torch.zeros(4, dtype=torch.int32, device="cuda") if multi else torch.zeros(4, dtype=torch.int32).pin_memory()
    remote_flag = 0
    if not multi:
        src = H.Pool.allocate(local, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.src_blocks, w.src_dtype)
        dst = H.Pool.allocate(local, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.dst_blocks, dst_dtype,
                              scales=scales, refcounts=w.prefix_lens is not None, fill_byte=0x5A)
        fill_source(src, w, 1234)
    else:
        # Every rank announces its pool (IPC handles, layer addresses); its partner maps it.
        if is_prefill:
            mine = src = H.Pool.allocate(local, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.src_blocks, "f16")
            fill_source(src, w, 1234 + rank)
        else:
            mine = dst = H.Pool.allocate(local, w.n_layers, w.n_kv_heads, w.head_dim, w.block_size, w.dst_blocks, dst_dtype,
                                         scales=scales, refcounts=w.prefix_lens is not None, fill_byte=0x5A)
        hs, off = H.ipc_export(mine.storage.data_ptr())
        hf, foff = H.ipc_export(flag.data_ptr())
        info = {"pool": (hs, off), "flag": (hf, foff), "base": mine.storage.data_ptr(), "bytes": mine.storage.numel(),
                "k": [int(p) for p in mine.k_ptrs], "v": [int(p) for p in mine.v_ptrs], "device": local}
        if mine.k_scales is not None:
            info["ks"] = H.ipc_export(mine.k_scales.data_ptr())
            info["vs"] = H.ipc_export(mine.v_scales.data_ptr())
        if mine.refcounts is not None:
            info["rc"] = H.ipc_export(mine.refcounts.data_ptr())
        infos = [None] * world
        dist.all_gather_object(infos, info)
        pi = infos[partner]
        base = H.ipc_import(*pi["pool"])
        rel = lambda p: base + (p - pi["base"])
        theirs = H.Pool.from_pointers(pi["device"], dst_dtype if is_prefill else "f16", w.n_kv_heads, w.head_dim, w.block_size,
                                      w.dst_blocks if is_prefill else w.src_blocks, [rel(p) for p in pi["k"]], [rel(p) for p in pi["v"]],
                                      H.ipc_import(*pi["ks"]) if "ks" in pi else 0, H.ipc_import(*pi["vs"]) if "vs" in pi else 0,
                                      H.ipc_import(*pi["rc"]) if "rc" in pi else 0)
        if is_prefill:
            dst, remote_base, remote_bytes = theirs, base, pi["bytes"]
            remote_flag = H.ipc_import(*pi["flag"])
        else:
            src_remote = theirs

    wire_msgs = None
    if multi:
        wire_msgs = exchange_tables(w, is_prefill, mover, partner, dst_dtype)
    batch = H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride, w.prefix_lens)
    plan = None
    if mover:
        plan = H.Plan(src_remote, dst, batch, None, flags | H.N.PLAN_PULL) if pull else H.Plan(src, dst, batch, None, flags)
        if args.bulk_tune:
            plan.tune_bulk(*[int(x) for x in args.bulk_tune.split(",")])
        if args.grid_tune:
            plan.tune_grid(args.grid_tune)
        if args.vec_tune:
            plan.tune_vector(*[int(x) for x in args.vec_tune.split(",")])
        if args.small_tune:
            plan.tune_small(*[int(x) for x in args.small_tune.split(",")])
    stream = torch.cuda.current_stream()
    # where the kernel publishes completion: the host-visible flag on one GPU; the decode GPU's flag across GPUs (its own
    # memory when it pulls, the mapped peer word when the prefill GPU pushes)
    done_flag = flag.data_ptr() if (not multi or pull) else (remote_flag if is_prefill else 0)
    waits_on_flag = multi and not pull and not is_prefill     # a pushed handoff is awaited by the decode rank
    if args.no_flag:
        done_flag = 0                                         # probe: the launch alone, nothing published

    def barrier():
        if multi:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- N > 1: the link's own yardstick, measured in this run: a copy-engine copy of 1 GiB from the prefill
    # pool into the paired decode pool, every pair at once, CUDA events, best of 5 (slowest pair reported) ----
    peer_copy = None
    if multi:
        nbytes = int(min(1 << 30, src.storage.numel() if is_prefill else 1 << 62, remote_bytes if is_prefill else 1 << 62))
        best = float("inf")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(6):
            barrier()
            if is_prefill:
                e0.record(stream)
                H.memcpy_enqueue(remote_base, src.storage.data_ptr(), nbytes, stream)
                e1.record(stream)
                torch.cuda.synchronize()
                if it:
                    best = min(best, e0.elapsed_time(e1))
        barrier()
        t = torch.tensor([(nbytes / (best * 1e-3) / 1e9) if is_prefill else 1e30], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        peer_copy = float(t.item())
        if not is_prefill:                           # the copy wrote over the head of the pool: restore the fill pattern
            dst.storage[: 1 << 30].fill_(0x5A)
        barrier()

    sampler.start()
    # ---- warm-up -------------------------------------------------------------------------
    gen = 0
    for _ in range(args.warmup):
        gen += 1
        if mover:
            plan.enqueue(stream, done_flag, gen)
        elif waits_on_flag:
            H.flag_wait_host(local, flag.data_ptr(), gen, 60_000_000)
    barrier()
    sampler.mark()

    # ---- timed: K handoffs, inputs resident in HBM -------------------------------------------
    small = is_small(w)
    t_wall0 = time.perf_counter()
    if mover:
        ms, gen = time_handoffs(H, plan, w, args.steps, stream, done_flag, gen)
    else:
        gen += args.steps
        if waits_on_flag:
            H.flag_wait_host(local, flag.data_ptr(), gen, 600_000_000)
        ms = 0.0                                      # the moving rank's CUDA events time the pair
    barrier()
    sampler.mark()
    ms_total = max_over_ranks(ms)

    stats_src = [plan.stats() if mover else None]
    if multi:                                       # rank 0 prints; the plan may live on its partner
        gathered = [None] * world
        dist.all_gather_object(gathered, None if stats_src[0] is None else
                               {f: getattr(stats_src[0], f) for f, _ in H.N.TkvStats._fields_})
        first = next(g for g in gathered if g is not None)
        stats_src = [type("Stats", (), first)]
    if args.sweep:
        if rank == 0:
            st = stats_src[0]
            per = ms_total / args.steps
            bytes_moved = st.bytes_written if multi else st.bytes_read + st.bytes_written
            print(json.dumps({"sweep": True, "workload": w.name, "n_gpus": world, "ms_per_step": round(per, 5),
                              "value": round(st.payload_bytes * pairs / (per * 1e-3) / 1e9, 2),
                              "achieved": round(bytes_moved / (per * 1e-3) / 1e9, 1), "peer_copy_GBps": peer_copy,
                              "kernel": KERNEL_NAMES.get(st.kernel_variant, "?"), "grid": [st.grid, st.block], "clocks": sampler.stop()}), flush=True)
        else:
            sampler.stop()
        if multi:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- end to end, device-resident pools: host tables -> plan update (H2D work list) -> kernel -> D2H flag
    e2e_steps = max(1, min(args.steps, 50))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        gen += 1
        if mover:
            plan.update(batch)
            plan.enqueue(stream, done_flag, gen)
            if not multi or pull:
                H.flag_wait_host(local, flag.data_ptr(), gen, 60_000_000)
        elif waits_on_flag:
            H.flag_wait_host(local, flag.data_ptr(), gen, 600_000_000)
    torch.cuda.synchronize()
    res_s = time.perf_counter() - t0
    barrier()
    res_s = max_over_ranks(res_s)

    # ---- parity, not timed: every moved row of every layer, at every N ------------------------
    parity = parity_step(H, w, batch, src, dst, is_prefill, partner, multi, local, scales)
    barrier()

    # ---- end to end, HOST buffers: the prompts' K/V sit in page-locked host memory in the contiguous
    # transfer layout (the reference's KvCacheTransfer); every step uploads the tables, runs the
    # from_transfer kernel, which pulls the payload over PCIe and stores it into the decode pool
    # (casting on the way for an E4M3 pool), and reads the completion flag back.
    host_steps = max(1, min(args.steps, args.host_steps))
    xfer = plan_h = None
    # bounded by host memory: at most ~8 GB of page-locked buffer; larger batches move their first layers only
    per_layer = w.payload_bytes // w.n_layers
    host_layers = int(max(1, min(w.n_layers, 8_000_000_000 // max(per_layer, 1))))
    if is_prefill:
        n_blocks = H.batch_blocks(batch, w.block_size)
        xfer = H.Transfer.allocate(host_layers, w.n_kv_heads, w.head_dim, w.block_size, n_blocks, "f16", device=local, host=True)
        hv = xfer.data.view(torch.int16)
        tile = torch.randint(-15000, 15000, (1 << 24,), dtype=torch.int16)          # finite F16 bit patterns
        for o in range(0, hv.numel(), tile.numel()):
            n = min(tile.numel(), hv.numel() - o)
            hv[o:o + n].copy_(tile[:n])
        plan_h = H.Plan.from_transfer(xfer, dst, batch, H.Shard(0, 0, w.n_kv_heads, 0, 0, host_layers),
                                      H.N.PLAN_FORCE_BULK if args.host_bulk else (0 if args.host_direct else H.N.PLAN_STAGE_HOST))
        if args.host_bulk and args.bulk_tune:
            plan_h.tune_bulk(*[int(x) for x in args.bulk_tune.split(",")])
        if args.host_vec_tune:
            plan_h.tune_vector(*[int(x) for x in args.host_vec_tune.split(",")])
    # this leg's kernel runs on the prefill GPU (its host holds the buffer) and publishes to the decode rank's flag
    host_done = flag.data_ptr() if not multi else (remote_flag if is_prefill else 0)
    barrier()
    for it in range(1 + host_steps):             # first pass is the warm-up
        if it == 1:
            barrier()
            t0 = time.perf_counter()
        gen += 1
        if is_prefill:
            plan_h.update(batch)
            plan_h.enqueue(stream, host_done, gen)
            if not multi:
                H.flag_wait_host(local, flag.data_ptr(), gen, 120_000_000)
        else:
            H.flag_wait_host(local, flag.data_ptr(), gen, 120_000_000)
    torch.cuda.synchronize()
    host_s = time.perf_counter() - t0
    barrier()
    host_s = max_over_ranks(host_s)
    host_h2d = (plan_h.stats().payload_bytes + plan_h.stats().worklist_bytes) if is_prefill else 0
    per_rank_h2d = torch.tensor([host_h2d * host_steps / host_s / 1e9 if is_prefill else 0.0], dtype=torch.float64, device="cuda")
    h2d_rates = [per_rank_h2d.clone() for _ in range(world)] if multi else [per_rank_h2d]
    if multi:
        dist.all_gather(h2d_rates, per_rank_h2d)
    del plan_h, xfer

    # ---- comparison baseline (N > 1): pack kernel -> NCCL send/recv -> scatter kernel ------------------
    nccl = None
    if multi and not args.no_nccl:
        nccl = nccl_baseline(H, w, batch, src, dst, is_prefill, partner, local, scales, max(3, min(args.steps, 10)), barrier)
    clocks = sampler.stop()

    if rank == 0:
        st = stats_src[0]
        payload_all = st.payload_bytes * pairs       # strong: the pairs' shares add up to the one batch; weak: every pair its own batch
        per_launch_ms = ms_total / args.steps
        value = payload_all / (per_launch_ms * 1e-3) / 1e9
        peak, peak_kind = measured_peaks()
        algo = st.bytes_read + st.bytes_written                     # one launch, one GPU
        kname = KERNEL_NAMES.get(st.kernel_variant, "?")
        ratio = NCU_TRAFFIC_RATIO.get(kname)
        if multi:
            wire = st.bytes_written                                  # what one prefill GPU stores into its decode GPU per launch
            achieved = wire / (per_launch_ms * 1e-3) / 1e9
            roofline = {"bound": "nvlink", "achieved": round(achieved, 1), "peak": round(peer_copy, 1), "unit": "GB/s",
                        "frac": round(achieved / peer_copy, 4), "traffic": int(wire), "algorithmic_bytes": int(wire),
                        "peak_source": "copy-engine copy of 1 GiB prefill pool -> paired decode pool measured in this run, every pair at once, best of 5, slowest pair",
                        "traffic_source": "wire bytes: what crosses from one prefill GPU to its decode GPU per launch (no ncu capture wraps a multi-rank run)",
                        "frac_of_nominal_900": round(achieved / 900.0, 4), "per": "pair, one direction"}
        else:
            achieved = algo / (per_launch_ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                        "frac": round(achieved / peak, 4), "traffic": (int(ratio * algo) if ratio else None),
                        "algorithmic_bytes": int(algo), "peak_source": f"{peak_kind} copy peak (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
                        "frac_of_nominal_8000": round(achieved / 8000.0, 4)}
        cfg = describe(w, world, small, args.push, args.gpu_order)
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(per_launch_ms, 5), "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": ("f32->f16" if w.src_dtype == "f32" else "u16") if dst_dtype == "f16" else "f16->e4m3",
            "data": "synthetic", "config": cfg,
            "launch": {"kernel": kname, "grid": [st.grid, st.block],
                       "runs_on": "the one GPU" if not multi else ("decode GPU (pull: loads over NVLink)" if pull else "prefill GPU (push: stores over NVLink)")},
            "parity": parity["parity"], "parity_detail": {k: v for k, v in parity.items() if k != "parity"},
            "roofline": roofline,
            "e2e": {"value": round(payload_all * host_layers / w.n_layers * host_steps / host_s / 1e9, 2), "unit": UNIT,
                    "h2d_bytes_per_step": int(host_h2d), "d2h_bytes_per_step": 4, "steps": host_steps,
                    "layers": host_layers, "h2d_GBps_per_prefill_rank": [round(float(r.item()), 2) for r in h2d_rates[:pairs]],
                    "what": "K/V of the batch in page-locked HOST memory (contiguous transfer layout) + host block tables -> "
                            "tkv_plan_update -> tkv_handoff_enqueue of a from_transfer plan (TKV_PLAN_STAGE_HOST: the copy engine brings "
                            "the buffer in one layer at a time while the previous layer's kernel stores into the decode pool) -> flag read back"},
            "e2e_resident": {"value": round(payload_all * e2e_steps / res_s / 1e9, 2), "unit": UNIT,
                             "h2d_bytes_per_step": int(st.worklist_bytes), "d2h_bytes_per_step": 4, "steps": e2e_steps,
                             "what": "same call sequence with the K/V already in the prefill GPU's paged pool (where prefill "
                                     "wrote it): host block tables -> tkv_plan_update -> tkv_handoff_enqueue -> flag read back"},
            "gpu_launches": args.steps,              # one handoff kernel per timed step
            "gpu_launches_whole_run": args.warmup + args.steps + e2e_steps + 1 + host_steps,
            "clocks": clocks,
        }
        if world > 2:
            line["e2e"]["prefill_gpus"] = [gpu_of(r) for r in range(pairs)]
        if nccl is not None:
            line["nccl_baseline"] = nccl
        if wire_msgs is not None:
            line["wire_messages"] = wire_msgs
        if not multi and not args.no_cpu:
            layers = sample_layers(w)
            v1, sample = time_cpu(w, 1, layers, 3)
            vall, _ = time_cpu(w, os.cpu_count() or 1, layers, 3)
            line["cpu_baseline"] = {"value": round(v1, 3), "unit": UNIT, "cores": 1, "kind": "port", "sample": sample,
                                    "all_cores": {"value": round(vall, 3), "cores": os.cpu_count() or 1}}
    if not multi and args.others and not (args.workload or args.single_tokens or args.layers or args.src_f32):
        # the other benchmark configurations on this GPU, device-timed and parity-checked the same way
        plan.destroy()
        del src, dst, plan
        torch.cuda.empty_cache()
        peak, _ = measured_peaks()
        line["other_configs"] = {name: quick_config(H, name, 20, peak) for name in ("cfg1", "cfg2", "cfg3", "cfg4")}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if multi:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------
# the FP8 cache's consumer: decode attention over the pool the handoff filled (not the driver's line)
# ----------------------------------------------------------------------------------------
def run_attention(args):
    """One decode step's attention for the config-3 batch: 32 layer launches back to back over the
    E4M3 + scales pool (or the F16 pool with --attn-f16) that a handoff has just filled.  Bytes
    counted: every cached K and V element of the batch once per layer, plus scales, q and out."""
    import torch
    from tempura_b200 import handoff as H
    torch.cuda.set_device(0)
    if args.attn_seqs:              # a wider batch of the same length distribution (how the kernel scales with bytes per launch)
        from tempura_b200 import workloads as W
        w = W.llama8b_fp8(pool_blocks=args.pool_blocks or 256 * args.attn_seqs + 64, n_seqs=args.attn_seqs)
        if args.layers:
            w.n_layers = args.layers
            w.name += f"-{args.layers}layers"
    else:
        w = pick_workload("cfg3", 1, args.pool_blocks or 4096, layers=args.layers)
    fp8 = not args.attn_f16
    src = H.Pool.allocate(0, w.n_layers, 8, 128, 16, w.src_blocks, "f16")
    fill_source(src, w, 77)
    if fp8:
        pool = H.Pool.allocate(0, w.n_layers, 8, 128, 16, w.dst_blocks, "e4m3", scales=True, fill_byte=0x5A)
        H.Plan(src, pool, H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride)).enqueue()
        tables_np = w.dst_tables
    else:
        pool, tables_np = src, w.src_tables
    n, n_q = len(w.seq_lens), 32
    tables = torch.from_numpy(tables_np.astype(np.int64)).to(torch.int32).cuda()
    lens = torch.from_numpy(w.seq_lens.astype(np.int64)).to(torch.int32).cuda()
    q = torch.randn((n, n_q, 128), device="cuda")
    max_len = int(w.seq_lens.max())
    sampler = ClockSampler(0)
    sampler.start()

    attn = H.DecodeAttention(pool, q, tables, lens, max_len, split_tokens=args.attn_split,
                             flags=(1 if args.attn_per_head else 0) | (2 if args.attn_mma_sync else 0),
                             total_kv_tokens=0 if args.attn_no_hint else int(w.seq_lens.astype(np.int64).sum()))
    for layer in range(w.n_layers):          # plain launches first (module load, argument structs)
        attn.enqueue(layer)
    torch.cuda.synchronize()
    # one decode step's 32 attention launches as a CUDA graph, so the host's launch cost is not what is timed
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for layer in range(w.n_layers):
            attn.enqueue(layer)
    step = graph.replay

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler.mark()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    sampler.mark()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    tokens = int(w.seq_lens.astype(np.int64).sum())
    blocks = int(((w.seq_lens.astype(np.int64) + 15) // 16).sum())
    es = 1 if fp8 else 2
    per_layer = tokens * 8 * 128 * 2 * es + (blocks * 8 * 2 * 4 if fp8 else 0) + 2 * n * n_q * 128 * 4
    algo = per_layer * w.n_layers
    peak, kind = measured_peaks()
    achieved = algo / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "paged_decode_attention_GBps", "value": round(achieved, 1), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 5), "us_per_layer": round(ms * 1e3 / w.n_layers, 2), "higher_is_better": True,
        "dtype": ("e4m3+scales -> f16 mma.sync, f32 accumulate" if fp8 else "f16 mma.sync, f32 accumulate") if (args.attn_mma_sync or args.attn_per_head)
                 else ("e4m3 x e4m3 / e4m3 x e5m2 tcgen05.mma, f32 accumulate in tensor memory" if fp8 else "f16 tcgen05.mma, f32 accumulate in tensor memory"),
        "data": "synthetic",
        "config": {"workload": w.name + "-decode-attention", "layers": w.n_layers, "kv_heads": 8, "q_heads": n_q, "head_dim": 128,
                   "n_seqs": n, "cached_tokens": tokens, "l2": "each layer's K/V is read once per step; a step reads more than L2 holds"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": None, "algorithmic_bytes": int(algo), "peak_source": f"{kind} copy peak"},
        "gpu_launches": (args.warmup + args.steps) * w.n_layers * 2, "clocks": clocks}), flush=True)



def run_prefill_attention(args):
    """--workload prefill: causal attention of one prompt's tokens over its own paged cache, one layer per launch, on the
    tcgen05 kernel (tkv_prefill_attn_enqueue): --prefill-tokens T new tokens after --prefill-start cached ones, the
    Llama-3.1-8B shape (32 query heads on 8 kv heads of 128 dims), E4M3 + scales pool filled by a handoff (or the F16
    pool with --attn-f16).  FLOPs counted: 4 * head_dim * query heads * sum over query tokens of the positions each
    attends to (both contractions, causal); the tensor-core work the kernel adds for its operand terms is not counted."""
    import torch
    from tempura_b200 import handoff as H
    from tempura_b200 import workloads as W
    torch.cuda.set_device(0)
    t, start = args.prefill_tokens, args.prefill_start
    total = start + t
    layers = args.layers or 4
    fp8 = not args.attn_f16
    blocks = (total + 15) // 16 + 8
    w = W.Workload("llama3.1-8b-prefill", layers, 8, 128, 16, blocks, blocks, np.array([total], dtype=np.uint32),
                   dst_dtype="e4m3" if fp8 else "f16", seed=9).build_tables()
    src = H.Pool.allocate(0, layers, 8, 128, 16, w.src_blocks, "f16")
    fill_source(src, w, 78)
    if fp8:
        pool = H.Pool.allocate(0, layers, 8, 128, 16, w.dst_blocks, "e4m3", scales=True, fill_byte=0x5A)
        H.Plan(src, pool, H.Batch(w.seq_lens, w.src_tables, w.dst_tables, w.table_stride)).enqueue()
        row_np = w.dst_tables[0]
    else:
        pool, row_np = src, w.src_tables[0]
    row = torch.from_numpy(row_np.astype(np.int64)).to(torch.int32).cuda()
    q = torch.randn((t, 32, 128), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    sampler = ClockSampler(0)
    sampler.start()
    pf_flags = 1 if args.prefill_single_tile else (2 if args.prefill_two_tiles else 0)
    outs = [H.prefill_attention(pool, l, q, row, start, status=status, flags=pf_flags) for l in range(layers)]     # plain launches first
    torch.cuda.synchronize()
    if int(status.item()):
        raise SystemExit(f"prefill attention reported status {int(status.item())}")
    # parity inside the run: a sample of query tokens against the decode kernel's mma.sync path (an independent kernel)
    pick = sorted({0, t // 3, t - 1})
    tabs = row.reshape(1, -1).expand(len(pick), -1).contiguous()
    lens = torch.tensor([start + i + 1 for i in pick], dtype=torch.int32, device="cuda")
    ref = H.decode_attention(pool, layers - 1, q[pick].contiguous(), tabs, lens, max_kv_len=total, flags=2)
    err = float((outs[-1][pick] - ref).abs().max())
    scale = float(ref.abs().max())
    if not err <= 4e-3 * max(scale, 1.0):
        raise SystemExit(f"prefill attention differs from the decode kernel on sampled tokens: max err {err:.3e}")
    def step():
        for l in range(layers):
            H.prefill_attention(pool, l, q, row, start, flags=pf_flags)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler.mark()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    sampler.mark()
    clocks = sampler.stop()
    ms = ev0.elapsed_time(ev1) / args.steps
    attended = t * start + t * (t + 1) // 2
    flops = 4.0 * 128 * 32 * attended * layers
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak_tf, kind = (float(json.load(open(path))["bf16_tflops"]), "measured") if os.path.exists(path) else (1590.0, "fallback")
    achieved = flops / (ms * 1e-3) / 1e12
    es = 1 if fp8 else 2
    print(json.dumps({
        "metric": "paged_prefill_attention_TFLOPs", "value": round(achieved, 1), "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 5), "us_per_layer": round(ms * 1e3 / layers, 2), "higher_is_better": True,
        "dtype": "e4m3 x e4m3 / e5m2 x e4m3 tcgen05.mma, f32 accumulate in tensor memory" if fp8 else "f16 tcgen05.mma, f32 accumulate in tensor memory",
        "data": "synthetic",
        "config": {"workload": w.name + ("-e4m3" if fp8 else "-f16"), "layers": layers, "kv_heads": 8, "q_heads": 32, "head_dim": 128,
                   "new_tokens": t, "cached_before": start, "l2": "K/V of one layer (%d MB) is re-read by every group of 32 query tokens, mostly from L2" % (total * 8 * 128 * 2 * es >> 20)},
        "parity": {"sampled_tokens": pick, "max_abs_err_vs_mma_sync_decode_kernel": err, "max_abs_value": scale},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(achieved / peak_tf, 4),
                     "traffic": None, "peak_source": f"{kind} cuBLAS bf16 burst peak (the kernel's FP8 MMAs run at twice that rate but it issues 2.5 times the counted work: two q terms, three probability terms)" if fp8 else f"{kind} cuBLAS bf16 burst peak"},
        "gpu_launches": (args.warmup + args.steps) * layers, "clocks": clocks}), flush=True)


def bench_prefix_index(args) -> None:
    """--workload prefix: the device-resident prefix index on the shared-prefix benchmark shape (64 prompts x
    8 192 tokens with a common 2 048-token prefix, one node per 16-token block).  A step is one lookup of the
    whole batch followed by its release; the value is prompt tokens resolved per second.  The CPU leg is the
    RadixTree oracle doing the same lookup + release on one host core."""
    import torch
    from tempura_b200 import handoff as H
    torch.cuda.set_device(0)
    rng = np.random.default_rng(77)
    n, length, pre, group = 64, 8192, 2048, 16
    shared = rng.integers(0, 32000, size=pre)
    tok = np.stack([np.concatenate([shared, rng.integers(0, 32000, size=length - pre)]) for _ in range(n)]).astype(np.int32)
    pages = np.arange(n * (length // group), dtype=np.int32).reshape(n, length // group)
    t, l, p = torch.from_numpy(tok).cuda(), torch.full((n,), length, dtype=torch.int32).cuda(), torch.from_numpy(pages).cuda()
    ix = H.PrefixIndex(0, 1 << 17, group)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    ix.insert(t, l, p)
    ev[1].record()
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        ix.lookup(t, l)
        ix.release(t, l)
    torch.cuda.synchronize()
    sampler.mark()
    # the output tensors are allocated once: a step is the two launches
    b = ix._batch(t, l)
    out_pages = torch.empty((n, length // group), dtype=torch.int32, device="cuda")
    matched = torch.empty(n, dtype=torch.int32, device="cuda")
    import ctypes as C
    from tempura_b200._native import lib
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ev[2].record()
    for _ in range(args.steps):
        lib().tkv_prefix_index_lookup(ix._h, C.byref(b), out_pages.data_ptr(), length // group, matched.data_ptr(), st)
        lib().tkv_prefix_index_release(ix._h, C.byref(b), st)
    ev[3].record()
    torch.cuda.synchronize()
    sampler.mark()
    clocks = sampler.stop()
    if not bool((matched == length // group).all()):
        raise SystemExit("prefix index: lookup did not match every node")
    ms = ev[2].elapsed_time(ev[3]) / args.steps
    from oracle.prefix_oracle import RadixOracle
    ref = RadixOracle(group)
    seqs = [row.tolist() for row in tok]
    ref.batch_insert(seqs, [row.tolist() for row in pages])
    t0 = time.perf_counter()
    ref.batch_lookup(seqs)
    ref.batch_release(seqs)
    cpu_s = time.perf_counter() - t0
    tokens = n * length
    print(json.dumps({
        "metric": "prefix_index_tokens_resolved_per_s", "value": round(tokens / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5), "insert_ms": round(ev[0].elapsed_time(ev[1]), 4),
        "higher_is_better": True, "dtype": "u64 hash keys, u32 pages", "data": "synthetic",
        "config": {"workload": "llama3.1-8b-prefix2048-64seq-prefix-index", "n_seqs": n, "tokens_per_seq": length, "shared_prefix": pre,
                   "group_tokens": group, "capacity": 1 << 17, "l2": "the table (5 MB) stays in L2: this call is latency-bound, not bandwidth-bound"},
        "cpu_baseline": {"value": round(tokens / cpu_s, 1), "unit": "tokens/s", "cores": 1, "kind": "port",
                         "sample": "the same 64 x 8192-token lookup + release through the RadixTree oracle, once"},
        "gpu_launches": (max(args.warmup, 3) + args.steps) * 2 + 2, "clocks": clocks}), flush=True)


def bench_admission(args) -> None:
    """--workload admit: the decode side's admission of the prefix-reuse batch (64 prompts sharing a resident
    2 048-token prefix, 128-512-token suffixes; 4 layers unless --layers says otherwise), wall clock from the
    prompts' token ids to the completed handoff, two ways: everything on the device (prefix index lookup -> page
    allocator -> handoff from device tables) and with the host in the loop (the same lookup, its answer copied
    to the host, pages popped from a host free list, a host-built plan).  Both end with the same bytes moved."""
    import torch
    from tempura_b200 import handoff as H
    from tempura_b200 import workloads as W
    torch.cuda.set_device(0)
    layers, blocks, bs = args.layers or 4, args.pool_blocks or 16384, 16
    w = W.llama8b_prefix(pool_blocks=blocks)
    n, pre = len(w.seq_lens), 2048
    rng = np.random.default_rng(91)
    system = rng.integers(0, 32000, size=pre)
    stride_tok = int(w.seq_lens.max())
    tok = np.zeros((n, stride_tok), dtype=np.int32)
    for q, m in enumerate(w.seq_lens):
        tok[q, :pre] = system
        tok[q, pre:int(m)] = rng.integers(0, 32000, size=int(m) - pre)
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.int64)).to(torch.int32).cuda()
    src = H.Pool.allocate(0, layers, 8, 128, bs, blocks, "f16")
    dst = H.Pool.allocate(0, layers, 8, 128, bs, blocks, "f16", refcounts=True, fill_byte=0x5A)
    src.storage.view(torch.int16).random_(0, 15000)
    tokens, lens = i32(tok), i32(w.seq_lens)
    src_tables = i32(w.src_tables.reshape(n, -1))
    stride = src_tables.shape[1]
    # the decode side: pages 0..127 hold the shared prefix and are indexed; the allocator owns the rest
    index, alloc = H.PrefixIndex(0, 1 << 16, bs), H.DevicePageAllocator(0, blocks)
    pre_tab = torch.zeros((1, pre // bs), dtype=torch.int32, device="cuda")
    alloc.allocate(pre_tab, i32([pre // bs]))
    index.insert(i32(system[None, :]), i32([pre]), pre_tab)
    host_free = list(range(blocks - 1, pre // bs - 1, -1))                     # the same stack, on the host
    pairs_cap = int(((w.seq_lens.astype(np.int64) + bs - 1) // bs).sum())
    plan_dev = H.Plan.with_capacity(src, dst, pairs_cap)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    dst_tables = torch.zeros((n, stride), dtype=torch.int32, device="cuda")
    matched_dev = torch.zeros(n, dtype=torch.int32, device="cuda")

    def device_path():
        index.lookup(tokens, lens, out_pages=dst_tables, out_matched=matched_dev)
        alloc.allocate(dst_tables, first=matched_dev, seq_lens=lens, block_size=bs)
        plan_dev.enqueue_device_tables(lens, src_tables, dst_tables, prefix_blocks=matched_dev, apply_refcounts=True, status=status)
        torch.cuda.synchronize()
        # undo, outside what a server would do per admission: give the pages and the references back
        alloc.free(dst_tables, first=matched_dev, seq_lens=lens, block_size=bs)
        index.release(tokens, lens)
        dst.refcounts.zero_()
        torch.cuda.synchronize()

    def host_path():
        matched, pages = index.lookup(tokens, lens)
        m, pg = matched.cpu().numpy(), pages.cpu().numpy()                     # the round trip
        tab = np.zeros((n, stride), dtype=np.uint32)
        taken = []
        for q in range(n):
            nb = (int(w.seq_lens[q]) + bs - 1) // bs
            tab[q, :m[q]] = pg[q, :m[q]]
            for i in range(m[q], nb):
                tab[q, i] = host_free.pop()
                taken.append(tab[q, i])
        plan = H.Plan(src, dst, H.Batch(w.seq_lens, w.src_tables, tab, stride, (m * bs).astype(np.uint32)))
        plan.enqueue()
        plan.refcount_apply(+1)
        torch.cuda.synchronize()
        plan.destroy()
        host_free.extend(reversed(taken))
        index.release(tokens, lens)
        dst.refcounts.zero_()
        torch.cuda.synchronize()
        return tab

    def timed(fn, steps):
        # only the admission itself is on the clock: from the call to the synchronize inside fn that follows the handoff
        best = []
        for _ in range(steps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            best.append(time.perf_counter() - t0)
        return statistics.median(best)

    for _ in range(max(args.warmup, 3)):
        device_path()
        host_path()
    if int(status.item()) != 0:
        raise SystemExit(f"admission: device work list refused the batch (status {int(status.item())})")
    tab = host_path()
    device_path()
    steps = min(args.steps, 50)
    t_dev, t_host = timed(device_path, steps), timed(host_path, steps)
    suffix_tokens = int((w.seq_lens.astype(np.int64) - pre).sum())
    payload = suffix_tokens * 8 * 128 * 2 * 2 * layers
    print(json.dumps({
        "metric": "admission_ms", "value": round(t_dev * 1e3, 4), "unit": "ms", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(t_dev * 1e3, 4), "higher_is_better": False, "dtype": "u16", "data": "synthetic",
        "host_in_the_loop_ms": round(t_host * 1e3, 4),
        "config": {"workload": w.name + f"-admission-{layers}layers", "n_seqs": n, "shared_prefix": pre, "suffix_tokens": suffix_tokens,
                   "payload_bytes": payload, "note": "wall clock per admission including giving pages and references back (both legs do it)"},
        "gpu_launches": None}), flush=True)

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "attn", "prefill", "prefix", "admit"])
    ap.add_argument("--prefill-tokens", type=int, default=4096, help="--workload prefill: new tokens of the prompt")
    ap.add_argument("--prefill-single-tile", action="store_true", help="--workload prefill: one query tile per CTA (TKV_PREFILL_SINGLE_TILE)")
    ap.add_argument("--prefill-two-tiles", action="store_true", help="--workload prefill: two query tiles per CTA (TKV_PREFILL_TWO_TILES)")
    ap.add_argument("--prefill-start", type=int, default=0, help="--workload prefill: tokens already cached before them")
    ap.add_argument("--attn-split", type=int, default=0, help="--workload attn: cached tokens per CTA (0 = library default)")
    ap.add_argument("--attn-no-hint", action="store_true", help="--workload attn: do not tell the library the batch's total cached tokens")
    ap.add_argument("--attn-seqs", type=int, default=None, help="--workload attn: this many prompts instead of the configuration's 16")
    ap.add_argument("--attn-per-head", action="store_true", help="--workload attn: the per-(sequence, kv head) CTA form")
    ap.add_argument("--attn-mma-sync", action="store_true", help="--workload attn: the warp-level mma.sync kernel instead of the tcgen05 one")
    ap.add_argument("--attn-f16", action="store_true", help="--workload attn: read the F16 pool instead of the E4M3 one")
    ap.add_argument("--pool-blocks", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="profiling aid: keep the batch, use fewer layers")
    ap.add_argument("--src-f32", action="store_true", help="probe: F32 source pool cast into the F16 pool (give --pool-blocks 8192)")
    ap.add_argument("--single-tokens", type=int, default=None, help="latency probe: one prompt of this many tokens (cfg2/cfg3 shape)")
    ap.add_argument("--variant", default="auto", choices=["auto", "vector", "bulk"])
    ap.add_argument("--bulk-tune", default=None, help="stages,ctas_per_sm,stage_bytes for the bulk-copy variant")
    ap.add_argument("--grid-tune", type=int, default=None, help="CTAs per SM cap for the register kernels")
    ap.add_argument("--vec-tune", default=None, help="bytes_per_access,unroll,store_hint for the register copy kernel (e.g. 32,8,0)")
    ap.add_argument("--flush-then-read", action="store_true", help="probe for small batches: after the L2 flush (a 256 MB write) read 256 MB, so L2 holds clean lines when the timed launch starts")
    ap.add_argument("--heads-per-pair", type=int, default=None, help="probe (cfg5): pools of this many kv heads, e.g. 2 at N = 2 reproduces one pair's share of the N = 8 run")
    ap.add_argument("--no-flag", action="store_true", help="probe (--sweep, one GPU): enqueue without a completion flag")
    ap.add_argument("--small-tune", default=None, help="flag_mode,inline_list of tkv_plan_tune_small (e.g. 1,1 = flag from the kernel, list from device memory)")
    ap.add_argument("--gpu-order", choices=["paired", "interleaved"], default="interleaved",
                    help="N > 2: which GPU a rank takes. interleaved (default) = prefill rank i on GPU 2i, its decode rank on GPU 2i+1; "
                         "paired = rank r on GPU r (prefill GPUs 0 .. N/2-1). NVLink rates are the same either way; host buffers reach "
                         "GPUs 0-3 of this pool's boxes at 115 GB/s together, so four prefill GPUs side by side halve the host-buffer leg")
    ap.add_argument("--push", action="store_true", help="N > 1: the prefill GPU's kernel stores into the decode pool (default for a same-dtype batch: the decode GPU pulls)")
    ap.add_argument("--peer-bulk", action="store_true", help="N > 1: bulk stores (shared -> peer global) instead of register stores")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sweep", action="store_true", help="tuning aid: the device-timed region only (no end-to-end legs, no parity step, no baselines)")
    ap.add_argument("--no-others", dest="others", action="store_false",
                    help="N = 1 default run: skip the other four configurations (extra keys of the line)")
    ap.add_argument("--no-nccl", action="store_true", help="N > 1: skip the pack -> NCCL send/recv -> scatter comparison")
    ap.add_argument("--host-bulk", action="store_true", help="host-buffer leg: bulk-copy ring reading the pinned buffer (experiment)")
    ap.add_argument("--host-direct", action="store_true", help="host-buffer leg: the kernel reads the pinned buffer itself instead of the copy engine staging it layer by layer")
    ap.add_argument("--host-vec-tune", default=None, help="host-buffer leg: bytes_per_access,unroll,store_hint of the register kernel that reads the pinned buffer (probe)")
    ap.add_argument("--host-steps", type=int, default=5, help="steps of the host-buffer end-to-end leg (PCIe-bound)")
    args = ap.parse_args()
    global FLUSH_THEN_READ
    FLUSH_THEN_READ = args.flush_then_read
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "prefix":
        return bench_prefix_index(args)
    if args.workload == "admit":
        return bench_admission(args)
    if args.workload == "prefill":
        return run_prefill_attention(args)
    if args.workload == "attn":
        run_attention(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
