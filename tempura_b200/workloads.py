"""The five handoff workloads of the benchmark definition, as shapes and seeded
block tables.  Values are synthetic; nothing here touches a dataset.

Lengths and permutations come from a counter-based 64-bit mixer so any subset can be
regenerated independently; the same arithmetic is restated in C by the CPU oracle and
the two are compared in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

_M = (1 << 64) - 1


def mix64(seed: int, stream: int, index) -> np.ndarray:
    """SplitMix64 finaliser over (seed, stream, index); vectorised over ``index``."""
    with np.errstate(over="ignore"):
        idx = np.asarray(index, dtype=np.uint64)
        z = (np.uint64((seed * 0x9E3779B97F4A7C15) & _M) + np.uint64((stream * 0xD1B54A32D192ED03) & _M) + idx)
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def permutation(n: int, seed: int, stream: int = 0) -> np.ndarray:
    """Fisher-Yates from the top index down, draws taken from ``mix64``."""
    out = np.arange(n, dtype=np.uint32)
    if n < 2:
        return out
    idx = np.arange(n, dtype=np.uint64)
    draws = (mix64(seed, stream, idx) % (idx + np.uint64(1))).astype(np.int64)
    o = out.tolist()
    d = draws.tolist()
    for i in range(n - 1, 0, -1):
        j = d[i]
        o[i], o[j] = o[j], o[i]
    return np.asarray(o, dtype=np.uint32)


def lengths(n: int, lo: int, hi: int, seed: int, stream: int = 0) -> np.ndarray:
    idx = np.arange(n, dtype=np.uint64)
    return (np.uint64(lo) + mix64(seed, stream, idx) % np.uint64(hi - lo + 1)).astype(np.uint32)


@dataclass
class Workload:
    name: str
    n_layers: int
    n_kv_heads: int
    head_dim: int
    block_size: int
    src_blocks: int                 # blocks in the prefill-side pool
    dst_blocks: int
    seq_lens: np.ndarray
    src_dtype: str = "f16"
    dst_dtype: str = "f16"
    prefix_lens: Optional[np.ndarray] = None
    outlier_channels: tuple = ()
    outlier_gain: float = 1.0
    sigma: float = 0.5
    seed: int = 0
    src_tables: np.ndarray = field(default=None)
    dst_tables: np.ndarray = field(default=None)
    table_stride: int = 0
    shared_prefix_blocks: Optional[np.ndarray] = None   # config 4: dst ids of the resident prefix

    @property
    def tokens_moved(self) -> int:
        pre = self.prefix_lens if self.prefix_lens is not None else 0
        return int((self.seq_lens.astype(np.int64) - pre).sum())

    @property
    def bytes_per_token(self) -> int:
        return 2 * self.n_layers * self.n_kv_heads * self.head_dim * {"f32": 4, "f16": 2, "e4m3": 1}[self.src_dtype]

    @property
    def payload_bytes(self) -> int:
        return self.tokens_moved * self.bytes_per_token

    def build_tables(self) -> "Workload":
        bs = self.block_size
        nb = (self.seq_lens.astype(np.int64) + bs - 1) // bs
        self.table_stride = int(nb.max()) if len(nb) else 1
        n = len(self.seq_lens)
        src_free = permutation(self.src_blocks, self.seed, 101)
        dst_free = permutation(self.dst_blocks, self.seed + 1, 202)
        self.src_tables = np.full((n, self.table_stride), 0xFFFFFFFF, dtype=np.uint32)
        self.dst_tables = np.full((n, self.table_stride), 0xFFFFFFFF, dtype=np.uint32)
        s = d = 0
        shared = None
        if self.prefix_lens is not None and len(self.prefix_lens) and int(self.prefix_lens.max()) > 0:
            # one common prefix: its destination blocks are drawn once and shared
            npre = int(self.prefix_lens.max()) // bs
            shared = dst_free[d:d + npre].copy()
            d += npre
            self.shared_prefix_blocks = shared
        for q in range(n):
            k = int(nb[q])
            if s + k > self.src_blocks or d + k > self.dst_blocks:
                raise ValueError("pool too small for the batch")
            self.src_tables[q, :k] = src_free[s:s + k]
            s += k
            pre_b = int(self.prefix_lens[q]) // bs if self.prefix_lens is not None else 0
            if pre_b:
                self.dst_tables[q, :pre_b] = shared[:pre_b]
            self.dst_tables[q, pre_b:k] = dst_free[d:d + k - pre_b]
            d += k - pre_b
        return self


def tinyllama_cpu(seed: int = 0) -> Workload:
    """TinyLlama-1.1B shape, one 512-token prompt, 1024-block pools, same device."""
    return Workload("tinyllama-1.1b-f16-1seq512", 22, 4, 64, 16, 1024, 1024,
                    np.array([512], dtype=np.uint32), seed=seed).build_tables()


def llama8b_f16(pool_blocks: int = 65536, n_seqs: int = 16, lo: int = 512, hi: int = 4096, seed: int = 0) -> Workload:
    """Llama-3.1-8B shape, 16 prompts of uniform length in [512, 4096]."""
    return Workload(f"llama3.1-8b-f16-{n_seqs}seq", 32, 8, 128, 16, pool_blocks, pool_blocks,
                    lengths(n_seqs, lo, hi, seed, 7), seed=seed).build_tables()


def llama8b_fp8(pool_blocks: int = 65536, n_seqs: int = 16, lo: int = 512, hi: int = 4096, seed: int = 0) -> Workload:
    """Same batch, E4M3 destination with per-(layer, kv-head, block) FP32 scales; a
    seeded 1 % of the head_dim channels (at least one) carries x20 outliers."""
    n_out = max(1, round(0.01 * 128))
    chans = tuple(int(c) for c in (mix64(seed, 9, np.arange(n_out, dtype=np.uint64)) % np.uint64(128)))
    w = Workload(f"llama3.1-8b-f16-to-e4m3-{n_seqs}seq", 32, 8, 128, 16, pool_blocks, pool_blocks,
                 lengths(n_seqs, lo, hi, seed, 7), dst_dtype="e4m3", outlier_channels=chans,
                 outlier_gain=20.0, seed=seed)
    return w.build_tables()


def llama8b_prefix(pool_blocks: int = 65536, n_seqs: int = 64, prefix: int = 2048, lo: int = 128, hi: int = 512,
                   seed: int = 0) -> Workload:
    """64 prompts share a resident 2048-token prefix; only the 128-512 token suffixes move."""
    suf = lengths(n_seqs, lo, hi, seed, 11)
    w = Workload(f"llama3.1-8b-f16-prefix{prefix}-{n_seqs}seq", 32, 8, 128, 16, pool_blocks, pool_blocks,
                 (suf + np.uint32(prefix)).astype(np.uint32),
                 prefix_lens=np.full(n_seqs, prefix, dtype=np.uint32), seed=seed)
    return w.build_tables()


def llama70b_f16(n_seqs: int = 32, seq_len: int = 4096, n_kv_heads: int = 8, n_layers: int = 80, seed: int = 0) -> Workload:
    """Llama-3.1-70B shape, 32 prompts of 4096 tokens; the pool is exactly the blocks
    needed, fully shuffled.  ``n_kv_heads`` is the per-pair share when sharded."""
    blocks = n_seqs * ((seq_len + 15) // 16)
    return Workload(f"llama3.1-70b-f16-{n_seqs}x{seq_len}-h{n_kv_heads}", n_layers, n_kv_heads, 128, 16, blocks, blocks,
                    np.full(n_seqs, seq_len, dtype=np.uint32), seed=seed).build_tables()
