"""Prefill / decode pairing of the ranks of one box (one process per GPU).

The reference pairs one prefill worker with one decode worker inside a process
(DisaggregatedPipeline::new, engine/src/disaggregated.rs:130-151).  Across GPUs the same
pairing is rank i (prefill) -> rank i + P (decode), P = world / 2, with the KV heads
split evenly over the P pairs (layers when there are fewer heads than pairs); the split
itself is computed by the C ABI (``tkv_pairing_make``) so that every language binding
agrees on it.  Each pool holds only its pair's share, so plans between paired pools use
pool-local numbering.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

from . import _native as N
from ._native import check, lib

import ctypes as C


@dataclass(frozen=True)
class Role:
    rank: int
    world: int
    pair: int             # index of the prefill/decode pair this rank belongs to
    is_prefill: bool
    partner: int          # rank of the other side of the pair
    head_begin: int       # this pair's share in GLOBAL (unsharded) numbering
    n_heads: int
    layer_begin: int
    n_layers: int


def pairings(world: int, n_layers: int, n_kv_heads: int) -> List[N.TkvPairing]:
    out = (N.TkvPairing * 8)()
    n = C.c_int32(0)
    check(lib().tkv_pairing_make(world, n_layers, n_kv_heads, out, 8, C.byref(n)))
    return [out[i] for i in range(n.value)]


def role_of(rank: int, world: int, n_layers: int, n_kv_heads: int) -> Role:
    """Which side of which pair ``rank`` plays, and the pair's share of heads and layers."""
    prs = pairings(world, n_layers, n_kv_heads)
    if world == 1:
        sh = prs[0].shard
        return Role(0, 1, 0, True, 0, sh.src_head_begin, sh.n_heads, sh.src_layer_begin, sh.n_layers)
    for i, pr in enumerate(prs):
        if rank in (pr.prefill_device, pr.decode_device):
            is_prefill = rank == pr.prefill_device
            sh = pr.shard
            return Role(rank, world, i, is_prefill, pr.decode_device if is_prefill else pr.prefill_device,
                        sh.src_head_begin, sh.n_heads, sh.src_layer_begin, sh.n_layers)
    raise ValueError(f"rank {rank} is in no pair of a {world}-rank box")


def gpu_of_rank(rank: int, world: int, order: str = "interleaved") -> int:
    """The CUDA ordinal a rank of a one-node job takes.  ``tkv_pairing_make`` numbers slots (prefill i, decode i + world/2);
    NVLink treats every placement of the slots alike, host memory does not: neighbouring GPUs share the host's links, so
    ``interleaved`` puts prefill slot i on GPU 2i and its decode slot on GPU 2i + 1 (four prefill GPUs then read host
    buffers at 216 GB/s instead of 115, measured on an 8-GPU B200 box).  ``paired`` keeps rank r on GPU r; two ranks are
    the same either way."""
    if order not in ("interleaved", "paired"):
        raise ValueError(f"unknown GPU order {order!r}")
    if not 0 <= rank < max(world, 1):
        raise ValueError(f"rank {rank} outside a {world}-rank job")
    if order == "paired" or world <= 2:
        return rank
    half = world // 2
    return 2 * rank if rank < half else 2 * (rank - half) + 1


def local_shard(role: Role) -> N.TkvShard:
    """The shard in pool-local numbering, for pools that hold exactly the pair's share."""
    return N.TkvShard(0, 0, role.n_heads, 0, 0, role.n_layers)
