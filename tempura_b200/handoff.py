"""Python face of the KV handoff C ABI.

Thin by design: torch supplies device memory and streams, everything that moves KV
bytes goes through ``libtkv.so``.  Names follow the reference's domain: pools of
paged blocks, block tables, shards, prefill and decode sides
(engine/src/kv_cache.rs, engine/src/cutile_kv_cache.rs, engine/src/disaggregated.rs
in the tempura repository).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _native as N
from ._native import TkvError, check, lib

_ELEM = {N.DTYPE_F32: 4, N.DTYPE_F16: 2, N.DTYPE_E4M3: 1}
_TORCH_VIEW = {N.DTYPE_F32: torch.float32, N.DTYPE_F16: torch.float16, N.DTYPE_E4M3: torch.uint8}
KvDtype = {"f32": N.DTYPE_F32, "f16": N.DTYPE_F16, "e4m3": N.DTYPE_E4M3}


def _u32(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.uint32))


def init(devices: Sequence[int]) -> None:
    """Enable peer access between the listed devices (once per process)."""
    arr = (C.c_int32 * len(devices))(*devices)
    check(lib().tkv_init(arr, len(devices)))


@dataclass
class Pool:
    """A paged KV pool on one device: per layer one K and one V tensor laid out
    ``[block][token_in_block][kv_head][head_dim]`` (GpuKvPagePool,
    engine/src/cutile_kv_cache.rs:1584-1602)."""
    device: int
    dtype: int
    n_layers: int
    n_kv_heads: int
    head_dim: int
    block_size: int
    total_blocks: int
    k_ptrs: np.ndarray
    v_ptrs: np.ndarray
    k_scales_ptr: int = 0
    v_scales_ptr: int = 0
    refcounts_ptr: int = 0
    # tensors that own the memory (None when built from foreign pointers)
    storage: Optional[torch.Tensor] = None
    k: List[torch.Tensor] = field(default_factory=list)
    v: List[torch.Tensor] = field(default_factory=list)
    k_scales: Optional[torch.Tensor] = None
    v_scales: Optional[torch.Tensor] = None
    refcounts: Optional[torch.Tensor] = None

    @property
    def elem_size(self) -> int:
        return _ELEM[self.dtype]

    @property
    def layer_bytes(self) -> int:
        return self.total_blocks * self.block_size * self.n_kv_heads * self.head_dim * self.elem_size

    @staticmethod
    def allocate(device: int, n_layers: int, n_kv_heads: int, head_dim: int, block_size: int,
                 total_blocks: int, dtype: str = "f16", scales: bool = False, refcounts: bool = False,
                 fill_byte: Optional[int] = 0xA5) -> "Pool":
        """One flat allocation carved into 2*n_layers layer tensors (so a decode
        process can export the whole pool with a single IPC handle)."""
        dt = KvDtype[dtype]
        dev = torch.device("cuda", device)
        layer_bytes = total_blocks * block_size * n_kv_heads * head_dim * _ELEM[dt]
        pad = (-layer_bytes) % 256
        stride = layer_bytes + pad
        storage = torch.empty(2 * n_layers * stride, dtype=torch.uint8, device=dev)
        if fill_byte is not None:
            storage.fill_(fill_byte)
        k, v = [], []
        for l in range(n_layers):
            k.append(storage[(2 * l) * stride:(2 * l) * stride + layer_bytes].view(_TORCH_VIEW[dt]))
            v.append(storage[(2 * l + 1) * stride:(2 * l + 1) * stride + layer_bytes].view(_TORCH_VIEW[dt]))
        pool = Pool(device, dt, n_layers, n_kv_heads, head_dim, block_size, total_blocks,
                    np.array([t.data_ptr() for t in k], dtype=np.uint64),
                    np.array([t.data_ptr() for t in v], dtype=np.uint64),
                    storage=storage, k=k, v=v)
        if scales:
            pool.k_scales = torch.full((n_layers, total_blocks, n_kv_heads), -123.0, dtype=torch.float32, device=dev)
            pool.v_scales = torch.full((n_layers, total_blocks, n_kv_heads), -123.0, dtype=torch.float32, device=dev)
            pool.k_scales_ptr, pool.v_scales_ptr = pool.k_scales.data_ptr(), pool.v_scales.data_ptr()
        if refcounts:
            pool.refcounts = torch.zeros(total_blocks, dtype=torch.int32, device=dev)
            pool.refcounts_ptr = pool.refcounts.data_ptr()
        return pool

    @staticmethod
    def from_pointers(device: int, dtype: str, n_kv_heads: int, head_dim: int, block_size: int,
                      total_blocks: int, k_ptrs: Sequence[int], v_ptrs: Sequence[int],
                      k_scales_ptr: int = 0, v_scales_ptr: int = 0, refcounts_ptr: int = 0) -> "Pool":
        """Describe memory owned elsewhere (another process's pool mapped through IPC,
        or an engine's own tensors)."""
        return Pool(device, KvDtype[dtype], len(k_ptrs), n_kv_heads, head_dim, block_size, total_blocks,
                    np.array(list(k_ptrs), dtype=np.uint64), np.array(list(v_ptrs), dtype=np.uint64),
                    k_scales_ptr, v_scales_ptr, refcounts_ptr)

    def blocks(self, layer: int, is_v: bool = False) -> torch.Tensor:
        """[total_blocks, block_size, n_kv_heads, head_dim] view of one layer."""
        t = (self.v if is_v else self.k)[layer]
        return t.view(self.total_blocks, self.block_size, self.n_kv_heads, self.head_dim)

    def c_struct(self) -> N.TkvPool:
        s = N.TkvPool(self.device, self.dtype, self.n_layers, self.n_kv_heads, self.head_dim,
                      self.block_size, self.total_blocks, 0,
                      self.k_ptrs.ctypes.data_as(C.POINTER(C.c_uint64)),
                      self.v_ptrs.ctypes.data_as(C.POINTER(C.c_uint64)),
                      self.k_scales_ptr, self.v_scales_ptr, self.refcounts_ptr)
        s._keep = (self.k_ptrs, self.v_ptrs)
        return s


@dataclass
class Batch:
    """Block tables and lengths of the prompts that finished prefill."""
    seq_lens: np.ndarray
    src_tables: np.ndarray
    dst_tables: np.ndarray
    table_stride: int
    prefix_lens: Optional[np.ndarray] = None
    table_layer_stride: int = 0

    def __post_init__(self):
        self.seq_lens = _u32(self.seq_lens)
        self.src_tables = _u32(self.src_tables).reshape(-1)
        self.dst_tables = _u32(self.dst_tables).reshape(-1)
        if self.prefix_lens is not None:
            self.prefix_lens = _u32(self.prefix_lens)

    def c_struct(self) -> N.TkvBatch:
        p = C.POINTER(C.c_uint32)
        s = N.TkvBatch(len(self.seq_lens), self.table_stride, self.table_layer_stride, 0,
                       self.seq_lens.ctypes.data_as(p),
                       self.prefix_lens.ctypes.data_as(p) if self.prefix_lens is not None else None,
                       self.src_tables.ctypes.data_as(p), self.dst_tables.ctypes.data_as(p))
        s._keep = self
        return s


@dataclass
class Transfer:
    """A contiguous transfer buffer (the batch form of KvCacheTransfer,
    engine/src/kv_cache.rs:514-522): per moved layer a K plane then a V plane of the moved
    blocks in work-list order.  ``data`` is a tensor on ``device``, or (``host``) a pinned
    host tensor that ``device``'s kernel reads or writes over PCIe."""
    data: torch.Tensor
    dtype: int
    device: int
    scales: Optional[torch.Tensor] = None
    host: bool = False

    @staticmethod
    def allocate(n_layers: int, n_heads: int, head_dim: int, block_size: int, n_blocks: int, dtype: str = "f16",
                 device: int = 0, scales: bool = False, fill_byte: Optional[int] = None, host: bool = False) -> "Transfer":
        dt = KvDtype[dtype]
        nbytes = int(lib().tkv_transfer_bytes(n_layers, n_heads, head_dim, block_size, dt, n_blocks))
        if host:
            data = torch.empty(max(nbytes, 16), dtype=torch.uint8, pin_memory=True)
        else:
            data = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=torch.device("cuda", device))
        if fill_byte is not None:
            data.fill_(fill_byte)
        sc = None
        if scales:
            shape = (2, n_layers, max(n_blocks, 1), n_heads)
            sc = (torch.full(shape, -123.0, dtype=torch.float32, pin_memory=True) if host else
                  torch.full(shape, -123.0, dtype=torch.float32, device=data.device))
        return Transfer(data, dt, device, sc, host)

    def planes(self, n_layers: int, n_blocks: int) -> torch.Tensor:
        """[layer][K|V][block][bytes of one block] view of the used part of the buffer."""
        used = self.data[: (self.data.numel() // max(2 * n_layers * n_blocks, 1)) * 2 * n_layers * n_blocks]
        return used.view(n_layers, 2, n_blocks, -1)

    def c_struct(self) -> N.TkvTransfer:
        return N.TkvTransfer(self.device, self.dtype, 1 if self.host else 0, 0, self.data.data_ptr(), self.data.numel(),
                             self.scales.data_ptr() if self.scales is not None else 0)


def batch_blocks(batch: "Batch", block_size: int) -> int:
    b = batch.c_struct()
    return int(lib().tkv_batch_blocks(C.byref(b), block_size))


def Shard(src_head_begin=0, dst_head_begin=0, n_heads=0, src_layer_begin=0, dst_layer_begin=0, n_layers=0) -> N.TkvShard:
    return N.TkvShard(src_head_begin, dst_head_begin, n_heads, src_layer_begin, dst_layer_begin, n_layers)


class Plan:
    """A validated, uploaded work list binding one batch to a source and a destination
    pool.  ``enqueue`` is asynchronous on a stream of the source device."""

    def __init__(self, src: Optional[Pool], dst: Optional[Pool], batch: Batch, shard: Optional[N.TkvShard] = None,
                 flags: int = 0, transfer: Optional[Transfer] = None):
        """``src`` and ``dst`` pools: the one-kernel handoff.  ``src`` and ``transfer``:
        gather into a contiguous buffer (to_transfer).  ``transfer`` and ``dst``: scatter a
        buffer into the pool (from_transfer)."""
        self.src, self.dst, self.transfer = src, dst, transfer
        self._h = C.c_void_p()
        b = batch.c_struct()
        sh = C.byref(shard) if shard is not None else None
        if transfer is None:
            self._s, self._d = src.c_struct(), dst.c_struct()
            self.launch_device = dst.device if flags & N.PLAN_PULL else src.device
            check(lib().tkv_plan_create(C.byref(self._s), C.byref(self._d), C.byref(b), sh, flags, C.byref(self._h)))
        elif dst is None:
            self._s, self._x = src.c_struct(), transfer.c_struct()
            self.launch_device = src.device
            check(lib().tkv_plan_create_to_transfer(C.byref(self._s), C.byref(self._x), C.byref(b), sh, flags,
                                                    C.byref(self._h)))
        else:
            assert src is None, "give either two pools, or one pool and a transfer buffer"
            self._d, self._x = dst.c_struct(), transfer.c_struct()
            self.launch_device = transfer.device
            check(lib().tkv_plan_create_from_transfer(C.byref(self._x), C.byref(self._d), C.byref(b), sh, flags,
                                                      C.byref(self._h)))

    @staticmethod
    def to_transfer(src: Pool, transfer: Transfer, batch: Batch, shard: Optional[N.TkvShard] = None, flags: int = 0) -> "Plan":
        return Plan(src, None, batch, shard, flags, transfer)

    @staticmethod
    def from_transfer(transfer: Transfer, dst: Pool, batch: Batch, shard: Optional[N.TkvShard] = None, flags: int = 0) -> "Plan":
        return Plan(None, dst, batch, shard, flags, transfer)

    def update(self, batch: Batch) -> None:
        b = batch.c_struct()
        check(lib().tkv_plan_update(self._h, C.byref(b)))

    def enqueue(self, stream: Optional[torch.cuda.Stream] = None, done_flag: int = 0, flag_value: int = 0) -> None:
        if stream is None:
            stream = torch.cuda.current_stream(self.launch_device)
        check(lib().tkv_handoff_enqueue(self._h, C.c_void_p(stream.cuda_stream), done_flag, flag_value))

    @staticmethod
    def with_capacity(src: Pool, dst: Pool, n_pairs: int, shard: Optional[N.TkvShard] = None, flags: int = 0) -> "Plan":
        """A plan sized for up to ``n_pairs`` block pairs per call, for :meth:`enqueue_device_tables`."""
        ids = np.arange(n_pairs, dtype=np.uint32)
        return Plan(src, dst, Batch(np.array([n_pairs * src.block_size], dtype=np.uint32), ids, ids, n_pairs), shard, flags)

    def enqueue_device_tables(self, seq_lens: torch.Tensor, src_tables: torch.Tensor, dst_tables: torch.Tensor,
                              prefix_lens: Optional[torch.Tensor] = None, apply_refcounts: bool = False,
                              status: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None,
                              done_flag: int = 0, flag_value: int = 0, prefix_blocks: Optional[torch.Tensor] = None) -> None:
        """The handoff with its work list built on the device from int32 tensors ``seq_lens [n]``, ``src_tables`` /
        ``dst_tables [n, stride]`` and optional ``prefix_lens [n]`` (as the device prefix index and page allocator
        leave them; ``prefix_blocks [n]`` gives the resident prefix in blocks instead); ``status`` (device int32) receives 0 or
        an error code."""
        for t in (seq_lens, src_tables, dst_tables, prefix_lens, status, prefix_blocks):
            assert t is None or (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous())
        assert src_tables.shape == dst_tables.shape and src_tables.shape[0] == seq_lens.numel()
        if stream is None:
            stream = torch.cuda.current_stream(self.launch_device)
        b = N.TkvDeviceBatch(src_tables.shape[0], src_tables.shape[1], 1 if apply_refcounts else 0, 0, seq_lens.data_ptr(),
                             prefix_lens.data_ptr() if prefix_lens is not None else 0, src_tables.data_ptr(), dst_tables.data_ptr(),
                             status.data_ptr() if status is not None else 0, prefix_blocks.data_ptr() if prefix_blocks is not None else 0)
        check(lib().tkv_handoff_enqueue_device_tables(self._h, C.byref(b), C.c_void_p(stream.cuda_stream), done_flag, flag_value))

    def refcount_apply(self, delta: int, stream: Optional[torch.cuda.Stream] = None) -> None:
        if stream is None:
            stream = torch.cuda.current_stream(self.launch_device)
        check(lib().tkv_refcount_apply(self._h, delta, C.c_void_p(stream.cuda_stream)))

    def tune_bulk(self, stages: int, ctas_per_sm: int, stage_bytes: int = 32768) -> None:
        check(lib().tkv_plan_tune_bulk(self._h, stages, ctas_per_sm, stage_bytes))

    def tune_vector(self, bytes_per_access: int, unroll: int = 8, store_hint: int = 0) -> None:
        check(lib().tkv_plan_tune_vector(self._h, bytes_per_access, unroll, store_hint))

    def tune_small(self, flag_mode: int = 0, inline_list: int = 0) -> None:
        check(lib().tkv_plan_tune_small(self._h, flag_mode, inline_list))

    def tune_grid(self, ctas_per_sm: int) -> None:
        check(lib().tkv_plan_tune_grid(self._h, ctas_per_sm))

    def device_error(self) -> int:
        out = C.c_uint32(0)
        check(lib().tkv_plan_error(self._h, C.byref(out)))
        return out.value

    def stats(self) -> N.TkvStats:
        st = N.TkvStats()
        check(lib().tkv_plan_stats(self._h, C.byref(st)))
        return st

    def destroy(self) -> None:
        if self._h:
            lib().tkv_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def handoff_noalloc(src: Pool, dst: Pool, batch: Batch, shard: Optional[N.TkvShard] = None,
                    stream: Optional[torch.cuda.Stream] = None) -> None:
    """Same-dtype handoff that allocates no device memory: the work list goes into a fixed
    array inside the library instead of a plan's buffer.  For callers that cannot call
    cudaMalloc when a handoff happens (HBM already owned by the KV pools, or a serving loop
    that must not stall the device).  Calls on one device share that array, so their GPU
    work must not overlap; at most 16384 block pairs and 128 layers per call."""
    if stream is None:
        stream = torch.cuda.current_stream(src.device)
    s, d, b = src.c_struct(), dst.c_struct(), batch.c_struct()
    check(lib().tkv_handoff_noalloc(C.byref(s), C.byref(d), C.byref(b),
                                    C.byref(shard) if shard is not None else None,
                                    C.c_void_p(stream.cuda_stream)))


def pairing_make(n_gpus: int, n_layers: int, n_kv_heads: int) -> List[N.TkvPairing]:
    out = (N.TkvPairing * 8)()
    n = C.c_int32(0)
    check(lib().tkv_pairing_make(n_gpus, n_layers, n_kv_heads, out, 8, C.byref(n)))
    return [out[i] for i in range(n.value)]


def flag_wait_host(device: int, flag_ptr: int, expected: int, timeout_us: int) -> None:
    check(lib().tkv_flag_wait_host(device, flag_ptr, expected, timeout_us))


def flag_wait_enqueue(stream: torch.cuda.Stream, flag_ptr: int, expected: int, max_spins: int, status_ptr: int) -> None:
    check(lib().tkv_flag_wait_enqueue(C.c_void_p(stream.cuda_stream), flag_ptr, expected, max_spins, status_ptr))


def cast(src: torch.Tensor, dst: torch.Tensor, src_dtype: str, dst_dtype: str) -> None:
    n = src.numel()
    assert dst.numel() == n and src.is_cuda and dst.is_cuda
    st = torch.cuda.current_stream(src.device)
    check(lib().tkv_cast(src.data_ptr(), KvDtype[src_dtype], dst.data_ptr(), KvDtype[dst_dtype], n,
                         C.c_void_p(st.cuda_stream)))


def memcpy_enqueue(dst_ptr: int, src_ptr: int, nbytes: int, stream: Optional[torch.cuda.Stream] = None) -> None:
    """One asynchronous copy-engine copy between two addresses the current device can reach (local memory, a mapped
    peer pool, pinned host memory): the reference's cuMemcpyDtoDAsync call sites (engine/src/cutile_kv_cache.rs:449-468)."""
    if stream is None:
        stream = torch.cuda.current_stream()
    check(lib().tkv_memcpy_enqueue(dst_ptr, src_ptr, nbytes, C.c_void_p(stream.cuda_stream)))


def bits_checksum(t: torch.Tensor, dtype: str) -> int:
    out = C.c_uint64(0)
    st = torch.cuda.current_stream(t.device)
    check(lib().tkv_bits_checksum(t.data_ptr(), KvDtype[dtype], t.numel(), C.c_void_p(st.cuda_stream), C.byref(out)))
    return out.value


def selfcheck_e4m3(skip_bits: int = 0) -> int:
    out = C.c_uint64(0)
    check(lib().tkv_selfcheck_e4m3(skip_bits, C.byref(out)))
    return out.value


def selfcheck_scaled_quant() -> int:
    out = C.c_uint64(0)
    check(lib().tkv_selfcheck_scaled_quant(C.byref(out)))
    return out.value


def selfcheck_tensor_cores():
    """Mismatch counts of the tcgen05 operand plumbing self-check: E4M3 K-major, E4M3 x E5M2 MN-major, F16 K-major, F16 MN-major."""
    out = (C.c_uint64 * 4)()
    check(lib().tkv_selfcheck_tensor_cores(out))
    return [int(v) for v in out]


def ipc_export(ptr: int):
    h = (C.c_uint8 * 64)()
    off = C.c_uint64(0)
    check(lib().tkv_ipc_export(ptr, h, C.byref(off)))
    return bytes(h), off.value


def ipc_import(handle: bytes, offset: int) -> int:
    h = (C.c_uint8 * 64)(*handle)
    out = C.c_uint64(0)
    check(lib().tkv_ipc_import(h, offset, C.byref(out)))
    return out.value


class DecodeAttention:
    """Decode attention over the paged pool with its output and split scratch allocated once, so
    a decode loop (or a CUDA graph capture) only issues launches.  ``q`` is f32
    ``[n_seqs, n_q_heads, head_dim]`` on the pool's device, ``tables`` int32
    ``[n_seqs, table_stride]`` block ids, ``kv_lens`` int32 ``[n_seqs]`` read by the kernel when
    it runs.  (OxideDecodeAttn::forward_batch_d2d_ptrs_{f16,e4m3},
    kernels/src/oxide_decode_attn_host.rs:682-760.)"""

    def __init__(self, pool: Pool, q: torch.Tensor, tables: torch.Tensor, kv_lens: torch.Tensor, max_kv_len: int,
                 sm_scale: Optional[float] = None, split_tokens: int = 0, flags: int = 0, total_kv_tokens: int = 0):
        assert q.is_cuda and q.dtype == torch.float32 and q.is_contiguous() and q.dim() == 3
        assert tables.is_cuda and tables.dtype == torch.int32 and tables.is_contiguous()
        assert kv_lens.is_cuda and kv_lens.dtype == torch.int32
        self.pool, self.q, self.tables, self.kv_lens = pool, q, tables, kv_lens
        n_seqs, n_q_heads, head_dim = q.shape
        self.sm_scale = 1.0 / float(head_dim) ** 0.5 if sm_scale is None else sm_scale
        self.out = torch.empty_like(q)
        need = int(lib().tkv_decode_attn_scratch_bytes(n_seqs, n_q_heads, head_dim, max_kv_len, split_tokens))
        self.scratch = torch.empty(max(need, 4) // 4, dtype=torch.float32, device=q.device)
        self._pool_c = pool.c_struct()
        self._args = {}
        self.status = torch.zeros(1, dtype=torch.int32, device=q.device)
        self._mk = lambda layer: N.TkvDecodeAttn(n_seqs, n_q_heads, tables.shape[1], layer, max_kv_len, self.sm_scale,
                                                 split_tokens, flags, q.data_ptr(), self.out.data_ptr(), tables.data_ptr(),
                                                 kv_lens.data_ptr(), self.scratch.data_ptr() if need else 0, need,
                                                 total_kv_tokens, self.status.data_ptr())

    def enqueue(self, layer: int, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        if stream is None:
            stream = torch.cuda.current_stream(self.pool.device)
        args = self._args.get(layer)
        if args is None:
            args = self._args[layer] = self._mk(layer)
        check(lib().tkv_decode_attn_enqueue(C.byref(self._pool_c), C.byref(args), C.c_void_p(stream.cuda_stream)))
        return self.out


def decode_attention(pool: Pool, layer: int, q: torch.Tensor, tables: torch.Tensor, kv_lens: torch.Tensor,
                     sm_scale: Optional[float] = None, max_kv_len: Optional[int] = None,
                     stream: Optional[torch.cuda.Stream] = None, split_tokens: int = 0, flags: int = 0) -> torch.Tensor:
    """One-shot form of :class:`DecodeAttention`; returns f32 of q's shape.  Raises if a bounded wait
    inside the kernel gave up."""
    if max_kv_len is None:
        max_kv_len = int(kv_lens.max().item()) if q.shape[0] else 0
    attn = DecodeAttention(pool, q, tables, kv_lens, max_kv_len, sm_scale, split_tokens, flags)
    out = attn.enqueue(layer, stream)
    if int(attn.status.item()) != 0:
        raise TkvError(int(attn.status.item()), "decode attention: a bounded wait inside the kernel gave up")
    return out


class PrefixIndex:
    """Device-resident ``RadixTree`` (engine/src/prefix_cache.rs:17-149): insert / lookup / release /
    evict_lru over a batch of token sequences, one launch per call, all state in HBM.  Sequences are
    int32 tensors ``[n_seqs, stride]`` on the index's device with int32 ``lens``; a node is
    ``group_tokens`` consecutive tokens (1 = the reference's per-token nodes, 16 = one per KV block)."""

    def __init__(self, device: int, capacity: int, group_tokens: int = 1):
        self.device, self.group_tokens = device, group_tokens
        h = C.c_void_p()
        check(lib().tkv_prefix_index_create(device, capacity, group_tokens, C.byref(h)))
        self._h = h

    def close(self) -> None:
        if self._h:
            lib().tkv_prefix_index_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _batch(self, tokens: torch.Tensor, lens: torch.Tensor, pages: Optional[torch.Tensor] = None,
               page_lens: Optional[torch.Tensor] = None) -> N.TkvPrefixBatch:
        for t in (tokens, lens, pages, page_lens):
            assert t is None or (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous() and t.device.index == self.device)
        assert tokens.dim() == 2 and lens.numel() == tokens.shape[0]
        return N.TkvPrefixBatch(tokens.shape[0], tokens.shape[1], pages.shape[1] if pages is not None else 0, 0,
                                tokens.data_ptr(), lens.data_ptr(), pages.data_ptr() if pages is not None else 0,
                                page_lens.data_ptr() if page_lens is not None else 0)

    def _stream(self, stream):
        return C.c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)

    def insert(self, tokens, lens, pages=None, page_lens=None, stream=None) -> None:
        b = self._batch(tokens, lens, pages, page_lens)
        check(lib().tkv_prefix_index_insert(self._h, C.byref(b), self._stream(stream)))

    def lookup(self, tokens, lens, stream=None, out_pages: Optional[torch.Tensor] = None, out_matched: Optional[torch.Tensor] = None):
        """Returns ``(matched, pages)``: int32 ``[n_seqs]`` matched nodes and int32 ``[n_seqs, nodes]`` page
        ids (-1 where a matched node has no page or past the match).  With ``out_pages`` (say the destination block
        tables) the pages of the matched nodes are written at the head of its rows and the rest is left alone."""
        b = self._batch(tokens, lens)
        if out_pages is None:
            n_nodes = max(tokens.shape[1] // self.group_tokens, 1)
            out_pages = torch.full((tokens.shape[0], n_nodes), -1, dtype=torch.int32, device=tokens.device)
        if out_matched is None:
            out_matched = torch.zeros(tokens.shape[0], dtype=torch.int32, device=tokens.device)
        assert out_pages.dtype == torch.int32 and out_pages.is_contiguous() and out_pages.shape[0] == tokens.shape[0]
        check(lib().tkv_prefix_index_lookup(self._h, C.byref(b), out_pages.data_ptr(), out_pages.shape[1], out_matched.data_ptr(),
                                            self._stream(stream)))
        return out_matched, out_pages

    def release(self, tokens, lens, stream=None) -> None:
        b = self._batch(tokens, lens)
        check(lib().tkv_prefix_index_release(self._h, C.byref(b), self._stream(stream)))

    def evict_lru(self, max_nodes: int = 1, stream=None):
        """Unlinks up to ``max_nodes`` nodes; returns ``(pages, nodes_unlinked)`` with the freed page ids on the host."""
        dev = f"cuda:{self.device}"
        pages = torch.full((max(max_nodes, 1),), -1, dtype=torch.int32, device=dev)
        counts = torch.zeros(2, dtype=torch.int32, device=dev)
        check(lib().tkv_prefix_index_evict_lru(self._h, max_nodes, pages.data_ptr(), pages.numel(), counts.data_ptr(),
                                               counts.data_ptr() + 4, self._stream(stream)))
        n_pages, n_nodes = (int(x) for x in counts.cpu())
        return pages[:n_pages].cpu().tolist(), n_nodes

    def set_key_bits(self, bits: int) -> None:
        """Test hook: cut the keys to ``bits`` bits so that prefixes collide (the guard must then turn them into misses)."""
        check(lib().tkv_prefix_index_set_key_bits(self._h, bits))

    def stats(self, stream=None) -> N.TkvPrefixIndexStats:
        st = N.TkvPrefixIndexStats()
        check(lib().tkv_prefix_index_stats(self._h, self._stream(stream), C.byref(st)))
        return st


class DevicePageAllocator:
    """``PageAllocator`` (engine/src/kv_cache.rs:762-797) with its free stack in HBM: one launch places (or
    returns) the pages of a whole batch straight in a device block table."""

    def __init__(self, device: int, total_pages: int):
        self.device = device
        h = C.c_void_p()
        check(lib().tkv_device_page_allocator_create(device, total_pages, C.byref(h)))
        self._h = h
        self.status = torch.zeros(1, dtype=torch.int32, device=f"cuda:{device}")

    def close(self) -> None:
        if self._h:
            lib().tkv_device_page_allocator_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _call(self, fn, tables, counts, first, stream, seq_lens, block_size):
        for t in (tables, counts, first, seq_lens):
            assert t is None or (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous() and t.device.index == self.device)
        b = N.TkvPageBatch(tables.shape[0], tables.shape[1], tables.data_ptr(), first.data_ptr() if first is not None else 0,
                           counts.data_ptr() if counts is not None else 0, seq_lens.data_ptr() if seq_lens is not None else 0, block_size, 0)
        st = C.c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)
        check(fn(self._h, C.byref(b), self.status.data_ptr(), st))

    def allocate(self, tables, counts=None, first=None, stream=None, seq_lens=None, block_size: int = 16) -> None:
        """Fills ``tables[s, first[s] : first[s] + counts[s]]``; without ``counts`` a row gets the blocks of ``seq_lens[s]``
        tokens that ``first[s]`` does not cover.  ``self.status`` (device int32) is 0 or an error code."""
        self._call(lib().tkv_device_page_allocator_allocate, tables, counts, first, stream, seq_lens, block_size)

    def free(self, tables, counts=None, first=None, stream=None, seq_lens=None, block_size: int = 16) -> None:
        self._call(lib().tkv_device_page_allocator_free, tables, counts, first, stream, seq_lens, block_size)

    def available(self, stream=None) -> int:
        out = C.c_uint32()
        st = C.c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)
        check(lib().tkv_device_page_allocator_available(self._h, st, C.byref(out)))
        return int(out.value)


def refcount_apply_device_tables(dst: Pool, dst_tables: torch.Tensor, prefix_blocks: torch.Tensor, delta: int,
                                 status: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None) -> None:
    """+1 / -1 on ``dst``'s reference counts for the first ``prefix_blocks[q]`` entries of every row of ``dst_tables``
    (int32 device tensors), launched on the pool's device."""
    for t in (dst_tables, prefix_blocks, status):
        assert t is None or (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous())
    b = N.TkvDeviceBatch(dst_tables.shape[0], dst_tables.shape[1], 0, 0, 0, 0, 0, dst_tables.data_ptr(),
                         status.data_ptr() if status is not None else 0, prefix_blocks.data_ptr())
    s = dst.c_struct()
    st = stream or torch.cuda.current_stream(dst.device)
    check(lib().tkv_refcount_apply_device_tables(C.byref(s), C.byref(b), delta, C.c_void_p(st.cuda_stream)))


def prefill_attention(pool: Pool, layer: int, q: torch.Tensor, table_row: torch.Tensor, start_pos: int,
                      sm_scale: Optional[float] = None, stream: Optional[torch.cuda.Stream] = None,
                      status: Optional[torch.Tensor] = None, flags: int = 0) -> torch.Tensor:
    """Causal attention of ``T`` new tokens of ONE sequence over its paged cache on the tcgen05 tensor cores (the
    prefill-side twin of ``decode_attention``): the tokens' K/V rows are already in the pool at positions
    ``start_pos .. start_pos + T - 1`` and query token ``t`` attends to positions ``0 .. start_pos + t``.  ``q`` is f32
    ``[T, 32, 128]``, ``table_row`` the sequence's int32 block table; 8 kv heads, 16-token blocks, F16 or E4M3 pool
    (per-block scales applied).  Raises ``TkvError`` for any other geometry (``causal_chunk_attention`` covers those)."""
    assert q.dtype == torch.float32 and q.is_contiguous() and q.dim() == 3
    table_row = table_row.to(torch.int32).contiguous()
    out = torch.empty_like(q)
    st = stream or torch.cuda.current_stream(q.device)
    args = N.TkvPrefillAttn(q.shape[0], q.shape[1], layer, start_pos, table_row.numel(),
                            float(sm_scale if sm_scale is not None else 1.0 / np.sqrt(q.shape[2])), flags, 0,
                            q.data_ptr(), out.data_ptr(), table_row.data_ptr(), status.data_ptr() if status is not None else 0)
    ps = pool.c_struct()
    check(lib().tkv_prefill_attn_enqueue(C.byref(ps), C.byref(args), C.c_void_p(st.cuda_stream)))
    return out


def causal_chunk_attention(pool: Pool, layer: int, q: torch.Tensor, table_row: torch.Tensor, start_pos: int,
                           sm_scale: Optional[float] = None, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Causal attention of ``T`` consecutive new tokens of ONE sequence over the paged pool (their K/V rows already
    written at positions ``start_pos .. start_pos + T - 1``): query token ``t`` attends to positions ``0 .. start_pos + t``.
    ``q`` is f32 ``[T, n_q_heads, head_dim]``, ``table_row`` the sequence's int32 block table.  Each query token is one
    row of the decode kernel (the rows share the table and differ in length), which is the right shape for a few
    tokens at a time -- speculative verification, short prefill chunks -- and reads the scaled E4M3 pool exactly as
    decode does; it is not a prefill-throughput kernel (K/V is fetched once per query token, mostly from L2).
    (cutile_flash_attn_heads_paged_e4m3, kernels/src/cutile_flash_attention.rs:868, is the reference's unscaled form.)"""
    t = q.shape[0]
    tables = table_row.reshape(1, -1).expand(t, -1).contiguous()
    kv_lens = torch.arange(start_pos + 1, start_pos + t + 1, dtype=torch.int32, device=q.device)
    return decode_attention(pool, layer, q, tables, kv_lens, sm_scale, max_kv_len=start_pos + t, stream=stream)
