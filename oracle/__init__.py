"""ctypes binding of the CPU oracle (``oracle/tkv_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Importers are the test-suite, the smoke check and the
benchmark's CPU-baseline leg; the shipped package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libtkv_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the system gcc (``make -C oracle``)."""
    srcs = [os.path.join(_HERE, f) for f in ("tkv_oracle.c", "tkv_oracle.h", "x86_f16c_check.c", "Makefile")]
    stale = force or not os.path.exists(_SO) or any(
        os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


class OrcPool(C.Structure):
    _fields_ = [
        ("n_layers", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
        ("block_size", C.c_uint32), ("total_blocks", C.c_uint32), ("elem_size", C.c_uint32),
        ("k_layers", C.POINTER(C.c_void_p)), ("v_layers", C.POINTER(C.c_void_p)),
        ("k_scales", C.POINTER(C.c_float)), ("v_scales", C.POINTER(C.c_float)),
    ]


class OrcBatch(C.Structure):
    _fields_ = [
        ("n_seqs", C.c_uint32),
        ("seq_lens", C.POINTER(C.c_uint32)), ("prefix_lens", C.POINTER(C.c_uint32)),
        ("src_tables", C.POINTER(C.c_uint32)), ("dst_tables", C.POINTER(C.c_uint32)),
        ("table_stride", C.c_uint32), ("table_layer_stride", C.c_uint32),
    ]


class OrcShard(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "src_head_begin", "dst_head_begin", "n_heads", "src_layer_begin", "dst_layer_begin", "n_layers")]


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(_SO)
    u8, u16, u32, u64, i64, f32, sz = C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64, C.c_int64, C.c_float, C.c_size_t
    vp, P = C.c_void_p, C.POINTER

    def sig(name, res, *args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("orc_f32_to_e4m3", u8, f32)
    sig("orc_e4m3_to_f32", f32, u8)
    sig("orc_f32_to_e4m3_legacy", u8, f32)
    sig("orc_f32_to_f16", u16, f32)
    sig("orc_f16_to_f32", f32, u16)
    sig("orc_f32_to_f16_scalar_fallback", u16, f32)
    sig("orc_block_scale", f32, u16, P(f32))
    sig("orc_quantize_scaled", u8, u16, f32)
    sig("orc_paged_row_offset", sz, P(u32), sz, sz, sz, sz, sz)
    sig("orc_pa_new", vp, sz); sig("orc_pa_delete", None, vp)
    sig("orc_pa_allocate", i64, vp); sig("orc_pa_free", None, vp, sz)
    sig("orc_pa_available", sz, vp); sig("orc_pa_in_use", sz, vp)
    sig("orc_bt_new", vp, sz); sig("orc_bt_delete", None, vp)
    sig("orc_bt_set_block", None, vp, sz, sz); sig("orc_bt_get_block", i64, vp, sz)
    sig("orc_bt_num_blocks", sz, vp); sig("orc_bt_as_slice", P(u32), vp)
    sig("orc_bt_clear", sz, vp, P(sz), sz)
    sig("orc_paged_gather", None, vp, P(u32), sz, sz, sz, sz, vp)
    sig("orc_paged_scatter", None, vp, P(u32), sz, sz, sz, sz, sz, vp)
    sig("orc_transfer_layer", None, P(f32), sz, sz, C.c_int, vp)
    for n in ("orc_handoff_copy", "orc_handoff_f16_to_e4m3", "orc_handoff_f32_to_f16", "orc_handoff_e4m3_to_f16",
              "orc_handoff_e4m3_to_f32", "orc_handoff_f32_to_e4m3"):
        sig(n, C.c_int, P(OrcPool), P(OrcPool), P(OrcBatch), P(OrcShard), C.c_int)
    sig("orc_refcount_apply", None, P(u32), P(OrcBatch), u32, C.c_int)
    sig("orc_paged_decode_attention", C.c_int, P(OrcPool), u32, P(f32), P(u32), u32, P(u32), u32, u32, f32, P(f32))
    sig("orc_bits_checksum_f32", u64, P(f32), sz)
    sig("orc_bits_checksum_f16_as_f32", u64, P(u16), sz)
    sig("orc_bits_checksum_e4m3_as_f32", u64, P(u8), sz)
    sig("orc_radix_new", vp); sig("orc_radix_delete", None, vp)
    sig("orc_radix_insert", None, vp, P(u32), sz, P(sz), sz)
    sig("orc_radix_lookup", sz, vp, P(u32), sz, P(sz), sz, P(sz))
    sig("orc_radix_release", None, vp, P(u32), sz)
    sig("orc_radix_evict_lru", sz, vp, P(sz), sz)
    sig("orc_radix_hit_count", u64, vp); sig("orc_radix_tokens_saved", u64, vp)
    sig("orc_radix_node_count", sz, vp); sig("orc_radix_ref_count", i64, vp, P(u32), sz)
    sig("orc_pt_new", vp, sz); sig("orc_pt_delete", None, vp)
    sig("orc_pt_store", None, vp, P(u32), sz, C.c_char_p, P(u32), sz, sz)
    sig("orc_pt_probe", sz, vp, P(u32), sz, C.c_char_p, P(u32), sz, P(sz))
    sig("orc_pt_release", None, vp, P(u32), sz, C.c_char_p)
    sig("orc_pt_len", sz, vp); sig("orc_pt_hit_count", u64, vp); sig("orc_pt_tokens_saved", u64, vp)
    sig("orc_pt_ref_count", i64, vp, P(u32), sz, C.c_char_p)
    sig("orc_ra_new", vp, sz); sig("orc_ra_delete", None, vp)
    sig("orc_ra_alloc", C.c_int, vp, sz, P(sz)); sig("orc_ra_free", None, vp, sz, sz)
    sig("orc_ra_try_extend", C.c_int, vp, sz, sz, sz)
    sig("orc_ra_free_pages", sz, vp); sig("orc_ra_allocated_pages", sz, vp)
    sig("orc_ra_free_runs", sz, vp, P(sz), P(sz), sz)
    sig("orc_mix64", u64, u64, u64, u64)
    sig("orc_gen_normal_f16", None, P(u16), sz, u64, u64, C.c_double, u32, P(u32), u32, C.c_double, sz)
    sig("orc_gen_permutation", None, P(u32), u32, u64, u64)
    sig("orc_gen_lengths", None, P(u32), u32, u32, u32, u64, u64)
    sig("orc_have_f16c", C.c_int)
    sig("orc_hw_f32_to_f16", u16, f32)
    sig("orc_hw_f16_to_f32", f32, u16)
    sig("orc_sweep_f32_to_f16", u64, vp, C.c_uint)
    _lib = L
    return L


# --------------------------------------------------------------------------
# numpy-facing helpers
# --------------------------------------------------------------------------
def _p(arr: np.ndarray, ctype):
    return arr.ctypes.data_as(C.POINTER(ctype))


def u32arr(x) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(x, dtype=np.uint32))


@dataclass
class HostPool:
    """A paged pool in host memory: one flat array per layer for K and for V,
    laid out [block][token_in_block][kv_head][head_dim] (the reference's
    PagedKvCache / GpuKvPagePool layout)."""
    n_layers: int
    n_kv_heads: int
    head_dim: int
    block_size: int
    total_blocks: int
    dtype: np.dtype
    k: list
    v: list
    k_scales: Optional[np.ndarray] = None
    v_scales: Optional[np.ndarray] = None

    @staticmethod
    def filled(n_layers, n_kv_heads, head_dim, block_size, total_blocks, dtype, fill_byte=0xA5,
               with_scales=False, scale_fill=-123.0):
        dtype = np.dtype(dtype)
        n = total_blocks * block_size * n_kv_heads * head_dim

        def mk():
            a = np.empty(n * dtype.itemsize, dtype=np.uint8)
            a[:] = fill_byte
            return a.view(dtype)

        hp = HostPool(n_layers, n_kv_heads, head_dim, block_size, total_blocks, dtype,
                      [mk() for _ in range(n_layers)], [mk() for _ in range(n_layers)])
        if with_scales:
            hp.k_scales = np.full((n_layers, total_blocks, n_kv_heads), scale_fill, dtype=np.float32)
            hp.v_scales = np.full((n_layers, total_blocks, n_kv_heads), scale_fill, dtype=np.float32)
        return hp

    def block_view(self, arr):
        return arr.reshape(self.total_blocks, self.block_size, self.n_kv_heads, self.head_dim)

    def c_struct(self):
        kp = (C.c_void_p * self.n_layers)(*[a.ctypes.data for a in self.k])
        vp = (C.c_void_p * self.n_layers)(*[a.ctypes.data for a in self.v])
        s = OrcPool(self.n_layers, self.n_kv_heads, self.head_dim, self.block_size,
                    self.total_blocks, self.dtype.itemsize,
                    C.cast(kp, C.POINTER(C.c_void_p)), C.cast(vp, C.POINTER(C.c_void_p)),
                    _p(self.k_scales, C.c_float) if self.k_scales is not None else None,
                    _p(self.v_scales, C.c_float) if self.v_scales is not None else None)
        s._keep = (kp, vp)
        return s


def make_batch(seq_lens, src_tables, dst_tables, table_stride, prefix_lens=None, table_layer_stride=0):
    seq_lens = u32arr(seq_lens)
    src_tables = u32arr(src_tables).reshape(-1)
    dst_tables = u32arr(dst_tables).reshape(-1)
    pre = u32arr(prefix_lens) if prefix_lens is not None else None
    b = OrcBatch(len(seq_lens), _p(seq_lens, C.c_uint32),
                 _p(pre, C.c_uint32) if pre is not None else None,
                 _p(src_tables, C.c_uint32), _p(dst_tables, C.c_uint32), table_stride, table_layer_stride)
    b._keep = (seq_lens, src_tables, dst_tables, pre)
    return b


def full_shard(src: HostPool, dst: HostPool) -> OrcShard:
    return OrcShard(0, 0, min(src.n_kv_heads, dst.n_kv_heads), 0, 0, min(src.n_layers, dst.n_layers))


_MODES = {"copy": "orc_handoff_copy", "f16_e4m3": "orc_handoff_f16_to_e4m3", "f32_f16": "orc_handoff_f32_to_f16",
          "e4m3_f16": "orc_handoff_e4m3_to_f16", "e4m3_f32": "orc_handoff_e4m3_to_f32", "f32_e4m3": "orc_handoff_f32_to_e4m3"}


def handoff(src: HostPool, dst: HostPool, batch: OrcBatch, shard: Optional[OrcShard] = None,
            mode: str = "copy", n_threads: int = 1) -> None:
    sh = shard if shard is not None else full_shard(src, dst)
    s, d = src.c_struct(), dst.c_struct()
    rc = getattr(lib(), _MODES[mode])(C.byref(s), C.byref(d), C.byref(batch), C.byref(sh), n_threads)
    if rc != 0:
        raise ValueError(f"oracle rejected the handoff arguments (code {rc})")


def paged_decode_attention(pool: HostPool, layer: int, q: np.ndarray, tables: np.ndarray, kv_lens, scale: float) -> np.ndarray:
    """q: [n_seqs, num_heads, head_dim] f32 -> out of the same shape."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    tables = u32arr(tables)
    kv_lens = u32arr(kv_lens)
    out = np.empty_like(q)
    s = pool.c_struct()
    rc = lib().orc_paged_decode_attention(C.byref(s), layer, _p(q, C.c_float), _p(tables.reshape(-1), C.c_uint32), tables.shape[1],
                                          _p(kv_lens, C.c_uint32), q.shape[0], q.shape[1], scale, _p(out, C.c_float))
    if rc != 0:
        raise ValueError(f"oracle rejected the attention arguments (code {rc})")
    return out


def refcount_apply(refcounts: np.ndarray, batch: OrcBatch, block_size: int, delta: int) -> None:
    assert refcounts.dtype == np.uint32
    lib().orc_refcount_apply(_p(refcounts, C.c_uint32), C.byref(batch), block_size, delta)


def gen_normal_f16(n, seed, stream, sigma=0.5, head_dim=0, outlier_channels: Sequence[int] = (),
                   outlier_gain=1.0, first_index=0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint16)
    oc = u32arr(list(outlier_channels)) if len(outlier_channels) else None
    lib().orc_gen_normal_f16(_p(out, C.c_uint16), n, seed, stream, sigma, head_dim,
                             _p(oc, C.c_uint32) if oc is not None else None,
                             len(outlier_channels), outlier_gain, first_index)
    return out


def gen_permutation(n, seed, stream=0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().orc_gen_permutation(_p(out, C.c_uint32), n, seed, stream)
    return out


def gen_lengths(n, lo, hi, seed, stream=0) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().orc_gen_lengths(_p(out, C.c_uint32), n, lo, hi, seed, stream)
    return out


def f32_to_e4m3(x: float) -> int:
    return lib().orc_f32_to_e4m3(C.c_float(x))


def e4m3_to_f32(b: int) -> float:
    return lib().orc_e4m3_to_f32(b)
