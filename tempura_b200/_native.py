"""ctypes view of ``libtkv.so``.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_lib = None


class TkvError(RuntimeError):
    """Mirror of the reference's ``KernelError`` (kernel-api/src/lib.rs:5-13) plus the
    CUDA, timeout and pool-exhaustion codes of the C ABI."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{STATUS_NAMES.get(code, code)}] {message}")
        self.code = code
        self.message = message


OK, ERR_DIMENSION_MISMATCH, ERR_INVALID_CONFIG, ERR_CUDA, ERR_TIMEOUT, ERR_POOL_EXHAUSTED = range(6)
STATUS_NAMES = {0: "Ok", 1: "DimensionMismatch", 2: "InvalidConfig", 3: "CudaError", 4: "Timeout", 5: "PoolExhausted"}
DTYPE_F32, DTYPE_F16, DTYPE_E4M3 = 0, 1, 2
PREFILL_SINGLE_TILE, PREFILL_TWO_TILES = 1, 2
PLAN_ALLOW_SHARED_DST, PLAN_FORCE_VECTOR, PLAN_FORCE_BULK, PLAN_INT_QUANTIZER, PLAN_PEER_BULK_STORES, PLAN_PULL, PLAN_STAGE_HOST = 1, 2, 4, 8, 16, 32, 64
ATTN_PER_HEAD_CTAS = 1
ATTN_MMA_SYNC = 2
VARIANT_VECTOR, VARIANT_BULK, VARIANT_FP8_WARP, VARIANT_FP8_GENERIC, VARIANT_CAST_GENERIC, VARIANT_FP8_STAGED, VARIANT_DEQUANT, VARIANT_CAST_VEC, VARIANT_WIDE = 1, 2, 3, 4, 5, 6, 7, 8, 9


class TkvPool(C.Structure):
    _fields_ = [
        ("device", C.c_int32), ("dtype", C.c_int32),
        ("n_layers", C.c_uint32), ("n_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
        ("block_size", C.c_uint32), ("total_blocks", C.c_uint32), ("reserved", C.c_uint32),
        ("k_layer_ptrs", C.POINTER(C.c_uint64)), ("v_layer_ptrs", C.POINTER(C.c_uint64)),
        ("k_scales", C.c_uint64), ("v_scales", C.c_uint64), ("refcounts", C.c_uint64),
    ]


class TkvBatch(C.Structure):
    _fields_ = [
        ("n_seqs", C.c_uint32), ("table_stride", C.c_uint32), ("table_layer_stride", C.c_uint32),
        ("reserved", C.c_uint32),
        ("seq_lens", C.POINTER(C.c_uint32)), ("prefix_lens", C.POINTER(C.c_uint32)),
        ("src_tables", C.POINTER(C.c_uint32)), ("dst_tables", C.POINTER(C.c_uint32)),
    ]


class TkvTransfer(C.Structure):
    _fields_ = [("device", C.c_int32), ("dtype", C.c_int32), ("host_memory", C.c_uint32), ("reserved", C.c_uint32),
                ("data", C.c_uint64), ("bytes", C.c_uint64), ("scales", C.c_uint64)]


class TkvDecodeAttn(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_seqs", "n_q_heads", "table_stride", "layer", "max_kv_len")] + [
        ("sm_scale", C.c_float), ("split_tokens", C.c_uint32), ("flags", C.c_uint32)] + [(n, C.c_uint64) for n in ("q", "out", "tables", "kv_lens", "scratch", "scratch_bytes", "total_kv_tokens", "status")]


class TkvPrefillAttn(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_tokens", "n_q_heads", "layer", "start_pos", "table_len")] + [("sm_scale", C.c_float)] + [
        (n, C.c_uint32) for n in ("flags", "reserved")] + [(n, C.c_uint64) for n in ("q", "out", "table", "status")]


class TkvPrefixBatch(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_seqs", "stride", "page_stride", "reserved")] + [
        (n, C.c_uint64) for n in ("tokens", "lens", "pages", "page_lens")]


class TkvPrefixIndexStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("hits", "tokens_saved", "live_nodes", "tombstones", "capacity", "ticks")] + [
        ("group_tokens", C.c_uint32), ("table_full", C.c_uint32), ("key_collisions", C.c_uint64)]


class TkvPageBatch(C.Structure):
    _fields_ = [("n_seqs", C.c_uint32), ("table_stride", C.c_uint32), ("tables", C.c_uint64), ("first", C.c_uint64), ("counts", C.c_uint64),
                ("seq_lens", C.c_uint64), ("block_size", C.c_uint32), ("reserved", C.c_uint32)]


class TkvDeviceBatch(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_seqs", "table_stride", "apply_refcounts", "reserved")] + [
        (n, C.c_uint64) for n in ("seq_lens", "prefix_lens", "src_tables", "dst_tables", "status", "prefix_blocks")]


class TkvCoordinatorConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_prefill", "n_decode", "block_size", "max_inflight_per_decode", "max_retries",
                                          "headroom_blocks")] + [("handoff_timeout", C.c_uint64)]


class TkvAdmission(C.Structure):
    _fields_ = [("request_id", C.c_uint64)] + [(n, C.c_uint32) for n in ("prefill_worker", "decode_worker", "blocks", "prefix_tokens")]


class TkvRequestInfo(C.Structure):
    _fields_ = [("request_id", C.c_uint64)] + [(n, C.c_uint32) for n in (
        "state", "prefill_worker", "decode_worker", "reserved_blocks", "prefix_tokens", "attempts")]


class TkvCoordinatorStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("submitted", "admitted", "handoffs_completed", "handoffs_failed", "retries", "fallbacks",
                                          "finished", "in_system", "waiting", "reserved_blocks")]


REQ_QUEUED, REQ_PREFILL, REQ_WAITING, REQ_ADMITTED, REQ_TRANSFER, REQ_DECODE, REQ_REPREFILL = range(7)
RETRY_HANDOFF, REPREFILL = 1, 2
PREFIX_NO_PAGE = 0xFFFFFFFF


class TkvSessionHeader(C.Structure):
    _fields_ = [("position", C.c_uint64), ("seed", C.c_uint64)] + [(n, C.c_uint32) for n in (
        "seq_len", "n_layers", "n_kv_heads", "head_dim", "block_size", "kv_dtype", "block_begin", "n_blocks",
        "piece_index", "piece_count", "n_logits", "reserved")]


class TkvShard(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "src_head_begin", "dst_head_begin", "n_heads", "src_layer_begin", "dst_layer_begin", "n_layers")]


class TkvPairing(C.Structure):
    _fields_ = [("prefill_device", C.c_int32), ("decode_device", C.c_int32), ("shard", TkvShard)]


class TkvStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "payload_bytes", "bytes_read", "bytes_written", "n_blocks", "n_chunks", "n_tokens",
        "n_prefix_refs", "worklist_bytes")] + [(n, C.c_uint32) for n in ("grid", "block", "kernel_variant", "peer")]


# every symbol include/tkv.h declares: name -> (restype, argtypes)
_u8p, _u32p, _u64p, _szp = C.POINTER(C.c_uint8), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_size_t)
_vp, _i32, _u32, _u64, _sz = C.c_void_p, C.c_int32, C.c_uint32, C.c_uint64, C.c_size_t
SIGNATURES = {
    "tkv_last_error": (None, [C.c_char_p, _sz]),
    "tkv_last_cuda_error": (_i32, []),
    "tkv_version": (C.c_char_p, []),
    "tkv_init": (_i32, [C.POINTER(_i32), _i32]),
    "tkv_shutdown": (_i32, []),
    "tkv_plan_create": (_i32, [C.POINTER(TkvPool), C.POINTER(TkvPool), C.POINTER(TkvBatch), C.POINTER(TkvShard), _u32, C.POINTER(_vp)]),
    "tkv_plan_create_to_transfer": (_i32, [C.POINTER(TkvPool), C.POINTER(TkvTransfer), C.POINTER(TkvBatch), C.POINTER(TkvShard), _u32, C.POINTER(_vp)]),
    "tkv_plan_create_from_transfer": (_i32, [C.POINTER(TkvTransfer), C.POINTER(TkvPool), C.POINTER(TkvBatch), C.POINTER(TkvShard), _u32, C.POINTER(_vp)]),
    "tkv_transfer_bytes": (_u64, [_u32, _u32, _u32, _u32, _i32, _u64]),
    "tkv_batch_blocks": (_u64, [C.POINTER(TkvBatch), _u32]),
    "tkv_plan_update": (_i32, [_vp, C.POINTER(TkvBatch)]),
    "tkv_plan_destroy": (_i32, [_vp]),
    "tkv_plan_stats": (_i32, [_vp, C.POINTER(TkvStats)]),
    "tkv_handoff_enqueue": (_i32, [_vp, _vp, _u64, _u32]),
    "tkv_handoff_noalloc": (_i32, [C.POINTER(TkvPool), C.POINTER(TkvPool), C.POINTER(TkvBatch), C.POINTER(TkvShard), _vp]),
    "tkv_plan_tune_bulk": (_i32, [_vp, _u32, _u32, _u32]),
    "tkv_plan_tune_vector": (_i32, [_vp, _u32, _u32, _u32]),
    "tkv_plan_tune_grid": (_i32, [_vp, _u32]),
    "tkv_plan_tune_small": (_i32, [_vp, _u32, _u32]),
    "tkv_plan_error": (_i32, [_vp, _u32p]),
    "tkv_flag_wait_host": (_i32, [_i32, _u64, _u32, _u64]),
    "tkv_flag_wait_enqueue": (_i32, [_vp, _u64, _u32, _u64, _u64]),
    "tkv_refcount_apply": (_i32, [_vp, _i32, _vp]),
    "tkv_pairing_make": (_i32, [_i32, _u32, _u32, C.POINTER(TkvPairing), _i32, C.POINTER(_i32)]),
    "tkv_cast": (_i32, [_u64, _i32, _u64, _i32, _u64, _vp]),
    "tkv_selfcheck_e4m3": (_i32, [_u32, _u64p]),
    "tkv_selfcheck_scaled_quant": (_i32, [_u64p]),
    "tkv_memcpy_enqueue": (_i32, [_u64, _u64, _u64, _vp]),
    "tkv_bits_checksum": (_i32, [_u64, _i32, _u64, _vp, _u64p]),
    "tkv_ipc_export": (_i32, [_u64, _u8p, _u64p]),
    "tkv_ipc_import": (_i32, [_u8p, _u64, _u64p]),
    "tkv_ipc_close": (_i32, [_u64, _u64]),
    "tkv_decode_attn_scratch_bytes": (_u64, [_u32, _u32, _u32, _u32, _u32]),
    "tkv_decode_attn_enqueue": (_i32, [C.POINTER(TkvPool), C.POINTER(TkvDecodeAttn), _vp]),
    "tkv_selfcheck_tensor_cores": (_i32, [_u64p]),
    "tkv_session_wire_size": (_sz, [C.POINTER(TkvSessionHeader)]),
    "tkv_session_pack": (_i32, [C.POINTER(TkvSessionHeader), _u32p, C.POINTER(C.c_float), _u8p, _sz, _szp]),
    "tkv_session_unpack": (_i32, [_u8p, _sz, C.POINTER(TkvSessionHeader), C.POINTER(_u32p), C.POINTER(C.POINTER(C.c_float))]),
    "tkv_page_allocator_new": (_vp, [_sz]),
    "tkv_page_allocator_delete": (None, [_vp]),
    "tkv_page_allocator_allocate": (_i32, [_vp, _szp]),
    "tkv_page_allocator_free": (None, [_vp, _sz]),
    "tkv_page_allocator_available": (_sz, [_vp]),
    "tkv_page_allocator_in_use": (_sz, [_vp]),
    "tkv_page_allocator_total": (_sz, [_vp]),
    "tkv_block_table_new": (_vp, [_sz]),
    "tkv_block_table_delete": (None, [_vp]),
    "tkv_block_table_set_block": (_i32, [_vp, _sz, _sz]),
    "tkv_block_table_get_block": (_i32, [_vp, _sz, _szp]),
    "tkv_block_table_num_blocks": (_sz, [_vp]),
    "tkv_block_table_max_blocks": (_sz, [_vp]),
    "tkv_block_table_as_slice": (_u32p, [_vp]),
    "tkv_block_table_clear": (_sz, [_vp, _szp, _sz]),
    "tkv_run_allocator_new": (_vp, [_sz]),
    "tkv_run_allocator_delete": (None, [_vp]),
    "tkv_run_allocator_alloc": (_i32, [_vp, _sz, _szp]),
    "tkv_run_allocator_free": (_i32, [_vp, _sz, _sz]),
    "tkv_run_allocator_try_extend": (_i32, [_vp, _sz, _sz, _sz]),
    "tkv_run_allocator_free_pages": (_sz, [_vp]),
    "tkv_run_allocator_allocated_pages": (_sz, [_vp]),
    "tkv_run_allocator_free_runs": (_sz, [_vp, _szp, _szp, _sz]),
    "tkv_prefix_index_create": (_i32, [_i32, _u64, _u32, C.POINTER(_vp)]),
    "tkv_prefix_index_destroy": (None, [_vp]),
    "tkv_prefix_index_insert": (_i32, [_vp, C.POINTER(TkvPrefixBatch), _vp]),
    "tkv_prefix_index_lookup": (_i32, [_vp, C.POINTER(TkvPrefixBatch), _u64, _u32, _u64, _vp]),
    "tkv_prefix_index_release": (_i32, [_vp, C.POINTER(TkvPrefixBatch), _vp]),
    "tkv_prefix_index_evict_lru": (_i32, [_vp, _u32, _u64, _u32, _u64, _u64, _vp]),
    "tkv_prefill_attn_enqueue": (_i32, [C.POINTER(TkvPool), C.POINTER(TkvPrefillAttn), _vp]),
    "tkv_prefix_index_stats": (_i32, [_vp, _vp, C.POINTER(TkvPrefixIndexStats)]),
    "tkv_prefix_index_set_key_bits": (_i32, [_vp, _u32]),
    "tkv_device_page_allocator_create": (_i32, [_i32, _u32, C.POINTER(_vp)]),
    "tkv_device_page_allocator_destroy": (None, [_vp]),
    "tkv_device_page_allocator_allocate": (_i32, [_vp, C.POINTER(TkvPageBatch), _u64, _vp]),
    "tkv_device_page_allocator_free": (_i32, [_vp, C.POINTER(TkvPageBatch), _u64, _vp]),
    "tkv_device_page_allocator_available": (_i32, [_vp, _vp, _u32p]),
    "tkv_handoff_enqueue_device_tables": (_i32, [_vp, C.POINTER(TkvDeviceBatch), _vp, _u64, _u32]),
    "tkv_refcount_apply_device_tables": (_i32, [C.POINTER(TkvPool), C.POINTER(TkvDeviceBatch), _i32, _vp]),
    "tkv_coordinator_new": (_vp, [C.POINTER(TkvCoordinatorConfig)]),
    "tkv_coordinator_delete": (None, [_vp]),
    "tkv_coordinator_set_headroom": (_i32, [_vp, _u32, _u64]),
    "tkv_coordinator_submit": (_i32, [_vp, _u64, _u32, _u32, _u32, _u32p]),
    "tkv_coordinator_next_prefill": (_i32, [_vp, _u32, _u64p]),
    "tkv_coordinator_prefill_done": (_i32, [_vp, _u64, _u32]),
    "tkv_coordinator_admit": (_sz, [_vp, C.POINTER(TkvAdmission), _sz]),
    "tkv_coordinator_handoff_started": (_i32, [_vp, _u64, _u64]),
    "tkv_coordinator_handoff_complete": (_i32, [_vp, _u64]),
    "tkv_coordinator_handoff_failed": (_i32, [_vp, _u64, _u32p]),
    "tkv_coordinator_timed_out": (_sz, [_vp, _u64, _u64p, _sz]),
    "tkv_coordinator_reprefill_done": (_i32, [_vp, _u64]),
    "tkv_coordinator_finish": (_i32, [_vp, _u64]),
    "tkv_coordinator_request": (_i32, [_vp, _u64, C.POINTER(TkvRequestInfo)]),
    "tkv_coordinator_stats": (_i32, [_vp, C.POINTER(TkvCoordinatorStats)]),
    "tkv_radix_tree_new": (_vp, []),
    "tkv_radix_tree_delete": (None, [_vp]),
    "tkv_radix_tree_insert": (None, [_vp, _u32p, _sz, _szp, _sz]),
    "tkv_radix_tree_lookup": (_sz, [_vp, _u32p, _sz, _szp, _sz, _szp]),
    "tkv_radix_tree_release": (None, [_vp, _u32p, _sz]),
    "tkv_radix_tree_evict_lru": (_sz, [_vp, _szp, _sz]),
    "tkv_radix_tree_hit_count": (_u64, [_vp]),
    "tkv_radix_tree_tokens_saved": (_u64, [_vp]),
    "tkv_radix_tree_node_count": (_sz, [_vp]),
    "tkv_prefix_table_new": (_vp, [_sz]),
    "tkv_prefix_table_delete": (None, [_vp]),
    "tkv_prefix_table_store": (None, [_vp, _u32p, _sz, C.c_char_p, _u32p, _sz, _sz]),
    "tkv_prefix_table_probe": (_sz, [_vp, _u32p, _sz, C.c_char_p, _u32p, _sz, _szp]),
    "tkv_prefix_table_release": (None, [_vp, _u32p, _sz, C.c_char_p]),
    "tkv_prefix_table_len": (_sz, [_vp]),
    "tkv_prefix_table_hit_count": (_u64, [_vp]),
    "tkv_prefix_table_tokens_saved": (_u64, [_vp]),
}


def lib() -> C.CDLL:
    """Loads the in-tree ``libtkv.so``; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU fallback for the KV handoff)")
    L = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)          # AttributeError here == header/library drift
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != 0:
        buf = C.create_string_buffer(512)
        lib().tkv_last_error(buf, 512)
        raise TkvError(rc, buf.value.decode(errors="replace"))
