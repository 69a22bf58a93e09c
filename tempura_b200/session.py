"""The handoff's metadata on the wire: ``SessionTransfer {cache, position, seed, last_logits}``
(engine/src/session.rs:194-200) as the checksummed message of ``tkv_session_pack`` /
``tkv_session_unpack``.  The K/V bytes do not travel in it: the cache is its geometry and the block table
that names its pages in the sender's pool, announced whole or in page-granular pieces.  No CUDA, no torch."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _native as N
from ._native import check, lib


def header(position: int, seed: int, seq_len: int, n_layers: int, n_kv_heads: int, head_dim: int, block_size: int, kv_dtype: int,
           block_begin: int, n_blocks: int, piece_index: int = 0, piece_count: int = 1, n_logits: int = 0) -> N.TkvSessionHeader:
    return N.TkvSessionHeader(position, seed, seq_len, n_layers, n_kv_heads, head_dim, block_size, kv_dtype, block_begin, n_blocks,
                              piece_index, piece_count, n_logits, 0)


def pack(h: N.TkvSessionHeader, blocks, logits=()) -> bytes:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint32)
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    size = lib().tkv_session_wire_size(C.byref(h))
    out = (C.c_uint8 * size)()
    written = C.c_size_t(0)
    check(lib().tkv_session_pack(C.byref(h), blocks.ctypes.data_as(C.POINTER(C.c_uint32)),
                                 logits.ctypes.data_as(C.POINTER(C.c_float)) if logits.size else None, out, size, C.byref(written)))
    return bytes(out[: written.value])


def unpack(msg: bytes) -> Tuple[N.TkvSessionHeader, np.ndarray, np.ndarray]:
    """Raises ``TkvError`` for a truncated, damaged or foreign message."""
    buf = (C.c_uint8 * max(len(msg), 1)).from_buffer_copy(msg if msg else b"\0")
    h = N.TkvSessionHeader()
    bp, lp = C.POINTER(C.c_uint32)(), C.POINTER(C.c_float)()
    check(lib().tkv_session_unpack(buf, len(msg), C.byref(h), C.byref(bp), C.byref(lp)))
    blocks = np.ctypeslib.as_array(bp, (h.n_blocks,)).copy() if h.n_blocks else np.zeros(0, np.uint32)
    logits = np.ctypeslib.as_array(lp, (h.n_logits,)).copy() if h.n_logits else np.zeros(0, np.float32)
    return h, blocks, logits


def pack_batch(seq_lens: Sequence[int], tables: np.ndarray, n_layers: int, n_kv_heads: int, head_dim: int, block_size: int, kv_dtype: int,
               seeds: Optional[Sequence[int]] = None, pieces: int = 1) -> List[bytes]:
    """One message per sequence (or ``pieces`` page-granular messages each): what a prefill worker announces for a
    batch of finished prompts.  ``tables[q]`` holds sequence q's block ids in the sender's pool."""
    out = []
    for q, length in enumerate(seq_lens):
        length = int(length)
        nb = (length + block_size - 1) // block_size
        cuts = np.linspace(0, nb, min(pieces, max(nb, 1)) + 1).astype(int)
        for i in range(len(cuts) - 1):
            b0, b1 = int(cuts[i]), int(cuts[i + 1])
            h = header(length, int(seeds[q]) if seeds is not None else q, length, n_layers, n_kv_heads, head_dim, block_size, kv_dtype,
                       b0, b1 - b0, i, len(cuts) - 1)
            out.append(pack(h, tables[q, b0:b1]))
    return out


def frame(messages: Sequence[bytes]) -> bytes:
    """Length-prefixed concatenation, so that a batch of messages can cross a byte stream."""
    return b"".join(len(m).to_bytes(4, "little") + m for m in messages)


def unframe(stream: bytes) -> List[bytes]:
    out, at = [], 0
    while at < len(stream):
        n = int.from_bytes(stream[at:at + 4], "little")
        out.append(stream[at + 4:at + 4 + n])
        at += 4 + n
    return out
