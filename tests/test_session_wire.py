"""SessionTransfer metadata on the wire (engine/src/session.rs:194-200): position, seed,
last logits, cache geometry and block table survive a pack / unpack round trip, pieces name
block ranges, and damaged or truncated messages are refused with the reference's error
classes.  Host logic only."""
import ctypes as C

import numpy as np
import pytest

from tempura_b200 import _build, _native as N


@pytest.fixture(scope="module")
def L():
    _build.build()
    return N.lib()


def header(**kw):
    base = dict(position=35, seed=42, seq_len=35, n_layers=32, n_kv_heads=8, head_dim=128, block_size=16,
                kv_dtype=N.DTYPE_F16, block_begin=0, n_blocks=3, piece_index=0, piece_count=1, n_logits=0, reserved=0)
    base.update(kw)
    return N.TkvSessionHeader(**base)


def pack(L, h, blocks, logits):
    blocks = np.ascontiguousarray(blocks, dtype=np.uint32)
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    size = L.tkv_session_wire_size(C.byref(h))
    out = (C.c_uint8 * size)()
    written = C.c_size_t(0)
    N.check(L.tkv_session_pack(C.byref(h), blocks.ctypes.data_as(C.POINTER(C.c_uint32)),
                               logits.ctypes.data_as(C.POINTER(C.c_float)), out, size, C.byref(written)))
    assert written.value == size
    return bytes(out)


def unpack(L, msg):
    buf = (C.c_uint8 * len(msg)).from_buffer_copy(msg)
    h = N.TkvSessionHeader()
    bp, lp = C.POINTER(C.c_uint32)(), C.POINTER(C.c_float)()
    N.check(L.tkv_session_unpack(buf, len(msg), C.byref(h), C.byref(bp), C.byref(lp)))
    blocks = np.ctypeslib.as_array(bp, (h.n_blocks,)).copy() if h.n_blocks else np.zeros(0, np.uint32)
    logits = np.ctypeslib.as_array(lp, (h.n_logits,)).copy() if h.n_logits else np.zeros(0, np.float32)
    return h, blocks, logits


def test_round_trip_matches_reference_fields(L):
    # engine/src/disaggregated.rs:292-303: position 3, seed 42, seq_len 3, vocab_size logits
    rng = np.random.default_rng(0)
    logits = rng.standard_normal(128256).astype(np.float32)
    h = header(position=3, seq_len=3, n_blocks=1, n_logits=logits.size)
    msg = pack(L, h, [977], logits)
    assert len(msg) == 8 + 64 + 4 + 4 * logits.size + 8
    g, blocks, got = unpack(L, msg)
    assert (g.position, g.seed, g.seq_len, g.n_layers, g.n_kv_heads, g.head_dim) == (3, 42, 3, 32, 8, 128)
    assert blocks.tolist() == [977] and np.array_equal(got.view(np.uint32), logits.view(np.uint32))


def test_page_granular_pieces(L):
    table = np.arange(100, 110, dtype=np.uint32)            # 10 blocks = 150 tokens
    pieces = []
    for i, (b0, n) in enumerate(((0, 4), (4, 4), (8, 2))):
        h = header(position=150, seq_len=150, block_begin=b0, n_blocks=n, piece_index=i, piece_count=3,
                   n_logits=5 if i == 2 else 0)
        pieces.append(pack(L, h, table[b0:b0 + n], np.arange(5, dtype=np.float32) if i == 2 else []))
    rebuilt = np.zeros(10, dtype=np.uint32)
    for msg in reversed(pieces):                             # any arrival order
        g, blocks, logits = unpack(L, msg)
        rebuilt[g.block_begin:g.block_begin + g.n_blocks] = blocks
        assert (logits.size == 5) == (g.piece_index == 2)
    assert np.array_equal(rebuilt, table)


def test_damaged_and_truncated_messages_are_refused(L):
    msg = bytearray(pack(L, header(), [1, 2, 3], []))
    with pytest.raises(N.TkvError) as e:
        unpack(L, bytes(msg[:-1]))
    assert e.value.code == N.ERR_DIMENSION_MISMATCH
    flipped = bytearray(msg)
    flipped[80] ^= 0x10                                       # inside the block table
    with pytest.raises(N.TkvError) as e:
        unpack(L, bytes(flipped))
    assert e.value.code == N.ERR_INVALID_CONFIG and "corrupt" in e.value.message
    wrong = bytearray(msg)
    wrong[0] = ord("X")
    with pytest.raises(N.TkvError) as e:
        unpack(L, bytes(wrong))
    assert e.value.code == N.ERR_INVALID_CONFIG
    with pytest.raises(N.TkvError):
        unpack(L, b"short")


def test_header_rules(L):
    with pytest.raises(N.TkvError) as e:
        pack(L, header(n_blocks=4), [1, 2, 3, 4], [])           # 35 tokens are 3 blocks
    assert e.value.code == N.ERR_DIMENSION_MISMATCH
    for bad in (dict(block_size=0), dict(kv_dtype=7), dict(piece_index=1), dict(position=36)):
        with pytest.raises(N.TkvError) as e:
            pack(L, header(**bad), [1, 2, 3], [])
        assert e.value.code == N.ERR_INVALID_CONFIG
    h = header()
    out = (C.c_uint8 * 16)()
    written = C.c_size_t(0)
    blocks = np.array([1, 2, 3], dtype=np.uint32)
    rc = L.tkv_session_pack(C.byref(h), blocks.ctypes.data_as(C.POINTER(C.c_uint32)), None, out, 16, C.byref(written))
    assert rc == N.ERR_DIMENSION_MISMATCH
