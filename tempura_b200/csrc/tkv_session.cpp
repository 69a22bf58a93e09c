// Wire form of the handoff's metadata: SessionTransfer {cache, position, seed, last_logits}
// (engine/src/session.rs:194-200) with the cache reduced to its geometry and block table,
// for a prefill process and a decode process that do not share an address space.  The
// reference derives serde traits for the struct and fixes no byte format; this one is
// little-endian, self-describing and checksummed, and can be cut into page-granular
// pieces (piece i names blocks [block_begin, block_begin + n_blocks) of the sequence) so a
// long prompt's blocks can be announced and moved as they are produced.  No CUDA here.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/tkv.h"

namespace tkv_internal {
int32_t set_error(int32_t code, int32_t cuda_code, const char* text);
}

namespace {

constexpr uint32_t kMagic = 0x53564B54u;  // "TKVS"
constexpr uint32_t kVersion = 1u;
constexpr size_t kFixed = 8 + sizeof(TkvSessionHeader);  // magic, version, header
constexpr size_t kTrailer = 8;                           // FNV-1a 64 of everything before it

uint64_t fnv1a(const uint8_t* p, size_t n) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (size_t i = 0; i < n; i++) {
        h ^= p[i];
        h *= 0x100000001B3ull;
    }
    return h;
}

int32_t fail(int32_t code, const char* fmt, unsigned long long a = 0, unsigned long long b = 0) {
    char buf[256];
    snprintf(buf, sizeof buf, fmt, a, b);
    return tkv_internal::set_error(code, 0, buf);
}

int32_t check_header(const TkvSessionHeader* h) {
    if (h->kv_dtype > TKV_DTYPE_E4M3) return fail(TKV_ERR_INVALID_CONFIG, "session header: unknown kv dtype %llu", h->kv_dtype);
    if (!h->block_size || !h->n_layers || !h->n_kv_heads || !h->head_dim)
        return fail(TKV_ERR_INVALID_CONFIG, "session header: zero-sized cache geometry");
    const uint64_t total = ((uint64_t)h->seq_len + h->block_size - 1) / h->block_size;
    if ((uint64_t)h->block_begin + h->n_blocks > total)
        return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (blocks named beyond the sequence)", total,
                    (uint64_t)h->block_begin + h->n_blocks);
    if (h->piece_count == 0 || h->piece_index >= h->piece_count)
        return fail(TKV_ERR_INVALID_CONFIG, "session header: piece %llu of %llu", h->piece_index, h->piece_count);
    if (h->position > h->seq_len) return fail(TKV_ERR_INVALID_CONFIG, "session header: position %llu beyond seq_len %llu", h->position, h->seq_len);
    return TKV_OK;
}

}  // namespace

extern "C" {

size_t tkv_session_wire_size(const TkvSessionHeader* h) {
    if (!h) return 0;
    return kFixed + (size_t)h->n_blocks * 4 + (size_t)h->n_logits * 4 + kTrailer;
}

int32_t tkv_session_pack(const TkvSessionHeader* h, const uint32_t* blocks, const float* logits, uint8_t* out, size_t cap,
                         size_t* written) {
    if (!h || !out || !written || (h->n_blocks && !blocks) || (h->n_logits && !logits))
        return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    int32_t rc = check_header(h);
    if (rc) return rc;
    const size_t need = tkv_session_wire_size(h);
    if (cap < need) return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (output buffer bytes)", need, cap);
    uint8_t* p = out;
    memcpy(p, &kMagic, 4);
    memcpy(p + 4, &kVersion, 4);
    memcpy(p + 8, h, sizeof *h);
    p += kFixed;
    memcpy(p, blocks, (size_t)h->n_blocks * 4);
    p += (size_t)h->n_blocks * 4;
    memcpy(p, logits, (size_t)h->n_logits * 4);
    p += (size_t)h->n_logits * 4;
    const uint64_t sum = fnv1a(out, (size_t)(p - out));
    memcpy(p, &sum, 8);
    *written = need;
    return TKV_OK;
}

int32_t tkv_session_unpack(const uint8_t* in, size_t len, TkvSessionHeader* h, const uint32_t** blocks, const float** logits) {
    if (!in || !h || !blocks || !logits) return fail(TKV_ERR_INVALID_CONFIG, "NULL argument");
    if (len < kFixed + kTrailer) return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (message bytes)", kFixed + kTrailer, len);
    uint32_t magic, version;
    memcpy(&magic, in, 4);
    memcpy(&version, in + 4, 4);
    if (magic != kMagic) return fail(TKV_ERR_INVALID_CONFIG, "not a session transfer message (magic %llx)", magic);
    if (version != kVersion) return fail(TKV_ERR_INVALID_CONFIG, "session transfer version %llu, this library reads %llu", version, kVersion);
    TkvSessionHeader tmp;
    memcpy(&tmp, in + 8, sizeof tmp);
    const size_t need = tkv_session_wire_size(&tmp);
    if (len != need) return fail(TKV_ERR_DIMENSION_MISMATCH, "dimension mismatch: expected %llu, got %llu (message bytes)", need, len);
    uint64_t sum;
    memcpy(&sum, in + len - kTrailer, 8);
    if (sum != fnv1a(in, len - kTrailer)) return fail(TKV_ERR_INVALID_CONFIG, "session transfer message is corrupt (checksum)");
    int32_t rc = check_header(&tmp);
    if (rc) return rc;
    *h = tmp;
    *blocks = reinterpret_cast<const uint32_t*>(in + kFixed);
    *logits = reinterpret_cast<const float*>(in + kFixed + (size_t)tmp.n_blocks * 4);
    return TKV_OK;
}

}  // extern "C"
