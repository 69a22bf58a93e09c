/*
 * x86_f16c_check.c -- TEST INFRASTRUCTURE ONLY.
 * Exposes the two x86 F16C conversions the reference calls directly
 * (engine/src/kv_cache.rs:29-67: _mm_cvtps_ph with _MM_FROUND_TO_NEAREST_INT,
 * _mm_cvtph_ps) so a test can sweep them against the portable restatement in
 * tkv_oracle.c.  Built only when the compiler targets F16C; otherwise the
 * probe reports "absent" and the test skips.
 */
#include <stdint.h>
#include <string.h>
#if defined(__F16C__)
#include <immintrin.h>
int orc_have_f16c(void) { return 1; }
uint16_t orc_hw_f32_to_f16(float x) {
    __m128 v = _mm_set_ss(x);
    __m128i h = _mm_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT);
    return (uint16_t)_mm_extract_epi16(h, 0);
}
float orc_hw_f16_to_f32(uint16_t h) {
    __m128i v = _mm_set1_epi16((short)h);
    return _mm_cvtss_f32(_mm_cvtph_ps(v));
}
/* sweeps every f32 whose low `skip_bits` bits are zero; returns mismatches */
uint64_t orc_sweep_f32_to_f16(uint16_t (*soft)(float), unsigned skip_bits) {
    uint64_t bad = 0;
    for (uint64_t b = 0; b < (1ull << 32); b += (1ull << skip_bits)) {
        uint32_t u = (uint32_t)b;
        float x;
        memcpy(&x, &u, 4);
        if (soft(x) != orc_hw_f32_to_f16(x)) bad++;
    }
    return bad;
}
#else
int orc_have_f16c(void) { return 0; }
uint16_t orc_hw_f32_to_f16(float x) { (void)x; return 0; }
float orc_hw_f16_to_f32(uint16_t h) { (void)h; return 0.0f; }
uint64_t orc_sweep_f32_to_f16(uint16_t (*soft)(float), unsigned skip_bits) { (void)soft; (void)skip_bits; return 0; }
#endif
