// AVX2 row dots for the Q4_K_M type mix (Q4_K, Q6_K, Q8_0) against q8 activations: the integer
// products run on vpmaddubsw / vpmaddwd, each 32-value activation block's integer sums are scaled
// in a float vector accumulator, one horizontal sum per row.  Same values as the scalar units up
// to fp32 summation order.  Counterpart of the reference's AVX2 kernels in crates/qdot
// (per-type row dots against quantised activations with no f32 materialisation).
#pragma once
#include <immintrin.h>
#include <stdint.h>

#include "../quant_units.cuh"

namespace blh {

#if defined(__AVX2__)
static inline float hsum8(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  return _mm_cvtss_f32(lo);
}

// row: K/256 super-blocks of 144 bytes (d, dmin, scales[12], qs[128]); xq: K codes; xds: {d, d*sum} per 32
static inline float row_dot_q4k_avx2(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  const __m256i m4 = _mm256_set1_epi8(0x0F), ones = _mm256_set1_epi16(1);
  __m256 acc = _mm256_setzero_ps();
  float mins = 0.f;
  for (int sb = 0; sb < K / 256; ++sb) {
    const uint8_t* p = row + (long)sb * 144;
    const float d = bl::half_bits_to_float((uint16_t)(p[0] | (p[1] << 8)));
    const float dmin = bl::half_bits_to_float((uint16_t)(p[2] | (p[3] << 8)));
    const uint8_t* s = p + 4;
    int sc[8], mn[8];
    for (int i = 0; i < 4; ++i) {
      sc[i] = s[i] & 63; mn[i] = s[4 + i] & 63;
      sc[4 + i] = (s[8 + i] & 0xF) | ((s[i] >> 6) << 4);
      mn[4 + i] = (s[8 + i] >> 4) | ((s[4 + i] >> 6) << 4);
    }
    const float* ds = xds + (long)sb * 16;
    const int8_t* a = xq + (long)sb * 256;
    for (int j = 0; j < 4; ++j) {
      const __m256i q = _mm256_loadu_si256((const __m256i*)(p + 16 + 32 * j));
      const __m256i lo = _mm256_and_si256(q, m4), hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), m4);
      const __m256i a0 = _mm256_loadu_si256((const __m256i*)(a + 64 * j)), a1 = _mm256_loadu_si256((const __m256i*)(a + 64 * j + 32));
      const __m256i p0 = _mm256_madd_epi16(_mm256_maddubs_epi16(lo, a0), ones);
      const __m256i p1 = _mm256_madd_epi16(_mm256_maddubs_epi16(hi, a1), ones);
      acc = _mm256_fmadd_ps(_mm256_set1_ps(d * (float)sc[2 * j] * ds[2 * (2 * j)]), _mm256_cvtepi32_ps(p0), acc);
      acc = _mm256_fmadd_ps(_mm256_set1_ps(d * (float)sc[2 * j + 1] * ds[2 * (2 * j + 1)]), _mm256_cvtepi32_ps(p1), acc);
      mins += dmin * ((float)mn[2 * j] * ds[2 * (2 * j) + 1] + (float)mn[2 * j + 1] * ds[2 * (2 * j + 1) + 1]);
    }
  }
  return hsum8(acc) - mins;
}

// resident Q6_K super-block of 224 bytes: ql[128] qh[64] sc[16] d pad
static inline float row_dot_q6k_avx2(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  const __m256i m4 = _mm256_set1_epi8(0x0F), m2 = _mm256_set1_epi8(0x03), one8 = _mm256_set1_epi8(1);
  __m256 acc = _mm256_setzero_ps();
  for (int sb = 0; sb < K / 256; ++sb) {
    const uint8_t* p = row + (long)sb * 224;
    const int8_t* sc = (const int8_t*)(p + 192);
    const float d = bl::half_bits_to_float((uint16_t)(p[208] | (p[209] << 8)));
    const float* ds = xds + (long)sb * 16;
    const int8_t* a = xq + (long)sb * 256;
    for (int n = 0; n < 2; ++n) {
      const __m256i l0 = _mm256_loadu_si256((const __m256i*)(p + 64 * n)), l1 = _mm256_loadu_si256((const __m256i*)(p + 64 * n + 32));
      const __m256i h = _mm256_loadu_si256((const __m256i*)(p + 128 + 32 * n));
      __m256i q[4];
      q[0] = _mm256_or_si256(_mm256_and_si256(l0, m4), _mm256_slli_epi16(_mm256_and_si256(h, m2), 4));
      q[1] = _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4));
      q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4));
      q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4));
      for (int g = 0; g < 4; ++g) {
        // values 128n + 32g .. +31 = activation block 4n + g; the two 16-value halves have scales 8n + 2g, 8n + 2g + 1
        const __m256i av = _mm256_loadu_si256((const __m256i*)(a + 128 * n + 32 * g));
        const int s0 = sc[8 * n + 2 * g], s1 = sc[8 * n + 2 * g + 1];
        const __m256i sv = _mm256_set_m128i(_mm_set1_epi16((short)s1), _mm_set1_epi16((short)s0));
        const __m256i qa = _mm256_maddubs_epi16(q[g], av);            // pairs q*a (q in 0..63)
        const __m256i sa = _mm256_maddubs_epi16(one8, av);            // pairs of a
        const __m256i t = _mm256_sub_epi16(qa, _mm256_slli_epi16(sa, 5));   // (q - 32) * a per pair, fits 16 bits
        const __m256i ps = _mm256_madd_epi16(t, sv);                  // times the group scale, summed to 32 bits
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d * ds[2 * (4 * n + g)]), _mm256_cvtepi32_ps(ps), acc);
      }
    }
  }
  return hsum8(acc);
}

// resident Q8_0 row: K codes then K/32 f16 scales
static inline float row_dot_q80_avx2(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  const __m256i ones = _mm256_set1_epi16(1);
  __m256 acc = _mm256_setzero_ps();
  const uint8_t* sc = row + K;
  for (int b = 0; b < K / 32; ++b) {
    const __m256i w = _mm256_loadu_si256((const __m256i*)(row + 32 * b));
    const __m256i av = _mm256_loadu_si256((const __m256i*)(xq + 32 * b));
    const __m256i p = _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_sign_epi8(w, w), _mm256_sign_epi8(av, w)), ones);
    const float dw = bl::half_bits_to_float((uint16_t)(sc[2 * b] | (sc[2 * b + 1] << 8)));
    acc = _mm256_fmadd_ps(_mm256_set1_ps(dw * xds[2 * b]), _mm256_cvtepi32_ps(p), acc);
  }
  return hsum8(acc);
}

// true and the dot in *out when a vector path serves this type
static inline bool row_dot_fast(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds, float* out) {
  if (K % 256) return false;
  switch (wtype) {
    case bl::WT_Q4_K: *out = row_dot_q4k_avx2(row, K, xq, xds); return true;
    case bl::WT_Q6_K: *out = row_dot_q6k_avx2(row, K, xq, xds); return true;
    case bl::WT_Q8_0: *out = row_dot_q80_avx2(row, K, xq, xds); return true;
  }
  return false;
}
#else
static inline bool row_dot_fast(int, const uint8_t*, int, const int8_t*, const float*, float*) { return false; }
#endif

}  // namespace blh
