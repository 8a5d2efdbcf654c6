// AVX-512 VNNI row dots (256-bit vpdpbusd through AVX-512VL) for Q4_K, Q5_K, Q6_K, Q8_0 and Q8_F32 rows against q8
// activations: one vpdpbusd replaces the vpmaddubsw + vpmaddwd pair of the AVX2 paths and cannot saturate.  Compiled
// with per-function target attributes and picked at run time (__builtin_cpu_supports), so the library still loads on
// a CPU without these instructions.  Same values as the scalar units up to fp32 summation order.  Counterpart of the
// reference's VNNI kernels in crates/qdot (src/lib.rs: dispatch by CPU feature, per-type row dots).
#pragma once
#include <immintrin.h>
#include <stdint.h>

#include "../quant_units.cuh"
#include "qdot_avx2.h"

namespace blh {

#if defined(__x86_64__) && defined(__AVX2__)
#define BLH_VNNI __attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni,avx2,fma")))

static inline bool cpu_has_vnni() {
  static const bool has = __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512vl") &&
                          __builtin_cpu_supports("avx512bw");
  return has;
}

BLH_VNNI static inline void k_scales(const uint8_t* s, int* sc, int* mn) {
  for (int i = 0; i < 4; ++i) {
    sc[i] = s[i] & 63; mn[i] = s[4 + i] & 63;
    sc[4 + i] = (s[8 + i] & 0xF) | ((s[i] >> 6) << 4);
    mn[4 + i] = (s[8 + i] >> 4) | ((s[4 + i] >> 6) << 4);
  }
}

BLH_VNNI static inline float row_dot_q4k_vnni(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  const __m256i m4 = _mm256_set1_epi8(0x0F), zero = _mm256_setzero_si256();
  __m256 acc = _mm256_setzero_ps();
  float mins = 0.f;
  for (int sb = 0; sb < K / 256; ++sb) {
    const uint8_t* p = row + (long)sb * 144;
    const float d = bl::half_bits_to_float((uint16_t)(p[0] | (p[1] << 8)));
    const float dmin = bl::half_bits_to_float((uint16_t)(p[2] | (p[3] << 8)));
    int sc[8], mn[8];
    k_scales(p + 4, sc, mn);
    const float* ds = xds + (long)sb * 16;
    const int8_t* a = xq + (long)sb * 256;
    for (int j = 0; j < 4; ++j) {
      const __m256i q = _mm256_loadu_si256((const __m256i*)(p + 16 + 32 * j));
      const __m256i lo = _mm256_and_si256(q, m4), hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), m4);
      const __m256i a0 = _mm256_loadu_si256((const __m256i*)(a + 64 * j)), a1 = _mm256_loadu_si256((const __m256i*)(a + 64 * j + 32));
      const __m256i p0 = _mm256_dpbusd_epi32(zero, lo, a0), p1 = _mm256_dpbusd_epi32(zero, hi, a1);
      acc = _mm256_fmadd_ps(_mm256_set1_ps(d * (float)sc[2 * j] * ds[2 * (2 * j)]), _mm256_cvtepi32_ps(p0), acc);
      acc = _mm256_fmadd_ps(_mm256_set1_ps(d * (float)sc[2 * j + 1] * ds[2 * (2 * j + 1)]), _mm256_cvtepi32_ps(p1), acc);
      mins += dmin * ((float)mn[2 * j] * ds[2 * (2 * j) + 1] + (float)mn[2 * j + 1] * ds[2 * (2 * j + 1) + 1]);
    }
  }
  return hsum8(acc) - mins;
}

// Q5_K super-block of 176 bytes: d, dmin, scales[12], qh[32], qs[128]; bit 2j / 2j + 1 of qh[i] is the fifth bit of the
// low / high nibble of qs[32 j + i]
BLH_VNNI static inline float row_dot_q5k_vnni(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  const __m256i m4 = _mm256_set1_epi8(0x0F), m1 = _mm256_set1_epi8(1), zero = _mm256_setzero_si256();
  __m256 acc = _mm256_setzero_ps();
  float mins = 0.f;
  for (int sb = 0; sb < K / 256; ++sb) {
    const uint8_t* p = row + (long)sb * 176;
    const float d = bl::half_bits_to_float((uint16_t)(p[0] | (p[1] << 8)));
    const float dmin = bl::half_bits_to_float((uint16_t)(p[2] | (p[3] << 8)));
    int sc[8], mn[8];
    k_scales(p + 4, sc, mn);
    const __m256i qh = _mm256_loadu_si256((const __m256i*)(p + 16));
    const float* ds = xds + (long)sb * 16;
    const int8_t* a = xq + (long)sb * 256;
    for (int j = 0; j < 4; ++j) {
      const __m256i q = _mm256_loadu_si256((const __m256i*)(p + 48 + 32 * j));
      const __m256i h0 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2 * j), m1), 4);
      const __m256i h1 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2 * j + 1), m1), 4);
      const __m256i lo = _mm256_or_si256(_mm256_and_si256(q, m4), h0);
      const __m256i hi = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(q, 4), m4), h1);
      const __m256i a0 = _mm256_loadu_si256((const __m256i*)(a + 64 * j)), a1 = _mm256_loadu_si256((const __m256i*)(a + 64 * j + 32));
      const __m256i p0 = _mm256_dpbusd_epi32(zero, lo, a0), p1 = _mm256_dpbusd_epi32(zero, hi, a1);
      acc = _mm256_fmadd_ps(_mm256_set1_ps(d * (float)sc[2 * j] * ds[2 * (2 * j)]), _mm256_cvtepi32_ps(p0), acc);
      acc = _mm256_fmadd_ps(_mm256_set1_ps(d * (float)sc[2 * j + 1] * ds[2 * (2 * j + 1)]), _mm256_cvtepi32_ps(p1), acc);
      mins += dmin * ((float)mn[2 * j] * ds[2 * (2 * j) + 1] + (float)mn[2 * j + 1] * ds[2 * (2 * j + 1) + 1]);
    }
  }
  return hsum8(acc) - mins;
}

// resident Q6_K super-block of 224 bytes: ql[128] qh[64] sc[16] d pad.  Per 16 values: scale * (sum q a - 32 sum a).
BLH_VNNI static inline float row_dot_q6k_vnni(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  const __m256i m4 = _mm256_set1_epi8(0x0F), m2 = _mm256_set1_epi8(0x03), one8 = _mm256_set1_epi8(1), zero = _mm256_setzero_si256();
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
        const __m256i av = _mm256_loadu_si256((const __m256i*)(a + 128 * n + 32 * g));
        const __m256i qa = _mm256_dpbusd_epi32(zero, q[g], av);                 // 8 sums of 4 products q * a
        const __m256i sa = _mm256_dpbusd_epi32(zero, one8, av);                 // 8 sums of 4 activations
        const __m256i t = _mm256_sub_epi32(qa, _mm256_slli_epi32(sa, 5));       // sum (q - 32) a
        // lanes 0..3 cover values 0..15 (scale 8n + 2g), lanes 4..7 values 16..31 (scale 8n + 2g + 1)
        const __m256i sv = _mm256_set_m128i(_mm_set1_epi32(sc[8 * n + 2 * g + 1]), _mm_set1_epi32(sc[8 * n + 2 * g]));
        acc = _mm256_fmadd_ps(_mm256_set1_ps(d * ds[2 * (4 * n + g)]), _mm256_cvtepi32_ps(_mm256_mullo_epi32(t, sv)), acc);
      }
    }
  }
  return hsum8(acc);
}

// int8 codes with f16 (Q8_0) or f32 (Q8_F32) scales after the codes; signed x signed through |w| and sign(a, w)
BLH_VNNI static inline float row_dot_q8_vnni(const uint8_t* row, int K, const int8_t* xq, const float* xds, bool f32_scales) {
  const __m256i zero = _mm256_setzero_si256();
  __m256 acc = _mm256_setzero_ps();
  const uint8_t* sc = row + K;
  for (int b = 0; b < K / 32; ++b) {
    const __m256i w = _mm256_loadu_si256((const __m256i*)(row + 32 * b));
    const __m256i av = _mm256_loadu_si256((const __m256i*)(xq + 32 * b));
    const __m256i pr = _mm256_dpbusd_epi32(zero, _mm256_abs_epi8(w), _mm256_sign_epi8(av, w));
    float dw;
    if (f32_scales) __builtin_memcpy(&dw, sc + 4 * b, 4);
    else dw = bl::half_bits_to_float((uint16_t)(sc[2 * b] | (sc[2 * b + 1] << 8)));
    acc = _mm256_fmadd_ps(_mm256_set1_ps(dw * xds[2 * b]), _mm256_cvtepi32_ps(pr), acc);
  }
  return hsum8(acc);
}

// true and the dot in *out when a VNNI path serves this type on this CPU
static inline bool row_dot_vnni(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds, float* out) {
  if (!cpu_has_vnni()) return false;
  switch (wtype) {
    case bl::WT_Q4_K: if (K % 256) return false; *out = row_dot_q4k_vnni(row, K, xq, xds); return true;
    case bl::WT_Q5_K: if (K % 256) return false; *out = row_dot_q5k_vnni(row, K, xq, xds); return true;
    case bl::WT_Q6_K: if (K % 256) return false; *out = row_dot_q6k_vnni(row, K, xq, xds); return true;
    case bl::WT_Q8_0: if (K % 32) return false; *out = row_dot_q8_vnni(row, K, xq, xds, false); return true;
    case bl::WT_Q8_F32: if (K % 32) return false; *out = row_dot_q8_vnni(row, K, xq, xds, true); return true;
  }
  return false;
}
#else
static inline bool cpu_has_vnni() { return false; }
static inline bool row_dot_vnni(int, const uint8_t*, int, const int8_t*, const float*, float*) { return false; }
#endif

}  // namespace blh
