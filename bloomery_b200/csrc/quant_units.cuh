// Weight "units": 64 consecutive values of one weight row, decoded in registers and
// dotted against the q8 activation form (int8 codes + {d, d*sum} per 32 values).
//
// The same code compiles for the device (sm_100a, dp4a) and for the host (scalar
// mirror used by the CPU engine and by the CPU tests), which is how the byte-level
// decode is checked without a GPU.  The reference keeps per-type device dots in
// crates/gpu/src/lib.rs (q4k_gemv, q6k_gemv), crates/gpu/src/kquant/*.rs and
// crates/gpu/src/q5.rs, and their CPU twins in crates/qdot/src/lib.rs.
//
// Resident layouts (what sits in HBM; values are never re-quantised, only re-laid):
//   Q4_K  the file's 144-byte superblocks, unchanged (16-byte aligned)
//   Q5_K  the file's 176-byte superblocks, unchanged
//   Q6_K  224-byte superblocks: ql[128] qh[64] scales[16] d(f16) pad[14]
//   Q8_0  per row: K int8 codes, then K/32 f16 scales, padded to 16 bytes
//   F16/BF16/F32 rows unchanged
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#define BL_HD __host__ __device__ __forceinline__
#else
#define BL_HD inline
#endif

namespace bl {

enum WType : int {
  WT_F32 = 0,
  WT_F16 = 1,
  WT_Q4_0 = 2,
  WT_Q4_1 = 3,
  WT_Q5_0 = 6,
  WT_Q5_1 = 7,
  WT_Q8_0 = 8,
  WT_Q2_K = 10,
  WT_Q3_K = 11,
  WT_Q4_K = 12,
  WT_Q5_K = 13,
  WT_Q6_K = 14,
  WT_BF16 = 30,
  WT_NVFP4 = 40,     // resident rows: K/2 code bytes, K/16 e4m3 scales, f32 tensor scale, pad to 16
  WT_FP8_B128 = 41,  // resident rows: K e4m3 codes, K/128 f32 scales (the 128x128 block scale, per row), pad to 16
  WT_Q8_F32 = 50,    // resident rows: K int8 codes, K/32 f32 scales, pad to 16 (IQ4_NL / IQ4_XS / MXFP4 / IQ2_XXS files land here)
};

struct u32x4 { uint32_t x, y, z, w; };

BL_HD int dot4(uint32_t a, uint32_t b, int c) {
#if defined(__CUDA_ARCH__)
  return __dp4a((int)a, (int)b, c);
#else
  for (int i = 0; i < 4; ++i) c += (int)(int8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
  return c;
#endif
}

// unsigned a (0..255 per byte) times signed b
BL_HD int dot4_us(uint32_t a, uint32_t b, int c) {
#if defined(__CUDA_ARCH__)
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
#else
  for (int i = 0; i < 4; ++i) c += (int)(uint8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
  return c;
#endif
}

BL_HD float half_bits_to_float(uint16_t h) {
#if defined(__CUDA_ARCH__)
  return __half2float(__ushort_as_half(h));
#else
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  __builtin_memcpy(&f, &bits, 4);
  return f;
#endif
}

BL_HD uint32_t ld32(const uint8_t* p) {
#if defined(__CUDA_ARCH__)
  return *reinterpret_cast<const uint32_t*>(p);
#else
  uint32_t v; __builtin_memcpy(&v, p, 4); return v;
#endif
}

BL_HD u32x4 ld128(const uint8_t* p) {
#if defined(__CUDA_ARCH__) && defined(BL_UNITS_GENERIC_LD)
  // a translation unit that reads weight units out of shared memory defines BL_UNITS_GENERIC_LD: a plain
  // load works in every address space, the read-only-cache load below only in global memory
  uint4 v = *reinterpret_cast<const uint4*>(p);
  return u32x4{v.x, v.y, v.z, v.w};
#elif defined(__CUDA_ARCH__)
  uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  return u32x4{v.x, v.y, v.z, v.w};
#else
  u32x4 v; __builtin_memcpy(&v, p, 16); return v;
#endif
}

// activation view for one unit: 64 codes (16 words) and the two {d, s} pairs
struct ActUnit {
  const uint32_t* q;   // 16 words, 16-byte aligned
  float d0, s0, d1, s1;
};

// ---------------------------------------------------------------------------------
// Q4_K
// ---------------------------------------------------------------------------------
struct Q4K {
  static constexpr int kType = WT_Q4_K;
  static constexpr int kSbBytes = 144;
  struct Regs { u32x4 q0, q1; uint32_t s0, s1, s2, dm; };
  static BL_HD long row_bytes(int K) { return (long)(K / 256) * kSbBytes; }
  // unit u of a row: superblock u/4, 64-value pair u%4
  static BL_HD void load(const uint8_t* row, int u, Regs& r) {
    const uint8_t* p = row + (long)(u >> 2) * kSbBytes;
    int j = u & 3;
    r.q0 = ld128(p + 16 + 32 * j);
    r.q1 = ld128(p + 32 + 32 * j);
    r.dm = ld32(p);
    r.s0 = ld32(p + 4); r.s1 = ld32(p + 8); r.s2 = ld32(p + 12);
  }
  static BL_HD void scale_min(const Regs& r, int i, int& sc, int& mn) {
    // 6-bit (scale, min) pair i of 8 from the 12 packed bytes
    int b = i & 3;
    uint32_t q_lo = (r.s0 >> (8 * b)) & 0xFF;     // bytes 0..3
    uint32_t q_mid = (r.s1 >> (8 * b)) & 0xFF;    // bytes 4..7
    uint32_t q_hi = (r.s2 >> (8 * b)) & 0xFF;     // bytes 8..11
    if (i < 4) { sc = q_lo & 63; mn = q_mid & 63; }
    else { sc = (q_hi & 0xF) | ((q_lo >> 6) << 4); mn = (q_hi >> 4) | ((q_mid >> 6) << 4); }
  }
  static BL_HD float dot(const Regs& r, int u, const ActUnit& a) {
    int j = u & 3;
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = dot4_us(w[i] & 0x0F0F0F0Fu, a.q[i], lo);
      hi = dot4_us((w[i] >> 4) & 0x0F0F0F0Fu, a.q[8 + i], hi);
    }
    int sc0, mn0, sc1, mn1;
    scale_min(r, 2 * j, sc0, mn0);
    scale_min(r, 2 * j + 1, sc1, mn1);
    float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF));
    float dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    float pos = a.d0 * (float)(sc0 * lo) + a.d1 * (float)(sc1 * hi);
    float neg = a.s0 * (float)mn0 + a.s1 * (float)mn1;
    return d * pos - dmin * neg;
  }
  // decode the unit's 64 values (for the embedding gather and the bf16 expander)
  static BL_HD void decode(const Regs& r, int u, float* out) {
    int j = u & 3;
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
    int sc0, mn0, sc1, mn1;
    scale_min(r, 2 * j, sc0, mn0);
    scale_min(r, 2 * j + 1, sc1, mn1);
    float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF));
    float dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    float d0 = d * sc0, m0 = dmin * mn0, d1 = d * sc1, m1 = dmin * mn1;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        uint32_t byte = (w[i] >> (8 * b)) & 0xFF;
        out[4 * i + b] = d0 * (float)(byte & 0xF) - m0;
        out[32 + 4 * i + b] = d1 * (float)(byte >> 4) - m1;
      }
  }
};

// ---------------------------------------------------------------------------------
// Q5_K
// ---------------------------------------------------------------------------------
struct Q5K {
  static constexpr int kType = WT_Q5_K;
  static constexpr int kSbBytes = 176;
  struct Regs { u32x4 q0, q1, h0, h1; uint32_t s0, s1, s2, dm; };
  static BL_HD long row_bytes(int K) { return (long)(K / 256) * kSbBytes; }
  static BL_HD void load(const uint8_t* row, int u, Regs& r) {
    const uint8_t* p = row + (long)(u >> 2) * kSbBytes;
    int j = u & 3;
    r.dm = ld32(p);
    r.s0 = ld32(p + 4); r.s1 = ld32(p + 8); r.s2 = ld32(p + 12);
    r.h0 = ld128(p + 16); r.h1 = ld128(p + 32);
    r.q0 = ld128(p + 48 + 32 * j);
    r.q1 = ld128(p + 64 + 32 * j);
  }
  static BL_HD void codes(const Regs& r, int u, uint32_t* lo5, uint32_t* hi5) {
    int j = u & 3;
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
    const uint32_t h[8] = {r.h0.x, r.h0.y, r.h0.z, r.h0.w, r.h1.x, r.h1.y, r.h1.z, r.h1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t hb0 = (h[i] >> (2 * j)) & 0x01010101u;
      uint32_t hb1 = (h[i] >> (2 * j + 1)) & 0x01010101u;
      lo5[i] = (w[i] & 0x0F0F0F0Fu) | (hb0 << 4);
      hi5[i] = ((w[i] >> 4) & 0x0F0F0F0Fu) | (hb1 << 4);
    }
  }
  static BL_HD float dot(const Regs& r, int u, const ActUnit& a) {
    int j = u & 3;
    uint32_t l5[8], h5[8];
    codes(r, u, l5, h5);
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = dot4_us(l5[i], a.q[i], lo);
      hi = dot4_us(h5[i], a.q[8 + i], hi);
    }
    Q4K::Regs t; t.s0 = r.s0; t.s1 = r.s1; t.s2 = r.s2;
    int sc0, mn0, sc1, mn1;
    Q4K::scale_min(t, 2 * j, sc0, mn0);
    Q4K::scale_min(t, 2 * j + 1, sc1, mn1);
    float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF));
    float dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    float pos = a.d0 * (float)(sc0 * lo) + a.d1 * (float)(sc1 * hi);
    float neg = a.s0 * (float)mn0 + a.s1 * (float)mn1;
    return d * pos - dmin * neg;
  }
  static BL_HD void decode(const Regs& r, int u, float* out) {
    int j = u & 3;
    uint32_t l5[8], h5[8];
    codes(r, u, l5, h5);
    Q4K::Regs t; t.s0 = r.s0; t.s1 = r.s1; t.s2 = r.s2;
    int sc0, mn0, sc1, mn1;
    Q4K::scale_min(t, 2 * j, sc0, mn0);
    Q4K::scale_min(t, 2 * j + 1, sc1, mn1);
    float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF));
    float dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    float d0 = d * sc0, m0 = dmin * mn0, d1 = d * sc1, m1 = dmin * mn1;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        out[4 * i + b] = d0 * (float)((l5[i] >> (8 * b)) & 0xFF) - m0;
        out[32 + 4 * i + b] = d1 * (float)((h5[i] >> (8 * b)) & 0xFF) - m1;
      }
  }
};

// ---------------------------------------------------------------------------------
// Q6_K (resident 224-byte superblocks)
// ---------------------------------------------------------------------------------
// Unit u of a superblock: half n = (u>>1)&1, 16-lane slice h = u&1.  It covers four
// runs of 16 values at 128n + 32g + 16h (g = 0..3); the activation gather below
// presents them to `dot` as if they were 64 consecutive values.
struct Q6K {
  static constexpr int kType = WT_Q6_K;
  static constexpr int kSbBytes = 224;
  static constexpr int kFileSbBytes = 210;
  struct Regs { u32x4 la, lb, h; uint32_t sc[4]; uint32_t d; };
  static BL_HD long row_bytes(int K) { return (long)(K / 256) * kSbBytes; }
  static BL_HD void load(const uint8_t* row, int u, Regs& r) {
    const uint8_t* p = row + (long)(u >> 2) * kSbBytes;
    int n = (u >> 1) & 1, h = u & 1;
    r.la = ld128(p + 64 * n + 16 * h);
    r.lb = ld128(p + 64 * n + 32 + 16 * h);
    r.h = ld128(p + 128 + 32 * n + 16 * h);
    u32x4 s = ld128(p + 192);
    r.sc[0] = s.x; r.sc[1] = s.y; r.sc[2] = s.z; r.sc[3] = s.w;
    r.d = ld32(p + 208) & 0xFFFF;
  }
  static BL_HD int scale(const Regs& r, int idx) {  // idx 0..15, signed byte
    // selects instead of a dynamically indexed register array (which would live in local memory)
    const int wi = idx >> 2;
    const uint32_t lo = (wi & 1) ? r.sc[1] : r.sc[0];
    const uint32_t hi = (wi & 1) ? r.sc[3] : r.sc[2];
    const uint32_t word = (wi & 2) ? hi : lo;
    return (int)(int8_t)((word >> (8 * (idx & 3))) & 0xFF);
  }
  // four groups g of four words (16 codes each), codes already centred (q - 32)
  static BL_HD void codes(const Regs& r, uint32_t c[4][4]) {
    const uint32_t la[4] = {r.la.x, r.la.y, r.la.z, r.la.w};
    const uint32_t lb[4] = {r.lb.x, r.lb.y, r.lb.z, r.lb.w};
    const uint32_t hh[4] = {r.h.x, r.h.y, r.h.z, r.h.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      c[0][i] = (la[i] & 0x0F0F0F0Fu) | (((hh[i] >> 0) & 0x03030303u) << 4);
      c[1][i] = (lb[i] & 0x0F0F0F0Fu) | (((hh[i] >> 2) & 0x03030303u) << 4);
      c[2][i] = ((la[i] >> 4) & 0x0F0F0F0Fu) | (((hh[i] >> 4) & 0x03030303u) << 4);
      c[3][i] = ((lb[i] >> 4) & 0x0F0F0F0Fu) | (((hh[i] >> 6) & 0x03030303u) << 4);
    }
  }
  // `aq` points at the superblock's 256 codes (64 words); `ads` at its 8 {d,s} pairs
  static BL_HD float dot_sb(const Regs& r, int u, const uint32_t* aq, const float* ads) {
    int n = (u >> 1) & 1, h = u & 1;
    uint32_t c[4][4];
    codes(r, c);
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint32_t* x = aq + (128 * n + 32 * g + 16 * h) / 4;
      int s = 0, sx = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s = dot4_us(c[g][i], x[i], s);
        sx = dot4(0x01010101u, x[i], sx);
      }
      s -= 32 * sx;
      acc += ads[2 * (4 * n + g)] * (float)(scale(r, 8 * n + 2 * g + h) * s);
    }
    return half_bits_to_float((uint16_t)r.d) * acc;
  }
  static BL_HD void decode(const Regs& r, int u, float* out /*64: g*16 + i*/) {
    int n = (u >> 1) & 1, h = u & 1;
    uint32_t c[4][4];
    codes(r, c);
    float d = half_bits_to_float((uint16_t)r.d);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float ds = d * (float)scale(r, 8 * n + 2 * g + h);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int b = 0; b < 4; ++b)
          out[16 * g + 4 * i + b] = ds * (float)((int)((c[g][i] >> (8 * b)) & 0xFF) - 32);
    }
  }
  // position inside the superblock of decoded element e (0..63) of unit u
  static BL_HD int value_index(int u, int e) {
    int n = (u >> 1) & 1, h = u & 1;
    return 128 * n + 32 * (e >> 4) + 16 * h + (e & 15);
  }
};

// ---------------------------------------------------------------------------------
// Q8_0 (resident: codes then f16 scales per row)
// ---------------------------------------------------------------------------------
struct Q80 {
  static constexpr int kType = WT_Q8_0;
  struct Regs { u32x4 q[4]; uint32_t dd; };
  static BL_HD long row_bytes(int K) { return (((long)K + K / 16) + 15) / 16 * 16; }
  static BL_HD void load(const uint8_t* row, int u, int K, Regs& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = ld128(row + 64 * u + 16 * i);
    r.dd = ld32(row + K + 4 * u);
  }
  static BL_HD float dot(const Regs& r, const ActUnit& a) {
    const uint32_t w[16] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w,
                            r.q[2].x, r.q[2].y, r.q[2].z, r.q[2].w, r.q[3].x, r.q[3].y, r.q[3].z, r.q[3].w};
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = dot4(w[i], a.q[i], lo);
      hi = dot4(w[8 + i], a.q[8 + i], hi);
    }
    float d0 = half_bits_to_float((uint16_t)(r.dd & 0xFFFF));
    float d1 = half_bits_to_float((uint16_t)(r.dd >> 16));
    return d0 * a.d0 * (float)lo + d1 * a.d1 * (float)hi;
  }
  static BL_HD void decode(const Regs& r, float* out) {
    float d0 = half_bits_to_float((uint16_t)(r.dd & 0xFFFF));
    float d1 = half_bits_to_float((uint16_t)(r.dd >> 16));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {r.q[i].x, r.q[i].y, r.q[i].z, r.q[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int b = 0; b < 4; ++b)
          out[16 * i + 4 * k + b] = (i < 2 ? d0 : d1) * (float)(int8_t)((w[k] >> (8 * b)) & 0xFF);
    }
  }
};





// ---------------------------------------------------------------------------------
// Q8_F32 (resident only): int8 codes with one f32 scale per 32 values, value = code * scale.
// The non-linear and grid types of the file format (IQ4_NL, IQ4_XS, MXFP4, IQ2_XXS) decode to exactly this form at
// load: their codes are small integers from a code book and every 32 values share one scale, so no value changes.
// ---------------------------------------------------------------------------------
struct Q8F {
  static constexpr int kType = WT_Q8_F32;
  struct Regs { u32x4 q[4]; uint32_t d0, d1; };
  static BL_HD long row_bytes(int K) { return (((long)K + K / 8) + 15) / 16 * 16; }
  static BL_HD void load(const uint8_t* row, int u, int K, Regs& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = ld128(row + 64 * u + 16 * i);
    r.d0 = ld32(row + K + 8 * u);
    r.d1 = ld32(row + K + 8 * u + 4);
  }
  static BL_HD float scale(uint32_t bits) { float f; __builtin_memcpy(&f, &bits, 4); return f; }
  static BL_HD float dot(const Regs& r, const ActUnit& a) {
    const uint32_t w[16] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w,
                            r.q[2].x, r.q[2].y, r.q[2].z, r.q[2].w, r.q[3].x, r.q[3].y, r.q[3].z, r.q[3].w};
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      lo = dot4(w[i], a.q[i], lo);
      hi = dot4(w[8 + i], a.q[8 + i], hi);
    }
    return scale(r.d0) * a.d0 * (float)lo + scale(r.d1) * a.d1 * (float)hi;
  }
  static BL_HD void decode(const Regs& r, float* out) {
    const float d0 = scale(r.d0), d1 = scale(r.d1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {r.q[i].x, r.q[i].y, r.q[i].z, r.q[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int b = 0; b < 4; ++b)
          out[16 * i + 4 * k + b] = (i < 2 ? d0 : d1) * (float)(int8_t)((w[k] >> (8 * b)) & 0xFF);
    }
  }
};

// ---------------------------------------------------------------------------------
// Q2_K: 84-byte file blocks re-laid to 96: qs[64] scales[16] d dmin pad[12].
// Unit u of a super-block: n = (u >> 1) & 1 picks the 32 code bytes, jp = u & 1 the bit pairs
// (shifts 4jp and 4jp + 2); its 64 values are consecutive.  value = d * (sc & 15) * q - dmin * (sc >> 4).
// ---------------------------------------------------------------------------------
struct Q2K {
  static constexpr int kType = WT_Q2_K;
  static constexpr int kSbBytes = 96;
  struct Regs { u32x4 q0, q1; uint32_t sc, dm; };
  static BL_HD long row_bytes(int K) { return (long)(K / 256) * kSbBytes; }
  static BL_HD void load(const uint8_t* row, int u, Regs& r) {
    const uint8_t* p = row + (long)(u >> 2) * kSbBytes;
    const int n = (u >> 1) & 1, jp = u & 1;
    r.q0 = ld128(p + 32 * n);
    r.q1 = ld128(p + 32 * n + 16);
    r.sc = ld32(p + 64 + 8 * n + 4 * jp);
    r.dm = ld32(p + 80);
  }
  static BL_HD float dot(const Regs& r, int u, const ActUnit& a) {
    const int jp = u & 1;
    const float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF)), dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const u32x4& q = (g & 1) ? r.q1 : r.q0;
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      const int shift = 4 * jp + 2 * (g >> 1);
      int s = 0, sx = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s = dot4_us((w[i] >> shift) & 0x03030303u, a.q[4 * g + i], s);
        sx = dot4(0x01010101u, a.q[4 * g + i], sx);
      }
      const uint32_t scb = (r.sc >> (8 * g)) & 0xFF;
      acc += ((g >> 1) ? a.d1 : a.d0) * (d * (float)(scb & 0xF) * (float)s - dmin * (float)(scb >> 4) * (float)sx);
    }
    return acc;
  }
  static BL_HD void decode(const Regs& r, int u, float* out) {
    const int jp = u & 1;
    const float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF)), dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const u32x4& q = (g & 1) ? r.q1 : r.q0;
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      const int shift = 4 * jp + 2 * (g >> 1);
      const uint32_t scb = (r.sc >> (8 * g)) & 0xFF;
      const float dl = d * (float)(scb & 0xF), ml = dmin * (float)(scb >> 4);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int b = 0; b < 4; ++b) out[16 * g + 4 * i + b] = (float)((w[i] >> (8 * b + shift)) & 3) * dl - ml;
    }
  }
};

// ---------------------------------------------------------------------------------
// Q3_K: 110-byte file blocks re-laid to 128: qs[64] hmask[32] sc[16] (the 6-bit scales unpacked to
// signed bytes, 32 already subtracted) d pad[14].  Units as for Q2_K.  value = d * sc * (q - (hbit ? 0 : 4)).
// ---------------------------------------------------------------------------------
struct Q3K {
  static constexpr int kType = WT_Q3_K;
  static constexpr int kSbBytes = 128;
  struct Regs { u32x4 q0, q1, h0, h1; uint32_t sc, d; };
  static BL_HD long row_bytes(int K) { return (long)(K / 256) * kSbBytes; }
  static BL_HD void load(const uint8_t* row, int u, Regs& r) {
    const uint8_t* p = row + (long)(u >> 2) * kSbBytes;
    const int n = (u >> 1) & 1, jp = u & 1;
    r.q0 = ld128(p + 32 * n);
    r.q1 = ld128(p + 32 * n + 16);
    r.h0 = ld128(p + 64);
    r.h1 = ld128(p + 80);
    r.sc = ld32(p + 96 + 8 * n + 4 * jp);
    r.d = ld32(p + 112) & 0xFFFF;
  }
  static BL_HD float dot(const Regs& r, int u, const ActUnit& a) {
    const int n = (u >> 1) & 1, jp = u & 1;
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const u32x4& q = (g & 1) ? r.q1 : r.q0;
      const u32x4& h = (g & 1) ? r.h1 : r.h0;
      const uint32_t w[4] = {q.x, q.y, q.z, q.w}, hw[4] = {h.x, h.y, h.z, h.w};
      const int shift = 4 * jp + 2 * (g >> 1), hbit = 4 * n + 2 * jp + (g >> 1);
      int s = 0, sh = 0, sx = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s = dot4_us((w[i] >> shift) & 0x03030303u, a.q[4 * g + i], s);
        sh = dot4_us((hw[i] >> hbit) & 0x01010101u, a.q[4 * g + i], sh);
        sx = dot4(0x01010101u, a.q[4 * g + i], sx);
      }
      const int sc = (int)(int8_t)((r.sc >> (8 * g)) & 0xFF);
      acc += ((g >> 1) ? a.d1 : a.d0) * (float)(sc * (s + 4 * sh - 4 * sx));
    }
    return half_bits_to_float((uint16_t)r.d) * acc;
  }
  static BL_HD void decode(const Regs& r, int u, float* out) {
    const int n = (u >> 1) & 1, jp = u & 1;
    const float d = half_bits_to_float((uint16_t)r.d);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const u32x4& q = (g & 1) ? r.q1 : r.q0;
      const u32x4& h = (g & 1) ? r.h1 : r.h0;
      const uint32_t w[4] = {q.x, q.y, q.z, q.w}, hw[4] = {h.x, h.y, h.z, h.w};
      const int shift = 4 * jp + 2 * (g >> 1), hbit = 4 * n + 2 * jp + (g >> 1);
      const float dl = d * (float)(int)(int8_t)((r.sc >> (8 * g)) & 0xFF);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int qq = (int)((w[i] >> (8 * b + shift)) & 3) - (((hw[i] >> (8 * b + hbit)) & 1) ? 0 : 4);
          out[16 * g + 4 * i + b] = (float)qq * dl;
        }
    }
  }
};

// ---------------------------------------------------------------------------------
// The 32-value block family Q4_0 / Q4_1 / Q5_0 / Q5_1, re-laid as planes so every load is aligned:
//   row = [codes K/2][fifth bits K/8 (5-bit types)][f16 d per block K/16][f16 m per block K/16 (_1 types)] pad 16
// Codes keep the file's nibble order (byte i of a block: low nibble = value i, high nibble = value i + 16).
// value = d * (q - 8 | 16)  (_0)   or   d * q + m  (_1)
// ---------------------------------------------------------------------------------
template <int BITS, bool HAS_MIN, int TYPE>
struct Q32 {
  static constexpr int kType = TYPE;
  struct Regs { u32x4 q0, q1; uint32_t h0, h1, dd, mm; };
  static BL_HD long off_d(int K) { return K / 2 + (BITS == 5 ? K / 8 : 0); }
  static BL_HD long row_bytes(int K) { return ((off_d(K) + K / 16 + (HAS_MIN ? K / 16 : 0)) + 15) / 16 * 16; }
  static BL_HD void load(const uint8_t* row, int u, int K, Regs& r) {
    r.q0 = ld128(row + 32 * u);
    r.q1 = ld128(row + 32 * u + 16);
    if (BITS == 5) { r.h0 = ld32(row + K / 2 + 8 * u); r.h1 = ld32(row + K / 2 + 8 * u + 4); } else { r.h0 = r.h1 = 0; }
    r.dd = ld32(row + off_d(K) + 4 * u);
    r.mm = HAS_MIN ? ld32(row + off_d(K) + K / 16 + 4 * u) : 0u;
  }
  // four fifth-bits (bits 0..3 of x) to bit 4 of four bytes
  static BL_HD uint32_t spread(uint32_t x) {
    return ((x & 1u) | ((x & 2u) << 7) | ((x & 4u) << 14) | ((x & 8u) << 21)) << 4;
  }
  // the eight code words of block b (values 0..31 in order) as unsigned bytes
  static BL_HD void codes(const Regs& r, int b, uint32_t* c) {
    const u32x4& q = b ? r.q1 : r.q0;
    const uint32_t h = b ? r.h1 : r.h0;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      c[j] = w[j] & 0x0F0F0F0Fu;
      c[4 + j] = (w[j] >> 4) & 0x0F0F0F0Fu;
      if (BITS == 5) { c[j] |= spread(h >> (4 * j)); c[4 + j] |= spread(h >> (16 + 4 * j)); }
    }
  }
  static BL_HD float dot(const Regs& r, const ActUnit& a) {
    float acc = 0.f;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      uint32_t c[8];
      codes(r, b, c);
      int s = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) s = dot4_us(c[j], a.q[8 * b + j], s);
      const float d = half_bits_to_float((uint16_t)(r.dd >> (16 * b)));
      const float da = b ? a.d1 : a.d0, sa = b ? a.s1 : a.s0;
      if (HAS_MIN) acc += d * da * (float)s + half_bits_to_float((uint16_t)(r.mm >> (16 * b))) * sa;
      else acc += d * (da * (float)s - (float)(BITS == 5 ? 16 : 8) * sa);
    }
    return acc;
  }
  static BL_HD void decode(const Regs& r, float* out) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      uint32_t c[8];
      codes(r, b, c);
      const float d = half_bits_to_float((uint16_t)(r.dd >> (16 * b)));
      const float m = HAS_MIN ? half_bits_to_float((uint16_t)(r.mm >> (16 * b))) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int q = (int)((c[j] >> (8 * k)) & 0xFF);
          out[32 * b + 4 * j + k] = HAS_MIN ? d * (float)q + m : d * (float)(q - (BITS == 5 ? 16 : 8));
        }
    }
  }
};
using Q40 = Q32<4, false, WT_Q4_0>;
using Q41 = Q32<4, true, WT_Q4_1>;
using Q50 = Q32<5, false, WT_Q5_0>;
using Q51 = Q32<5, true, WT_Q5_1>;

// ---------------------------------------------------------------------------------
// E4M3 and E2M1 scalar decoders (host and device)
// ---------------------------------------------------------------------------------
BL_HD float e4m3_to_float(uint8_t b) {
  const int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 0) v = (float)m * 0.001953125f;                 // subnormal: m * 2^-9
  else if (e == 15 && m == 7) v = __builtin_nanf("");        // the one NaN encoding (no infinities)
  else {
    uint32_t bits = (uint32_t)(e + 120) << 23 | (uint32_t)m << 20;   // 2^(e-7) * (1 + m/8)
    __builtin_memcpy(&v, &bits, 4);
  }
  return s ? -v : v;
}


// four E4M3 bytes of one word -> four floats (the hardware converter on the device)
BL_HD void e4m3x4_to_float(uint32_t w, float* o) {
#if defined(__CUDA_ARCH__)
  uint32_t h0, h1;
  asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %2; cvt.rn.f16x2.e4m3x2 %0, lo; cvt.rn.f16x2.e4m3x2 %1, hi; }"
      : "=r"(h0), "=r"(h1) : "r"(w));
  const __half2 a = *reinterpret_cast<__half2*>(&h0), b = *reinterpret_cast<__half2*>(&h1);
  const float2 fa = __half22float2(a), fb = __half22float2(b);
  o[0] = fa.x; o[1] = fa.y; o[2] = fb.x; o[3] = fb.y;
#else
  for (int b = 0; b < 4; ++b) o[b] = e4m3_to_float((uint8_t)(w >> (8 * b)));
#endif
}

// two E2M1 magnitudes per lookup: code & 7 -> {0, 0.5, 1, 1.5, 2, 3, 4, 6} * 2
BL_HD int e2m1_x2(uint32_t code) {
  const int mag = (int)((0x0C08060403020100ull >> (8 * (code & 7))) & 0xFF);
  return (code & 8) ? -mag : mag;
}

// ---------------------------------------------------------------------------------
// NVFP4: 16-value groups, E2M1 codes (low nibble first), E4M3 group scale, f32 tensor scale.
// Codes are doubled to small integers and dotted with the q8 activations (the reference
// runs NVFP4 experts on int8 activations too: crates/gpu/src/gemm/gemm32.rs, gemm_nvfp4p).
// ---------------------------------------------------------------------------------
struct NvFp4 {
  static constexpr int kType = WT_NVFP4;
  struct Regs { u32x4 q0, q1; uint32_t sc; float g; };
  static BL_HD long row_bytes(int K) { return (((long)K / 2 + K / 16 + 4) + 15) / 16 * 16; }
  static BL_HD void load(const uint8_t* row, int u, int K, Regs& r) {
    r.q0 = ld128(row + 32 * u);
    r.q1 = ld128(row + 32 * u + 16);
    r.sc = ld32(row + K / 2 + 4 * u);
    uint32_t gb = ld32(row + K / 2 + K / 16);
    __builtin_memcpy(&r.g, &gb, 4);
  }
  // eight nibbles of one word -> two words of int8 (values x2)
  static BL_HD void expand(uint32_t w, uint32_t& lo4, uint32_t& hi4) {
    lo4 = 0; hi4 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo4 |= (uint32_t)(uint8_t)e2m1_x2((w >> (4 * i)) & 0xF) << (8 * i);
      hi4 |= (uint32_t)(uint8_t)e2m1_x2((w >> (16 + 4 * i)) & 0xF) << (8 * i);
    }
  }
  static BL_HD float dot(const Regs& r, const uint32_t* aq /*16 words*/, const float* ad /*d of the two 32-blocks*/) {
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {                 // group g: values 16g..16g+15 = words 2g, 2g+1 of codes
      int s = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t lo4, hi4;
        expand(w[2 * g + h], lo4, hi4);
        s = dot4(lo4, aq[4 * g + 2 * h], s);
        s = dot4(hi4, aq[4 * g + 2 * h + 1], s);
      }
      acc += e4m3_to_float((uint8_t)(r.sc >> (8 * g))) * ad[g >> 1] * (float)s;
    }
    return acc * r.g * 0.5f;
  }
  static BL_HD void decode(const Regs& r, float* out) {
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const float sc = e4m3_to_float((uint8_t)(r.sc >> (8 * g))) * r.g * 0.5f;
#pragma unroll
      for (int i = 0; i < 16; ++i) out[16 * g + i] = sc * (float)e2m1_x2((w[2 * g + i / 8] >> (4 * (i & 7))) & 0xF);
    }
  }
};

// ---------------------------------------------------------------------------------
// FP8 block-scaled (E4M3 codes, one f32 scale per 128 values of the row)
// ---------------------------------------------------------------------------------
struct Fp8B128 {
  static constexpr int kType = WT_FP8_B128;
  struct Regs { u32x4 q[4]; float sc; };
  static BL_HD long row_bytes(int K) { return (((long)K + K / 32) + 15) / 16 * 16; }
  static BL_HD void load(const uint8_t* row, int u, int K, Regs& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) r.q[i] = ld128(row + 64 * u + 16 * i);
    uint32_t sb = ld32(row + K + 4 * (u >> 1));
    __builtin_memcpy(&r.sc, &sb, 4);
  }
  static BL_HD float dot(const Regs& r, const uint32_t* aq, const float* ad) {
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {r.q[i].x, r.q[i].y, r.q[i].z, r.q[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
      {
        float wv[4];
        e4m3x4_to_float(w[k], wv);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const float xv = (float)(int8_t)((aq[4 * i + k] >> (8 * b)) & 0xFF);
          if (i < 2) acc0 = wv[b] * xv + acc0; else acc1 = wv[b] * xv + acc1;
        }
      }
    }
    return r.sc * (ad[0] * acc0 + ad[1] * acc1);
  }
  static BL_HD void decode(const Regs& r, float* out) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t w[4] = {r.q[i].x, r.q[i].y, r.q[i].z, r.q[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int b = 0; b < 4; ++b) out[16 * i + 4 * k + b] = r.sc * e4m3_to_float((uint8_t)(w[k] >> (8 * b)));
    }
  }
};

// ---------------------------------------------------------------------------------
// Uniform interface used by the templated kernels:
//   T::loadu(row, u, K, regs)                     fetch unit u of a weight row
//   T::dotu(regs, u, xq_row_words, xds_row)       dot with a q8 activation row
//   T::decodeu(regs, u, out64), T::pos(u, e)      decoded values and their positions
// ---------------------------------------------------------------------------------
struct F2 { float x, y; };

template <class T> struct Unit;

template <> struct Unit<Q4K> {
  using Regs = Q4K::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int, Regs& r) { Q4K::load(row, u, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return Q4K::dot(r, u, a);
  }
  static BL_HD void decodeu(const Regs& r, int u, float* o) { Q4K::decode(r, u, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};
template <> struct Unit<Q5K> {
  using Regs = Q5K::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int, Regs& r) { Q5K::load(row, u, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return Q5K::dot(r, u, a);
  }
  static BL_HD void decodeu(const Regs& r, int u, float* o) { Q5K::decode(r, u, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};
template <> struct Unit<Q6K> {
  using Regs = Q6K::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int, Regs& r) { Q6K::load(row, u, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    int sb = u >> 2;
    return Q6K::dot_sb(r, u, xq + 64 * sb, reinterpret_cast<const float*>(xds + 8 * sb));
  }
  static BL_HD void decodeu(const Regs& r, int u, float* o) { Q6K::decode(r, u, o); }
  static BL_HD int pos(int u, int e) { return 256 * (u >> 2) + Q6K::value_index(u, e); }
};
template <> struct Unit<Q8F> {
  using Regs = Q8F::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int K, Regs& r) { Q8F::load(row, u, K, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return Q8F::dot(r, a);
  }
  static BL_HD void decodeu(const Regs& r, int, float* o) { Q8F::decode(r, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};
template <> struct Unit<Q80> {
  using Regs = Q80::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int K, Regs& r) { Q80::load(row, u, K, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return Q80::dot(r, a);
  }
  static BL_HD void decodeu(const Regs& r, int, float* o) { Q80::decode(r, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};


template <> struct Unit<Q2K> {
  using Regs = Q2K::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int, Regs& r) { Q2K::load(row, u, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return Q2K::dot(r, u, a);
  }
  static BL_HD void decodeu(const Regs& r, int u, float* o) { Q2K::decode(r, u, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};
template <> struct Unit<Q3K> {
  using Regs = Q3K::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int, Regs& r) { Q3K::load(row, u, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return Q3K::dot(r, u, a);
  }
  static BL_HD void decodeu(const Regs& r, int u, float* o) { Q3K::decode(r, u, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};

template <int BITS, bool HAS_MIN, int TYPE> struct Unit<Q32<BITS, HAS_MIN, TYPE>> {
  using T32 = Q32<BITS, HAS_MIN, TYPE>;
  using Regs = typename T32::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int K, Regs& r) { T32::load(row, u, K, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    ActUnit a{xq + 16 * u, xds[2 * u].x, xds[2 * u].y, xds[2 * u + 1].x, xds[2 * u + 1].y};
    return T32::dot(r, a);
  }
  static BL_HD void decodeu(const Regs& r, int, float* o) { T32::decode(r, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};

template <> struct Unit<NvFp4> {
  using Regs = NvFp4::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int K, Regs& r) { NvFp4::load(row, u, K, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    const float ad[2] = {xds[2 * u].x, xds[2 * u + 1].x};
    return NvFp4::dot(r, xq + 16 * u, ad);
  }
  static BL_HD void decodeu(const Regs& r, int, float* o) { NvFp4::decode(r, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};
template <> struct Unit<Fp8B128> {
  using Regs = Fp8B128::Regs;
  static BL_HD void loadu(const uint8_t* row, int u, int K, Regs& r) { Fp8B128::load(row, u, K, r); }
  static BL_HD float dotu(const Regs& r, int u, const uint32_t* xq, const F2* xds) {
    const float ad[2] = {xds[2 * u].x, xds[2 * u + 1].x};
    return Fp8B128::dot(r, xq + 16 * u, ad);
  }
  static BL_HD void decodeu(const Regs& r, int, float* o) { Fp8B128::decode(r, o); }
  static BL_HD int pos(int u, int e) { return 64 * u + e; }
};

// ---------------------------------------------------------------------------------
// Activation registers of one unit: 16 code words and up to four {d, s} pairs, fetched
// once (from shared or global memory) and reused against several weight rows.
//   ActOf<T>::load(xq_row_words, xds_row, u, regs);  ActOf<T>::dot(wregs, u, regs)
// ---------------------------------------------------------------------------------
struct ActRegs { uint32_t q[16]; float d[4]; float s[4]; };

BL_HD void ld_act128(const uint32_t* p, uint32_t* o) {
#if defined(__CUDA_ARCH__)
  uint4 v = *reinterpret_cast<const uint4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
#else
  __builtin_memcpy(o, p, 16);
#endif
}

template <class T> struct ActOf {
  // 64 consecutive values: Q4_K, Q5_K, Q8_0
  static BL_HD void load(const uint32_t* xq, const F2* xds, int u, ActRegs& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) ld_act128(xq + 16 * u + 4 * i, a.q + 4 * i);
    a.d[0] = xds[2 * u].x; a.s[0] = xds[2 * u].y; a.d[1] = xds[2 * u + 1].x; a.s[1] = xds[2 * u + 1].y;
  }
  static BL_HD float dot(const typename Unit<T>::Regs& r, int u, const ActRegs& a) {
    ActUnit au{a.q, a.d[0], a.s[0], a.d[1], a.s[1]};
    if constexpr (T::kType == WT_Q8_0 || T::kType == WT_Q8_F32 || T::kType == WT_Q4_0 || T::kType == WT_Q4_1 || T::kType == WT_Q5_0 ||
                  T::kType == WT_Q5_1) return T::dot(r, au);
    else return T::dot(r, u, au);
  }
};

template <> struct ActOf<Q6K> {
  static BL_HD void load(const uint32_t* xq, const F2* xds, int u, ActRegs& a) {
    const int sb = u >> 2, n = (u >> 1) & 1, h = u & 1;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      ld_act128(xq + 64 * sb + (128 * n + 32 * g + 16 * h) / 4, a.q + 4 * g);
      a.d[g] = xds[8 * sb + 4 * n + g].x;
    }
  }
  static BL_HD float dot(const Q6K::Regs& r, int u, const ActRegs& a) {
    const int n = (u >> 1) & 1, h = u & 1;
    uint32_t c[4][4];
    Q6K::codes(r, c);
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      int s = 0, sx = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s = dot4_us(c[g][i], a.q[4 * g + i], s);
        sx = dot4(0x01010101u, a.q[4 * g + i], sx);
      }
      s -= 32 * sx;
      acc += a.d[g] * (float)(Q6K::scale(r, 8 * n + 2 * g + h) * s);
    }
    return half_bits_to_float((uint16_t)r.d) * acc;
  }
};

template <> struct ActOf<NvFp4> {
  static BL_HD void load(const uint32_t* xq, const F2* xds, int u, ActRegs& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) ld_act128(xq + 16 * u + 4 * i, a.q + 4 * i);
    a.d[0] = xds[2 * u].x; a.d[1] = xds[2 * u + 1].x;
  }
  static BL_HD float dot(const NvFp4::Regs& r, int, const ActRegs& a) { return NvFp4::dot(r, a.q, a.d); }
};
template <> struct ActOf<Fp8B128> {
  static BL_HD void load(const uint32_t* xq, const F2* xds, int u, ActRegs& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) ld_act128(xq + 16 * u + 4 * i, a.q + 4 * i);
    a.d[0] = xds[2 * u].x; a.d[1] = xds[2 * u + 1].x;
  }
  static BL_HD float dot(const Fp8B128::Regs& r, int, const ActRegs& a) { return Fp8B128::dot(r, a.q, a.d); }
};

// Resident row size for a weight type and row length.
BL_HD long resident_row_bytes(int wtype, int K) {
  switch (wtype) {
    case WT_Q4_K: return Q4K::row_bytes(K);
    case WT_Q5_K: return Q5K::row_bytes(K);
    case WT_Q6_K: return Q6K::row_bytes(K);
    case WT_Q8_0: return Q80::row_bytes(K);
    case WT_Q8_F32: return Q8F::row_bytes(K);
    case WT_Q2_K: return Q2K::row_bytes(K);
    case WT_Q3_K: return Q3K::row_bytes(K);
    case WT_Q4_0: return Q40::row_bytes(K);
    case WT_Q4_1: return Q41::row_bytes(K);
    case WT_Q5_0: return Q50::row_bytes(K);
    case WT_Q5_1: return Q51::row_bytes(K);
    case WT_NVFP4: return NvFp4::row_bytes(K);
    case WT_FP8_B128: return Fp8B128::row_bytes(K);
    case WT_F32: return 4L * K;
    case WT_F16: case WT_BF16: return 2L * K;
  }
  return -1;
}

}  // namespace bl
