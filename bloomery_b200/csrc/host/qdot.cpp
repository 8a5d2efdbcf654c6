// CPU quantised dots: the scalar mirror of the device units (bit-for-bit the same
// integer sums and the same fp32 operation order per unit) plus AVX2 paths chosen at
// run time.  Serves three purposes: the byte-level oracle for the CUDA kernels, the
// CPU engine's matmul (the --cpu-moe host path), and the cold-expert host leg.
// Counterpart of crates/qdot (lib.rs:1-108: per-type row dots against quantised
// activations with no f32 materialisation, scalar mirrors beside the SIMD kernels).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <immintrin.h>

#include "../quant_units.cuh"
#include "pool.h"
#include "qdot_avx2.h"
#include "qdot_vnni.h"

using namespace bl;

namespace {

template <class T>
float row_dot_scalar(const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  using U = Unit<T>;
  // mirror of the device reduction: lane l sums units l, l+32, ...; then a xor butterfly
  float lane_acc[32];
  for (int l = 0; l < 32; ++l) lane_acc[l] = 0.f;
  const int nunits = K / 64;
  for (int u = 0; u < nunits; ++u) {
    typename U::Regs r;
    U::loadu(row, u, K, r);
    lane_acc[u & 31] += U::dotu(r, u, reinterpret_cast<const uint32_t*>(xq), reinterpret_cast<const F2*>(xds));
  }
  for (int o = 16; o > 0; o >>= 1) {
    float nxt[32];
    for (int l = 0; l < 32; ++l) nxt[l] = lane_acc[l] + lane_acc[l ^ o];
    std::memcpy(lane_acc, nxt, sizeof(nxt));
  }
  return lane_acc[0];
}

float row_dot_any(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  switch (wtype) {
    case WT_Q4_K: return row_dot_scalar<Q4K>(row, K, xq, xds);
    case WT_Q5_K: return row_dot_scalar<Q5K>(row, K, xq, xds);
    case WT_Q6_K: return row_dot_scalar<Q6K>(row, K, xq, xds);
    case WT_Q8_0: return row_dot_scalar<Q80>(row, K, xq, xds);
    case WT_Q8_F32: return row_dot_scalar<Q8F>(row, K, xq, xds);
    case WT_NVFP4: return row_dot_scalar<NvFp4>(row, K, xq, xds);
    case WT_FP8_B128: return row_dot_scalar<Fp8B128>(row, K, xq, xds);
    case WT_Q2_K: return row_dot_scalar<Q2K>(row, K, xq, xds);
    case WT_Q3_K: return row_dot_scalar<Q3K>(row, K, xq, xds);
    case WT_Q4_0: return row_dot_scalar<Q40>(row, K, xq, xds);
    case WT_Q4_1: return row_dot_scalar<Q41>(row, K, xq, xds);
    case WT_Q5_0: return row_dot_scalar<Q50>(row, K, xq, xds);
    case WT_Q5_1: return row_dot_scalar<Q51>(row, K, xq, xds);
  }
  return NAN;
}

template <class T>
void row_decode(const uint8_t* row, int K, float* out) {
  using U = Unit<T>;
  for (int u = 0; u < K / 64; ++u) {
    typename U::Regs r;
    U::loadu(row, u, K, r);
    float v[64];
    U::decodeu(r, u, v);
    for (int e = 0; e < 64; ++e) out[U::pos(u, e)] = v[e];
  }
}

}  // namespace

extern "C" {

// the vector path's dot of one row (tests compare it with the scalar mirror); returns 0 when there is none
int blh_row_dot_fast(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds, float* out) {
  return blh::row_dot_fast(wtype, row, K, xq, xds, out) ? 1 : 0;
}

// the AVX-512 VNNI path's dot of one row; 0 when the CPU lacks the instructions or the type has no such path
int blh_row_dot_vnni(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds, float* out) {
  return blh::row_dot_vnni(wtype, row, K, xq, xds, out) ? 1 : 0;
}
int blh_cpu_has_vnni() { return blh::cpu_has_vnni() ? 1 : 0; }

long blh_resident_row_bytes(int wtype, int K) { return resident_row_bytes(wtype, K); }

// q8 activation form, identical rounding to the device (round-to-nearest-even)
void blh_act_q8(const float* x, int M, int K, int8_t* codes, float* ds) {
  for (int m = 0; m < M; ++m)
    for (int b = 0; b < K / 32; ++b) {
      const float* xb = x + (long)m * K + b * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(xb[i]));
      float d = amax / 127.0f;
      float inv = d > 0.f ? 1.0f / d : 0.f;
      int sum = 0;
      for (int i = 0; i < 32; ++i) {
        int q = (int)std::nearbyintf(xb[i] * inv);
        q = q < -127 ? -127 : q > 127 ? 127 : q;
        codes[(long)m * K + b * 32 + i] = (int8_t)q;
        sum += q;
      }
      ds[((long)m * (K / 32) + b) * 2] = d;
      ds[((long)m * (K / 32) + b) * 2 + 1] = d * (float)sum;
    }
}

// out[m, r] = W[r, :] . act[m, :] over resident rows; threads from the shared pool
int blh_gemv(int wtype, const uint8_t* w, int rows, int K, const int8_t* xq, const float* xds, int M, float* out,
             long out_stride) {
  long rb = resident_row_bytes(wtype, K);
  if (rb <= 0 || K % 64) return -1;
  blh::Pool::instance().parallel_for(rows, 64, [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r)
      for (int m = 0; m < M; ++m)
        out[(long)m * out_stride + r] = row_dot_any(wtype, w + (long)r * rb, K, xq + (long)m * K, xds + (long)m * (K / 32) * 2);
  });
  return 0;
}

int blh_decode_rows(int wtype, const uint8_t* w, int rows, int K, float* out) {
  long rb = resident_row_bytes(wtype, K);
  if (rb <= 0) return -1;
  for (int r = 0; r < rows; ++r) {
    const uint8_t* row = w + (long)r * rb;
    float* o = out + (long)r * K;
    switch (wtype) {
      case WT_Q4_K: row_decode<Q4K>(row, K, o); break;
      case WT_Q5_K: row_decode<Q5K>(row, K, o); break;
      case WT_Q6_K: row_decode<Q6K>(row, K, o); break;
      case WT_Q8_0: row_decode<Q80>(row, K, o); break;
      case WT_Q8_F32: row_decode<Q8F>(row, K, o); break;
      case WT_NVFP4: row_decode<NvFp4>(row, K, o); break;
      case WT_FP8_B128: row_decode<Fp8B128>(row, K, o); break;
      case WT_Q2_K: row_decode<Q2K>(row, K, o); break;
      case WT_Q3_K: row_decode<Q3K>(row, K, o); break;
      case WT_Q4_0: row_decode<Q40>(row, K, o); break;
      case WT_Q4_1: row_decode<Q41>(row, K, o); break;
      case WT_Q5_0: row_decode<Q50>(row, K, o); break;
      case WT_Q5_1: row_decode<Q51>(row, K, o); break;
      default: return -1;
    }
  }
  return 0;
}

}  // extern "C"
