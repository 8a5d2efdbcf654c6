// Argument block and activation prologues shared by the decode GEMV kernels: the register-streaming kernel
// (decode_gemv.cu) and the shared-memory staged one (decode_staged.cu).
#pragma once
#include "common.cuh"

namespace bl {

struct GemvSeg {
  const uint8_t* w;
  int rows;
  int wtype;
  int blk0;        // first block of this segment
  int nblk;        // blocks that share this segment's rows evenly
  long row_bytes;
};

struct GemvArgs {
  GemvSeg seg[4];
  int nseg;
  int K;
  int M;
  const float* x;          // input A: fp32 rows, RMS-normalised and quantised in the prologue
  long x_stride;
  const float* gain;
  float eps;
  const int8_t* xq;        // input B: rows already in q8 form
  const float2* xds;
  float* out;
  long out_stride;
  const float* resid;
  long resid_stride;
  unsigned* fault;
  int layer;
  ReduceIn red;            // n_ranks > 0: x is "x + sum of every rank's partial rows" (consumer half)
  PushOut push;            // n_ranks > 0: the result is a partial update pushed to every rank (producer half)
  int stage_bytes;         // staged kernel: bytes of shared memory reserved for a block's weight rows
  int rpb_max;             // staged kernel: most rows any block owns
  int dbg;                 // staged kernel: timing-experiment switches (0 in normal use)
  // Weights that a LATER launch will stream (the next layer's projections): every block asks L2 to fetch its
  // share of each span before it waits for its predecessor, so that launch finds them on chip.
  const uint8_t* pf_ptr[6];
  long pf_bytes[6];
  int n_pf;
};

// One thread per block: ask L2 to prefetch this block's 1 / gridDim.x share of each span (16-byte granules).
__device__ __forceinline__ void prefetch_spans_l2(const uint8_t* const* ptr, const long* bytes, int n) {
  for (int i = 0; i < n; ++i) {
    const long share = ((bytes[i] + gridDim.x - 1) / gridDim.x + 15) & ~15L;
    const long lo = (long)blockIdx.x * share;
    long left = bytes[i] - lo;
    left = left < share ? left : share;
    left &= ~15L;
    for (long o = 0; o < left; o += 32768) {
      const unsigned n_b = (unsigned)((left - o) < 32768 ? (left - o) : 32768);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr[i] + lo + o), "r"(n_b) : "memory");
    }
  }
}


// ---- shared-memory layout of a q8 activation row ----------------------------------------
// The codes of a K-value row are kept in 16-byte chunks.  Layout 0 is linear.  The staged kernels read a
// row with lane u fetching the four chunks of weight unit u, which in a linear row lie 64 bytes apart from the
// next lane's (a 4-way bank conflict on every load); layouts 1 and 2 store chunk c where consecutive lanes
// read consecutive chunks:
//   1  units of 64 consecutive values (every type but Q6_K): chunk 4u + i sits at i * nunits + u
//   2  Q6_K units (four runs of 16 values, 32 apart): chunk 16 sb + 8 n + 2 g + h sits at g * nunits + (4 sb + 2 n + h)
__device__ __forceinline__ int act_chunk_pos(int c, int nunits, int layout) {
  if (layout == 1) return (c & 3) * nunits + (c >> 2);
  if (layout == 2) return ((c >> 1) & 3) * nunits + 4 * (c >> 4) + 2 * ((c >> 3) & 1) + (c & 1);
  return c;
}

// Activation registers of weight unit u out of a shared-memory row in layout 1 / 2 (act_chunk_pos): every load of
// a warp touches 32 consecutive 16-byte chunks, so none meets a bank conflict.  `sds` stays linear.
template <class T> struct StagedAct {
  static constexpr int kLayout = 1;
  static __device__ __forceinline__ void load(const int8_t* sq, const float2* sds, int u, int nunits, ActRegs& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(sq + ((long)(i * nunits + u) << 4));
      a.q[4 * i] = v.x; a.q[4 * i + 1] = v.y; a.q[4 * i + 2] = v.z; a.q[4 * i + 3] = v.w;
    }
    const float4 ds = *reinterpret_cast<const float4*>(sds + 2 * u);
    a.d[0] = ds.x; a.s[0] = ds.y; a.d[1] = ds.z; a.s[1] = ds.w;
  }
};
template <> struct StagedAct<Q6K> {
  static constexpr int kLayout = 2;
  static __device__ __forceinline__ void load(const int8_t* sq, const float2* sds, int u, int nunits, ActRegs& a) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 v = *reinterpret_cast<const uint4*>(sq + ((long)(g * nunits + u) << 4));
      a.q[4 * g] = v.x; a.q[4 * g + 1] = v.y; a.q[4 * g + 2] = v.z; a.q[4 * g + 3] = v.w;
    }
    const int sb = u >> 2, n = (u >> 1) & 1;
    const float4 d01 = *reinterpret_cast<const float4*>(sds + 8 * sb + 4 * n);
    const float4 d23 = *reinterpret_cast<const float4*>(sds + 8 * sb + 4 * n + 2);
    a.d[0] = d01.x; a.d[1] = d01.z; a.d[2] = d23.x; a.d[3] = d23.z;
  }
};
__host__ __device__ inline int staged_layout(int wtype) { return wtype == WT_Q6_K ? 2 : 1; }

// ---- activation prologue ------------------------------------------------------------
// sq/sds receive q8(x * gain) WITHOUT the RMS scale; s_scale[m] receives the scale.
template <int MB, bool FLOATW>
__device__ __forceinline__ void prologue_norm(const GemvArgs& a, int8_t* sq, float2* sds, float* sx, float* s_scale,
                                              double* red, int layout = 0) {
  const int K = a.K, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool reduce = a.red.n_ranks > 0;
  __shared__ int s_gave_up;
  ReduceWait rw{0u, 0ull, &s_gave_up};
  if (reduce) {
    if (tid == 0) s_gave_up = (a.red.fault && *a.red.fault != 0xFFFFFFFFu) ? 1 : 0;   // a poisoned engine no longer waits
    __syncthreads();
    rw.epoch = site_epoch(a.red.step, a.red.sites_per_step, a.red.site_index);
  }
#pragma unroll 1
  for (int m = 0; m < MB; ++m) {
    const int ms = m < a.M ? m : a.M - 1;
    const float* x = a.x + (long)ms * a.x_stride;
    float ss = 0.f;
    for (int i0 = tid * 8; i0 < K; i0 += 256 * 8) {
      float4 x0, x1;
      if (reduce) {
        x0 = *reinterpret_cast<const float4*>(x + i0); x1 = *reinterpret_cast<const float4*>(x + i0 + 4);
        float acc8[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        reduce_sum8(a.red, rw, ms, i0, acc8);
        x0 = make_float4(acc8[0], acc8[1], acc8[2], acc8[3]); x1 = make_float4(acc8[4], acc8[5], acc8[6], acc8[7]);
        if (blockIdx.x == 0 && m < a.M) {
          *reinterpret_cast<float4*>(a.red.x_out + (long)m * a.red.x_out_stride + i0) = x0;
          *reinterpret_cast<float4*>(a.red.x_out + (long)m * a.red.x_out_stride + i0 + 4) = x1;
        }
      } else {
        x0 = *reinterpret_cast<const float4*>(x + i0); x1 = *reinterpret_cast<const float4*>(x + i0 + 4);
      }
      float4 g0 = __ldg(reinterpret_cast<const float4*>(a.gain + i0)), g1 = __ldg(reinterpret_cast<const float4*>(a.gain + i0 + 4));
      float v[8] = {x0.x * g0.x, x0.y * g0.y, x0.z * g0.z, x0.w * g0.w, x1.x * g1.x, x1.y * g1.y, x1.z * g1.z, x1.w * g1.w};
      ss += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const float d = amax / 127.0f, inv = d > 0.f ? 1.0f / d : 0.f;
      int q[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { q[j] = max(-127, min(127, __float2int_rn(v[j] * inv))); sum += q[j]; }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      uint2 packed;
      packed.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | ((unsigned)(q[3] & 0xFF) << 24);
      packed.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | ((unsigned)(q[7] & 0xFF) << 24);
      *reinterpret_cast<uint2*>(sq + (long)m * K + act_chunk_pos(i0 >> 4, K / 64, layout) * 16 + (i0 & 15)) = packed;
      if ((tid & 3) == 0) sds[(long)m * (K / 32) + i0 / 32] = make_float2(d, d * (float)sum);
      if (FLOATW) {
        *reinterpret_cast<float4*>(sx + (long)m * K + i0) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(sx + (long)m * K + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
    double tot = warp_sum_d((double)ss);
    if (lane == 0) red[m * 8 + warp] = tot;
  }
  __syncthreads();
  if (tid < MB) {
    double all = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) all += red[tid * 8 + w];
    s_scale[tid] = 1.0f / sqrtf((float)(all / (double)K) + a.eps);
  }
  __syncthreads();
}

template <int MB>
__device__ __forceinline__ void prologue_q8in(const GemvArgs& a, int8_t* sq, float2* sds, float* s_scale, int layout = 0) {
  const int K = a.K, tid = threadIdx.x;
  for (int i = tid; i < MB * K / 16; i += 256) {
    int m = (i * 16) / K;
    const int ms = m < a.M ? m : a.M - 1;
    const int c = i - m * (K / 16);
    reinterpret_cast<uint4*>(sq)[m * (K / 16) + act_chunk_pos(c, K / 64, layout)] = reinterpret_cast<const uint4*>(a.xq + (long)ms * K)[c];
  }
  for (int i = tid; i < MB * (K / 32); i += 256) {
    int m = i / (K / 32);
    const int ms = m < a.M ? m : a.M - 1;
    sds[i] = a.xds[(long)ms * (K / 32) + (i - m * (K / 32))];
  }
  if (tid < MB) s_scale[tid] = 1.0f;
  __syncthreads();
}


}  // namespace bl
