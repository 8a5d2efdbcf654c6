// Quantised GEMV for the decode chain (m <= 8 activation rows), weights dequantised
// in registers and dotted with dp4a against q8 activations.
//
// One launch covers up to four weight segments that share an input (q, k, v
// projections; or one matrix), each with its own block type.  A warp owns one weight
// row at a time and loops over row groups (persistent grid sized to the SM count), so
// the RMSNorm + q8 prologue runs once per block, not once per 8 rows.
//
// Blackwell specifics: the first row group of every block is pulled into L2 with a
// bulk prefetch (cp.async.bulk.prefetch.L2) *before* griddepcontrol.wait, so under
// programmatic dependent launch the weight stream of kernel N+1 overlaps the tail of
// kernel N.  Behavioural counterpart of q4k_gemv/q6k_gemv(_mcol) in
// crates/gpu/src/lib.rs:1604-1632 and qwen3moe_qkv_q4k / qwen3moe_o_resid_q4k in
// crates/gpu/src/arch/qwen3moe/proj.rs: fixed lane split and a fixed xor-butterfly, so
// reruns are bit-identical and each row of an m-row call equals its own 1-row call.
#include "common.cuh"

namespace bl {

int g_use_pdl = 1;

struct GemvSeg {
  const uint8_t* w;
  int rows;
  int wtype;
  long row_bytes;
};

struct GemvArgs {
  GemvSeg seg[4];
  int nseg;
  int total_groups;  // sum over segments of ceil(rows / 8)
  int K;
  int M;
  // input A: fp32 rows to be RMS-normalised and quantised in the prologue
  const float* x;
  long x_stride;
  const float* gain;
  float eps;
  // input B: rows already in q8 form
  const int8_t* xq;
  const float2* xds;
  // outputs
  float* out;
  long out_stride;
  const float* resid;  // optional, same layout as out
  long resid_stride;
  int8_t* xq_out;      // optional: block 0 publishes the prologue's q8 rows
  float2* xds_out;
  unsigned* fault;
  int layer;
};

__device__ __forceinline__ void l2_prefetch_bulk(const void* p, unsigned bytes) {
  // bytes must be a multiple of 16 and p 16-byte aligned
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

template <class T, int MB>
__device__ __forceinline__ void row_dot(const uint8_t* row, int K, int lane, const int8_t* sq, const float2* sds,
                                        float (&acc)[MB]) {
  using U = Unit<T>;
  const int nunits = K / 64;
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  for (int u = lane; u < nunits; u += 32) {
    typename U::Regs r;
    U::loadu(row, u, K, r);
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      acc[m] += U::dotu(r, u, reinterpret_cast<const uint32_t*>(sq + (long)m * K),
                        reinterpret_cast<const F2*>(sds + (long)m * (K / 32)));
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = warp_sum(acc[m]);
}

template <int MB>
__device__ __forceinline__ void row_dot_float(const uint8_t* row, int wtype, int K, int lane, const float* sx,
                                              float (&acc)[MB]) {
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  for (int i = lane * 4; i < K; i += 128) {
    float w0, w1, w2, w3;
    if (wtype == WT_F32) {
      float4 v = __ldg(reinterpret_cast<const float4*>(row) + i / 4);
      w0 = v.x; w1 = v.y; w2 = v.z; w3 = v.w;
    } else if (wtype == WT_F16) {
      uint2 v = __ldg(reinterpret_cast<const uint2*>(row) + i / 4);
      float2 a = __half22float2(*reinterpret_cast<__half2*>(&v.x));
      float2 b = __half22float2(*reinterpret_cast<__half2*>(&v.y));
      w0 = a.x; w1 = a.y; w2 = b.x; w3 = b.y;
    } else {
      uint2 v = __ldg(reinterpret_cast<const uint2*>(row) + i / 4);
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v.x));
      float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v.y));
      w0 = a.x; w1 = a.y; w2 = b.x; w3 = b.y;
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const float4 xv = *reinterpret_cast<const float4*>(sx + (long)m * K + i);
      acc[m] = fmaf(w0, xv.x, fmaf(w1, xv.y, fmaf(w2, xv.z, fmaf(w3, xv.w, acc[m]))));
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = warp_sum(acc[m]);
}

// NORM: input A (fp32 + RMSNorm prologue); otherwise input B (q8 rows copied to smem).
// FLOATW: some segment holds F32/F16/BF16 rows, so normalised fp32 rows are kept too.
template <int MB, bool NORM, bool FLOATW>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  int8_t* sq = reinterpret_cast<int8_t*>(smem);
  float2* sds = reinterpret_cast<float2*>(smem + (size_t)MB * K);
  float* red = reinterpret_cast<float*>(sds + (size_t)MB * (K / 32));
  float* sx = red + 64;  // only when FLOATW
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // Which row does this warp own in row group g?  Groups are laid out per segment.
  auto locate = [&](int g, int& s, int& row) {
    int gs = 0;
    s = 0;
#pragma unroll 1
    for (; s < a.nseg; ++s) {
      int ng = (a.seg[s].rows + 7) >> 3;
      if (g < gs + ng) break;
      gs += ng;
    }
    row = (g - gs) * 8 + warp;
  };

  // weights do not depend on the predecessor: start them towards L2 now
  for (int g = blockIdx.x, it = 0; g < a.total_groups && it < 2; g += gridDim.x, ++it) {
    int s, row;
    locate(g, s, row);
    if (s < a.nseg && row < a.seg[s].rows && lane == 0 && (a.seg[s].row_bytes & 15) == 0)
      l2_prefetch_bulk(a.seg[s].w + (long)row * a.seg[s].row_bytes, (unsigned)a.seg[s].row_bytes);
  }
  pdl_wait();

  if (NORM) {
#pragma unroll 1
    for (int m = 0; m < MB; ++m) {
      const int ms = m < a.M ? m : a.M - 1;
      block_rmsnorm_q8(a.x + (long)ms * a.x_stride, a.gain, K, a.eps, sq + (long)m * K, sds + (long)m * (K / 32), red,
                       FLOATW ? sx + (long)m * K : nullptr);
    }
    if (a.xq_out && blockIdx.x == 0) {
      for (int i = tid; i < a.M * K / 16; i += 256)
        reinterpret_cast<uint4*>(a.xq_out)[i] = reinterpret_cast<const uint4*>(sq)[i];
      for (int i = tid; i < a.M * (K / 32); i += 256) a.xds_out[i] = sds[i];
    }
  } else {
    for (int i = tid; i < MB * K / 16; i += 256) {
      int m = (i * 16) / K;
      const int ms = m < a.M ? m : a.M - 1;
      reinterpret_cast<uint4*>(sq)[i] =
          reinterpret_cast<const uint4*>(a.xq + (long)ms * K)[i - m * (K / 16)];
    }
    for (int i = tid; i < MB * (K / 32); i += 256) {
      int m = i / (K / 32);
      const int ms = m < a.M ? m : a.M - 1;
      sds[i] = a.xds[(long)ms * (K / 32) + (i - m * (K / 32))];
    }
    __syncthreads();
  }
  pdl_launch();

  int out_base[4];
  {
    int o = 0;
    for (int s = 0; s < 4; ++s) { out_base[s] = o; if (s < a.nseg) o += a.seg[s].rows; }
  }

#pragma unroll 1
  for (int g = blockIdx.x; g < a.total_groups; g += gridDim.x) {
    int s, row;
    locate(g, s, row);
    if (s >= a.nseg || row >= a.seg[s].rows) continue;
    const uint8_t* wrow = a.seg[s].w + (long)row * a.seg[s].row_bytes;
    float acc[MB];
    switch (a.seg[s].wtype) {
      case WT_Q4_K: row_dot<Q4K, MB>(wrow, K, lane, sq, sds, acc); break;
      case WT_Q6_K: row_dot<Q6K, MB>(wrow, K, lane, sq, sds, acc); break;
      case WT_Q5_K: row_dot<Q5K, MB>(wrow, K, lane, sq, sds, acc); break;
      case WT_Q8_0: row_dot<Q80, MB>(wrow, K, lane, sq, sds, acc); break;
      default:
        if (FLOATW) row_dot_float<MB>(wrow, a.seg[s].wtype, K, lane, sx, acc);
        else {
#pragma unroll
          for (int m = 0; m < MB; ++m) acc[m] = __int_as_float(0x7fc00000);
        }
    }
    if (lane == 0) {
      const int col = out_base[s] + row;
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < a.M) {
          float v = acc[m];
          if (a.resid) v += a.resid[(long)m * a.resid_stride + col];
          a.out[(long)m * a.out_stride + col] = v;
        }
      }
    }
  }
}

static size_t gemv_smem(int MB, int K, bool floatw) {
  size_t b = (size_t)MB * K + (size_t)MB * (K / 32) * 8 + 64 * 4;
  if (floatw) b += (size_t)MB * K * 4;
  return b;
}

template <int MB, bool NORM, bool FLOATW>
static cudaError_t gemv_launch(const GemvArgs& a, int grid, cudaStream_t st) {
  size_t smem = gemv_smem(MB, a.K, FLOATW);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemv_kernel<MB, NORM, FLOATW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_set = true;
  }
  return launch(gemv_kernel<MB, NORM, FLOATW>, dim3(grid), dim3(256), smem, st, a);
}

template <bool NORM, bool FLOATW>
static cudaError_t gemv_dispatch_mb(const GemvArgs& a, int mb, int grid, cudaStream_t st) {
  switch (mb) {
    case 1: return gemv_launch<1, NORM, FLOATW>(a, grid, st);
    case 2: return gemv_launch<2, NORM, FLOATW>(a, grid, st);
    case 4: return gemv_launch<4, NORM, FLOATW>(a, grid, st);
    default: return gemv_launch<8, NORM, FLOATW>(a, grid, st);
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

void bl_set_pdl(int on) { g_use_pdl = on ? 1 : 0; }

// out[m, :] = (resid[m, :] +) W_seg * act(m), for up to four weight segments.
//   norm != 0: act = q8(RMSNorm(x[m]) * gain); else act = (xq, xds) given.
// Returns 0, a negative contract code, or a positive cudaError_t.
int bl_gemv(int nseg, const void* const* w, const int* rows, const int* wtypes, int K, int M,
            int norm, const float* x, long x_stride, const float* gain, float eps,
            const int8_t* xq, const float* xds,
            float* out, long out_stride, const float* resid, long resid_stride,
            int8_t* xq_out, float* xds_out, unsigned* fault, int layer, int sm_count, cudaStream_t st) {
  BL_REQUIRE(nseg >= 1 && nseg <= 4, BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && M <= 8, BL_ERR_SHAPE);
  BL_REQUIRE(K > 0 && K % 256 == 0, BL_ERR_SHAPE);
  GemvArgs a = {};
  a.nseg = nseg;
  bool floatw = false;
  int groups = 0;
  for (int s = 0; s < nseg; ++s) {
    long rb = resident_row_bytes(wtypes[s], K);
    BL_REQUIRE(rb > 0, BL_ERR_TYPE);
    BL_REQUIRE(((uintptr_t)w[s] & 15) == 0, BL_ERR_ALIGN);
    a.seg[s] = GemvSeg{(const uint8_t*)w[s], rows[s], wtypes[s], rb};
    if (wtypes[s] == WT_F32 || wtypes[s] == WT_F16 || wtypes[s] == WT_BF16) floatw = true;
    groups += (rows[s] + 7) / 8;
  }
  BL_REQUIRE(!(floatw && !norm), BL_ERR_TYPE);
  a.total_groups = groups;
  a.K = K; a.M = M;
  a.x = x; a.x_stride = x_stride; a.gain = gain; a.eps = eps;
  a.xq = xq; a.xds = (const float2*)xds;
  a.out = out; a.out_stride = out_stride; a.resid = resid; a.resid_stride = resid_stride;
  a.xq_out = xq_out; a.xds_out = (float2*)xds_out;
  a.fault = fault; a.layer = layer;
  int mb = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  BL_REQUIRE(gemv_smem(mb, K, floatw) <= 200 * 1024, BL_ERR_LIMIT);
  int grid = groups < sm_count * 4 ? groups : sm_count * 4;
  cudaError_t e;
  if (norm) e = floatw ? gemv_dispatch_mb<true, true>(a, mb, grid, st) : gemv_dispatch_mb<true, false>(a, mb, grid, st);
  else e = gemv_dispatch_mb<false, false>(a, mb, grid, st);
  return (int)e;
}

}  // extern "C"
