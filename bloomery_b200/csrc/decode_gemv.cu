// Quantised GEMV for the decode chain (m <= 8 activation rows), weights dequantised
// in registers and dotted with dp4a against q8 activations.
//
// Decode at one row is latency-bound, not bandwidth-bound, so the kernel is shaped to
// keep one DRAM round trip on the critical path:
//   * a warp owns R weight rows at a time and issues every load of its first tile into
//     registers BEFORE griddepcontrol.wait and before the activation prologue, so under
//     programmatic dependent launch the weight stream of kernel N+1 overlaps the tail
//     of kernel N and its own RMSNorm prologue;
//   * the prologue needs no second pass: q8 codes of x*gain do not depend on the RMS
//     scale (it is a per-row scalar), so sum-of-squares and quantisation run in one
//     sweep and the scale multiplies the finished dot products;
//   * blocks are type-uniform (a tile of 8*R rows never straddles two weight segments),
//     which keeps block-wide barriers out of divergent code.
// One launch covers up to four weight segments that share an input (q, k, v).
//
// Behavioural counterpart of q4k_gemv/q6k_gemv(_mcol) in crates/gpu/src/lib.rs:1604-1632
// and qwen3moe_qkv_q4k / qwen3moe_o_resid_q4k in crates/gpu/src/arch/qwen3moe/proj.rs:
// fixed lane split and a fixed xor-butterfly, so reruns are bit-identical and each row of
// an m-row call equals its own 1-row call.
#include "gemv_common.cuh"

namespace bl {

int g_use_pdl = 1;

// ---- the rows of one warp ---------------------------------------------------------------
// A warp owns rows [r_lo, r_hi) of its segment and walks them R at a time; every load of a
// chunk is issued before anything is computed.  C = units per lane per inner step.
// `between` runs once per block, after the very first loads are in flight.
template <class T, int MB, int R, int C, class Between>
__device__ __forceinline__ void rows_q(const GemvArgs& a, const GemvSeg& s, int r_lo, int r_hi, int out_col0,
                                       const int8_t* sq, const float2* sds, const float* s_scale, Between&& between) {
  using U = Unit<T>;
  const int K = a.K, lane = threadIdx.x & 31;
  const int nunits = K / 64;
  const unsigned push_epoch = a.push.n_ranks > 0 ? site_epoch(a.push.step, a.push.sites_per_step, a.push.site_index) : 0u;
  for (int r0 = r_lo; r0 < r_hi || r0 == r_lo; r0 += R) {
    float acc[R][MB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
    for (int base = 0; base < nunits; base += 32 * C) {
      typename U::Regs regs[R][C];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int u = base + c * 32 + lane;
          // rows past the end re-read the segment's last row (their result is dropped)
          const int rr = min(r0 + r, s.rows - 1);
          if (u < nunits) U::loadu(s.w + (long)rr * s.row_bytes, u, K, regs[r][c]);
        }
      between();
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int u = base + c * 32 + lane;
        if (u < nunits) {
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            // the block's activation rows sit in the conflict-free chunk layout of its weight type
            ActRegs act;
            StagedAct<T>::load(sq + (long)m * K, sds + (long)m * (K / 32), u, nunits, act);
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r][m] += ActOf<T>::dot(regs[r][c], u, act);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MB; ++m) acc[r][m] = warp_sum(acc[r][m]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r0 + r < r_hi) {
          const int col = out_col0 + r0 + r;
#pragma unroll
          for (int m = 0; m < MB; ++m)
            if (m < a.M) {
              float v = acc[r][m] * s_scale[m];
              if (a.push.n_ranks > 0) { push_store(a.push, push_epoch, (long)m * a.out_stride + col, v); continue; }
              if (a.resid) v += a.resid[(long)m * a.resid_stride + col];
              a.out[(long)m * a.out_stride + col] = v;
            }
        }
      }
    }
    if (r0 + R >= r_hi) break;
  }
}

// float weights (F32 / F16 / BF16) against fp32 x*gain rows
template <int MB, int R, class Between>
__device__ __forceinline__ void rows_f(const GemvArgs& a, const GemvSeg& s, int r_lo, int r_hi, int out_col0,
                                       const float* sx, const float* s_scale, Between&& between) {
  const int K = a.K, lane = threadIdx.x & 31;
  const unsigned push_epoch = a.push.n_ranks > 0 ? site_epoch(a.push.step, a.push.sites_per_step, a.push.site_index) : 0u;
  for (int r0 = r_lo; r0 < r_hi || r0 == r_lo; r0 += R) {
    float acc[R][MB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
    for (int i = lane * 8; i < K; i += 256) {
      float wv[R][8];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint8_t* row = s.w + (long)min(r0 + r, s.rows - 1) * s.row_bytes;
        if (s.wtype == WT_F32) {
          float4 p = __ldg(reinterpret_cast<const float4*>(row) + i / 4), q = __ldg(reinterpret_cast<const float4*>(row) + i / 4 + 1);
          wv[r][0] = p.x; wv[r][1] = p.y; wv[r][2] = p.z; wv[r][3] = p.w; wv[r][4] = q.x; wv[r][5] = q.y; wv[r][6] = q.z; wv[r][7] = q.w;
        } else {
          uint4 p = __ldg(reinterpret_cast<const uint4*>(row) + i / 8);
          const uint32_t ws[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = (s.wtype == WT_F16) ? __half22float2(*reinterpret_cast<const __half2*>(&ws[j]))
                                           : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ws[j]));
            wv[r][2 * j] = f.x; wv[r][2 * j + 1] = f.y;
          }
        }
      }
      between();
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        const float4 x0 = *reinterpret_cast<const float4*>(sx + (long)m * K + i);
        const float4 x1 = *reinterpret_cast<const float4*>(sx + (long)m * K + i + 4);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float t = acc[r][m];
          t = fmaf(wv[r][0], x0.x, t); t = fmaf(wv[r][1], x0.y, t); t = fmaf(wv[r][2], x0.z, t); t = fmaf(wv[r][3], x0.w, t);
          t = fmaf(wv[r][4], x1.x, t); t = fmaf(wv[r][5], x1.y, t); t = fmaf(wv[r][6], x1.z, t); t = fmaf(wv[r][7], x1.w, t);
          acc[r][m] = t;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MB; ++m) acc[r][m] = warp_sum(acc[r][m]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r0 + r < r_hi) {
          const int col = out_col0 + r0 + r;
#pragma unroll
          for (int m = 0; m < MB; ++m)
            if (m < a.M) {
              float v = acc[r][m] * s_scale[m];
              if (a.push.n_ranks > 0) { push_store(a.push, push_epoch, (long)m * a.out_stride + col, v); continue; }
              if (a.resid) v += a.resid[(long)m * a.resid_stride + col];
              a.out[(long)m * a.out_stride + col] = v;
            }
        }
    }
    if (r0 + R >= r_hi) break;
  }
}

// FAM: 0 = ggml integer-dot types, 1 = those plus float rows, 2 = block-scaled float planes (NVFP4, FP8).
// One kernel per family keeps the register budget of the K-quant bodies free of the plane decoders.
template <int MB, int R, int C, bool NORM, int FAM>
__global__ void __launch_bounds__(256, 2) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  int8_t* sq = reinterpret_cast<int8_t*>(smem);
  float2* sds = reinterpret_cast<float2*>(smem + (size_t)MB * K);
  double* red = reinterpret_cast<double*>(sds + (size_t)MB * (K / 32));
  float* s_scale = reinterpret_cast<float*>(red + MB * 8);
  float* sx = s_scale + 8;  // only when FLOATW

  if (a.n_pf > 0 && threadIdx.x == 0) prefetch_spans_l2(a.pf_ptr, a.pf_bytes, a.n_pf);
  int si = 0, col0 = 0;
#pragma unroll
  for (int q = 1; q < 4; ++q)
    if (q < a.nseg && (int)blockIdx.x >= a.seg[q].blk0) { si = q; }
  for (int q = 0; q < si; ++q) col0 += a.seg[q].rows;
  // a block serves one weight type: its q8 activation rows take the chunk layout that type's units read without
  // bank conflicts (act_chunk_pos); float rows read the fp32 copy instead
  const int act_layout = staged_layout(a.seg[si].wtype);
  bool ready = false;
  auto between = [&]() {
    if (!ready) {
      pdl_wait();
      if (NORM) prologue_norm<MB, FAM == 1>(a, sq, sds, sx, s_scale, red, act_layout);
      else prologue_q8in<MB>(a, sq, sds, s_scale, act_layout);
      pdl_launch();
      ready = true;
    }
  };
  {
    const GemvSeg& s = a.seg[si];
    // even split of the segment's rows over its warps
    const int W = s.nblk * 8, wg = ((int)blockIdx.x - s.blk0) * 8 + (threadIdx.x >> 5);
    const int rpw = (s.rows + W - 1) / W;
    const int r_lo = min(s.rows, wg * rpw), r_hi = min(s.rows, r_lo + rpw);
    if constexpr (FAM == 2) {
      switch (s.wtype) {
        case WT_NVFP4: rows_q<NvFp4, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_FP8_B128: rows_q<Fp8B128, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q2_K: rows_q<Q2K, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q3_K: rows_q<Q3K, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q4_0: rows_q<Q40, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q4_1: rows_q<Q41, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q5_0: rows_q<Q50, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q5_1: rows_q<Q51, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        default: break;
      }
    } else {
      switch (s.wtype) {
        case WT_Q4_K: rows_q<Q4K, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q6_K: rows_q<Q6K, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q5_K: rows_q<Q5K, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q8_0: rows_q<Q80, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        case WT_Q8_F32: rows_q<Q8F, MB, R, C>(a, s, r_lo, r_hi, col0, sq, sds, s_scale, between); break;
        default:
          if (FAM == 1) rows_f<MB, R>(a, s, r_lo, r_hi, col0, sx, s_scale, between);
      }
    }
  }
  between();
}

static size_t gemv_smem(int MB, int K, bool floatw) {
  size_t b = (size_t)MB * K + (size_t)MB * (K / 32) * 8 + MB * 8 * 8 + 8 * 4;
  if (floatw) b += (size_t)MB * K * 4;
  return b;
}

template <int MB, int R, int C, bool NORM, int FAM>
static cudaError_t gemv_launch(const GemvArgs& a, int grid, cudaStream_t st) {
  size_t smem = gemv_smem(MB, a.K, FAM == 1);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemv_kernel<MB, R, C, NORM, FAM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_set = true;
  }
  return launch(gemv_kernel<MB, R, C, NORM, FAM>, dim3(grid), dim3(256), smem, st, a);
}

template <int R, int C, bool NORM, int FAM>
static cudaError_t gemv_dispatch_mb(const GemvArgs& a, int mb, int grid, cudaStream_t st) {
  switch (mb) {
    case 1: return gemv_launch<1, R, C, NORM, FAM>(a, grid, st);
    case 2: return gemv_launch<2, R, C, NORM, FAM>(a, grid, st);
    case 4: return gemv_launch<4, R, C, NORM, FAM>(a, grid, st);
    default: return gemv_launch<8, R, C, NORM, FAM>(a, grid, st);
  }
}

template <bool NORM, int FAM>
static cudaError_t gemv_dispatch_shape(const GemvArgs& a, int mb, int R, int C, int grid, cudaStream_t st) {
  if (C == 2) return gemv_dispatch_mb<1, 2, NORM, FAM>(a, mb, grid, st);
  if (R >= 3) return gemv_dispatch_mb<3, 1, NORM, FAM>(a, mb, grid, st);
  if (R == 2) return gemv_dispatch_mb<2, 1, NORM, FAM>(a, mb, grid, st);
  return gemv_dispatch_mb<1, 1, NORM, FAM>(a, mb, grid, st);
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
            const void* red_desc, const void* push_desc, unsigned* fault, int layer, int sm_count,
            int n_pf, const void* const* pf_ptr, const long* pf_bytes, cudaStream_t st) {
  BL_REQUIRE(nseg >= 1 && nseg <= 4, BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && M <= 8, BL_ERR_SHAPE);
  BL_REQUIRE(K > 0 && K % 256 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(!norm || (K % 2048 == 0 || K % 64 == 0), BL_ERR_SHAPE);
  BL_REQUIRE(n_pf >= 0 && n_pf <= 6, BL_ERR_SHAPE);
  GemvArgs a = {};
  a.n_pf = n_pf;
  for (int i = 0; i < n_pf; ++i) {
    BL_REQUIRE(((uintptr_t)pf_ptr[i] & 15) == 0 && pf_bytes[i] >= 0, BL_ERR_ALIGN);
    a.pf_ptr[i] = (const uint8_t*)pf_ptr[i]; a.pf_bytes[i] = pf_bytes[i];
  }
  a.nseg = nseg;
  bool floatw = false, planes = false, ggml = false;
  double total_bytes = 0;
  long rbs[4];
  for (int s = 0; s < nseg; ++s) {
    rbs[s] = resident_row_bytes(wtypes[s], K);
    BL_REQUIRE(rbs[s] > 0, BL_ERR_TYPE);
    BL_REQUIRE(((uintptr_t)w[s] & 15) == 0, BL_ERR_ALIGN);
    BL_REQUIRE(rows[s] >= 1, BL_ERR_SHAPE);
    total_bytes += (double)rows[s] * rbs[s];
    if (wtypes[s] == WT_F32 || wtypes[s] == WT_F16 || wtypes[s] == WT_BF16) floatw = true;
    else if (wtypes[s] == WT_NVFP4 || wtypes[s] == WT_FP8_B128 || wtypes[s] == WT_Q4_0 || wtypes[s] == WT_Q4_1 ||
             wtypes[s] == WT_Q5_0 || wtypes[s] == WT_Q5_1 || wtypes[s] == WT_Q2_K || wtypes[s] == WT_Q3_K) planes = true;
    else ggml = true;
  }
  BL_REQUIRE(!(floatw && !norm), BL_ERR_TYPE);
  BL_REQUIRE(!(planes && (floatw || ggml)), BL_ERR_TYPE);   // one family per call
  const int mb = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  // One wave: at most two resident blocks per SM; each segment gets a share of the blocks
  // in proportion to its bytes, never more blocks than it has 8-row groups.
  const int budget = 2 * sm_count;
  const int C = (K / 64 > 32) ? 2 : 1;
  int grid = 0, rpw_max = 1;
  for (int s = 0; s < nseg; ++s) {
    int nb = (int)((double)budget * ((double)rows[s] * rbs[s] / total_bytes));
    const int cap = (rows[s] + 7) / 8;
    nb = nb < 1 ? 1 : nb > cap ? cap : nb;
    a.seg[s] = GemvSeg{(const uint8_t*)w[s], rows[s], wtypes[s], grid, nb, rbs[s]};
    grid += nb;
    const int rpw = (rows[s] + nb * 8 - 1) / (nb * 8);
    rpw_max = rpw > rpw_max ? rpw : rpw_max;
  }
  int R = C == 2 ? 1 : (rpw_max >= 3 ? 3 : rpw_max);
  if (mb == 8 && R > 2) R = 2;
  a.K = K; a.M = M;
  a.x = x; a.x_stride = x_stride; a.gain = gain; a.eps = eps;
  a.xq = xq; a.xds = (const float2*)xds;
  a.out = out; a.out_stride = out_stride; a.resid = resid; a.resid_stride = resid_stride;
  a.fault = fault; a.layer = layer;
  if (red_desc) { a.red = *(const ReduceIn*)red_desc; BL_REQUIRE(norm && a.red.n_ranks <= kMaxRanks && a.red.H == K, BL_ERR_SHAPE); }
  if (push_desc) { a.push = *(const PushOut*)push_desc; BL_REQUIRE(a.push.n_ranks <= kMaxRanks, BL_ERR_SHAPE); }
  BL_REQUIRE(gemv_smem(mb, K, floatw) <= 200 * 1024, BL_ERR_LIMIT);
  cudaError_t e;
  if (planes) e = norm ? gemv_dispatch_shape<true, 2>(a, mb, R, C, grid, st) : gemv_dispatch_shape<false, 2>(a, mb, R, C, grid, st);
  else if (norm) e = floatw ? gemv_dispatch_shape<true, 1>(a, mb, R, C, grid, st) : gemv_dispatch_shape<true, 0>(a, mb, R, C, grid, st);
  else e = gemv_dispatch_shape<false, 0>(a, mb, R, C, grid, st);
  return (int)e;
}

}  // extern "C"
