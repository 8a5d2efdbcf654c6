// Decode-time mixture-of-experts chain (m <= 8 rows), expert ids read on the device:
//   1. router           RMSNorm prologue + fp32 router GEMV + top-k by the last-arriving
//                       block (softmax / renormalised, or sigmoid + selection bias with
//                       optional group-limited choice); publishes the q8 normed rows
//   2. gate_up_sel      gate·x and up·x of the chosen experts, SwiGLU, q8 of the result
//   3. down_combine     y = resid + sum_j w_j * down_j(act_j), slots in ascending order
//
// Contracts followed from the reference: softmax router math and tie rule
// (crates/gpu/src/route_softmax.rs:28-58: max, exp f32, f64 sum, top-k desc prob with
// ties to the smaller id, chosen probs renormalised; non-finite logit -> router fault,
// NaN weights); sigmoid "noaux" rule where the bias steers the choice only
// (crates/model/src/arch/noaux.rs:23-94); combine order (crates/gpu/src/arch/qwen3moe/
// experts.rs:36-45); the elsewhere-sentinel for slots another tier serves
// (crates/gpu/src/kquant/sel.rs doc).  The completion counter instead of a grid barrier
// is the reference's measured choice (docs/gpu-design.md:52-64).
#include "common.cuh"

namespace bl {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

struct RouterArgs {
  const float* x; long x_stride;       // [M, K] residual stream
  const float* gain; float eps;
  const uint8_t* w; int wtype;         // [E, K] F32 / F16 / BF16
  const float* bias;                   // [E] selection bias (sigmoid mode) or null
  int K, E, M, top_k;
  int mode;                            // 0 softmax, 1 sigmoid
  int renorm;                          // renormalise chosen weights
  float scale;                         // weights multiplier after renormalisation
  int n_group, topk_group;             // group-limited routing (1,1 = off)
  float* logits;                       // [M, E] scratch
  int* ids;                            // [M, top_k]
  float* wts;                          // [M, top_k]
  int8_t* xq_out; float2* xds_out;     // q8 of the normed rows [M, K]
  float* xn_out;                       // optional fp32 normed rows [M, K]
  unsigned* counter;                   // completion ticket, zero at rest
  unsigned* heat;                      // optional [E] routed-count histogram (residency rule)
  unsigned* fault; int layer;
};

template <int MB>
__global__ void __launch_bounds__(256) router_kernel(const RouterArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  float* sx = reinterpret_cast<float*>(smem);                 // [MB][K]
  int8_t* sq = reinterpret_cast<int8_t*>(sx + (size_t)MB * K);  // [MB][K]
  float2* sds = reinterpret_cast<float2*>(sq + (size_t)MB * K);
  float* red = reinterpret_cast<float*>(sds + (size_t)MB * (K / 32));
  __shared__ unsigned s_ticket;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  {  // router rows towards L2 ahead of the dependency wait
    int e = blockIdx.x * 8 + warp;
    long rb = resident_row_bytes(a.wtype, K);
    if (e < a.E && lane == 0)
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.w + e * rb), "r"((unsigned)rb) : "memory");
  }
  pdl_wait();
#pragma unroll 1
  for (int m = 0; m < MB; ++m) {
    const int ms = m < a.M ? m : a.M - 1;
    block_rmsnorm_q8(a.x + (long)ms * a.x_stride, a.gain, K, a.eps, sq + (long)m * K, sds + (long)m * (K / 32), red,
                     sx + (long)m * K);
  }
  pdl_launch();
  // every block holds the same normed rows; each publishes a slice of the q8 form
  {
    const int nb32 = K / 32;
    for (int b = blockIdx.x; b < nb32; b += gridDim.x) {
      for (int m = 0; m < a.M; ++m) {
        if (tid < 8) reinterpret_cast<uint32_t*>(a.xq_out + (long)m * K + b * 32)[tid] =
            reinterpret_cast<const uint32_t*>(sq + (long)m * K + b * 32)[tid];
        if (tid == 8) a.xds_out[(long)m * nb32 + b] = sds[(long)m * nb32 + b];
        if (a.xn_out && tid >= 32 && tid < 64) a.xn_out[(long)m * K + b * 32 + (tid - 32)] = sx[(long)m * K + b * 32 + (tid - 32)];
      }
    }
  }
  const int e = blockIdx.x * 8 + warp;
  if (e < a.E) {
    const uint8_t* row = a.w + (long)e * resident_row_bytes(a.wtype, K);
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0.f;
    for (int i = lane * 4; i < K; i += 128) {
      float w0, w1, w2, w3;
      if (a.wtype == WT_F32) {
        float4 v = __ldg(reinterpret_cast<const float4*>(row) + i / 4);
        w0 = v.x; w1 = v.y; w2 = v.z; w3 = v.w;
      } else if (a.wtype == WT_F16) {
        uint2 v = __ldg(reinterpret_cast<const uint2*>(row) + i / 4);
        float2 p = __half22float2(*reinterpret_cast<__half2*>(&v.x));
        float2 q = __half22float2(*reinterpret_cast<__half2*>(&v.y));
        w0 = p.x; w1 = p.y; w2 = q.x; w3 = q.y;
      } else {
        uint2 v = __ldg(reinterpret_cast<const uint2*>(row) + i / 4);
        float2 p = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v.x));
        float2 q = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v.y));
        w0 = p.x; w1 = p.y; w2 = q.x; w3 = q.y;
      }
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        const float4 xv = *reinterpret_cast<const float4*>(sx + (long)m * K + i);
        acc[m] = fmaf(w0, xv.x, fmaf(w1, xv.y, fmaf(w2, xv.z, fmaf(w3, xv.w, acc[m]))));
      }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      float v = warp_sum(acc[m]);
      if (lane == 0 && m < a.M) a.logits[(long)m * a.E + e] = v;
    }
  }
  // completion ticket: the last block to arrive routes every row
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(a.counter, 1u);
  __syncthreads();
  if (s_ticket != gridDim.x - 1) return;
  __threadfence();
  if (tid == 0) *a.counter = 0u;  // at rest again for the next replay

  constexpr int EPL = kMaxExperts / 32;  // experts per lane, strided: e = lane + 32 i
  for (int m = warp; m < a.M; m += 8) {
    float sc[EPL];     // choice score
    float wv[EPL];     // weight value
    bool finite = true;
    float mxl = -INFINITY;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      int ee = lane + 32 * i;
      float v = ee < a.E ? __ldcg(a.logits + (long)m * a.E + ee) : -INFINITY;
      if (ee < a.E && !isfinite(v)) finite = false;
      sc[i] = v;
      mxl = fmaxf(mxl, v);
    }
    finite = __all_sync(0xffffffffu, finite);
    if (!finite) {
      if (lane == 0) raise_fault(a.fault, a.layer, FS_ROUTER);
      if (lane < a.top_k) { a.wts[(long)m * a.top_k + lane] = __int_as_float(0x7fc00000); a.ids[(long)m * a.top_k + lane] = 0; }
      continue;
    }
    if (a.mode == 0) {
      mxl = warp_max(mxl);
      double part = 0.0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        float ex = (lane + 32 * i < a.E) ? expf(sc[i] - mxl) : 0.f;
        wv[i] = ex;
        part += (double)ex;
      }
      double tot = warp_sum_d(part);
#pragma unroll
      for (int i = 0; i < EPL; ++i) { wv[i] = wv[i] / (float)tot; sc[i] = (lane + 32 * i < a.E) ? wv[i] : -INFINITY; }
    } else {
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        int ee = lane + 32 * i;
        float sg = 1.0f / (1.0f + expf(-sc[i]));
        wv[i] = sg;
        sc[i] = ee < a.E ? sg + (a.bias ? a.bias[ee] : 0.f) : -INFINITY;
      }
    }
    // group-limited choice: keep the topk_group groups with the largest sum of their two best scores
    if (a.n_group > 1) {
      const int gsz = a.E / a.n_group;
      float gscore[16];
      for (int g = 0; g < a.n_group && g < 16; ++g) {
        float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          int ee = lane + 32 * i;
          if (ee < a.E && ee / gsz == g) { float v = sc[i]; if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v; }
        }
        // merge (b1, b2) pairs across lanes
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
          float n1 = fmaxf(b1, o1);
          float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
          b1 = n1; b2 = n2;
        }
        gscore[g] = b1 + b2;
      }
      unsigned keep = 0;
      for (int t = 0; t < a.topk_group; ++t) {
        int best = -1; float bv = -INFINITY;
        for (int g = 0; g < a.n_group && g < 16; ++g)
          if (!((keep >> g) & 1) && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
        if (best >= 0) keep |= 1u << best;
      }
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        int ee = lane + 32 * i;
        if (ee < a.E && !((keep >> (ee / gsz)) & 1)) sc[i] = -INFINITY;
      }
    }
    // top-k: k rounds of warp arg-max, larger score first, ties to the smaller id
    int my_id = 0; float my_w = 0.f;
    double wsum = 0.0;
    for (int t = 0; t < a.top_k; ++t) {
      float bv = -INFINITY; int bi = 0x7fffffff; float bw = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        int ee = lane + 32 * i;
        if (ee < a.E && (sc[i] > bv || (sc[i] == bv && ee < bi))) { bv = sc[i]; bi = ee; bw = wv[i]; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        float ow = __shfl_xor_sync(0xffffffffu, bw, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bw = ow; }
      }
      if ((bi & 31) == lane) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) if (i == (bi >> 5)) sc[i] = -INFINITY;
      }
      if (lane == t) { my_id = bi; my_w = bw; }
      wsum += (double)bw;  // slot order, same in every lane
    }
    if (lane < a.top_k) {
      float w = my_w;
      if (a.renorm) w = w / (float)wsum;
      w *= a.scale;
      a.ids[(long)m * a.top_k + lane] = my_id;
      a.wts[(long)m * a.top_k + lane] = w;
      if (a.heat) atomicAdd(a.heat + my_id, 1u);
    }
  }
}

// ------------------------------------------------------------------------------------
// gate·up·SwiGLU over device-side expert ids
// grid (I/32, n_used, M), 256 threads: warp w computes activation rows 4w..4w+3 of the chunk
// ------------------------------------------------------------------------------------
struct GateUpArgs {
  const int8_t* xq; const float2* xds;   // [M, K] q8
  const int* ids;                        // [M, n_used]
  const int* slot_map;                   // optional [E]: expert id -> resident slot (or kExpertElsewhere)
  const uint8_t* gate; const uint8_t* up; int gtype, utype;   // stacks [E_slots, I, K]
  int K, I, E, n_used, M;
  int8_t* actq; float2* actds;           // [M, n_used, I] q8
  float* act_f32;                        // optional fp32 copy
  unsigned* fault; int layer;
};

template <class TG, class TU>
__device__ __forceinline__ void gate_up_rows(const uint8_t* g0, const uint8_t* u0, long grb, long urb, int K, int lane,
                                             const int8_t* sq, const float2* sds, float (&gacc)[4], float (&uacc)[4]) {
  using UG = Unit<TG>; using UU = Unit<TU>;
  const int nunits = K / 64;
#pragma unroll
  for (int r = 0; r < 4; ++r) { gacc[r] = 0.f; uacc[r] = 0.f; }
  for (int u = lane; u < nunits; u += 32) {
    typename UG::Regs rg[4];
    typename UU::Regs ru[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) { UG::loadu(g0 + r * grb, u, K, rg[r]); UU::loadu(u0 + r * urb, u, K, ru[r]); }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      gacc[r] += UG::dotu(rg[r], u, reinterpret_cast<const uint32_t*>(sq), reinterpret_cast<const F2*>(sds));
      uacc[r] += UU::dotu(ru[r], u, reinterpret_cast<const uint32_t*>(sq), reinterpret_cast<const F2*>(sds));
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) { gacc[r] = warp_sum(gacc[r]); uacc[r] = warp_sum(uacc[r]); }
}

__global__ void __launch_bounds__(256) gate_up_sel_kernel(const GateUpArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int K = a.K;
  int8_t* sq = reinterpret_cast<int8_t*>(smem);
  float2* sds = reinterpret_cast<float2*>(smem + K);
  __shared__ float s_act[32];
  const int chunk = blockIdx.x, j = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_launch();
  int e = a.ids[(long)m * a.n_used + j];
  const long ob = ((long)m * a.n_used + j) * a.I + chunk * 32;
  bool skip = false, bad = false;
  if (e == kExpertElsewhere) skip = true;
  else if (e < 0 || e >= a.E) { skip = true; bad = true; }
  else if (a.slot_map) { e = a.slot_map[e]; if (e < 0) skip = true; }
  if (skip) {
    if (bad && tid == 0 && chunk == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID);
    if (tid < 32) {
      a.actq[ob + tid] = 0;
      if (a.act_f32) a.act_f32[ob + tid] = bad ? __int_as_float(0x7fc00000) : 0.f;
    }
    if (tid == 0) a.actds[ob / 32] = bad ? make_float2(__int_as_float(0x7fc00000), 0.f) : make_float2(0.f, 0.f);
    return;
  }
  for (int i = tid; i < K / 16; i += 256)
    reinterpret_cast<uint4*>(sq)[i] = reinterpret_cast<const uint4*>(a.xq + (long)m * K)[i];
  for (int i = tid; i < K / 32; i += 256) sds[i] = a.xds[(long)m * (K / 32) + i];
  __syncthreads();
  const long grb = resident_row_bytes(a.gtype, K), urb = resident_row_bytes(a.utype, K);
  const long row0 = (long)e * a.I + chunk * 32 + warp * 4;
  const uint8_t* g0 = a.gate + row0 * grb;
  const uint8_t* u0 = a.up + row0 * urb;
  float gacc[4], uacc[4];
  const int key = a.gtype * 64 + a.utype;
  switch (key) {
    case WT_Q4_K * 64 + WT_Q4_K: gate_up_rows<Q4K, Q4K>(g0, u0, grb, urb, K, lane, sq, sds, gacc, uacc); break;
    case WT_Q5_K * 64 + WT_Q5_K: gate_up_rows<Q5K, Q5K>(g0, u0, grb, urb, K, lane, sq, sds, gacc, uacc); break;
    case WT_Q6_K * 64 + WT_Q6_K: gate_up_rows<Q6K, Q6K>(g0, u0, grb, urb, K, lane, sq, sds, gacc, uacc); break;
    case WT_Q8_0 * 64 + WT_Q8_0: gate_up_rows<Q80, Q80>(g0, u0, grb, urb, K, lane, sq, sds, gacc, uacc); break;
    default:
#pragma unroll
      for (int r = 0; r < 4; ++r) { gacc[r] = __int_as_float(0x7fc00000); uacc[r] = 0.f; }
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float g = gacc[r];
      s_act[warp * 4 + r] = (g / (1.0f + expf(-g))) * uacc[r];
    }
  }
  __syncthreads();
  if (warp == 0) {
    float v = s_act[lane];
    float d, s;
    int8_t q = q8_lane(v, d, s);
    a.actq[ob + lane] = q;
    if (a.act_f32) a.act_f32[ob + lane] = v;
    if (lane == 0) a.actds[ob / 32] = make_float2(d, s);
  }
}

// ------------------------------------------------------------------------------------
// down projection of every chosen expert + router-weighted sum + residual, one launch
// grid (H/8, M), 256 threads: warp w owns output row 8*blockIdx.x + w
// ------------------------------------------------------------------------------------
struct DownArgs {
  const int8_t* actq; const float2* actds;  // [M, n_used, I]
  const int* ids; const float* wts;         // [M, n_used]
  const int* slot_map;
  const uint8_t* down; int dtype;           // stack [E_slots, H, I]
  int I, H, E, n_used, M;
  const float* resid; long resid_stride;    // [M, H] or null
  const float* extra; long extra_stride;    // optional addend (shared expert / host leg sum)
  float* out; long out_stride;
  unsigned* fault; int layer;
};

template <class T>
__device__ __forceinline__ float down_row(const DownArgs& a, int m, int d, int lane, const int8_t* sq, const float2* sds,
                                          const int* s_slot, const float* s_w) {
  using U = Unit<T>;
  const int upe = a.I / 64;              // units per expert row
  const int total = a.n_used * upe;
  const long rb = resident_row_bytes(T::kType, a.I);
  // per-slot partial sums kept separate, then added in ascending slot order
  float part[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) part[j] = 0.f;
  for (int t = lane; t < total; t += 32) {
    const int j = t / upe, u = t - j * upe;
    const int e = s_slot[j];
    if (e < 0) continue;
    typename U::Regs r;
    U::loadu(a.down + ((long)e * a.H + d) * rb, u, a.I, r);
    float v = U::dotu(r, u, reinterpret_cast<const uint32_t*>(sq + (long)j * a.I),
                      reinterpret_cast<const F2*>(sds + (long)j * (a.I / 32)));
#pragma unroll
    for (int jj = 0; jj < kMaxTopK; ++jj) if (jj == j) part[jj] += v;
  }
  float y = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) {
    if (j < a.n_used) y = fmaf(s_w[j], warp_sum(part[j]), y);
  }
  return y;
}

__global__ void __launch_bounds__(256) down_combine_kernel(const DownArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  int8_t* sq = reinterpret_cast<int8_t*>(smem);                              // [n_used][I]
  float2* sds = reinterpret_cast<float2*>(smem + (size_t)a.n_used * a.I);    // [n_used][I/32]
  __shared__ int s_slot[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  const int m = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_launch();
  if (tid < a.n_used) {
    int e = a.ids[(long)m * a.n_used + tid];
    float w = a.wts[(long)m * a.n_used + tid];
    if (e == kExpertElsewhere) e = -1;
    else if (e < 0 || e >= a.E) { e = -2; }
    else if (a.slot_map) { e = a.slot_map[e]; if (e < 0) e = -1; }
    s_slot[tid] = e; s_w[tid] = w;
  }
  const long n16 = (long)a.n_used * a.I / 16;
  for (long i = tid; i < n16; i += 256)
    reinterpret_cast<uint4*>(sq)[i] = reinterpret_cast<const uint4*>(a.actq + (long)m * a.n_used * a.I)[i];
  const long nds = (long)a.n_used * (a.I / 32);
  for (long i = tid; i < nds; i += 256) sds[i] = a.actds[(long)m * nds + i];
  __syncthreads();
  bool bad = false;
  for (int j = 0; j < a.n_used; ++j) bad |= (s_slot[j] == -2);
  const int d = blockIdx.x * 8 + warp;
  if (d >= a.H) return;
  float y;
  switch (a.dtype) {
    case WT_Q4_K: y = down_row<Q4K>(a, m, d, lane, sq, sds, s_slot, s_w); break;
    case WT_Q6_K: y = down_row<Q6K>(a, m, d, lane, sq, sds, s_slot, s_w); break;
    case WT_Q5_K: y = down_row<Q5K>(a, m, d, lane, sq, sds, s_slot, s_w); break;
    case WT_Q8_0: y = down_row<Q80>(a, m, d, lane, sq, sds, s_slot, s_w); break;
    default: y = __int_as_float(0x7fc00000);
  }
  if (lane == 0) {
    if (bad) { y = __int_as_float(0x7fc00000); if (d == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID); }
    if (a.extra) y += a.extra[(long)m * a.extra_stride + d];
    if (a.resid) y += a.resid[(long)m * a.resid_stride + d];
    a.out[(long)m * a.out_stride + d] = y;
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

int bl_router(const float* x, long x_stride, const float* gain, float eps, const void* w, int wtype, const float* bias,
              int K, int E, int M, int top_k, int mode, int renorm, float scale, int n_group, int topk_group,
              float* logits, int* ids, float* wts, int8_t* xq_out, float* xds_out, float* xn_out, unsigned* counter,
              unsigned* heat, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(E >= 1 && E <= kMaxExperts, BL_ERR_LIMIT);
  BL_REQUIRE(top_k >= 1 && top_k <= kMaxTopK && top_k <= E, BL_ERR_LIMIT);
  BL_REQUIRE(K % 128 == 0 && M >= 1 && M <= 8, BL_ERR_SHAPE);
  BL_REQUIRE(wtype == WT_F32 || wtype == WT_F16 || wtype == WT_BF16, BL_ERR_TYPE);
  BL_REQUIRE(n_group >= 1 && n_group <= 16 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group, BL_ERR_SHAPE);
  RouterArgs a{x, x_stride, gain, eps, (const uint8_t*)w, wtype, bias, K, E, M, top_k, mode, renorm, scale, n_group,
               topk_group, logits, ids, wts, xq_out, (float2*)xds_out, xn_out, counter, heat, fault, layer};
  int mb = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  size_t smem = (size_t)mb * K * 5 + (size_t)mb * (K / 32) * 8 + 256;
  BL_REQUIRE(smem <= 200 * 1024, BL_ERR_LIMIT);
  dim3 grid((E + 7) / 8);
#define BL_ROUTER_CASE(MBV)                                                                                  \
  {                                                                                                          \
    static bool set = false;                                                                                 \
    if (!set) { cudaFuncSetAttribute(router_kernel<MBV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); set = true; } \
    return (int)launch(router_kernel<MBV>, grid, dim3(256), smem, st, a);                                    \
  }
  switch (mb) {
    case 1: BL_ROUTER_CASE(1)
    case 2: BL_ROUTER_CASE(2)
    case 4: BL_ROUTER_CASE(4)
    default: BL_ROUTER_CASE(8)
  }
#undef BL_ROUTER_CASE
}

int bl_gate_up_sel(const int8_t* xq, const float* xds, const int* ids, const int* slot_map, const void* gate,
                   const void* up, int gtype, int utype, int K, int I, int E, int n_used, int M, int8_t* actq,
                   float* actds, float* act_f32, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(K % 256 == 0 && I % 32 == 0 && M >= 1 && n_used >= 1 && n_used <= kMaxTopK, BL_ERR_SHAPE);
  BL_REQUIRE(gtype == utype, BL_ERR_TYPE);
  BL_REQUIRE(gtype == WT_Q4_K || gtype == WT_Q5_K || gtype == WT_Q6_K || gtype == WT_Q8_0, BL_ERR_TYPE);
  GateUpArgs a{xq, (const float2*)xds, ids, slot_map, (const uint8_t*)gate, (const uint8_t*)up, gtype, utype, K, I, E,
               n_used, M, actq, (float2*)actds, act_f32, fault, layer};
  size_t smem = (size_t)K + (size_t)(K / 32) * 8;
  return (int)launch(gate_up_sel_kernel, dim3(I / 32, n_used, M), dim3(256), smem, st, a);
}

int bl_down_combine(const int8_t* actq, const float* actds, const int* ids, const float* wts, const int* slot_map,
                    const void* down, int dtype, int I, int H, int E, int n_used, int M, const float* resid,
                    long resid_stride, const float* extra, long extra_stride, float* out, long out_stride,
                    unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(I % 256 == 0 || (dtype == WT_Q8_0 && I % 64 == 0), BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && n_used >= 1 && n_used <= kMaxTopK, BL_ERR_SHAPE);
  BL_REQUIRE(dtype == WT_Q4_K || dtype == WT_Q5_K || dtype == WT_Q6_K || dtype == WT_Q8_0, BL_ERR_TYPE);
  DownArgs a{actq, (const float2*)actds, ids, wts, slot_map, (const uint8_t*)down, dtype, I, H, E, n_used, M, resid,
             resid_stride, extra, extra_stride, out, out_stride, fault, layer};
  size_t smem = (size_t)n_used * I + (size_t)n_used * (I / 32) * 8;
  BL_REQUIRE(smem <= 160 * 1024, BL_ERR_LIMIT);
  static bool set = false;
  if (!set) { cudaFuncSetAttribute(down_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024); set = true; }
  return (int)launch(down_combine_kernel, dim3((H + 7) / 8, M), dim3(256), smem, st, a);
}

}  // extern "C"
