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
#include "route.cuh"

namespace bl {

// block-scaled planes and the re-laid 32-value block types share one kernel family
static inline bool is_plane_family(int t) {
  return t == WT_NVFP4 || t == WT_FP8_B128 || t == WT_Q4_0 || t == WT_Q4_1 || t == WT_Q5_0 || t == WT_Q5_1 || t == WT_Q2_K || t == WT_Q3_K;
}


// grid = E blocks (one expert each), 256 threads.  A thread owns 8 consecutive values per
// 2048-value chunk; the router row, gain and x are loaded together, the dot product of
// w with x*gain and the sum of squares run in the same sweep, and the RMS scale multiplies
// the finished logit (so nothing waits for a normalisation pass).
template <int MB>
__global__ void __launch_bounds__(256) router_kernel(const RouterArgs a0) {
  __shared__ float s_dot[8][MB];
  __shared__ double s_ss[8][MB];
  __shared__ float s_scale[MB];
  const int K = a0.K;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e = blockIdx.x;
  RouterArgs a = a0;                      // row group blockIdx.y: rows [8 y, 8 y + M)
  if (blockIdx.y > 0) {
    const long r0 = (long)blockIdx.y * MB;
    a.x += r0 * a.x_stride; a.logits += r0 * a.E;
    if (a.xq_out) { a.xq_out += r0 * K; a.xds_out += r0 * (K / 32); }
    if (a.xn_out) a.xn_out += r0 * K;
  }
  a.M = min(MB, a0.M - (int)blockIdx.y * MB);
  const long rb = resident_row_bytes(a.wtype, K);
  const uint8_t* row = a.w + (long)e * rb;

  float dot[MB], ss[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) { dot[m] = 0.f; ss[m] = 0.f; }
  bool waited = false;
  __shared__ int s_gave_up;
  ReduceWait rw{0u, 0ull, &s_gave_up};
  for (int i0 = tid * 8; i0 < K; i0 += 2048) {
    float wv[8];
    if (a.wtype == WT_F32) {
      float4 p = __ldg(reinterpret_cast<const float4*>(row) + i0 / 4), q = __ldg(reinterpret_cast<const float4*>(row) + i0 / 4 + 1);
      wv[0] = p.x; wv[1] = p.y; wv[2] = p.z; wv[3] = p.w; wv[4] = q.x; wv[5] = q.y; wv[6] = q.z; wv[7] = q.w;
    } else {
      uint4 p = __ldg(reinterpret_cast<const uint4*>(row) + i0 / 8);
      const uint32_t ws[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = (a.wtype == WT_F16) ? __half22float2(*reinterpret_cast<const __half2*>(&ws[j]))
                                       : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ws[j]));
        wv[2 * j] = f.x; wv[2 * j + 1] = f.y;
      }
    }
    float4 g0 = __ldg(reinterpret_cast<const float4*>(a.gain + i0)), g1 = __ldg(reinterpret_cast<const float4*>(a.gain + i0 + 4));
    if (!waited) {
      pdl_wait(); waited = true;
      if (a.red.n_ranks > 0) {
        if (tid == 0) s_gave_up = (a.red.fault && *a.red.fault != 0xFFFFFFFFu) ? 1 : 0;   // a poisoned engine no longer waits
        __syncthreads();
        rw.epoch = site_epoch(a.red.step, a.red.sites_per_step, a.red.site_index);
      }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      const int ms = m < a.M ? m : a.M - 1;
      const float* xr = a.x + (long)ms * a.x_stride;
      float4 x0, x1;
      if (a.red.n_ranks > 0) {
        x0 = *reinterpret_cast<const float4*>(xr + i0); x1 = *reinterpret_cast<const float4*>(xr + i0 + 4);
        float acc8[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
        reduce_sum8(a.red, rw, ms, i0, acc8);
        x0 = make_float4(acc8[0], acc8[1], acc8[2], acc8[3]); x1 = make_float4(acc8[4], acc8[5], acc8[6], acc8[7]);
        if (e == 0 && m < a.M) {
          *reinterpret_cast<float4*>(a.red.x_out + (long)m * a.red.x_out_stride + i0) = x0;
          *reinterpret_cast<float4*>(a.red.x_out + (long)m * a.red.x_out_stride + i0 + 4) = x1;
        }
      } else {
        x0 = *reinterpret_cast<const float4*>(xr + i0); x1 = *reinterpret_cast<const float4*>(xr + i0 + 4);
      }
      ss[m] += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
      float t = dot[m];
      t = fmaf(wv[0], x0.x * g0.x, t); t = fmaf(wv[1], x0.y * g0.y, t); t = fmaf(wv[2], x0.z * g0.z, t); t = fmaf(wv[3], x0.w * g0.w, t);
      t = fmaf(wv[4], x1.x * g1.x, t); t = fmaf(wv[5], x1.y * g1.y, t); t = fmaf(wv[6], x1.z * g1.z, t); t = fmaf(wv[7], x1.w * g1.w, t);
      dot[m] = t;
    }
  }
  if (!waited) {
    pdl_wait();
    if (a.red.n_ranks > 0) {
      if (tid == 0) s_gave_up = (a.red.fault && *a.red.fault != 0xFFFFFFFFu) ? 1 : 0;   // a poisoned engine no longer waits
      __syncthreads();
      rw.epoch = site_epoch(a.red.step, a.red.sites_per_step, a.red.site_index);
    }
  }
  pdl_launch();
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    float d = warp_sum(dot[m]);
    double q = warp_sum_d((double)ss[m]);
    if (lane == 0) { s_dot[warp][m] = d; s_ss[warp][m] = q; }
  }
  __syncthreads();
  if (tid < MB) {
    float d = 0.f; double q = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) { d += s_dot[w][tid]; q += s_ss[w][tid]; }
    const float scale = (float)(1.0 / sqrt(q / (double)K + (double)a.eps));
    s_scale[tid] = scale;
    if (tid < a.M) { a.logits[(long)tid * a.E + e] = d * scale; __threadfence(); }
  }
  __syncthreads();
  __shared__ int s_last;
  if (a.ticket) {
    // every logit of this block is stored: take a ticket; the block that draws the last one routes the rows
    if (tid == 0) {
      __threadfence();
      const unsigned t = atomicAdd(a.ticket + blockIdx.y, 1u);
      s_last = (t == gridDim.x - 1) ? 1 : 0;
      if (s_last) a.ticket[blockIdx.y] = 0u;         // zero again for the next launch (graph replay)
    }
    __syncthreads();
  }
  // every block knows the scale; block b publishes 32-value blocks b, b + E, ... of the q8 rows
  if (a.xq_out) {
    const int nb32 = K / 32;
    for (int b = e * 8 + warp; b < nb32 * a.M; b += gridDim.x * 8) {
      const int m = b / nb32, bb = b - m * nb32;
      const int i = bb * 32 + lane;
      const float xv = a.red.n_ranks > 0 ? reduce_value(a.red, rw, a.x + (long)m * a.x_stride, m, i) : a.x[(long)m * a.x_stride + i];
      const float v = xv * a.gain[i] * s_scale[m];
      float d, sm;
      int8_t qv = q8_lane(v, d, sm);
      a.xq_out[(long)m * K + i] = qv;
      if (a.xn_out) a.xn_out[(long)m * K + i] = v;
      if (lane == 0) a.xds_out[(long)m * nb32 + bb] = make_float2(d, sm);
    }
  }
  if (a.ticket && s_last) {
    __shared__ RouteShared rs;
    __threadfence();
    RouteParams p = a.route;
    p.logits = a.logits;
    for (int m = 0; m < a.M; ++m) {
      int id; float w;
      const bool ok = route_block(p, m, rs, id, w);
      if (a.pf_gate) {
        // prediction: publish the predicted slots for the prefetch launch that follows (one SM alone cannot issue
        // tens of megabytes of prefetches fast enough; the follower spreads them over the whole card)
        if (warp == 0 && lane < p.top_k) {
          int e = ok ? rs.ids[lane] : -1;
          if (e >= 0 && a.pf_slot_map) e = a.pf_slot_map[e];
          a.ids[(long)m * p.top_k + lane] = e;
        }
        __syncthreads();
        continue;
      }
      if (warp == 0) {
        if (!ok && lane == 0) raise_fault(a.fault, a.layer, FS_ROUTER);
        if (lane < p.top_k) {
          a.ids[(long)m * p.top_k + lane] = ok ? id : -3;
          a.wts[(long)m * p.top_k + lane] = w;
          if (ok && a.heat) atomicAdd(a.heat + id, 1u);
        }
      }
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------------------------
// gate·up·SwiGLU over device-side expert ids
// grid (I/32, n_used, M), 256 threads: warp w computes activation rows 4w..4w+3 of the chunk
// ------------------------------------------------------------------------------------
struct GateUpArgs {
  const int8_t* xq; const float2* xds;   // [M, K] q8
  RouteParams route;                     // route.logits == null: ids are given
  int* ids;                              // [M, n_used] read (given) or written (routed here)
  float* wts;                            // [M, n_used] written when routed here
  unsigned* heat;                        // optional [E] routed-count histogram
  const int* slot_map;                   // optional [E]: expert id -> resident slot (or kExpertElsewhere)
  const uint8_t* gate; const uint8_t* up; int gtype, utype;   // stacks [E_slots, I, K]
  int K, I, E, n_used, M;
  int8_t* actq; float2* actds;           // [M, n_used, I] q8
  float* act_f32;                        // optional fp32 copy
  unsigned* fault; int layer;
  const uint8_t* down; long down_expert_bytes;   // optional: the down stack, whose chosen matrices L2 is asked to prefetch
};

// two activation outputs (2 gate rows + 2 up rows) of one warp
template <class T>
__device__ __forceinline__ void gate_up_rows(const uint8_t* g0, const uint8_t* u0, long rb, int K, int lane,
                                             const int8_t* xq, const float2* xds, float (&gacc)[2], float (&uacc)[2]) {
  using U = Unit<T>;
  const int nunits = K / 64;
#pragma unroll
  for (int r = 0; r < 2; ++r) { gacc[r] = 0.f; uacc[r] = 0.f; }
  for (int u = lane; u < nunits; u += 32) {
    typename U::Regs rg[2], ru[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) { U::loadu(g0 + r * rb, u, K, rg[r]); U::loadu(u0 + r * rb, u, K, ru[r]); }
    ActRegs act;   // activations straight from L2, behind the weight loads already in flight
    ActOf<T>::load(reinterpret_cast<const uint32_t*>(xq), reinterpret_cast<const F2*>(xds), u, act);
#pragma unroll
    for (int r = 0; r < 2; ++r) { gacc[r] += ActOf<T>::dot(rg[r], u, act); uacc[r] += ActOf<T>::dot(ru[r], u, act); }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) { gacc[r] = warp_sum(gacc[r]); uacc[r] = warp_sum(uacc[r]); }
}

// grid (I/32, n_used, M), 256 threads: warp w computes activation rows 4w..4w+3 of the chunk.
// When route.logits is set, warp 0 of every block routes row m itself (redundantly, from
// the router launch's logits) so no block waits on a completion counter; block (0, 0, m)
// also publishes ids / weights / heat for the launches that follow.
// FAM 0 = ggml integer-dot types, FAM 2 = block-scaled float planes (one kernel per family keeps
// the plane decoders out of the K-quant bodies' register budget)
template <int FAM>
__global__ void __launch_bounds__(256, 2) gate_up_sel_kernel(const GateUpArgs a) {
  const int K = a.K;
  __shared__ float s_act[32];
  __shared__ int s_e;
  const int chunk = blockIdx.x, j = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_launch();
  if (a.route.logits) {
    // block-wide rank counting: measured faster here than top_k rounds of a single warp's arg-max
    __shared__ RouteShared rs;
    int id; float w;
    const bool ok = route_block(a.route, m, rs, id, w);
    if (tid == 0) s_e = ok ? rs.ids[j] : -3;
    if (chunk == 0 && j == 0 && warp == 0) {
      if (!ok && lane == 0) raise_fault(a.fault, a.layer, FS_ROUTER);
      if (lane < a.n_used) {
        a.ids[(long)m * a.n_used + lane] = ok ? id : 0;
        a.wts[(long)m * a.n_used + lane] = w;
        if (ok && a.heat) atomicAdd(a.heat + id, 1u);
      }
    }
  } else if (tid == 0) {
    s_e = a.ids[(long)m * a.n_used + j];
  }
  __syncthreads();
  int e = s_e;
  const long ob = ((long)m * a.n_used + j) * a.I + chunk * 32;
  bool skip = false, bad = false;
  if (e == kExpertElsewhere) skip = true;
  else if (e == -3) { skip = true; bad = true; }                 // router fault: NaN downstream
  else if (e < 0 || e >= a.E) { skip = true; bad = true; if (tid == 0 && chunk == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID); }
  else if (a.slot_map) { e = a.slot_map[e]; if (e < 0) skip = true; }
  if (skip) {
    if (tid < 32) {
      a.actq[ob + tid] = 0;
      if (a.act_f32) a.act_f32[ob + tid] = bad ? __int_as_float(0x7fc00000) : 0.f;
    }
    if (tid == 0) a.actds[ob / 32] = bad ? make_float2(__int_as_float(0x7fc00000), 0.f) : make_float2(0.f, 0.f);
    return;
  }
  const long rb = resident_row_bytes(a.gtype, K);
  const int8_t* xq = a.xq + (long)m * K;
  const float2* xds = a.xds + (long)m * (K / 32);
  if (a.down && tid == 32) {
    // the down launch that follows streams expert e's matrix: this block asks L2 for its 1 / gridDim.x share
    const long share = (a.down_expert_bytes / gridDim.x) & ~15L;
    for (long o = 0; o < share; o += 32768) {
      const unsigned nb = (unsigned)((share - o) < 32768 ? (share - o) : 32768);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.down + (long)e * a.down_expert_bytes + (long)chunk * share + o), "r"(nb) : "memory");
    }
  }
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const long row0 = (long)e * a.I + chunk * 32 + warp * 4 + half * 2;
    const uint8_t* g0 = a.gate + row0 * rb;
    const uint8_t* u0 = a.up + row0 * rb;
    float gacc[2], uacc[2];
    if constexpr (FAM == 2) {
      switch (a.gtype) {
        case WT_NVFP4: gate_up_rows<NvFp4>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_FP8_B128: gate_up_rows<Fp8B128>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q2_K: gate_up_rows<Q2K>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q3_K: gate_up_rows<Q3K>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q4_0: gate_up_rows<Q40>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q4_1: gate_up_rows<Q41>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q5_0: gate_up_rows<Q50>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q5_1: gate_up_rows<Q51>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        default: gacc[0] = gacc[1] = __int_as_float(0x7fc00000); uacc[0] = uacc[1] = 0.f;
      }
    } else {
      switch (a.gtype) {
        case WT_Q4_K: gate_up_rows<Q4K>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q5_K: gate_up_rows<Q5K>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q6_K: gate_up_rows<Q6K>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q8_0: gate_up_rows<Q80>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        case WT_Q8_F32: gate_up_rows<Q8F>(g0, u0, rb, K, lane, xq, xds, gacc, uacc); break;
        default: gacc[0] = gacc[1] = __int_as_float(0x7fc00000); uacc[0] = uacc[1] = 0.f;
      }
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float g = gacc[r];
        s_act[warp * 4 + half * 2 + r] = (g / (1.0f + expf(-g))) * uacc[r];
      }
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
  PushOut push;                             // n_ranks > 0: the result is this rank's partial update
};

// UPL = units per lane (all loaded before any is used: one DRAM round trip per row)
template <class T, int UPL>
__device__ __forceinline__ float down_row(const DownArgs& a, int m, int d, int lane, const int* s_slot, const float* s_w) {
  using U = Unit<T>;
  const int upe = a.I / 64;              // units per expert row
  const int total = a.n_used * upe;
  const long rb = resident_row_bytes(T::kType, a.I);
  typename U::Regs regs[UPL];
  int jj[UPL], uu[UPL];
#pragma unroll
  for (int c = 0; c < UPL; ++c) {
    const int t = lane + 32 * c;
    jj[c] = -1; uu[c] = 0;
    if (t < total) {
      const int j = t / upe;
      const int e = s_slot[j];
      if (e >= 0) { jj[c] = j; uu[c] = t - j * upe; U::loadu(a.down + ((long)e * a.H + d) * rb, uu[c], a.I, regs[c]); }
    }
  }
  // per-slot partial sums kept separate, then added in ascending slot order
  float part[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) part[j] = 0.f;
#pragma unroll
  for (int c = 0; c < UPL; ++c) {
    if (jj[c] >= 0) {
      ActRegs act;
      const long ab = ((long)m * a.n_used + jj[c]) * a.I;
      ActOf<T>::load(reinterpret_cast<const uint32_t*>(a.actq + ab), reinterpret_cast<const F2*>(a.actds + ab / 32), uu[c], act);
      float v = ActOf<T>::dot(regs[c], uu[c], act);
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j) if (j == jj[c]) part[j] += v;
    }
  }
  // router-weighted sum over slots in ascending order inside the lane, then one butterfly
  float y = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) {
    if (j < a.n_used) y = fmaf(s_w[j], part[j], y);
  }
  return warp_sum(y);
}

template <int UPL, int FAM>
__global__ void __launch_bounds__(256, UPL <= 3 ? 2 : 1) down_combine_kernel(const DownArgs a) {
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
  __syncthreads();
  bool bad = false;
  for (int j = 0; j < a.n_used; ++j) bad |= (s_slot[j] == -2);
  const int d = blockIdx.x * 8 + warp;
  if (d < a.H) {
    float y;
    if constexpr (FAM == 2) {
      switch (a.dtype) {
        case WT_NVFP4: y = down_row<NvFp4, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_FP8_B128: y = down_row<Fp8B128, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q2_K: y = down_row<Q2K, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q3_K: y = down_row<Q3K, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q4_0: y = down_row<Q40, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q4_1: y = down_row<Q41, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q5_0: y = down_row<Q50, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q5_1: y = down_row<Q51, UPL>(a, m, d, lane, s_slot, s_w); break;
        default: y = __int_as_float(0x7fc00000);
      }
    } else {
      switch (a.dtype) {
        case WT_Q4_K: y = down_row<Q4K, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q6_K: y = down_row<Q6K, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q5_K: y = down_row<Q5K, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q8_0: y = down_row<Q80, UPL>(a, m, d, lane, s_slot, s_w); break;
        case WT_Q8_F32: y = down_row<Q8F, UPL>(a, m, d, lane, s_slot, s_w); break;
        default: y = __int_as_float(0x7fc00000);
      }
    }
    if (lane == 0) {
      if (bad) { y = __int_as_float(0x7fc00000); if (d == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID); }
      if (a.extra) y += a.extra[(long)m * a.extra_stride + d];
      if (a.push.n_ranks > 0) {
        push_store(a.push, site_epoch(a.push.step, a.push.sites_per_step, a.push.site_index), (long)m * a.out_stride + d, y);
      } else {
        if (a.resid) y += a.resid[(long)m * a.resid_stride + d];
        a.out[(long)m * a.out_stride + d] = y;
      }
    }
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

// Router logits (RMS scale applied) for M rows + the q8 form of the normed rows.
// ticket != null (one zeroed word per group of 8 rows): the launch also routes, i.e. writes ids / wts (and heat).
int bl_router(const float* x, long x_stride, const float* gain, float eps, const void* w, int wtype,
              int K, int E, int M, float* logits, int8_t* xq_out, float* xds_out, float* xn_out,
              const void* red_desc, unsigned* fault, int layer,
              unsigned* ticket, const float* bias, int top_k, int mode, int renorm, float scale, int n_group, int topk_group,
              int* ids, float* wts, unsigned* heat,
              const void* pf_gate, const void* pf_up, const void* pf_down, long pf_gate_bytes, long pf_down_bytes,
              const int* pf_slot_map, cudaStream_t st) {
  BL_REQUIRE(E >= 1 && E <= kMaxExperts, BL_ERR_LIMIT);
  BL_REQUIRE(K % 256 == 0 && M >= 1 && M <= 8 * 65535, BL_ERR_SHAPE);
  BL_REQUIRE(wtype == WT_F32 || wtype == WT_F16 || wtype == WT_BF16, BL_ERR_TYPE);
  RouterArgs a{};
  a.x = x; a.x_stride = x_stride; a.gain = gain; a.eps = eps; a.w = (const uint8_t*)w; a.wtype = wtype;
  a.K = K; a.E = E; a.M = M; a.logits = logits; a.xq_out = xq_out; a.xds_out = (float2*)xds_out; a.xn_out = xn_out;
  a.fault = fault; a.layer = layer;
  if (red_desc) { a.red = *(const ReduceIn*)red_desc; BL_REQUIRE(M <= kMaxRows && a.red.n_ranks <= kMaxRanks && a.red.H == K, BL_ERR_SHAPE); }
  if (ticket) {
    BL_REQUIRE(E % 4 == 0 && top_k >= 1 && top_k <= kMaxTopK && top_k <= E && n_group >= 1 && n_group <= 16 && E % n_group == 0 &&
               topk_group >= 1 && topk_group <= n_group && ((ids && wts) || pf_gate), BL_ERR_SHAPE);
    a.ticket = ticket; a.ids = ids; a.wts = wts; a.heat = heat;
    if (pf_gate) {
      BL_REQUIRE(pf_up && pf_down && pf_gate_bytes > 0 && pf_down_bytes > 0 && (((uintptr_t)pf_gate | (uintptr_t)pf_up | (uintptr_t)pf_down) & 15) == 0 &&
                 pf_gate_bytes % 16 == 0 && pf_down_bytes % 16 == 0, BL_ERR_ALIGN);
      a.pf_gate = (const uint8_t*)pf_gate; a.pf_up = (const uint8_t*)pf_up; a.pf_down = (const uint8_t*)pf_down;
      a.pf_gate_bytes = pf_gate_bytes; a.pf_down_bytes = pf_down_bytes; a.pf_slot_map = pf_slot_map;
    }
    a.route = RouteParams{nullptr, bias, E, top_k, mode, renorm, scale, n_group, topk_group};
  }
  int mb = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  dim3 grid(E, (M + mb - 1) / mb);
  switch (mb) {
    case 1: return (int)launch(router_kernel<1>, grid, dim3(256), 0, st, a);
    case 2: return (int)launch(router_kernel<2>, grid, dim3(256), 0, st, a);
    case 4: return (int)launch(router_kernel<4>, grid, dim3(256), 0, st, a);
    default: return (int)launch(router_kernel<8>, grid, dim3(256), 0, st, a);
  }
}

// Asks L2 to prefetch the gate / up (and optionally down) matrices of the experts named in ids[n] (negative = skip),
// 32 KB pieces dealt round-robin over the blocks; lane 0 of every warp issues.
__global__ void __launch_bounds__(256) prefetch_experts_kernel(const int* ids, int n, const uint8_t* gate, const uint8_t* up,
                                                               const uint8_t* down, long gate_bytes, long down_bytes) {
  pdl_wait();
  pdl_launch();
  const long gn = gate_bytes / 32768, dn = down ? down_bytes / 32768 : 0, per = 2 * gn + dn;
  const long total = per * n;
  const int wid = blockIdx.x * 8 + (threadIdx.x >> 5), nw = gridDim.x * 8;
  if ((threadIdx.x & 31) != 0) return;
  for (long c = wid; c < total; c += nw) {
    const int q = (int)(c / per);
    const long r = c - (long)q * per;
    const int e = ids[q];
    if (e < 0) continue;
    const uint8_t* src = r < gn ? gate + e * gate_bytes + r * 32768
                       : r < 2 * gn ? up + e * gate_bytes + (r - gn) * 32768
                       : down + e * down_bytes + (r - 2 * gn) * 32768;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(32768u) : "memory");
  }
}

// Standalone routing of M rows from logits (tests, prefill, host paths): one warp per row.
__global__ void __launch_bounds__(256) route_rows_kernel(RouteParams p, int M, int* ids, float* wts, unsigned* heat,
                                                         unsigned* fault, int layer) {
  __shared__ RouteShared rs;
  pdl_wait();
  pdl_launch();
  const int m = blockIdx.x, lane = threadIdx.x & 31;
  int id; float w;
  const bool ok = route_block(p, m, rs, id, w);
  if (threadIdx.x >= 32) return;
  if (!ok && lane == 0) raise_fault(fault, layer, FS_ROUTER);
  if (lane < p.top_k) {
    ids[(long)m * p.top_k + lane] = ok ? id : 0;
    wts[(long)m * p.top_k + lane] = w;
    if (ok && heat) atomicAdd(heat + id, 1u);
  }
}

int bl_prefetch_experts(const int* ids, int n, const void* gate, const void* up, const void* down, long gate_bytes,
                        long down_bytes, int blocks, cudaStream_t st) {
  BL_REQUIRE(n >= 1 && gate && up && gate_bytes > 0 && blocks >= 1, BL_ERR_SHAPE);
  BL_REQUIRE((((uintptr_t)gate | (uintptr_t)up | (uintptr_t)down) & 15) == 0 && gate_bytes % 16 == 0 && down_bytes % 16 == 0, BL_ERR_ALIGN);
  return (int)launch(prefetch_experts_kernel, dim3(blocks), dim3(256), 0, st, ids, n, (const uint8_t*)gate, (const uint8_t*)up,
                     (const uint8_t*)down, gate_bytes, down_bytes);
}

int bl_route_rows(const float* logits, const float* bias, int E, int M, int top_k, int mode, int renorm, float scale,
                  int n_group, int topk_group, int* ids, float* wts, unsigned* heat, unsigned* fault, int layer,
                  cudaStream_t st) {
  BL_REQUIRE(E >= 4 && E % 4 == 0 && E <= kMaxExperts && top_k >= 1 && top_k <= kMaxTopK && top_k <= E, BL_ERR_LIMIT);
  BL_REQUIRE(n_group >= 1 && n_group <= 16 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group, BL_ERR_SHAPE);
  RouteParams p{logits, bias, E, top_k, mode, renorm, scale, n_group, topk_group};
  return (int)launch(route_rows_kernel, dim3(M), dim3(256), 0, st, p, M, ids, wts, heat, fault, layer);
}

// route_logits != null: every block routes its row from the logits (and block 0 writes
// ids / wts / heat); otherwise ids are read as given.
int bl_gate_up_sel(const int8_t* xq, const float* xds, const float* route_logits, const float* bias, int top_k_mode,
                   int renorm, float scale, int n_group, int topk_group, int* ids, float* wts, unsigned* heat,
                   const int* slot_map, const void* gate, const void* up, int gtype, int utype, int K, int I, int E,
                   int n_used, int M, int8_t* actq, float* actds, float* act_f32, unsigned* fault, int layer,
                   const void* down, long down_expert_bytes, cudaStream_t st) {
  BL_REQUIRE(K % 256 == 0 && I % 32 == 0 && M >= 1 && n_used >= 1 && n_used <= kMaxTopK, BL_ERR_SHAPE);
  BL_REQUIRE(gtype == utype, BL_ERR_TYPE);
  BL_REQUIRE(gtype == WT_Q4_K || gtype == WT_Q5_K || gtype == WT_Q6_K || gtype == WT_Q8_0 || gtype == WT_Q8_F32 || is_plane_family(gtype), BL_ERR_TYPE);
  BL_REQUIRE(E % 4 == 0 && E <= kMaxExperts && n_group >= 1 && n_group <= 16 && E % n_group == 0, BL_ERR_LIMIT);
  GateUpArgs a{};
  a.xq = xq; a.xds = (const float2*)xds;
  a.route = RouteParams{route_logits, bias, E, n_used, top_k_mode, renorm, scale, n_group, topk_group};
  a.ids = ids; a.wts = wts; a.heat = heat; a.slot_map = slot_map;
  a.gate = (const uint8_t*)gate; a.up = (const uint8_t*)up; a.gtype = gtype; a.utype = utype;
  a.K = K; a.I = I; a.E = E; a.n_used = n_used; a.M = M;
  a.actq = actq; a.actds = (float2*)actds; a.act_f32 = act_f32; a.fault = fault; a.layer = layer;
  BL_REQUIRE(((uintptr_t)down & 15) == 0 && down_expert_bytes % 16 == 0, BL_ERR_ALIGN);
  a.down = (const uint8_t*)down; a.down_expert_bytes = down_expert_bytes;
  if (is_plane_family(gtype)) return (int)launch(gate_up_sel_kernel<2>, dim3(I / 32, n_used, M), dim3(256), 0, st, a);
  return (int)launch(gate_up_sel_kernel<0>, dim3(I / 32, n_used, M), dim3(256), 0, st, a);
}

int bl_down_combine(const int8_t* actq, const float* actds, const int* ids, const float* wts, const int* slot_map,
                    const void* down, int dtype, int I, int H, int E, int n_used, int M, const float* resid,
                    long resid_stride, const float* extra, long extra_stride, float* out, long out_stride,
                    const void* push_desc, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(I % 256 == 0 || ((dtype == WT_Q8_0 || dtype == WT_Q8_F32 || (is_plane_family(dtype) && dtype != WT_FP8_B128 && dtype != WT_Q2_K && dtype != WT_Q3_K)) && I % 64 == 0) ||
             (dtype == WT_FP8_B128 && I % 128 == 0), BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && n_used >= 1 && n_used <= kMaxTopK, BL_ERR_SHAPE);
  BL_REQUIRE(dtype == WT_Q4_K || dtype == WT_Q5_K || dtype == WT_Q6_K || dtype == WT_Q8_0 || dtype == WT_Q8_F32 || is_plane_family(dtype), BL_ERR_TYPE);
  DownArgs a{actq, (const float2*)actds, ids, wts, slot_map, (const uint8_t*)down, dtype, I, H, E, n_used, M, resid,
             resid_stride, extra, extra_stride, out, out_stride, fault, layer, PushOut{}};
  if (push_desc) { a.push = *(const PushOut*)push_desc; BL_REQUIRE(a.push.n_ranks <= kMaxRanks && M <= kMaxRows, BL_ERR_SHAPE); }
  const long total = (long)n_used * (I / 64);
  BL_REQUIRE(total <= 512, BL_ERR_LIMIT);
  dim3 grid((H + 7) / 8, M);
  if (is_plane_family(dtype)) {
    if (total <= 96) return (int)launch(down_combine_kernel<3, 2>, grid, dim3(256), 0, st, a);
    if (total <= 192) return (int)launch(down_combine_kernel<6, 2>, grid, dim3(256), 0, st, a);
    return (int)launch(down_combine_kernel<16, 2>, grid, dim3(256), 0, st, a);
  }
  if (total <= 96) return (int)launch(down_combine_kernel<3, 0>, grid, dim3(256), 0, st, a);
  if (total <= 192) return (int)launch(down_combine_kernel<6, 0>, grid, dim3(256), 0, st, a);
  return (int)launch(down_combine_kernel<16, 0>, grid, dim3(256), 0, st, a);
}

}  // extern "C"
