// One launch for the whole mixture-of-experts half of a decode layer (one activation row):
//   RMSNorm + router logits + top-k + gate.x / up.x of the chosen experts + SwiGLU + q8 + down projection +
//   router-weighted sum + residual.
//
// A thread-block cluster of 16 CTAs serves one chosen expert (grid = 16 x n_used, one CTA per SM).  Everything
// the three launches of the plain chain hand to one another through L2 (logits, routing, the expert's activation
// row) stays on chip: CTAs exchange it through distributed shared memory (st.shared::cluster on mapa addresses)
// and meet at the cluster's hardware barrier, so a layer's expert half costs one launch and two cluster barriers
// instead of three launches.
//
//   phase 0  (before griddepcontrol.wait) the CTA's 1/16 of the router matrix arrives by bulk copy
//   phase 1  x -> sum of squares, x*gain (fp32, for the router), q8(RMSNorm(x)*gain) (for the experts)
//   phase 2  logits of the CTA's E/16 experts, written into every peer's logit row         -> cluster barrier
//   phase 3  top-k (each CTA by itself, block-wide rank counting); cluster j takes slot j's expert
//   phase 4  bulk copies: the CTA's I/16 gate rows + up rows and its H/16 down rows of that expert
//   phase 5  gate.x, up.x, SwiGLU of those rows, written into every peer's activation row  -> cluster barrier
//   phase 6  q8 of the expert's activation row (each CTA by itself)
//   phase 7  the CTA's H/16 rows of the down projection -> partial row p_j (global)
//   phase 8  completion ticket per row slice: the last of the n_used clusters adds
//            x_out = x (+ extra) + sum_j w_j p_j over the slots in ascending order
//
// Arithmetic of the logits, the routing, the activations and their q8 form is that of router_kernel /
// gate_up_sel_kernel (same sums in the same order); the down projection sums each slot's row first and weights it
// afterwards, so its last bits differ from down_combine_kernel (tests hold both to the fp32 reference).
// The reference keeps these as separate launches (crates/gpu/src/route_softmax.rs, arch/qwen3moe/experts.rs);
// clusters and distributed shared memory are what lets them fuse here.
#include "staged.cuh"

namespace bl {

constexpr int kCl = 16;                // CTAs per cluster

struct MoeClusterArgs {
  const float* x;                        // [H] residual row (input)
  const float* gain; float eps;
  const uint8_t* rw; int rtype;          // router rows [E, H]: F32 / F16 / BF16
  RouteParams route;                     // logits field unused
  const int* slot_map;                   // optional [E]
  const uint8_t* gate; const uint8_t* up; int gtype;   // [E_slots, I, rb_g]
  const uint8_t* down; int dtype;                      // [E_slots, H, rb_d]
  int H, I, E, n_used;
  const float* extra;                    // optional [H] addend (shared expert, host leg)
  float* parts;                          // scratch [n_used, H]: the slots' unweighted down rows
  unsigned* tickets;                     // [kCl] zero between launches
  float* x_out;                          // [H] new residual row (must not alias x)
  float* logits; int* ids; float* wts; unsigned* heat;   // published for traces, residency, the host tier
  unsigned* fault; int layer;
  long long* probe;
};

struct MoeClusterSmem {                  // byte offsets into dynamic shared memory
  int rd, gu, xg, xq, xds, logits, act, actq, ads, total;
};

__host__ __device__ inline MoeClusterSmem moe_cluster_layout(int H, int I, int E, int rtype, int gtype, int dtype) {
  const long r_bytes = (long)(E / kCl) * H * (rtype == WT_F32 ? 4 : 2);
  const long d_bytes = (long)(H / kCl) * resident_row_bytes(dtype, I);
  const long g_bytes = (long)2 * (I / kCl) * resident_row_bytes(gtype, H);
  MoeClusterSmem s;
  long o = 0;
  auto take = [&](long n) { long at = o; o += (n + 127) / 128 * 128; return (int)at; };
  s.rd = take(r_bytes > d_bytes ? r_bytes : d_bytes);   // router rows, later the down rows
  s.gu = take(g_bytes);
  s.xg = take((long)H * 4);
  s.xq = take(H);
  s.xds = take((long)(H / 32) * 8);
  s.logits = take((long)E * 4);
  s.act = take((long)I * 4);
  s.actq = take(I);
  s.ads = take((long)(I / 32) * 8);
  s.total = (int)o;
  return s;
}

// two rows of K <= 1024 values per warp pass (lanes 0..15 row a, 16..31 row b), one row otherwise
template <class T>
__device__ __forceinline__ void down_rows_cluster(const uint8_t* sw, long rb, int I, int nrows, const int8_t* actq,
                                                  const float2* ads, float* s_p) {
  using U = Unit<T>;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int upe = I / 64;
  if (upe <= 16) {
    const int half = lane >> 4, hl = lane & 15;
    for (int r0 = warp * 2; r0 < nrows; r0 += 16) {
      const int r = r0 + half;
      float acc = 0.f;
      if (r < nrows && hl < upe) {
        typename U::Regs regs;
        U::loadu(sw + (long)r * rb, hl, I, regs);
        ActRegs act;
        StagedAct<T>::load(actq, ads, hl, upe, act);
        acc = ActOf<T>::dot(regs, hl, act);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (hl == 0 && r < nrows) s_p[r] = acc;
    }
  } else {
    for (int r = warp; r < nrows; r += 8) {
      float acc = 0.f;
      for (int u = lane; u < upe; u += 32) {
        typename U::Regs regs;
        U::loadu(sw + (long)r * rb, u, I, regs);
        ActRegs act;
        StagedAct<T>::load(actq, ads, u, upe, act);
        acc += ActOf<T>::dot(regs, u, act);
      }
      acc = warp_sum(acc);
      if (lane == 0) s_p[r] = acc;
    }
  }
}

template <int FAM>
__global__ void __launch_bounds__(256, 1) moe_cluster_kernel(const MoeClusterArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar_r, bar_gu, bar_d;
  __shared__ float s_dot[8][8];
  __shared__ double s_ss[8];
  __shared__ float s_scale;
  __shared__ float s_p[512];
  __shared__ int s_e, s_last;
  __shared__ RouteShared rs;
  const int H = a.H, I = a.I, E = a.E;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned c = cluster_ctarank();
  const int j = blockIdx.y;
  const MoeClusterSmem L = moe_cluster_layout(H, I, E, a.rtype, a.gtype, a.dtype);
  uint8_t* s_rd = smem + L.rd;
  uint8_t* s_gu = smem + L.gu;
  float* s_xg = reinterpret_cast<float*>(smem + L.xg);
  int8_t* s_xq = reinterpret_cast<int8_t*>(smem + L.xq);
  float2* s_xds = reinterpret_cast<float2*>(smem + L.xds);
  float* s_logits = reinterpret_cast<float*>(smem + L.logits);
  float* s_act = reinterpret_cast<float*>(smem + L.act);
  int8_t* s_actq = reinterpret_cast<int8_t*>(smem + L.actq);
  float2* s_ads = reinterpret_cast<float2*>(smem + L.ads);
  const int epc = E / kCl, apc = I / kCl, rpc = H / kCl;       // experts, activation rows, output rows per CTA
  const int rbytes = a.rtype == WT_F32 ? 4 : 2;
  const long rb_g = resident_row_bytes(a.gtype, H), rb_d = resident_row_bytes(a.dtype, I);

  // ---- phase 0: this CTA's router rows (they never depend on the predecessor) ----------------------
  probe_mark(a.probe, 0);
  if (tid == 0) {
    mbar_init(&bar_r, 1); mbar_init(&bar_gu, 1); mbar_init(&bar_d, 1);
    const uint32_t nb = (uint32_t)((long)epc * H * rbytes);
    mbar_expect_tx(&bar_r, nb);
    bulk_load_chunks(s_rd, a.rw + (long)c * epc * H * rbytes, nb, &bar_r);
  }
  __syncthreads();
  pdl_wait();
  pdl_launch();
  probe_mark(a.probe, 1);

  // ---- phase 1: the row, its sum of squares, x*gain, and (after the scale is known) its q8 form ------
  {
    float ss = 0.f;
    for (int i0 = tid * 8; i0 < H; i0 += 2048) {
      const float4 x0 = *reinterpret_cast<const float4*>(a.x + i0), x1 = *reinterpret_cast<const float4*>(a.x + i0 + 4);
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(a.gain + i0)), g1 = __ldg(reinterpret_cast<const float4*>(a.gain + i0 + 4));
      ss += x0.x * x0.x + x0.y * x0.y + x0.z * x0.z + x0.w * x0.w + x1.x * x1.x + x1.y * x1.y + x1.z * x1.z + x1.w * x1.w;
      *reinterpret_cast<float4*>(s_xg + i0) = make_float4(x0.x * g0.x, x0.y * g0.y, x0.z * g0.z, x0.w * g0.w);
      *reinterpret_cast<float4*>(s_xg + i0 + 4) = make_float4(x1.x * g1.x, x1.y * g1.y, x1.z * g1.z, x1.w * g1.w);
    }
    const double q = warp_sum_d((double)ss);
    if (lane == 0) s_ss[warp] = q;
    __syncthreads();
    if (tid == 0) {
      double tot = 0.0;
#pragma unroll
      for (int w = 0; w < 8; ++w) tot += s_ss[w];
      s_scale = (float)(1.0 / sqrt(tot / (double)H + (double)a.eps));
    }
    __syncthreads();
  }
  const float scale = s_scale;
  {
    // q8 of x * gain * scale per 32 values, in the layout the gate / up units read
    const int nb32 = H / 32, layout = staged_layout(a.gtype), nunits = H / 64;
    for (int b = warp; b < nb32; b += 8) {
      const int i = b * 32 + lane;
      const float v = a.x[i] * a.gain[i] * scale;
      float d, sm;
      const int8_t qv = q8_lane(v, d, sm);
      s_xq[act_chunk_pos(i >> 4, nunits, layout) * 16 + (i & 15)] = qv;
      if (lane == 0) s_xds[b] = make_float2(d, sm);
    }
  }
  probe_mark(a.probe, 2);

  // ---- phase 2: logits of this CTA's experts --------------------------------------------------------
  bool ok = mbar_wait(&bar_r, 0, a.fault, a.layer);
  {
    float dot[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) dot[k] = 0.f;
    for (int e0 = 0; e0 < epc; e0 += 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k) dot[k] = 0.f;
      for (int i0 = tid * 8; i0 < H; i0 += 2048) {
        const float4 y0 = *reinterpret_cast<const float4*>(s_xg + i0), y1 = *reinterpret_cast<const float4*>(s_xg + i0 + 4);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (e0 + k < epc) {
            const uint8_t* row = s_rd + (long)(e0 + k) * H * rbytes;
            float wv[8];
            if (a.rtype == WT_F32) {
              const float4 p = *(reinterpret_cast<const float4*>(row) + i0 / 4), q = *(reinterpret_cast<const float4*>(row) + i0 / 4 + 1);
              wv[0] = p.x; wv[1] = p.y; wv[2] = p.z; wv[3] = p.w; wv[4] = q.x; wv[5] = q.y; wv[6] = q.z; wv[7] = q.w;
            } else {
              const uint4 p = *(reinterpret_cast<const uint4*>(row) + i0 / 8);
              const uint32_t ws[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 f = (a.rtype == WT_F16) ? __half22float2(*reinterpret_cast<const __half2*>(&ws[q]))
                                                     : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ws[q]));
                wv[2 * q] = f.x; wv[2 * q + 1] = f.y;
              }
            }
            float t = dot[k];
            t = fmaf(wv[0], y0.x, t); t = fmaf(wv[1], y0.y, t); t = fmaf(wv[2], y0.z, t); t = fmaf(wv[3], y0.w, t);
            t = fmaf(wv[4], y1.x, t); t = fmaf(wv[5], y1.y, t); t = fmaf(wv[6], y1.z, t); t = fmaf(wv[7], y1.w, t);
            dot[k] = t;
          }
        }
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = warp_sum(dot[k]);
        if (lane == 0) s_dot[warp][k] = d;
      }
      __syncthreads();
      if (tid < 8 * kCl) {
        // thread (k, peer): the logit of expert e0 + k goes into peer's logit row
        const int k = tid / kCl, peer = tid % kCl;
        if (e0 + k < epc) {
          float d = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) d += s_dot[w][k];
          const float logit = ok ? d * scale : kNaN;
          const int e = (int)c * epc + e0 + k;
          st_peer_f32(peer_addr(s_logits + e, (unsigned)peer), logit);
          if (j == 0 && peer == 0 && a.logits) a.logits[e] = logit;
        }
      }
      __syncthreads();
    }
  }
  cluster_sync_all();
  probe_mark(a.probe, 3);

  // ---- phase 3: routing (every CTA by itself), phase 4: this CTA's rows of the chosen expert ---------
  {
    int id; float w;
    const bool rok = route_block(a.route, 0, rs, id, w, s_logits);
    __syncthreads();                    // every warp is done with the raw scores before the final weights replace them
    if (warp == 0) {
      if (lane < a.n_used) { rs.ids[lane] = rok ? id : -3; rs.wraw[lane] = w; }
      __syncwarp();
      if (j == 0 && c == 0) {
        if (!rok && lane == 0) raise_fault(a.fault, a.layer, FS_ROUTER);
        if (lane < a.n_used) {
          a.ids[lane] = rok ? id : -3;
          a.wts[lane] = w;
          if (rok && a.heat) atomicAdd(a.heat + id, 1u);
        }
      }
      if (lane == 0) {
        int e = rs.ids[j];
        if (e == kExpertElsewhere) e = -1;
        else if (e < 0 || e >= E) { e = -2; if (c == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID); }
        else if (a.slot_map) { e = a.slot_map[e]; if (e < 0) e = -1; }
        if (e >= 0) {
          const uint32_t gb = (uint32_t)(apc * rb_g), db = (uint32_t)(rpc * rb_d);
          mbar_expect_tx(&bar_gu, 2 * gb);
          bulk_load_chunks(s_gu, a.gate + ((long)e * I + (long)c * apc) * rb_g, gb, &bar_gu);
          bulk_load_chunks(s_gu + gb, a.up + ((long)e * I + (long)c * apc) * rb_g, gb, &bar_gu);
          mbar_expect_tx(&bar_d, db);                    // the router rows are no longer read: their room takes the down rows
          bulk_load_chunks(s_rd, a.down + ((long)e * H + (long)c * rpc) * rb_d, db, &bar_d);
        }
        s_e = e;
      }
    }
    __syncthreads();
  }
  const int e = s_e;
  probe_mark(a.probe, 4);

  // ---- phase 5: gate.x, up.x, SwiGLU of this CTA's activation rows -> every peer's activation row -----
  if (e >= 0) ok = mbar_wait(&bar_gu, 0, a.fault, a.layer) && ok;
  probe_mark(a.probe, 5);
  for (int r0 = warp * 2; r0 < apc; r0 += 16) {
    float gacc[2] = {0.f, 0.f}, uacc[2] = {0.f, 0.f};
    if (e >= 0) {
      const uint8_t* g0 = s_gu + (long)r0 * rb_g;
      const uint8_t* u0 = s_gu + (long)apc * rb_g + (long)r0 * rb_g;
      if constexpr (FAM == 0) {
        switch (a.gtype) {
          case WT_Q4_K: gate_up_rows_staged<Q4K>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q5_K: gate_up_rows_staged<Q5K>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q6_K: gate_up_rows_staged<Q6K>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q8_0: gate_up_rows_staged<Q80>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          default: gacc[0] = gacc[1] = kNaN;
        }
      } else {
        switch (a.gtype) {
          case WT_NVFP4: gate_up_rows_staged<NvFp4>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_FP8_B128: gate_up_rows_staged<Fp8B128>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q2_K: gate_up_rows_staged<Q2K>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q3_K: gate_up_rows_staged<Q3K>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q4_0: gate_up_rows_staged<Q40>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q4_1: gate_up_rows_staged<Q41>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q5_0: gate_up_rows_staged<Q50>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          case WT_Q5_1: gate_up_rows_staged<Q51>(g0, u0, rb_g, H, lane, s_xq, s_xds, gacc, uacc); break;
          default: gacc[0] = gacc[1] = kNaN;
        }
      }
    }
    // lanes 0..15: row r0 to peer lane; lanes 16..31: row r0 + 1 to peer lane - 16
    const int rr = lane >> 4;
    if (r0 + rr < apc) {
      const float g = gacc[rr];
      float v = (g / (1.0f + expf(-g))) * uacc[rr];
      if (e == -1) v = 0.f;
      else if (e < 0 || !ok) v = kNaN;
      st_peer_f32(peer_addr(s_act + (int)c * apc + r0 + rr, (unsigned)(lane & 15)), v);
    }
  }
  cluster_sync_all();
  probe_mark(a.probe, 6);

  // ---- phase 6: q8 of the expert's activation row --------------------------------------------------
  {
    const int nb32 = I / 32, layout = staged_layout(a.dtype), upe = I / 64;
    for (int b = warp; b < nb32; b += 8) {
      const int i = b * 32 + lane;
      const float v = s_act[i];
      float d, sm;
      const int8_t qv = q8_lane(v, d, sm);
      s_actq[act_chunk_pos(i >> 4, upe, layout) * 16 + (i & 15)] = qv;
      if (lane == 0) s_ads[b] = make_float2(d, sm);
    }
  }
  __syncthreads();

  // ---- phase 7: this CTA's rows of the down projection ---------------------------------------------
  if (e >= 0) ok = mbar_wait(&bar_d, 0, a.fault, a.layer) && ok;
  probe_mark(a.probe, 7);
  if (e >= 0) {
    if constexpr (FAM == 0) {
      switch (a.dtype) {
        case WT_Q4_K: down_rows_cluster<Q4K>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q5_K: down_rows_cluster<Q5K>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q6_K: down_rows_cluster<Q6K>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q8_0: down_rows_cluster<Q80>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        default: ok = false;
      }
    } else {
      switch (a.dtype) {
        case WT_NVFP4: down_rows_cluster<NvFp4>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_FP8_B128: down_rows_cluster<Fp8B128>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q2_K: down_rows_cluster<Q2K>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q3_K: down_rows_cluster<Q3K>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q4_0: down_rows_cluster<Q40>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q4_1: down_rows_cluster<Q41>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q5_0: down_rows_cluster<Q50>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        case WT_Q5_1: down_rows_cluster<Q51>(s_rd, rb_d, I, rpc, s_actq, s_ads, s_p); break;
        default: ok = false;
      }
    }
  }
  __syncthreads();
  probe_mark(a.probe, 8);
  for (int r = tid; r < rpc; r += 256) {
    float p = 0.f;
    if (e >= 0) p = ok ? s_p[r] : kNaN;
    else if (e == -2) p = kNaN;
    a.parts[(long)j * H + (long)c * rpc + r] = p;
  }

  // ---- phase 8: the last cluster to finish this row slice adds the slots up --------------------------
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned t = atomicAdd(a.tickets + c, 1u);
    s_last = (t == (unsigned)a.n_used - 1u) ? 1 : 0;
    if (s_last) a.tickets[c] = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int r = tid; r < rpc; r += 256) {
    const int d = (int)c * rpc + r;
    float y = 0.f;
    for (int q = 0; q < a.n_used; ++q) y = fmaf(rs.wraw[q], __ldcg(a.parts + (long)q * H + d), y);
    if (a.extra) y += a.extra[d];
    a.x_out[d] = y + a.x[d];
  }
  probe_mark(a.probe, 9);
}

extern long long* g_stage_probe;

}  // namespace bl

using namespace bl;

// 0 when the cluster launch serves this shape on this device (16-CTA clusters, one per chosen expert, all
// resident at once), a negative contract code otherwise; `smem_bytes` receives the dynamic shared memory it needs.
static int moe_cluster_check(int H, int I, int E, int n_used, int rtype, int gtype, int utype, int dtype, int* smem_bytes) {
  BL_REQUIRE(H % (kCl * 8) == 0 && H % 256 == 0 && I % (kCl * 2) == 0 && I % 64 == 0 && E % kCl == 0 && E <= kMaxExperts, BL_ERR_SHAPE);
  BL_REQUIRE(H / kCl <= 512 && n_used >= 1 && n_used <= kMaxTopK, BL_ERR_SHAPE);
  BL_REQUIRE(rtype == WT_F32 || rtype == WT_F16 || rtype == WT_BF16, BL_ERR_TYPE);
  BL_REQUIRE(gtype == utype, BL_ERR_TYPE);
  const long rb_g = resident_row_bytes(gtype, H), rb_d = resident_row_bytes(dtype, I);
  BL_REQUIRE(rb_g > 0 && rb_d > 0 && rb_g % 16 == 0 && rb_d % 16 == 0, BL_ERR_TYPE);
  BL_REQUIRE(gtype != WT_F32 && gtype != WT_F16 && gtype != WT_BF16 && dtype != WT_F32 && dtype != WT_F16 && dtype != WT_BF16, BL_ERR_TYPE);
  BL_REQUIRE((I % 256 == 0) || dtype == WT_Q8_0 || dtype == WT_NVFP4 || dtype == WT_Q4_0 || dtype == WT_Q4_1 || dtype == WT_Q5_0 ||
             dtype == WT_Q5_1 || (dtype == WT_FP8_B128 && I % 128 == 0), BL_ERR_SHAPE);
  const MoeClusterSmem L = moe_cluster_layout(H, I, E, rtype, gtype, dtype);
  BL_REQUIRE(L.total + 10 * 1024 <= 227 * 1024, BL_ERR_LIMIT);      // static shared memory of the kernel rides on top
  BL_REQUIRE((long)2 * (I / kCl) * rb_g < (1 << 20) && (long)(H / kCl) * rb_d < (1 << 20), BL_ERR_LIMIT);
  *smem_bytes = L.total;
  return 0;
}

template <int FAM>
static int moe_cluster_launch(const MoeClusterArgs& a, int smem, int n_used, cudaStream_t st, bool query_only) {
  static int max_clusters = -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kCl, n_used, 1);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCl; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (max_clusters < 0) {
    cudaError_t e = cudaFuncSetAttribute(moe_cluster_kernel<FAM>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_cluster_kernel<FAM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 217 * 1024);
    if (e != cudaSuccess) { cudaGetLastError(); return BL_ERR_LIMIT; }
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, moe_cluster_kernel<FAM>, &cfg);
    if (e != cudaSuccess) { cudaGetLastError(); n = 0; }
    max_clusters = n;
  }
  // every chosen expert's cluster must be resident at once, or the launch would run in waves
  if (max_clusters < n_used) return BL_ERR_LIMIT;
  if (query_only) return 0;
  cfg.numAttrs = g_use_pdl ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, moe_cluster_kernel<FAM>, a);
}

static int fam_of(int t) { return (t == WT_Q4_K || t == WT_Q5_K || t == WT_Q6_K || t == WT_Q8_0) ? 0 : 2; }

extern "C" {

// Most clusters of `size` CTAs (each with `smem` bytes of dynamic shared memory, 256 threads) resident at once.
int bl_max_active_clusters(int size, int smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(size, 64, 1);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = (size_t)smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = size; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaFuncSetAttribute(moe_cluster_kernel<0>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
  cudaFuncSetAttribute(moe_cluster_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 217 * 1024);
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, moe_cluster_kernel<0>, &cfg) != cudaSuccess) { cudaGetLastError(); return -1; }
  return n;
}

// Whether bl_moe_cluster serves this shape on the current device (0 = yes).
int bl_moe_cluster_fits(int H, int I, int E, int n_used, int rtype, int gtype, int utype, int dtype) {
  int smem = 0;
  const int rc = moe_cluster_check(H, I, E, n_used, rtype, gtype, utype, dtype, &smem);
  if (rc != 0) return rc;
  if (fam_of(gtype) != fam_of(dtype)) return BL_ERR_TYPE;
  MoeClusterArgs a{};
  return fam_of(gtype) == 0 ? moe_cluster_launch<0>(a, smem, n_used, nullptr, true) : moe_cluster_launch<2>(a, smem, n_used, nullptr, true);
}

// The expert half of a decode layer for ONE activation row, in one cluster launch (see the head of this file).
// parts: scratch [n_used * H] floats; tickets: 16 zeroed words (left zero); x_out must not alias x.
int bl_moe_cluster(const float* x, const float* gain, float eps, const void* rw, int rtype, const float* bias, int mode,
                   int renorm, float scale, int n_group, int topk_group, const int* slot_map, const void* gate, const void* up,
                   int gtype, int utype, const void* down, int dtype, int H, int I, int E, int n_used, const float* extra,
                   float* parts, unsigned* tickets, float* x_out, float* logits, int* ids, float* wts, unsigned* heat,
                   unsigned* fault, int layer, cudaStream_t st) {
  int smem = 0;
  const int rc = moe_cluster_check(H, I, E, n_used, rtype, gtype, utype, dtype, &smem);
  if (rc != 0) return rc;
  BL_REQUIRE(fam_of(gtype) == fam_of(dtype), BL_ERR_TYPE);
  BL_REQUIRE(x != x_out && ids && wts && parts && tickets, BL_ERR_SHAPE);
  BL_REQUIRE(E % 4 == 0 && n_group >= 1 && n_group <= 16 && E % n_group == 0 && topk_group >= 1 && topk_group <= n_group, BL_ERR_LIMIT);
  BL_REQUIRE((((uintptr_t)rw | (uintptr_t)gate | (uintptr_t)up | (uintptr_t)down | (uintptr_t)x | (uintptr_t)gain) & 15) == 0, BL_ERR_ALIGN);
  MoeClusterArgs a{x, gain, eps, (const uint8_t*)rw, rtype,
                   RouteParams{nullptr, bias, E, n_used, mode, renorm, scale, n_group, topk_group}, slot_map,
                   (const uint8_t*)gate, (const uint8_t*)up, gtype, (const uint8_t*)down, dtype, H, I, E, n_used, extra, parts,
                   tickets, x_out, logits, ids, wts, heat, fault, layer, g_stage_probe};
  return fam_of(gtype) == 0 ? moe_cluster_launch<0>(a, smem, n_used, st, false) : moe_cluster_launch<2>(a, smem, n_used, st, false);
}

}  // extern "C"
