// Routing shared by the decode MoE kernels: argument blocks and the block-wide top-k by rank counting.
#pragma once
#include "common.cuh"

namespace bl {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

// Routing parameters shared by the router launch and its consumers.
struct RouteParams {
  const float* logits;   // [M, E]
  const float* bias;     // [E] selection bias (sigmoid mode) or null
  int E, top_k, mode, renorm;
  float scale;
  int n_group, topk_group;
};

struct RouterArgs {
  const float* x; long x_stride;       // [M, K] residual stream
  const float* gain; float eps;
  const uint8_t* w; int wtype;         // [E, K] F32 / F16 / BF16
  int K, E, M;
  float* logits;                       // [M, E]
  int8_t* xq_out; float2* xds_out;     // q8 of the normed rows [M, K]
  float* xn_out;                       // optional fp32 normed rows [M, K]
  unsigned* fault; int layer;
  ReduceIn red;                        // n_ranks > 0: x = x + sum of every rank's partial rows
  // ticket != null: the block that finishes last (completion ticket, one word per row group, zero between
  // launches) turns the logits into (ids, weights) for the launches that follow and counts the picks
  unsigned* ticket;
  RouteParams route;                   // route.logits is ignored here (the kernel's own logits are routed)
  int* ids; float* wts;                // [M, top_k]
  unsigned* heat;                      // optional [E] routed-count histogram
  // Prediction form (pf_gate != null, with a ticket): the launch runs on the layer's INPUT rows, ahead of the
  // attention launches, and its last block asks L2 to prefetch the gate / up / down matrices of the route.top_k
  // best-scoring experts of each row.  Nothing is published: the real routing still happens on the real rows.
  const uint8_t* pf_gate; const uint8_t* pf_up; const uint8_t* pf_down;
  long pf_gate_bytes, pf_down_bytes;   // bytes of one expert's matrix in each stack
  const int* pf_slot_map;              // optional [E]: expert id -> resident slot (negative = not on this device)
};

// Block-wide routing of one row by rank counting: every thread owns up to two experts,
// reads all scores from shared memory and counts how many beat its own (larger score, or
// equal score at a smaller id); an expert of rank r < top_k is slot r.  No serial arg-max
// rounds, so it is short enough to run redundantly in every consumer block.  Softmax
// weights need only the chosen logits: w_j = exp(l_j - l_top) / sum over the chosen
// (renormalised) or over all experts (not renormalised).
struct __align__(16) RouteShared {
  float sc[kMaxExperts];
  float wv[kMaxExperts];
  float gs[16];
  int ids[kMaxTopK];
  float wraw[kMaxTopK];
  float total;
};

// `smem_logits`: the row's logits in shared memory (a kernel that computed them itself); null = read p.logits.
__device__ __forceinline__ bool route_block(const RouteParams& p, int m, RouteShared& sh, int& my_id, float& my_w,
                                            const float* smem_logits = nullptr) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  bool nonfinite = false;
  for (int e = tid; e < p.E; e += nthr) {
    const float l = smem_logits ? smem_logits[e] : __ldcg(p.logits + (long)m * p.E + e);
    if (!isfinite(l)) nonfinite = true;
    if (p.mode == 0) { sh.sc[e] = l; sh.wv[e] = l; }
    else { const float sg = 1.0f / (1.0f + expf(-l)); sh.wv[e] = sg; sh.sc[e] = sg + (p.bias ? p.bias[e] : 0.f); }
  }
  if (tid < kMaxTopK) { sh.ids[tid] = 0; sh.wraw[tid] = 0.f; }
  if (__syncthreads_or(nonfinite)) { my_id = 0; my_w = __int_as_float(0x7fc00000); return false; }
  if (p.n_group > 1) {
    const int gsz = p.E / p.n_group;
    if (tid < p.n_group) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int i = 0; i < gsz; ++i) { const float v = sh.sc[tid * gsz + i]; if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) b2 = v; }
      sh.gs[tid] = b1 + b2;
    }
    __syncthreads();
    bool drop[2] = {false, false};
    int c = 0;
    for (int e = tid; e < p.E; e += nthr, ++c) {
      const int g = e / gsz;
      const float mine = sh.gs[g];
      int rank = 0;
      for (int o = 0; o < p.n_group; ++o) rank += (sh.gs[o] > mine || (sh.gs[o] == mine && o < g)) ? 1 : 0;
      drop[c & 1] = rank >= p.topk_group;
    }
    c = 0;
    for (int e = tid; e < p.E; e += nthr, ++c) if (drop[c & 1]) sh.sc[e] = -INFINITY;
    __syncthreads();
  }
  for (int e = tid; e < p.E; e += nthr) {
    const float v = sh.sc[e];
    if (v == -INFINITY) continue;
    int rank = 0;
    for (int o = 0; o < p.E; o += 4) {
      const float4 q = *reinterpret_cast<const float4*>(sh.sc + o);
      rank += (q.x > v || (q.x == v && o < e)) ? 1 : 0;
      rank += (q.y > v || (q.y == v && o + 1 < e)) ? 1 : 0;
      rank += (q.z > v || (q.z == v && o + 2 < e)) ? 1 : 0;
      rank += (q.w > v || (q.w == v && o + 3 < e)) ? 1 : 0;
    }
    if (rank < p.top_k) { sh.ids[rank] = e; sh.wraw[rank] = sh.wv[e]; }
  }
  if (p.mode == 0 && !p.renorm && tid < 32) {
    double part = 0.0;
    float top = -INFINITY;
    for (int e = tid; e < p.E; e += 32) top = fmaxf(top, sh.wv[e]);
    top = warp_max(top);
    for (int e = tid; e < p.E; e += 32) part += (double)expf(sh.wv[e] - top);
    part = warp_sum_d(part);
    if (tid == 0) sh.total = (float)part;
  }
  __syncthreads();
  const int t = tid & 31;
  my_id = t < p.top_k ? sh.ids[t] : 0;
  float w = 0.f;
  if (t < p.top_k) {
    if (p.mode == 0) {
      const float top = sh.wraw[0];
      w = expf(sh.wraw[t] - top);
      if (p.renorm) {
        double sum = 0.0;
        for (int j = 0; j < p.top_k; ++j) sum += (double)expf(sh.wraw[j] - top);
        w = w / (float)sum;
      } else {
        w = w / sh.total;
      }
    } else {
      w = sh.wraw[t];
      if (p.renorm) {
        double sum = 0.0;
        for (int j = 0; j < p.top_k; ++j) sum += (double)sh.wraw[j];
        w = w / (float)sum;
      }
    }
    w *= p.scale;
  }
  my_w = w;
  return true;
}


// The same routing by ONE warp, for the common shape (one expert group, at most 256 experts, a multiple of 32):
// no block barriers, so a kernel can route in warp 0 while its other warps fetch activations.  Scores, ranks,
// weights and tie rule are those of route_block (same sums in the same order: the results are bit-equal).
struct __align__(16) RouteWarpShared {
  int ids[kMaxTopK];
  float wraw[kMaxTopK];
};

__device__ __forceinline__ bool route_warp_ok(const RouteParams& p) { return p.n_group <= 1 && p.E <= 256 && (p.E % 32) == 0; }

__device__ __forceinline__ bool route_warp(const RouteParams& p, int m, RouteWarpShared& sh, int lane, int& my_id, float& my_w) {
  const int per = p.E / 32;
  float sc[8], wv[8];
  bool nonfinite = false;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    sc[c] = 0.f; wv[c] = 0.f;
    if (c < per) {
      const int e = lane + 32 * c;
      const float l = __ldcg(p.logits + (long)m * p.E + e);
      if (!isfinite(l)) nonfinite = true;
      if (p.mode == 0) { sc[c] = l; wv[c] = l; }
      else { const float sg = 1.0f / (1.0f + expf(-l)); wv[c] = sg; sc[c] = sg + (p.bias ? p.bias[e] : 0.f); }
    }
  }
  if (lane < kMaxTopK) { sh.ids[lane] = 0; sh.wraw[lane] = 0.f; }
  if (__any_sync(0xffffffffu, nonfinite)) { my_id = 0; my_w = __int_as_float(0x7fc00000); return false; }
  // top_k rounds of a warp arg-max (larger score wins, equal scores go to the smaller id: the order rank counting
  // gives); a single warp has no spare lanes for all-pairs counting, and a round is ~50 dependent instructions
  for (int r = 0; r < p.top_k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int c = 0; c < 8; ++c)
      if (c < per && sc[c] > bv) { bv = sc[c]; bi = lane + 32 * c; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == (bi & 31)) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c == (bi >> 5)) { sh.ids[r] = bi; sh.wraw[r] = wv[c]; sc[c] = -INFINITY; }
    }
  }
  float total = 1.f;
  if (p.mode == 0 && !p.renorm) {
    float top = -INFINITY;
#pragma unroll
    for (int c = 0; c < 8; ++c) if (c < per) top = fmaxf(top, wv[c]);
    top = warp_max(top);
    double part = 0.0;
#pragma unroll
    for (int c = 0; c < 8; ++c) if (c < per) part += (double)expf(wv[c] - top);
    total = (float)warp_sum_d(part);
  }
  __syncwarp();
  my_id = lane < p.top_k ? sh.ids[lane] : 0;
  float w = 0.f;
  if (lane < p.top_k) {
    if (p.mode == 0) {
      const float top = sh.wraw[0];
      w = expf(sh.wraw[lane] - top);
      if (p.renorm) {
        double sum = 0.0;
        for (int j = 0; j < p.top_k; ++j) sum += (double)expf(sh.wraw[j] - top);
        w = w / (float)sum;
      } else {
        w = w / total;
      }
    } else {
      w = sh.wraw[lane];
      if (p.renorm) {
        double sum = 0.0;
        for (int j = 0; j < p.top_k; ++j) sum += (double)sh.wraw[j];
        w = w / (float)sum;
      }
    }
    w *= p.scale;
  }
  my_w = w;
  return true;
}

}  // namespace bl
