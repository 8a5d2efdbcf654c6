// Sampler on the card: one block per row runs the whole chain on the logits where they
// already are, so a sampled request costs one 4-byte token readback instead of a 600 KB
// logits row.
//
//   penalties (repeat / frequency / presence over the recent window)
//   -> top-k by radix select on order-preserving keys (4 passes of 8 bits; ties to the
//      smaller id) -> bitonic sort of the survivors (logit descending, id ascending)
//   -> min-p (logit >= max + ln(min_p)) and top-p (shortest prefix whose mass, normalised
//      over ALL top-k survivors and untempered, reaches top_p)
//   -> temperature -> softmax in f64 -> one draw u * total over the running sums, u from
//      xoshiro256** seeded through splitmix64 with a per-row draw counter (53-bit uniform)
//
// This is the chain of the host oracle (serve/sampler.py) and of the reference
// (crates/sampler/src/lib.rs:190-346); temperature <= 0 is the arg-max after penalties.
// top_k is capped at kMaxCand (1024) on the card; top_k = 0 ("all") samples from the 1024
// best, which carries all but a vanishing share of the mass.
//
// Few rows: one block per row leaves the card idle while 1,024 threads walk 150 k logits five
// times, so up to 8 rows take two launches.  sample_select_kernel splits a row's vocabulary over
// kSelBlocks blocks; each applies the penalties to its slice and writes its own top-k (same keys,
// same tie rule, in ascending id order) to a candidate list; sample_rows_kernel then runs unchanged
// on that list (ids through an index array).  The global top-k is a subset of the union of the
// slices' top-k and the list keeps id order, so the picked token is the same, bit for bit.
#include "common.cuh"

namespace bl {

constexpr int kMaxCand = 1024;

struct SampleArgs {
  const float* logits; long stride; int V; int M;
  const int* recent; int recent_stride; const int* n_recent;   // [M, recent_stride] window (newest last), counts
  const float* params;      // [M, 8]: temperature, top_k, top_p, min_p, repeat_penalty, frequency_penalty, presence_penalty, repeat_last_n
  const unsigned long long* seeds;   // [M]
  unsigned long long* draws;         // [M] draws made so far (advanced here)
  float* work;              // [M, V] scratch row for penalised logits (only touched when penalties apply)
  int* out_token;           // [M]
  int* out_n_cand;          // optional [M]
  unsigned* fault;
  const int* ids;           // optional [M, stride]: id of entry i of a row (a candidate list); null = i itself
  int penalties_done;       // the rows already carry their penalties (candidate lists do)
};

constexpr int kSelBlocks = 32;

__device__ __forceinline__ unsigned key_of(float v) {
  // order-preserving map float -> u32 (larger float = larger key); NaN sorts lowest
  if (v != v) return 0u;
  unsigned b = __float_as_uint(v + 0.0f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long rotl64(unsigned long long x, int k) { return (x << k) | (x >> (64 - k)); }

__device__ double xoshiro_draw(unsigned long long seed, unsigned long long n_before) {
  unsigned long long z = seed, s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    z += 0x9E3779B97F4A7C15ull;
    unsigned long long x = z;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    s[i] = x ^ (x >> 31);
  }
  unsigned long long out = 0;
  for (unsigned long long i = 0; i <= n_before; ++i) {
    out = rotl64(s[1] * 5ull, 7) * 9ull;
    const unsigned long long t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl64(s[3], 45);
  }
  return (double)(out >> 11) * (1.0 / 9007199254740992.0);
}

// Inclusive prefix sum over the block's 1024 threads (one value each), fixed order.
__device__ __forceinline__ double block_scan_d(double v, double* warp_tot /* [32] shared */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    double w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  return v + (warp > 0 ? warp_tot[warp - 1] : 0.0);
}
__device__ __forceinline__ unsigned block_scan_u(unsigned v, unsigned* warp_tot /* [32] shared */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  return v + (warp > 0 ? warp_tot[warp - 1] : 0u);
}

__global__ void __launch_bounds__(1024) sample_rows_kernel(const SampleArgs a) {
  __shared__ unsigned hist[256];
  __shared__ unsigned s_prefix, s_need, s_count;
  __shared__ float c_val[kMaxCand];
  __shared__ int c_id[kMaxCand];
  __shared__ double s_red[32];
  __shared__ int s_keep, s_pick;
  const int m = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  const float* P = a.params + (long)m * 8;
  const float temperature = P[0], top_p = P[2], min_p = P[3], rep = P[4], freq = P[5], pres = P[6];
  int top_k = (int)P[1];
  const int last_n = (int)P[7];
  const int V = a.V;
  const float* row = a.logits + (long)m * a.stride;
  // ---- penalties --------------------------------------------------------------------------
  const int n_rec = a.n_recent ? min(a.n_recent[m], a.recent_stride) : 0;
  const int win = min(n_rec, max(last_n, 0));
  const bool penal = !a.penalties_done && win > 0 && (rep != 1.0f || freq != 0.0f || pres != 0.0f);
  const int* ids = a.ids ? a.ids + (long)m * a.stride : nullptr;
  if (penal) {
    float* w = a.work + (long)m * V;
    for (int i = tid; i < V; i += 1024) w[i] = row[i];
    __syncthreads();
    const int* rec = a.recent + (long)m * a.recent_stride + (n_rec - win);
    for (int i = tid; i < win; i += 1024) {
      const int t = rec[i];
      if (t < 0 || t >= V) continue;
      bool first = true;                       // once per distinct token: the first occurrence does it
      int count = 0;
      for (int j = 0; j < win; ++j) { if (rec[j] == t) { if (j < i) first = false; ++count; } }
      if (!first) continue;
      float l = row[t];
      l = (l <= 0.f) ? l * rep : l / rep;
      w[t] = l - ((float)count * freq + pres);
    }
    __syncthreads();
    row = w;
  }
  // ---- greedy -----------------------------------------------------------------------------
  if (temperature <= 0.f) top_k = 1;
  if (top_k <= 0 || top_k > kMaxCand) top_k = kMaxCand;
  if (top_k > V) top_k = V;
  // ---- radix select: the key of the top_k-th best ---------------------------------------------
  if (tid == 0) { s_prefix = 0u; s_need = (unsigned)top_k; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < V; i += 1024) {
      const unsigned k = key_of(row[i]);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xFF], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned need = s_need, acc = 0;
      int b = 255;
      for (; b > 0; --b) { if (acc + hist[b] >= need) break; acc += hist[b]; }
      s_need = need - acc;                 // how many are still wanted inside bucket b
      s_prefix = prefix | ((unsigned)b << shift);
    }
    __syncthreads();
  }
  const unsigned kth = s_prefix;            // key of the k-th best; s_need of the ties at kth are wanted
  // ---- gather: everything above kth, then the lowest-id ties at kth ----------------------------
  if (tid == 0) s_count = 0u;
  __syncthreads();
  for (int i = tid; i < V; i += 1024) {
    const float v = row[i];
    if (key_of(v) > kth) { const unsigned p = atomicAdd(&s_count, 1u); if (p < kMaxCand) { c_val[p] = v; c_id[p] = ids ? ids[i] : i; } }
  }
  __syncthreads();
  {
    // ties at kth: the s_need lowest ids.  Each thread owns a contiguous id range, counts its
    // ties, a block scan turns counts into positions, so id order is kept without a serial scan.
    __shared__ unsigned s_wt[32];
    const unsigned base = s_count, want = s_need;
    const int per = (V + 1023) / 1024;
    const int i0 = tid * per, i1 = min(V, i0 + per);
    unsigned mine = 0;
    for (int i = i0; i < i1; ++i) mine += key_of(row[i]) == kth ? 1u : 0u;
    const unsigned incl = block_scan_u(mine, s_wt);
    unsigned pos = incl - mine;
    for (int i = i0; i < i1 && pos < want; ++i)
      if (key_of(row[i]) == kth) {
        if (base + pos < kMaxCand) { c_val[base + pos] = row[i]; c_id[base + pos] = ids ? ids[i] : i; }
        ++pos;
      }
    __syncthreads();
    if (tid == 0) s_count = min(base + want, (unsigned)kMaxCand);
  }
  __syncthreads();
  const int n = (int)s_count;
  // ---- bitonic sort: logit descending, id ascending ---------------------------------------------
  for (int i = n + tid; i < kMaxCand; i += 1024) { c_val[i] = -INFINITY; c_id[i] = 0x7fffffff; }
  __syncthreads();
  for (int k2 = 2; k2 <= kMaxCand; k2 <<= 1) {
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      const int i = tid, l = i ^ j;
      if (l > i) {
        const float vi = c_val[i], vl = c_val[l];
        const int ii = c_id[i], il = c_id[l];
        const bool i_first = key_of(vi) > key_of(vl) || (key_of(vi) == key_of(vl) && ii < il);   // i ranks before l
        const bool up = (i & k2) == 0;
        if (up ? !i_first : i_first) { c_val[i] = vl; c_val[l] = vi; c_id[i] = il; c_id[l] = ii; }
      }
      __syncthreads();
    }
  }
  if (a.out_n_cand && tid == 0) a.out_n_cand[m] = n;
  if (n <= 1 || temperature <= 0.f || !(c_val[0] > -INFINITY) || c_val[0] == INFINITY) {
    if (tid == 0) a.out_token[m] = (n >= 1 && c_id[0] != 0x7fffffff) ? c_id[0] : 0;
    return;
  }
  // ---- min-p and top-p (untempered, normalised over all top-k survivors) -------------------------
  // one candidate per thread; every sum is a block scan in thread order, so reruns are bit-identical
  const float mx = c_val[0];
  const bool live = tid < n;
  const double e1 = live ? exp((double)(c_val[tid] - mx)) : 0.0;
  const double cum1 = block_scan_d(e1, s_red);
  __shared__ double s_norm, s_total, s_u;
  if (tid == 1023) s_norm = cum1;
  if (tid == 0) s_keep = n;
  __syncthreads();
  const double norm = s_norm;
  if (min_p > 0.f) {
    const float floor_v = mx + logf(min_p);
    if (live && c_val[tid] < floor_v) atomicMin(&s_keep, max(1, tid));       // sorted: survivors are a prefix
  }
  __syncthreads();
  if (top_p < 1.0f) {
    if (live && cum1 / norm >= (double)top_p) atomicMin(&s_keep, tid + 1);     // shortest prefix reaching top_p
  }
  __syncthreads();
  const int keep = s_keep;
  // ---- temperature, softmax in f64, one draw ------------------------------------------------------
  const double inv_t = 1.0 / (double)temperature;
  const double e2 = tid < keep ? exp((double)(c_val[tid] - mx) * inv_t) : 0.0;
  const double cum2 = block_scan_d(e2, s_red);
  if (tid == 1023) s_total = cum2;
  if (tid == 0) {
    const unsigned long long nd = a.draws ? a.draws[m] : 0ull;
    s_u = keep > 1 ? xoshiro_draw(a.seeds ? a.seeds[m] : 0ull, nd) : 0.0;
    if (a.draws && keep > 1) a.draws[m] = nd + 1ull;
    s_pick = keep - 1;
  }
  __syncthreads();
  const double u = s_u * s_total;
  if (keep > 1 && tid < keep && cum2 > u) atomicMin(&s_pick, tid);               // first running sum above u
  __syncthreads();
  if (tid == 0) {
    a.out_token[m] = c_id[keep > 1 ? s_pick : 0];
    if (a.out_n_cand) a.out_n_cand[m] = keep;
  }
}

// Stage 1 of the few-row form: block (slice, row) selects the slice's top_k and writes them in ascending id order to
// cand_val / cand_id [M][kSelBlocks][cap]; unused cells hold NaN (the lowest key) and id INT_MAX.
struct SelectArgs {
  const float* logits; long stride; int V;
  const int* recent; int recent_stride; const int* n_recent;
  const float* params;
  float* cand_val; int* cand_id; int cap;
};

__global__ void __launch_bounds__(1024) sample_select_kernel(const SelectArgs a) {
  __shared__ unsigned hist[256];
  __shared__ unsigned s_prefix, s_need;
  __shared__ unsigned s_wt[32];
  extern __shared__ float s_slice[];                     // the slice's (penalised) logits
  const int blk = blockIdx.x, m = blockIdx.y, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  const float* P = a.params + (long)m * 8;
  const float temperature = P[0], rep = P[4], freq = P[5], pres = P[6];
  int top_k = (int)P[1];
  const int last_n = (int)P[7];
  const int per_blk = (a.V + kSelBlocks - 1) / kSelBlocks;
  const int v0 = blk * per_blk, v1 = min(a.V, v0 + per_blk), n = max(0, v1 - v0);
  const float* row = a.logits + (long)m * a.stride;
  for (int i = tid; i < n; i += 1024) s_slice[i] = row[v0 + i];
  __syncthreads();
  const int n_rec = a.n_recent ? min(a.n_recent[m], a.recent_stride) : 0;
  const int win = min(n_rec, max(last_n, 0));
  if (win > 0 && (rep != 1.0f || freq != 0.0f || pres != 0.0f)) {
    const int* rec = a.recent + (long)m * a.recent_stride + (n_rec - win);
    for (int i = tid; i < win; i += 1024) {
      const int t = rec[i];
      if (t < v0 || t >= v1) continue;
      bool first = true;
      int count = 0;
      for (int j = 0; j < win; ++j) { if (rec[j] == t) { if (j < i) first = false; ++count; } }
      if (!first) continue;
      float l = row[t];
      l = (l <= 0.f) ? l * rep : l / rep;
      s_slice[t - v0] = l - ((float)count * freq + pres);
    }
    __syncthreads();
  }
  if (temperature <= 0.f) top_k = 1;
  if (top_k <= 0 || top_k > kMaxCand) top_k = kMaxCand;
  top_k = min(top_k, a.cap);
  float* out_v = a.cand_val + ((long)m * kSelBlocks + blk) * a.cap;
  int* out_i = a.cand_id + ((long)m * kSelBlocks + blk) * a.cap;
  const int want_all = min(top_k, n);
  for (int i = want_all + tid; i < a.cap; i += 1024) { out_v[i] = __int_as_float(0x7fc00000); out_i[i] = 0x7fffffff; }
  if (n == 0) return;
  // radix select of the slice's want_all-th best key
  if (tid == 0) { s_prefix = 0u; s_need = (unsigned)want_all; }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int i = tid; i < n; i += 1024) {
      const unsigned k = key_of(s_slice[i]);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 0xFF], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned need = s_need, acc = 0;
      int b = 255;
      for (; b > 0; --b) { if (acc + hist[b] >= need) break; acc += hist[b]; }
      s_need = need - acc;
      s_prefix = prefix | ((unsigned)b << shift);
    }
    __syncthreads();
  }
  const unsigned kth = s_prefix, ties_wanted = s_need;
  // ordered gather: every thread owns a contiguous id range; two block scans give the positions of the entries above
  // kth and of the lowest-id ties at kth, so the list comes out in ascending id order
  const int per = (n + 1023) / 1024;
  const int i0 = min(n, tid * per), i1 = min(n, i0 + per);
  unsigned above = 0, ties = 0;
  for (int i = i0; i < i1; ++i) { const unsigned k = key_of(s_slice[i]); above += k > kth; ties += k == kth; }
  const unsigned tie_incl = block_scan_u(ties, s_wt);
  unsigned tie_pos = tie_incl - ties;                                   // ties before this thread's range
  unsigned take = 0;                                                    // entries of this range that are kept
  {
    unsigned tp = tie_pos;
    for (int i = i0; i < i1; ++i) {
      const unsigned k = key_of(s_slice[i]);
      if (k > kth) ++take;
      else if (k == kth) { if (tp < ties_wanted) ++take; ++tp; }
    }
  }
  const unsigned take_incl = block_scan_u(take, s_wt);
  unsigned pos = take_incl - take;
  for (int i = i0; i < i1; ++i) {
    const unsigned k = key_of(s_slice[i]);
    bool keep = k > kth;
    if (k == kth) { keep = tie_pos < ties_wanted; ++tie_pos; }
    if (keep) { if (pos < (unsigned)a.cap) { out_v[pos] = s_slice[i]; out_i[pos] = v0 + i; } ++pos; }
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

// work: M*V floats of scratch (written only for rows with penalties); draws: per-row counters.
int bl_sample_rows(const float* logits, long stride, int V, int M, const int* recent, int recent_stride,
                   const int* n_recent, const float* params, const unsigned long long* seeds, unsigned long long* draws,
                   float* work, int* out_token, int* out_n_cand, unsigned* fault, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && V >= 1 && params != nullptr && out_token != nullptr, BL_ERR_SHAPE);
  SampleArgs a{logits, stride, V, M, recent, recent_stride, n_recent, params, seeds, draws, work, out_token, out_n_cand, fault,
               nullptr, 0};
  return (int)launch(sample_rows_kernel, dim3(M), dim3(1024), 0, st, a);
}

// The few-row form (M <= 8 is where it pays): cand_val / cand_id are caller-owned scratch of M * 32 * cap cells, cap =
// the largest top_k of the rows (at most 1024; rows with top_k <= 0 need 1024).  Same picks as bl_sample_rows.
int bl_sample_rows_split(const float* logits, long stride, int V, int M, const int* recent, int recent_stride,
                         const int* n_recent, const float* params, const unsigned long long* seeds,
                         unsigned long long* draws, float* cand_val, int* cand_id, int cap, int* out_token,
                         int* out_n_cand, unsigned* fault, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && V >= 1 && params != nullptr && out_token != nullptr && cand_val && cand_id, BL_ERR_SHAPE);
  BL_REQUIRE(cap >= 1 && cap <= kMaxCand, BL_ERR_LIMIT);
  const int per_blk = (V + kSelBlocks - 1) / kSelBlocks;
  const size_t smem = (size_t)per_blk * 4;
  BL_REQUIRE(smem <= 200 * 1024, BL_ERR_LIMIT);
  static bool set = false;
  if (!set) { cudaFuncSetAttribute(sample_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); set = true; }
  SelectArgs sa{logits, stride, V, recent, recent_stride, n_recent, params, cand_val, cand_id, cap};
  cudaError_t e = launch(sample_select_kernel, dim3(kSelBlocks, M), dim3(1024), smem, st, sa);
  if (e != cudaSuccess) return (int)e;
  const int L = kSelBlocks * cap;
  SampleArgs a{cand_val, (long)L, L, M, nullptr, 0, nullptr, params, seeds, draws, nullptr, out_token, out_n_cand, fault,
               cand_id, 1};
  return (int)launch(sample_rows_kernel, dim3(M), dim3(1024), 0, st, a);
}

}  // extern "C"
