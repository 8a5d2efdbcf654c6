// Decode-time multi-head latent attention (DeepSeek-V2/V3, Kimi-K2 shape: latent 512 + RoPE 64).
//
// The cache keeps one row of 576 f16 values per position and layer: the RMS-normalised
// compressed KV latent c (512) followed by the rotated shared key part (64).  Attention
// runs in the latent space ("absorbed" form):
//
//   1. mla_kv_append   RMSNorm(c) * gain, interleaved-pair RoPE on the 64 rope dims, f16 append
//   2. mla_q_absorb    per head: RoPE on q_rope, q_lat = W_kb[h]^T q_nope  -> q' [M, n_q, 576] (pre-scaled)
//   3. mla_flash_seg   split-K online softmax of q' against the latent rows on warp-level tensor-core tiles
//                      (16 heads = the M dimension); the value of a key is its first 512 entries (one read
//                      serves K and V)
//   4. mla_merge_vup   merge segments ascending, v = W_vb[h] * latent (128 x 512 per head), q8 for o_proj
//
// The reference's latent flash and its absorbed-q f32 GEMV: crates/gpu/src/flash.rs,
// crates/gpu/src/q8f32.rs (f32-activation sites "router, absorbed MLA q").  W_kb is kept as
// [head][nope][512] and W_vb as [head][v_dim][512], both f32 or bf16 (the per-head products keep
// f32 activations).
#include "common.cuh"

namespace bl {

constexpr int kMlaPage = 64;
constexpr int kLat = 512;
constexpr int kRope = 64;
constexpr int kRow = kLat + kRope;      // 576 values per cached position
constexpr int kTile = 32;
constexpr int kRowPad = kRow + 8;       // shared-memory row stride in halves: 16-byte reads by key lanes do not collide
constexpr int kHeadsPerBlock = 16;      // 8 warps x 2 heads

struct MlaAppendArgs {
  const float* kv;         // [M, stride]: 512 latent values then 64 rope values
  long stride;
  const float* gain;       // [512]
  const float* inv_freq;   // [32]
  float eps;
  int M;
  const int* row_pos;
  const int* row_seq;
  const int* block_table;
  int max_pages, n_pages;
  __half* cache;           // [n_pages][64][576]
  unsigned* fault;
  int layer;
};

// grid (M), 256 threads
__global__ void __launch_bounds__(256) mla_kv_append_kernel(const MlaAppendArgs a) {
  __shared__ double red[8];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_launch();
  const int seq = a.row_seq[m];
  if (seq < 0) return;
  const int pos = a.row_pos[m];
  const float* src = a.kv + (long)m * a.stride;
  const float x0 = src[tid], x1 = src[tid + 256];
  double ss = warp_sum_d((double)(x0 * x0) + (double)(x1 * x1));
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  double tot = 0.0;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float scale = (float)(1.0 / sqrt(tot / (double)kLat + (double)a.eps));
  const int pslot = pos / kMlaPage;
  const int page = (pos >= 0 && pslot < a.max_pages) ? a.block_table[(long)seq * a.max_pages + pslot] : -1;
  if (page < 0 || page >= a.n_pages) {
    if (tid == 0) raise_fault(a.fault, a.layer, FS_PAGE);
    return;
  }
  __half* dst = a.cache + ((long)page * kMlaPage + (pos % kMlaPage)) * kRow;
  dst[tid] = __float2half_rn((scale * a.gain[tid]) * x0);
  dst[tid + 256] = __float2half_rn((scale * a.gain[tid + 256]) * x1);
  if (tid < kRope / 2) {
    const float r0 = src[kLat + 2 * tid], r1 = src[kLat + 2 * tid + 1];
    float s, c;
    sincosf((float)pos * a.inv_freq[tid], &s, &c);
    dst[kLat + 2 * tid] = __float2half_rn(fmaf(r0, c, -(r1 * s)));
    dst[kLat + 2 * tid + 1] = __float2half_rn(fmaf(r0, s, r1 * c));
  }
}

template <typename W> __device__ __forceinline__ float wf(const W* p, long i);
template <> __device__ __forceinline__ float wf<float>(const float* p, long i) { return p[i]; }
template <> __device__ __forceinline__ float wf<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }

// eight consecutive weights as floats (16-byte loads for bf16, two for f32)
template <typename W> __device__ __forceinline__ void load8(const W* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}

struct MlaQArgs {
  const float* q;          // [M, stride]: head h at h * (nope + 64): nope values then 64 rope values
  long stride;
  const void* w_kb;        // [n_q][nope][512]
  const float* inv_freq;
  float scale;             // softmax scale folded into q'
  int n_q, nope, M;
  const int* row_pos;
  const int* row_seq;
  float* q_lat;            // [M, n_q, 576]
};

// grid (n_q, M), 256 threads: thread t owns latent columns 2t, 2t+1
template <typename W>
__global__ void __launch_bounds__(256) mla_q_absorb_kernel(const MlaQArgs a) {
  __shared__ float sq[128];
  const int h = blockIdx.x, m = blockIdx.y, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  if (a.row_seq[m] < 0) return;
  const float* src = a.q + (long)m * a.stride + (long)h * (a.nope + kRope);
  if (tid < a.nope) sq[tid] = src[tid];
  float* out = a.q_lat + ((long)m * a.n_q + h) * kRow;
  if (tid >= 128 && tid < 128 + kRope / 2) {
    const int j = tid - 128;
    const float r0 = src[a.nope + 2 * j], r1 = src[a.nope + 2 * j + 1];
    float s, c;
    sincosf((float)a.row_pos[m] * a.inv_freq[j], &s, &c);
    out[kLat + 2 * j] = fmaf(r0, c, -(r1 * s)) * a.scale;
    out[kLat + 2 * j + 1] = fmaf(r0, s, r1 * c) * a.scale;
  }
  __syncthreads();
  const W* w = reinterpret_cast<const W*>(a.w_kb) + (long)h * a.nope * kLat;
  float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
  for (int n = 0; n < a.nope; ++n) {
    const float qn = sq[n];
    a0 = fmaf(wf<W>(w, (long)n * kLat + 2 * tid), qn, a0);
    a1 = fmaf(wf<W>(w, (long)n * kLat + 2 * tid + 1), qn, a1);
  }
  out[2 * tid] = a0 * a.scale;
  out[2 * tid + 1] = a1 * a.scale;
}

struct MlaFlashArgs {
  const float* q_lat;      // [M, n_q, 576]
  const __half* cache;
  const int* row_pos;
  const int* row_seq;
  const int* block_table;
  int max_pages, n_pages;
  int n_q, M, n_seg, ctx_limit;
  float* part_ml;          // [M, n_q, n_seg, 2]
  float* part_acc;         // [M, n_q, n_seg, 512]
  unsigned* fault;
  int layer;
};

__device__ __forceinline__ void mla_cp16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

constexpr int kPStride = 40;            // f16 row stride of the probability tile (32 keys + pad: conflict-free fragment loads)
constexpr int kSStride = 33;            // f32 row stride of the score tile

// grid (n_seg, ceil(n_q / 16), M), 256 threads = 8 warps; one block = 16 heads x one key segment.
// The 16 heads are the M dimension of warp-level tensor-core tiles (m16n8k16, f16 operands, f32 accumulate):
//   scores  S[16 x 32] = Q[16 x 576] K^T   warps (w, w + 4) share key columns 8(w & 3).., each half of the 576 depth
//   softmax            warp w owns head rows 2w, 2w + 1 (running max / sum in registers, probabilities to f16)
//   values  O[16 x 512] += P[16 x 32] V    warp w owns latent columns 64w..64w + 63 (V fragments by ldmatrix.trans
//                                          from the same rows the keys were read from)
// The cache is f16 already, so the K / V tiles feed the tensor cores as they arrive (cp.async, two stages).
__global__ void __launch_bounds__(256, 2) mla_flash_seg_kernel(const MlaFlashArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  __half* sq = reinterpret_cast<__half*>(smem);                                  // [16][584] f16, pre-scaled q'
  __half* skv = sq + kHeadsPerBlock * kRowPad;                                   // [2][32][584]
  float* ss = reinterpret_cast<float*>(skv + 2 * kTile * kRowPad);              // [16][33] scores
  float* spart = ss + kHeadsPerBlock * kSStride;                                 // [4][16][8] upper-half partial scores
  __half* sp = reinterpret_cast<__half*>(spart + 4 * 16 * 8);                    // [16][40] probabilities
  float* scorr = reinterpret_cast<float*>(sp + kHeadsPerBlock * kPStride);       // [16]
  const int seg = blockIdx.x, hb = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  pdl_wait();
  pdl_launch();
  const int seq = a.row_seq[m];
  if (seq < 0) return;
  const int n_keys = a.row_pos[m] + 1;
  const bool bad = n_keys <= 0 || n_keys > a.ctx_limit;
  if (bad && tid == 0 && seg == 0 && hb == 0) raise_fault(a.fault, a.layer, FS_KEY_COUNT);
  const int n_tiles = bad ? 0 : (n_keys + kTile - 1) / kTile;
  const int tps = (n_tiles + a.n_seg - 1) / a.n_seg;
  const int t0 = seg * tps, t1 = min(n_tiles, t0 + tps);
  if (!bad && t0 >= t1) return;                  // past the row's last key tile: the merge does not read this segment
  const int h0 = hb * kHeadsPerBlock;
  const int n_heads = min(kHeadsPerBlock, a.n_q - h0);
  for (int i = tid; i < kHeadsPerBlock * kRow; i += 256) {
    const int r = i / kRow, c = i - r * kRow;
    sq[r * kRowPad + c] = __float2half_rn(r < n_heads ? a.q_lat[((long)m * a.n_q + h0 + r) * kRow + c] : 0.f);
  }

  const int* bt = a.block_table + (long)seq * a.max_pages;
  auto issue_tile = [&](int tl, int stage) {
    const int key0 = tl * kTile;
    int page = bt[key0 / kMlaPage];
    page = (page < 0 || page >= a.n_pages) ? 0 : page;     // the append kernel raises the fault; stay in bounds
    const __half* base = a.cache + ((long)page * kMlaPage + (key0 % kMlaPage)) * kRow;
    constexpr int CH = kRow / 8;                            // 72 chunks of 16 bytes per row
    for (int c = tid; c < kTile * CH; c += 256) {
      const int r = c / CH, cc = c % CH;
      mla_cp16(skv + ((size_t)stage * kTile + r) * kRowPad + cc * 8, base + (long)r * kRow + cc * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float acc[8][4];                               // latent columns 64 warp + 8 j + {2t, 2t+1}, rows g and g + 8
#pragma unroll
  for (int j = 0; j < 8; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
  float mx[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};    // of head rows 2 warp, 2 warp + 1

  if (t0 < t1) issue_tile(t0, 0);
  for (int tl = t0; tl < t1; ++tl) {
    const int stage = (tl - t0) & 1;
    if (tl + 1 < t1) { issue_tile(tl + 1, stage ^ 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
    else { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
    __syncthreads();
    __half* kv = skv + (size_t)stage * kTile * kRowPad;
    const int kmax = min(kTile, n_keys - tl * kTile);
    if (kmax < kTile) {                          // rows past the last key: their probability is 0, keep 0 * x finite
      for (int i = tid; i < (kTile - kmax) * (kRowPad / 2); i += 256)
        reinterpret_cast<uint32_t*>(kv + (size_t)kmax * kRowPad)[i] = 0u;
      __syncthreads();
    }
    // ---- scores ----------------------------------------------------------------------------------
    {
      const int nt = warp & 3, kh = warp >> 2;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const __half* qa = sq + g * kRowPad + 2 * t;
      const __half* kb = kv + (size_t)(nt * 8 + g) * kRowPad + 2 * t;
#pragma unroll 6
      for (int ks = kh * 18; ks < kh * 18 + 18; ++ks) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa + ks * 16);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(qa + 8 * kRowPad + ks * 16);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(qa + 8 * kRowPad + ks * 16 + 8);
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kb + ks * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kb + ks * 16 + 8);
        mma_f16_16816(c, a0, a1, a2, a3, b0, b1);
      }
      if (kh == 1) {
        float* o = spart + nt * 128;
        o[g * 8 + 2 * t] = c[0]; o[g * 8 + 2 * t + 1] = c[1]; o[(g + 8) * 8 + 2 * t] = c[2]; o[(g + 8) * 8 + 2 * t + 1] = c[3];
      }
      __syncthreads();
      if (kh == 0) {
        const float* o = spart + nt * 128;
        const int col = nt * 8 + 2 * t;
        const bool m0 = col < kmax, m1 = col + 1 < kmax;
        ss[g * kSStride + col] = m0 ? c[0] + o[g * 8 + 2 * t] : -INFINITY;
        ss[g * kSStride + col + 1] = m1 ? c[1] + o[g * 8 + 2 * t + 1] : -INFINITY;
        ss[(g + 8) * kSStride + col] = m0 ? c[2] + o[(g + 8) * 8 + 2 * t] : -INFINITY;
        ss[(g + 8) * kSStride + col + 1] = m1 ? c[3] + o[(g + 8) * 8 + 2 * t + 1] : -INFINITY;
      }
    }
    __syncthreads();
    // ---- online softmax: warp w owns head rows 2w, 2w + 1 --------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = 2 * warp + h;
      const float sc = ss[r * kSStride + lane];
      const float nm = fmaxf(mx[h], warp_max(sc));
      const float corr = (mx[h] == -INFINITY) ? 0.f : __expf(mx[h] - nm);
      const float pr = (sc == -INFINITY) ? 0.f : __expf(sc - nm);
      l[h] = l[h] * corr + warp_sum(pr);
      mx[h] = nm;
      sp[r * kPStride + lane] = __float2half_rn(pr);
      if (lane == 0) scorr[r] = corr;
    }
    __syncthreads();
    // ---- values: warp w owns latent columns 64w .. 64w + 63 --------------------------------------------
    {
      const float c_lo = scorr[g], c_hi = scorr[g + 8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { acc[j][0] *= c_lo; acc[j][1] *= c_lo; acc[j][2] *= c_hi; acc[j][3] *= c_hi; }
      const __half* pa = sp + g * kPStride + 2 * t;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(pa + ks * 16);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(pa + 8 * kPStride + ks * 16);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(pa + ks * 16 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(pa + 8 * kPStride + ks * 16 + 8);
        // lane l addresses row (l & 7) of matrix (l >> 3): matrices 0, 1 = keys 16ks + 0..7, + 8..15 of column tile j,
        // matrices 2, 3 = the same keys of column tile j + 1
        const __half* vrow = kv + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kRowPad + 64 * warp + (lane >> 4) * 8;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vrow + j * 8);
          mma_f16_16816(acc[j], a0, a1, a2, a3, b[0], b[1]);
          mma_f16_16816(acc[j + 1], a0, a1, a2, a3, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  // partial results of this segment
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 2 * warp + h;
    if (r < n_heads && lane == 0) {
      const long pidx = ((long)m * a.n_q + h0 + r) * a.n_seg + seg;
      a.part_ml[pidx * 2] = bad ? __int_as_float(0x7fc00000) : mx[h];
      a.part_ml[pidx * 2 + 1] = l[h];
    }
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = g + 8 * hh;
    if (r < n_heads) {
      const long pidx = ((long)m * a.n_q + h0 + r) * a.n_seg + seg;
      float* o = a.part_acc + pidx * kLat + 64 * warp + 2 * t;
#pragma unroll
      for (int j = 0; j < 8; ++j) *reinterpret_cast<float2*>(o + 8 * j) = make_float2(acc[j][2 * hh], acc[j][2 * hh + 1]);
    }
  }
}

struct MlaMergeArgs {
  const float* part_ml;
  const float* part_acc;
  const void* w_vb;        // [n_q][v_dim][512]
  int n_q, n_seg, M, v_dim;
  const int* row_seq;
  const int* row_pos;
  int ctx_limit;
  float* out;              // optional fp32 [M, n_q * v_dim]
  int8_t* outq;            // q8 codes [M, n_q * v_dim]
  float2* outds;           // [M, n_q * v_dim / 32]
};

// grid (n_q, M), 256 threads
template <typename W>
__global__ void __launch_bounds__(256) mla_merge_vup_kernel(const MlaMergeArgs a) {
  __shared__ float slat[kLat];
  __shared__ float so[128];
  const int h = blockIdx.x, m = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // weights do not depend on the launch before this one: the first row group is fetched ahead of the wait
  const W* w = reinterpret_cast<const W*>(a.w_vb) + (long)h * a.v_dim * kLat;
  auto load_group = [&](int r0, float (&dst)[4][16]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int r = r0 + 8 * q;
      if (r < a.v_dim) {
        load8<W>(w + (long)r * kLat + 8 * lane, dst[q]);
        load8<W>(w + (long)r * kLat + 256 + 8 * lane, dst[q] + 8);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[q][i] = 0.f;
      }
    }
  };
  float cur[4][16];
  load_group(warp, cur);
  pdl_wait();
  pdl_launch();
  if (a.row_seq[m] < 0) return;
  const long p0 = ((long)m * a.n_q + h) * a.n_seg;
  int used = a.n_seg;                                       // segments past the row's last key tile weigh 0
  {
    const int n_keys = a.row_pos[m] + 1;
    if (n_keys > 0 && n_keys <= a.ctx_limit) {
      const int n_tiles = (n_keys + kTile - 1) / kTile;
      const int tps = (n_tiles + a.n_seg - 1) / a.n_seg;
      used = (n_tiles + tps - 1) / tps;
    }
  }
  float mx = -INFINITY;
  bool nan = false;
#pragma unroll 8
  for (int s = 0; s < used; ++s) {
    const float v = a.part_ml[(p0 + s) * 2];
    nan |= (v != v);
    mx = fmaxf(mx, v);
  }
  float n0 = 0.f, n1 = 0.f, den = 0.f;
#pragma unroll 8
  for (int s = 0; s < used; ++s) {                          // ascending segment order, fixed; loads of 8 segments in flight
    const float ms = a.part_ml[(p0 + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
    den = fmaf(a.part_ml[(p0 + s) * 2 + 1], w, den);
    n0 = fmaf(a.part_acc[(p0 + s) * kLat + tid], w, n0);
    n1 = fmaf(a.part_acc[(p0 + s) * kLat + tid + 256], w, n1);
  }
  const float qnan = __int_as_float(0x7fc00000);
  slat[tid] = nan ? qnan : n0 / den;
  slat[tid + 256] = nan ? qnan : n1 / den;
  __syncthreads();
  // value up-projection: warp w takes rows w, w + 8, ...; four rows at a time so that eight 16-byte weight loads
  // are in flight; lane l covers latent columns 8l..8l+7 and 256 + 8l..  The first group's weights were fetched
  // before the partials were merged, each later group's while the one before it is multiplied.
  float xl[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) { xl[i] = slat[8 * lane + i]; xl[8 + i] = slat[256 + 8 * lane + i]; }
  for (int r0 = warp; r0 < a.v_dim; r0 += 32) {
    float nxt[4][16];
    const bool more = r0 + 32 < a.v_dim;
    if (more) load_group(r0 + 32, nxt);
    float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int i = 0; i < 16; ++i) acc4[q] = fmaf(cur[q][i], xl[i], acc4[q]);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float v = warp_sum(acc4[q]);
      if (lane == 0 && r0 + 8 * q < a.v_dim) so[r0 + 8 * q] = v;
    }
    if (more) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int i = 0; i < 16; ++i) cur[q][i] = nxt[q][i];
    }
  }
  __syncthreads();
  if (tid < a.v_dim) {
    const float o = so[tid];
    const long width = (long)a.n_q * a.v_dim, col = (long)h * a.v_dim + tid;
    if (a.out) a.out[(long)m * width + col] = o;
    float d, s;
    const int8_t q = q8_lane(o, d, s);
    a.outq[(long)m * width + col] = q;
    if (lane == 0) a.outds[((long)m * width + col) / 32] = make_float2(d, s);
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

int bl_mla_kv_append(const float* kv, long stride, const float* gain, const float* inv_freq, float eps, int kv_lora,
                     int rope_dim, int M, const int* row_pos, const int* row_seq, const int* block_table, int max_pages,
                     int n_pages, void* cache, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(kv_lora == kLat && rope_dim == kRope && M >= 1, BL_ERR_SHAPE);
  MlaAppendArgs a{kv, stride, gain, inv_freq, eps, M, row_pos, row_seq, block_table, max_pages, n_pages,
                  (__half*)cache, fault, layer};
  return (int)launch(mla_kv_append_kernel, dim3(M), dim3(256), 0, st, a);
}

// wtype: 0 = f32, 30 = bf16
int bl_mla_q_absorb(const float* q, long stride, const void* w_kb, int wtype, const float* inv_freq, float scale, int n_q,
                    int nope, int kv_lora, int rope_dim, int M, const int* row_pos, const int* row_seq, float* q_lat,
                    cudaStream_t st) {
  BL_REQUIRE(kv_lora == kLat && rope_dim == kRope && nope >= 1 && nope <= 128 && M >= 1, BL_ERR_SHAPE);
  BL_REQUIRE(wtype == 0 || wtype == 30, BL_ERR_TYPE);
  MlaQArgs a{q, stride, w_kb, inv_freq, scale, n_q, nope, M, row_pos, row_seq, q_lat};
  if (wtype == 0) return (int)launch(mla_q_absorb_kernel<float>, dim3(n_q, M), dim3(256), 0, st, a);
  return (int)launch(mla_q_absorb_kernel<__nv_bfloat16>, dim3(n_q, M), dim3(256), 0, st, a);
}

int bl_mla_flash_decode(const float* q_lat, const void* cache, const int* row_pos, const int* row_seq,
                        const int* block_table, int max_pages, int n_pages, int n_q, int M, int n_seg, int ctx_limit,
                        float* part_ml, float* part_acc, const void* w_vb, int wtype, int v_dim, float* out, int8_t* outq,
                        float* outds, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(n_q >= 1 && M >= 1 && n_seg >= 1 && v_dim >= 32 && v_dim <= 128 && v_dim % 32 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(wtype == 0 || wtype == 30, BL_ERR_TYPE);
  const size_t smem = (size_t)kHeadsPerBlock * kRowPad * 2 + (size_t)2 * kTile * kRowPad * 2 +
                      (size_t)(kHeadsPerBlock * kSStride + 4 * 16 * 8) * 4 + (size_t)kHeadsPerBlock * kPStride * 2 + 16 * 4;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(mla_flash_seg_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  MlaFlashArgs f{q_lat, (const __half*)cache, row_pos, row_seq, block_table, max_pages, n_pages, n_q, M, n_seg, ctx_limit,
                 part_ml, part_acc, fault, layer};
  cudaError_t e = launch(mla_flash_seg_kernel, dim3(n_seg, (n_q + kHeadsPerBlock - 1) / kHeadsPerBlock, M), dim3(256), smem, st, f);
  if (e != cudaSuccess) return (int)e;
  MlaMergeArgs g{part_ml, part_acc, w_vb, n_q, n_seg, M, v_dim, row_seq, row_pos, ctx_limit, out, outq, (float2*)outds};
  if (wtype == 0) return (int)launch(mla_merge_vup_kernel<float>, dim3(n_q, M), dim3(256), 0, st, g);
  return (int)launch(mla_merge_vup_kernel<__nv_bfloat16>, dim3(n_q, M), dim3(256), 0, st, g);
}

}  // extern "C"
