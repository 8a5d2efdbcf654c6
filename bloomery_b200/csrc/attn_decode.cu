// Decode-time attention over a paged KV cache (GQA, head size 128 or 64):
//   1. qk_norm_rope_append  per-head RMSNorm (optional) + NEOX RoPE + KV append
//   2. flash_decode_seg     split-K online-softmax over a fixed number of segments
//   3. flash_decode_merge   merge segments ascending, then quantise to q8 for o_proj
//
// Everything data-dependent (positions, sequence of each row, block table, live key
// count) is read from device buffers, so one captured graph serves every step; the
// segment grid is fixed per graph (the reference fixes 80: crates/gpu/src/flash_gqa.rs:350).
// Numeric contract followed (crates/gpu/src/rope_neox.rs:1-40, flash_gqa.rs:1-45): f32
// squares with f64 sums, NEOX pairs (i, i + HEAD/2) with fma forms, K and V rounded once
// to f16 (RNE); masked keys weigh exactly 0 and are never loaded; a key count of 0 or
// beyond the context raises FS_KEY_COUNT and writes NaN.
//
// KV layout per layer: [n_pages][n_kv][PAGE][HEAD] f16 for K and the same for V,
// PAGE = 64 positions.  block_table[seq][i] names the page of positions 64i..64i+63.
#include "common.cuh"

namespace bl {

constexpr int kPage = 64;
constexpr int kKeyTile = 32;

struct RopeArgs {
  const float* qkv;      // [M, (n_q + 2 n_kv) * HEAD]
  long qkv_stride;
  const float* q_gain;   // [HEAD] or null
  const float* k_gain;   // [HEAD] or null
  const float* inv_freq; // [HEAD/2]
  float eps;
  float q_scale;         // 1/sqrt(HEAD) folded into q
  int n_q, n_kv;
  int M;
  const int* row_pos;    // [M]
  const int* row_seq;    // [M], < 0 = padding row
  const int* block_table;
  int max_pages;         // per sequence
  int n_pages;           // pool size (bounds check)
  __half* k_cache;
  __half* v_cache;
  float* q_out;          // [M, n_q, HEAD]
  unsigned* fault;
  int layer;
  __nv_bfloat16* q_bf16; // optional [n_q, M, HEAD] (head-major rows for the prompt GEMMs)
  int kv_q8;             // the caches hold q8_0 rows: HEAD/32 f16 scales, then HEAD int8 codes (34 bytes per 32 values)
};

// q8_0 key/value rows: per position and KV head HEAD / 32 f16 scales followed by HEAD int8 codes
template <int HEAD> struct KvQ8 {
  static constexpr int kRowBytes = HEAD / 32 * 34;
  static constexpr int kCodes = HEAD / 16;       // byte offset of the codes (4-byte aligned for both head sizes)
};

template <int HEAD>
__global__ void __launch_bounds__(HEAD / 2) qk_norm_rope_append_kernel(const RopeArgs a) {
  constexpr int HALF = HEAD / 2;
  __shared__ double red[HALF / 32];
  const int head = blockIdx.x, m = blockIdx.y, i = threadIdx.x;
  pdl_wait();
  pdl_launch();
  const int seq = a.row_seq[m];
  if (seq < 0) return;
  const int pos = a.row_pos[m];
  const float* src = a.qkv + (long)m * a.qkv_stride + (long)head * HEAD;
  float x0 = src[i], x1 = src[i + HALF];
  const bool is_q = head < a.n_q, is_k = !is_q && head < a.n_q + a.n_kv;
  if (is_q || is_k) {
    const float* gain = is_q ? a.q_gain : a.k_gain;
    if (gain) {
      double ss = warp_sum_d((double)(x0 * x0) + (double)(x1 * x1));
      if ((i & 31) == 0) red[i >> 5] = ss;
      __syncthreads();
      double tot = 0.0;
#pragma unroll
      for (int w = 0; w < HALF / 32; ++w) tot += red[w];
      float scale = (float)(1.0 / sqrt(tot / (double)HEAD + (double)a.eps));
      x0 = (scale * gain[i]) * x0;
      x1 = (scale * gain[i + HALF]) * x1;
    }
    float ang = (float)pos * a.inv_freq[i];
    float s, c;
    sincosf(ang, &s, &c);
    float y0 = fmaf(x0, c, -(x1 * s));
    float y1 = fmaf(x0, s, x1 * c);
    x0 = y0; x1 = y1;
  }
  if (is_q) {
    if (a.q_out) {
      float* q = a.q_out + ((long)m * a.n_q + head) * HEAD;
      q[i] = x0 * a.q_scale;
      q[i + HALF] = x1 * a.q_scale;
    }
    if (a.q_bf16) {
      __nv_bfloat16* q = a.q_bf16 + ((long)head * a.M + m) * HEAD;
      q[i] = __float2bfloat16_rn(x0 * a.q_scale);
      q[i + HALF] = __float2bfloat16_rn(x1 * a.q_scale);
    }
    return;
  }
  const int kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
  const int pslot = pos / kPage;
  int page = (pslot < a.max_pages) ? a.block_table[(long)seq * a.max_pages + pslot] : -1;
  if (page < 0 || page >= a.n_pages) {
    if (i == 0) raise_fault(a.fault, a.layer, FS_PAGE);
    return;
  }
  if (a.kv_q8) {
    // this thread's two values sit in blocks i / 32 and (i + HALF) / 32; a warp holds both blocks whole
    using Q = KvQ8<HEAD>;
    uint8_t* row = reinterpret_cast<uint8_t*>(is_k ? a.k_cache : a.v_cache) +
                   (((long)page * a.n_kv + kvh) * kPage + (pos % kPage)) * Q::kRowBytes;
    const __half d0 = __float2half_rn(warp_max(fabsf(x0)) * (1.0f / 127.0f));
    const __half d1 = __float2half_rn(warp_max(fabsf(x1)) * (1.0f / 127.0f));
    const float f0 = __half2float(d0), f1 = __half2float(d1);
    const int q0 = f0 > 0.f ? max(-127, min(127, __float2int_rn(x0 / f0))) : 0;
    const int q1 = f1 > 0.f ? max(-127, min(127, __float2int_rn(x1 / f1))) : 0;
    row[Q::kCodes + i] = (uint8_t)(int8_t)q0;
    row[Q::kCodes + i + HALF] = (uint8_t)(int8_t)q1;
    if ((i & 31) == 0) {
      reinterpret_cast<__half*>(row)[i >> 5] = d0;
      reinterpret_cast<__half*>(row)[(i + HALF) >> 5] = d1;
    }
    return;
  }
  __half* dst = (is_k ? a.k_cache : a.v_cache) + (((long)page * a.n_kv + kvh) * kPage + (pos % kPage)) * HEAD;
  dst[i] = __float2half_rn(x0);
  dst[i + HALF] = __float2half_rn(x1);
}

struct FlashArgs {
  const float* q;        // [M, n_q, HEAD], pre-scaled
  const __half* k_cache;
  const __half* v_cache;
  const int* row_pos;
  const int* row_seq;
  const int* block_table;
  int max_pages, n_pages;
  int n_q, n_kv, M, n_seg;
  int ctx_limit;
  float* part_ml;        // [M, n_q, n_seg, 2]
  float* part_acc;       // [M, n_q, n_seg, HEAD]
  unsigned* fault;
  int layer;
  int kv_q8;             // the caches hold q8_0 rows (KvQ8): tiles are expanded to f16 as they are staged
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// grid (n_seg, n_kv, M); 256 threads = 8 warps; warp w serves q heads w, w+8, ... of the group
template <int HEAD, int HPW, bool Q8 = false>
__global__ void __launch_bounds__(256) flash_decode_seg_kernel(const FlashArgs a) {
  constexpr int KSTR = HEAD + 8;      // padded f16 row stride for K: conflict-free 16-byte reads by key lanes
  constexpr int DPL = HEAD / 32;      // output dims per lane
  extern __shared__ __align__(16) uint8_t smem[];
  const int G = a.n_q / a.n_kv;
  float* sq = reinterpret_cast<float*>(smem);                              // [G][HEAD]
  __half* sk = reinterpret_cast<__half*>(smem + (size_t)G * HEAD * 4);     // [2][32][KSTR]
  __half* sv = sk + 2 * kKeyTile * KSTR;                                   // [2][32][HEAD]
  const int seg = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  pdl_wait();
  pdl_launch();
  const int seq = a.row_seq[m];
  if (seq < 0) return;
  const int n_keys = a.row_pos[m] + 1;
  const bool bad = n_keys <= 0 || n_keys > a.ctx_limit;
  if (bad && tid == 0 && seg == 0 && kvh == 0) raise_fault(a.fault, a.layer, FS_KEY_COUNT);

  const int n_tiles = bad ? 0 : (n_keys + kKeyTile - 1) / kKeyTile;
  const int tps = (n_tiles + a.n_seg - 1) / a.n_seg;
  const int t0 = seg * tps, t1 = min(n_tiles, t0 + tps);
  if (!bad && t0 >= t1) return;                  // past the row's last key tile: the merge does not read this segment

  for (int i = tid; i < G * HEAD; i += 256)
    sq[i] = a.q[((long)m * a.n_q + (long)kvh * G) * HEAD + i];

  const int* bt = a.block_table + (long)seq * a.max_pages;
  auto issue_tile = [&](int t, int stage) {
    const int key0 = t * kKeyTile;
    int page = bt[key0 / kPage];
    page = (page < 0 || page >= a.n_pages) ? 0 : page;  // fault is raised by the append kernel; stay in bounds
    constexpr int CH = HEAD / 8;  // 16-byte chunks per row
    if constexpr (Q8) {
      // q8_0 rows: eight codes and their block's scale per step, written to the same f16 tiles the dot loops read
      using Q = KvQ8<HEAD>;
      const long baseq = (((long)page * a.n_kv + kvh) * kPage + (key0 % kPage)) * Q::kRowBytes;
      const uint8_t* kq = reinterpret_cast<const uint8_t*>(a.k_cache) + baseq;
      const uint8_t* vq = reinterpret_cast<const uint8_t*>(a.v_cache) + baseq;
      for (int c = tid; c < kKeyTile * CH; c += 256) {
        const int r = c / CH, cc = c % CH;
        auto expand = [&](const uint8_t* rowp, __half* dst) {
          const float d = __half2float(reinterpret_cast<const __half*>(rowp)[cc >> 2]);
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(rowp + Q::kCodes + cc * 8);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(rowp + Q::kCodes + cc * 8 + 4);
          __half2 h[4];
          h[0] = __floats2half2_rn(d * (float)(int8_t)(w0 & 0xFF), d * (float)(int8_t)((w0 >> 8) & 0xFF));
          h[1] = __floats2half2_rn(d * (float)(int8_t)((w0 >> 16) & 0xFF), d * (float)(int8_t)(w0 >> 24));
          h[2] = __floats2half2_rn(d * (float)(int8_t)(w1 & 0xFF), d * (float)(int8_t)((w1 >> 8) & 0xFF));
          h[3] = __floats2half2_rn(d * (float)(int8_t)((w1 >> 16) & 0xFF), d * (float)(int8_t)(w1 >> 24));
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(h);
        };
        expand(kq + (long)r * Q::kRowBytes, sk + ((size_t)stage * kKeyTile + r) * KSTR + cc * 8);
        expand(vq + (long)r * Q::kRowBytes, sv + ((size_t)stage * kKeyTile + r) * HEAD + cc * 8);
      }
      cp_async_commit();
      return;
    }
    const long base = (((long)page * a.n_kv + kvh) * kPage + (key0 % kPage)) * HEAD;
    for (int c = tid; c < kKeyTile * CH; c += 256) {
      int r = c / CH, cc = c % CH;
      cp_async16(sk + ((size_t)stage * kKeyTile + r) * KSTR + cc * 8, a.k_cache + base + (long)r * HEAD + cc * 8);
      cp_async16(sv + ((size_t)stage * kKeyTile + r) * HEAD + cc * 8, a.v_cache + base + (long)r * HEAD + cc * 8);
    }
    cp_async_commit();
  };

  float mx[HPW], l[HPW], acc[HPW][DPL];
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    mx[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }

  if (t0 < t1) issue_tile(t0, 0);
  for (int t = t0; t < t1; ++t) {
    const int stage = (t - t0) & 1;
    if (t + 1 < t1) { issue_tile(t + 1, stage ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const int key = t * kKeyTile + lane;
    const __half* krow = sk + ((size_t)stage * kKeyTile + lane) * KSTR;
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
      const int hg = warp + 8 * h;
      if (hg < G) {
        const float* qh = sq + hg * HEAD;
        float s = 0.f;
#pragma unroll
        for (int d = 0; d < HEAD; d += 8) {
          uint4 kv = *reinterpret_cast<const uint4*>(krow + d);
          float4 q0 = *reinterpret_cast<const float4*>(qh + d);
          float4 q1 = *reinterpret_cast<const float4*>(qh + d + 4);
          float2 k0 = __half22float2(*reinterpret_cast<__half2*>(&kv.x));
          float2 k1 = __half22float2(*reinterpret_cast<__half2*>(&kv.y));
          float2 k2 = __half22float2(*reinterpret_cast<__half2*>(&kv.z));
          float2 k3 = __half22float2(*reinterpret_cast<__half2*>(&kv.w));
          s = fmaf(q0.x, k0.x, s); s = fmaf(q0.y, k0.y, s); s = fmaf(q0.z, k1.x, s); s = fmaf(q0.w, k1.y, s);
          s = fmaf(q1.x, k2.x, s); s = fmaf(q1.y, k2.y, s); s = fmaf(q1.z, k3.x, s); s = fmaf(q1.w, k3.y, s);
        }
        if (key >= n_keys) s = -INFINITY;
        float tmax = warp_max(s);
        float nm = fmaxf(mx[h], tmax);
        float corr = (mx[h] == -INFINITY) ? 0.f : __expf(mx[h] - nm);
        float p = (s == -INFINITY) ? 0.f : __expf(s - nm);
        l[h] = l[h] * corr + warp_sum(p);
        mx[h] = nm;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] *= corr;
        const __half* vbase = sv + (size_t)stage * kKeyTile * HEAD + lane * DPL;
        const int kmax = min(kKeyTile, n_keys - t * kKeyTile);  // masked keys are never read
#pragma unroll 4
        for (int k = 0; k < kmax; ++k) {
          float pk = __shfl_sync(0xffffffffu, p, k);
          const __half* vr = vbase + (size_t)k * HEAD;
          if constexpr (DPL == 4) {
            uint2 vv = *reinterpret_cast<const uint2*>(vr);
            float2 v0 = __half22float2(*reinterpret_cast<__half2*>(&vv.x));
            float2 v1 = __half22float2(*reinterpret_cast<__half2*>(&vv.y));
            acc[h][0] = fmaf(pk, v0.x, acc[h][0]); acc[h][1] = fmaf(pk, v0.y, acc[h][1]);
            acc[h][2] = fmaf(pk, v1.x, acc[h][2]); acc[h][3] = fmaf(pk, v1.y, acc[h][3]);
          } else {
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[h][d] = fmaf(pk, __half2float(vr[d]), acc[h][d]);
          }
        }
      }
    }
    __syncthreads();
  }

#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int hg = warp + 8 * h;
    if (hg < G) {
      const int qh = kvh * G + hg;
      const long pidx = ((long)m * a.n_q + qh) * a.n_seg + seg;
      if (lane == 0) {
        a.part_ml[pidx * 2] = bad ? __int_as_float(0x7fc00000) : mx[h];
        a.part_ml[pidx * 2 + 1] = l[h];
      }
#pragma unroll
      for (int d = 0; d < DPL; ++d) a.part_acc[pidx * HEAD + lane * DPL + d] = acc[h][d];
    }
  }
}


// ------------------------------------------------------------------------------------
// The same segment pass on warp-level tensor-core tiles (opt-in: bl_set_flash_mma).
// One block = one KV head x one key segment; its G <= 16 query heads are the M dimension of
// m16n8k16 f16 tiles (rows past G are zero):
//   scores  S[16 x 32] = Q[16 x HEAD] K^T    warps (w, w + 4) share key columns 8(w & 3).., each half of the depth
//   softmax            warp w owns head rows 2w, 2w + 1
//   values  O[16 x HEAD] += P[16 x 32] V     warp w owns output columns (HEAD / 8) w ..
// K and V rows are f16 in the cache already and feed the tensor cores as they arrive.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void fa_mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fa_ldmatrix_x2_trans(uint32_t (&r)[2], const void* smem_row) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

template <int HEAD>
__global__ void __launch_bounds__(256, 2) flash_decode_seg_mma_kernel(const FlashArgs a) {
  constexpr int STR = HEAD + 8;                  // f16 row stride of q, K and V tiles: fragment loads do not collide
  constexpr int KS = HEAD / 16;                  // k-steps of the score product
  constexpr int NT = HEAD / 64;                  // 8-column output tiles per warp in the value product
  constexpr int PSTR = 40, SSTR = 33;
  extern __shared__ __align__(16) uint8_t smem[];
  __half* sq = reinterpret_cast<__half*>(smem);                         // [16][STR]
  __half* sk = sq + 16 * STR;                                           // [2][32][STR]
  __half* sv = sk + 2 * kKeyTile * STR;                                 // [2][32][STR]
  float* ss = reinterpret_cast<float*>(sv + 2 * kKeyTile * STR);       // [16][33]
  float* spart = ss + 16 * SSTR;                                        // [4][16][8]
  __half* sp = reinterpret_cast<__half*>(spart + 512);                  // [16][40]
  float* scorr = reinterpret_cast<float*>(sp + 16 * PSTR);              // [16]
  const int G = a.n_q / a.n_kv;
  const int seg = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  pdl_wait();
  pdl_launch();
  const int seq = a.row_seq[m];
  if (seq < 0) return;
  const int n_keys = a.row_pos[m] + 1;
  const bool bad = n_keys <= 0 || n_keys > a.ctx_limit;
  if (bad && tid == 0 && seg == 0 && kvh == 0) raise_fault(a.fault, a.layer, FS_KEY_COUNT);
  const int n_tiles = bad ? 0 : (n_keys + kKeyTile - 1) / kKeyTile;
  const int tps = (n_tiles + a.n_seg - 1) / a.n_seg;
  const int t0 = seg * tps, t1 = min(n_tiles, t0 + tps);
  if (!bad && t0 >= t1) return;
  for (int i = tid; i < 16 * HEAD; i += 256) {
    const int r = i / HEAD, c = i - r * HEAD;
    sq[r * STR + c] = __float2half_rn(r < G ? a.q[((long)m * a.n_q + (long)kvh * G + r) * HEAD + c] : 0.f);
  }
  const int* bt = a.block_table + (long)seq * a.max_pages;
  auto issue_tile = [&](int tl, int stage) {
    const int key0 = tl * kKeyTile;
    int page = bt[key0 / kPage];
    page = (page < 0 || page >= a.n_pages) ? 0 : page;
    const long base = (((long)page * a.n_kv + kvh) * kPage + (key0 % kPage)) * HEAD;
    constexpr int CH = HEAD / 8;
    for (int c = tid; c < kKeyTile * CH; c += 256) {
      const int r = c / CH, cc = c % CH;
      cp_async16(sk + ((size_t)stage * kKeyTile + r) * STR + cc * 8, a.k_cache + base + (long)r * HEAD + cc * 8);
      cp_async16(sv + ((size_t)stage * kKeyTile + r) * STR + cc * 8, a.v_cache + base + (long)r * HEAD + cc * 8);
    }
    cp_async_commit();
  };
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
  float mx[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  if (t0 < t1) issue_tile(t0, 0);
  for (int tl = t0; tl < t1; ++tl) {
    const int stage = (tl - t0) & 1;
    if (tl + 1 < t1) { issue_tile(tl + 1, stage ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const __half* kt = sk + (size_t)stage * kKeyTile * STR;
    __half* vt = sv + (size_t)stage * kKeyTile * STR;
    const int kmax = min(kKeyTile, n_keys - tl * kKeyTile);
    if (kmax < kKeyTile) {                        // value rows past the last key: weight 0, keep 0 * x finite
      for (int i = tid; i < (kKeyTile - kmax) * (STR / 2); i += 256) reinterpret_cast<uint32_t*>(vt + (size_t)kmax * STR)[i] = 0u;
      __syncthreads();
    }
    {
      const int nt = warp & 3, kh = warp >> 2;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const __half* qa = sq + g * STR + 2 * t;
      const __half* kb = kt + (size_t)(nt * 8 + g) * STR + 2 * t;
#pragma unroll
      for (int ks = kh * (KS / 2); ks < (kh + 1) * (KS / 2); ++ks) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(qa + ks * 16);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(qa + 8 * STR + ks * 16);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(qa + 8 * STR + ks * 16 + 8);
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kb + ks * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kb + ks * 16 + 8);
        fa_mma_16816(c, a0, a1, a2, a3, b0, b1);
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
        ss[g * SSTR + col] = m0 ? c[0] + o[g * 8 + 2 * t] : -INFINITY;
        ss[g * SSTR + col + 1] = m1 ? c[1] + o[g * 8 + 2 * t + 1] : -INFINITY;
        ss[(g + 8) * SSTR + col] = m0 ? c[2] + o[(g + 8) * 8 + 2 * t] : -INFINITY;
        ss[(g + 8) * SSTR + col + 1] = m1 ? c[3] + o[(g + 8) * 8 + 2 * t + 1] : -INFINITY;
      }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = 2 * warp + h;
      const float sc = ss[r * SSTR + lane];
      const float nm = fmaxf(mx[h], warp_max(sc));
      const float corr = (mx[h] == -INFINITY) ? 0.f : __expf(mx[h] - nm);
      const float pr = (sc == -INFINITY) ? 0.f : __expf(sc - nm);
      l[h] = l[h] * corr + warp_sum(pr);
      mx[h] = nm;
      sp[r * PSTR + lane] = __float2half_rn(pr);
      if (lane == 0) scorr[r] = corr;
    }
    __syncthreads();
    {
      const float c_lo = scorr[g], c_hi = scorr[g + 8];
#pragma unroll
      for (int j = 0; j < NT; ++j) { acc[j][0] *= c_lo; acc[j][1] *= c_lo; acc[j][2] *= c_hi; acc[j][3] *= c_hi; }
      const __half* pa = sp + g * PSTR + 2 * t;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(pa + ks * 16);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(pa + 8 * PSTR + ks * 16);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(pa + ks * 16 + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(pa + 8 * PSTR + ks * 16 + 8);
        // lanes 0..15 address the 16 key rows of this k-step (matrix 0: rows 0..7, matrix 1: rows 8..15)
        const __half* vrow = vt + (size_t)(ks * 16 + (lane & 15)) * STR + (HEAD / 8) * warp;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          uint32_t b[2];
          fa_ldmatrix_x2_trans(b, vrow + j * 8);
          fa_mma_16816(acc[j], a0, a1, a2, a3, b[0], b[1]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = 2 * warp + h;
    if (r < G && lane == 0) {
      const long pidx = ((long)m * a.n_q + (long)kvh * G + r) * a.n_seg + seg;
      a.part_ml[pidx * 2] = bad ? __int_as_float(0x7fc00000) : mx[h];
      a.part_ml[pidx * 2 + 1] = l[h];
    }
  }
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = g + 8 * hh;
    if (r < G) {
      const long pidx = ((long)m * a.n_q + (long)kvh * G + r) * a.n_seg + seg;
      float* o = a.part_acc + pidx * HEAD + (HEAD / 8) * warp + 2 * t;
#pragma unroll
      for (int j = 0; j < NT; ++j) *reinterpret_cast<float2*>(o + 8 * j) = make_float2(acc[j][2 * hh], acc[j][2 * hh + 1]);
    }
  }
}

int g_flash_mma = 0;

struct MergeArgs {
  const float* part_ml;
  const float* part_acc;
  int n_q, n_seg, M;
  const int* row_seq;
  const int* row_pos;  // with ctx_limit: lets the merge skip the segments the row's keys never reach
  int ctx_limit;
  float* out;        // optional fp32 [M, n_q*HEAD]
  int8_t* outq;      // q8 codes [M, n_q*HEAD]
  float2* outds;     // [M, n_q*HEAD/32]
};

// grid (n_q, M), HEAD threads
template <int HEAD>
__global__ void __launch_bounds__(HEAD) flash_decode_merge_kernel(const MergeArgs a) {
  const int qh = blockIdx.x, m = blockIdx.y, d = threadIdx.x;
  pdl_wait();
  pdl_launch();
  if (a.row_seq[m] < 0) return;
  const long p0 = ((long)m * a.n_q + qh) * a.n_seg;
  // segments beyond the row's last key tile hold weight 0: the same split as the segment kernel says how many are live
  int used = a.n_seg;
  {
    const int n_keys = a.row_pos[m] + 1;
    if (n_keys > 0 && n_keys <= a.ctx_limit) {
      const int n_tiles = (n_keys + kKeyTile - 1) / kKeyTile;
      const int tps = (n_tiles + a.n_seg - 1) / a.n_seg;
      used = (n_tiles + tps - 1) / tps;
    }
  }
  float mx = -INFINITY;
  bool nan = false;
#pragma unroll 8
  for (int s = 0; s < used; ++s) {
    float v = a.part_ml[(p0 + s) * 2];
    nan |= (v != v);
    mx = fmaxf(mx, v);
  }
  float num = 0.f, den = 0.f;
#pragma unroll 8
  for (int s = 0; s < used; ++s) {  // ascending segment order, fixed; the loads of eight segments are in flight together
    float ms = a.part_ml[(p0 + s) * 2];
    float w = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
    den = fmaf(a.part_ml[(p0 + s) * 2 + 1], w, den);
    num = fmaf(a.part_acc[(p0 + s) * HEAD + d], w, num);
  }
  float o = nan ? __int_as_float(0x7fc00000) : num / den;
  const long col = (long)qh * HEAD + d;
  const long width = (long)a.n_q * HEAD;
  if (a.out) a.out[(long)m * width + col] = o;
  float ds_d, ds_s;
  int8_t q = q8_lane(o, ds_d, ds_s);
  a.outq[(long)m * width + col] = q;
  if ((d & 31) == 0) a.outds[((long)m * width + col) / 32] = make_float2(ds_d, ds_s);
}

}  // namespace bl

using namespace bl;

static int rope_append_go(const float* qkv, long qkv_stride, const float* q_gain, const float* k_gain, const float* inv_freq,
                          float eps, float q_scale, int head, int n_q, int n_kv, int M, const int* row_pos,
                          const int* row_seq, const int* block_table, int max_pages, int n_pages, void* k_cache,
                          void* v_cache, float* q_out, unsigned* fault, int layer, int kv_q8, cudaStream_t st) {
  BL_REQUIRE(head == 128 || head == 64, BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && n_q >= 1 && n_kv >= 1, BL_ERR_SHAPE);
  RopeArgs a{qkv, qkv_stride, q_gain, k_gain, inv_freq, eps, q_scale, n_q, n_kv, M, row_pos, row_seq, block_table,
             max_pages, n_pages, (__half*)k_cache, (__half*)v_cache, q_out, fault, layer, nullptr, kv_q8};
  dim3 grid(n_q + 2 * n_kv, M);
  if (head == 128) return (int)launch(qk_norm_rope_append_kernel<128>, grid, dim3(64), 0, st, a);
  return (int)launch(qk_norm_rope_append_kernel<64>, grid, dim3(32), 0, st, a);
}

extern "C" {

int bl_qk_norm_rope_append(const float* qkv, long qkv_stride, const float* q_gain, const float* k_gain,
                           const float* inv_freq, float eps, float q_scale, int head, int n_q, int n_kv, int M,
                           const int* row_pos, const int* row_seq, const int* block_table, int max_pages, int n_pages,
                           void* k_cache, void* v_cache, float* q_out, unsigned* fault, int layer, cudaStream_t st) {
  return rope_append_go(qkv, qkv_stride, q_gain, k_gain, inv_freq, eps, q_scale, head, n_q, n_kv, M, row_pos, row_seq,
                        block_table, max_pages, n_pages, k_cache, v_cache, q_out, fault, layer, 0, st);
}

// The same with q8_0 caches: rows of head / 32 f16 scales followed by head int8 codes (34 bytes per 32 values), written
// with one scale per 32 values of the normalised, rotated row.  (The reference: crates/gpu/src/rope_neox.rs, the q8_0
// append; --cache-type-k / -v q8_0.)
int bl_qk_norm_rope_append_q8(const float* qkv, long qkv_stride, const float* q_gain, const float* k_gain,
                              const float* inv_freq, float eps, float q_scale, int head, int n_q, int n_kv, int M,
                              const int* row_pos, const int* row_seq, const int* block_table, int max_pages, int n_pages,
                              void* k_cache, void* v_cache, float* q_out, unsigned* fault, int layer, cudaStream_t st) {
  return rope_append_go(qkv, qkv_stride, q_gain, k_gain, inv_freq, eps, q_scale, head, n_q, n_kv, M, row_pos, row_seq,
                        block_table, max_pages, n_pages, k_cache, v_cache, q_out, fault, layer, 1, st);
}

// 1: the segment pass runs on tensor-core tiles (flash_decode_seg_mma_kernel); 0: the fp32 kernel
void bl_set_flash_mma(int on) { bl::g_flash_mma = on ? 1 : 0; }

}  // extern "C"

static int flash_decode_go(const float* q, const void* k_cache, const void* v_cache, const int* row_pos, const int* row_seq,
                           const int* block_table, int max_pages, int n_pages, int head, int n_q, int n_kv, int M, int n_seg,
                           int ctx_limit, float* part_ml, float* part_acc, float* out, int8_t* outq, float* outds,
                           unsigned* fault, int layer, int kv_q8, cudaStream_t st) {
  BL_REQUIRE(head == 128 || head == 64, BL_ERR_SHAPE);
  BL_REQUIRE(n_kv >= 1 && n_q >= 1 && n_q % n_kv == 0 && n_q / n_kv <= 16, BL_ERR_SHAPE);
  BL_REQUIRE(n_seg >= 1 && M >= 1, BL_ERR_SHAPE);
  // the block table of a row holds max_pages pages of 64 positions: a context limit past that would index beyond it
  BL_REQUIRE(max_pages >= 1 && (long)ctx_limit <= (long)max_pages * kPage, BL_ERR_SHAPE);
  const int G = n_q / n_kv;
  FlashArgs a{q, (const __half*)k_cache, (const __half*)v_cache, row_pos, row_seq, block_table, max_pages, n_pages,
              n_q, n_kv, M, n_seg, ctx_limit, part_ml, part_acc, fault, layer, kv_q8};
  dim3 grid(n_seg, n_kv, M);
  size_t smem = (size_t)G * head * 4 + 2 * kKeyTile * (head + 8) * 2 + 2 * kKeyTile * head * 2;
  cudaError_t e;
  if (kv_q8) {
    // q8_0 caches: the fp32 segment kernel with tiles expanded to f16 as they are staged
    if (head == 128) {
      if (G <= 8) e = launch(flash_decode_seg_kernel<128, 1, true>, grid, dim3(256), smem, st, a);
      else {
        cudaFuncSetAttribute(flash_decode_seg_kernel<128, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
        e = launch(flash_decode_seg_kernel<128, 2, true>, grid, dim3(256), smem, st, a);
      }
    } else {
      if (G <= 8) e = launch(flash_decode_seg_kernel<64, 1, true>, grid, dim3(256), smem, st, a);
      else e = launch(flash_decode_seg_kernel<64, 2, true>, grid, dim3(256), smem, st, a);
    }
  } else if (g_flash_mma) {
    const size_t sm2 = (size_t)(16 + 4 * kKeyTile) * (head + 8) * 2 + (16 * 33 + 512) * 4 + 16 * 40 * 2 + 64;
    static bool set128 = false, set64 = false;
    if (head == 128) {
      if (!set128) { cudaFuncSetAttribute(flash_decode_seg_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm2); set128 = true; }
      e = launch(flash_decode_seg_mma_kernel<128>, grid, dim3(256), sm2, st, a);
    } else {
      if (!set64) { cudaFuncSetAttribute(flash_decode_seg_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm2); set64 = true; }
      e = launch(flash_decode_seg_mma_kernel<64>, grid, dim3(256), sm2, st, a);
    }
  } else if (head == 128) {
    if (G <= 8) e = launch(flash_decode_seg_kernel<128, 1>, grid, dim3(256), smem, st, a);
    else {
      cudaFuncSetAttribute(flash_decode_seg_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      e = launch(flash_decode_seg_kernel<128, 2>, grid, dim3(256), smem, st, a);
    }
  } else {
    if (G <= 8) e = launch(flash_decode_seg_kernel<64, 1>, grid, dim3(256), smem, st, a);
    else e = launch(flash_decode_seg_kernel<64, 2>, grid, dim3(256), smem, st, a);
  }
  if (e != cudaSuccess) return (int)e;
  MergeArgs mg{part_ml, part_acc, n_q, n_seg, M, row_seq, row_pos, ctx_limit, out, outq, (float2*)outds};
  if (head == 128) return (int)launch(flash_decode_merge_kernel<128>, dim3(n_q, M), dim3(128), 0, st, mg);
  return (int)launch(flash_decode_merge_kernel<64>, dim3(n_q, M), dim3(64), 0, st, mg);
}

extern "C" {

// Scratch: part_ml [M*n_q*n_seg*2] and part_acc [M*n_q*n_seg*head] floats, caller-owned.
int bl_flash_decode(const float* q, const void* k_cache, const void* v_cache, const int* row_pos, const int* row_seq,
                    const int* block_table, int max_pages, int n_pages, int head, int n_q, int n_kv, int M, int n_seg,
                    int ctx_limit, float* part_ml, float* part_acc, float* out, int8_t* outq, float* outds,
                    unsigned* fault, int layer, cudaStream_t st) {
  return flash_decode_go(q, k_cache, v_cache, row_pos, row_seq, block_table, max_pages, n_pages, head, n_q, n_kv, M, n_seg,
                         ctx_limit, part_ml, part_acc, out, outq, outds, fault, layer, 0, st);
}

// The same over q8_0 caches (see bl_qk_norm_rope_append_q8).
int bl_flash_decode_q8(const float* q, const void* k_cache, const void* v_cache, const int* row_pos, const int* row_seq,
                       const int* block_table, int max_pages, int n_pages, int head, int n_q, int n_kv, int M, int n_seg,
                       int ctx_limit, float* part_ml, float* part_acc, float* out, int8_t* outq, float* outds,
                       unsigned* fault, int layer, cudaStream_t st) {
  return flash_decode_go(q, k_cache, v_cache, row_pos, row_seq, block_table, max_pages, n_pages, head, n_q, n_kv, M, n_seg,
                         ctx_limit, part_ml, part_acc, out, outq, outds, fault, layer, 1, st);
}

}  // extern "C"

// ======================================================================================
// Allocation-free variant of bl_flash_decode (declared in bloomery_no_alloc.h).
//
// Some hosts of this library may not allocate device memory at the moment they need
// attention: code running inside someone else's memory plan (a serving process whose
// whole HBM budget was handed out at start-up and whose allocator is closed), a real-time
// loop where a cudaMalloc would stall every stream of the device, or a plug-in that is
// given input and output buffers and nothing else.  The split-K partials that
// bl_flash_decode takes from the caller live here in one file-scope device array instead.
//
// Limit: M * n_q * n_seg <= kStaticCells (8192) and head <= 128, i.e. 4 MiB + 64 KiB of
// device memory, held by every GPU on which this library is loaded, until the process
// ends.  Larger shapes are refused with BL_ERR_LIMIT; nothing is launched.
//
// The array is shared by every call and keeps the last call's contents.  Nothing in it
// has to start at zero: the segment kernel writes every cell the merge kernel reads
// (empty segments write weight 0).  Two calls that overlap on the GPU (different streams,
// or two host threads) race on it; callers serialise them on one stream.
//
// The first call on a device resolves the array's device address with
// cudaGetSymbolAddress (in host code the array's name is only a host-side handle, not a
// device pointer).  Make that first call before any stream capture begins.
// ======================================================================================
namespace bl {
constexpr long kStaticCells = 8192;
constexpr int kStaticHead = 128;
static __device__ __align__(256) float g_flash_static_scratch[kStaticCells * (kStaticHead + 2)];
static float* g_flash_static_ptr[64] = {nullptr};
}  // namespace bl

extern "C" int bl_flash_decode_static(const float* q, const void* k_cache, const void* v_cache, const int* row_pos,
                                      const int* row_seq, const int* block_table, int max_pages, int n_pages, int head,
                                      int n_q, int n_kv, int M, int n_seg, int ctx_limit, float* out, int8_t* outq,
                                      float* outds, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(head == 128 || head == 64, BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && n_q >= 1 && n_seg >= 1, BL_ERR_SHAPE);
  BL_REQUIRE((long)M * n_q * n_seg <= kStaticCells, BL_ERR_LIMIT);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  BL_REQUIRE(dev >= 0 && dev < 64, BL_ERR_LIMIT);
  if (g_flash_static_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_flash_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_flash_static_ptr[dev] = p;
  }
  float* part_ml = g_flash_static_ptr[dev];                       // kStaticCells * 2 floats
  float* part_acc = g_flash_static_ptr[dev] + kStaticCells * 2;   // kStaticCells * head floats
  return bl_flash_decode(q, k_cache, v_cache, row_pos, row_seq, block_table, max_pages, n_pages, head, n_q, n_kv, M,
                         n_seg, ctx_limit, part_ml, part_acc, out, outq, outds, fault, layer, st);
}
