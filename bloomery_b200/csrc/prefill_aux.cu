// Helpers of the prompt (prefill) path around the tcgen05 GEMM: block-quantised weights
// expanded to bf16, RMSNorm to bf16, the expert permutation (count, scatter, gather) and
// the slot-ordered combine.  The reference groups prompt rows by expert on the device in
// gemm_route / grouped_buckets (crates/gpu/src/gemm/kernels.rs:88, q4k_sel.rs:492) and sums
// slots in ascending order (crates/gpu/src/arch/qwen3moe/experts.rs:36-45).
#include "common.cuh"

namespace bl {

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint4 o;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  return o;
}

// Units in row-major order are also in output order (64 u + e for every type but Q6_K), so a warp's 32 units are
// 4 KiB of contiguous output: each lane parks its 128 bytes in shared memory and the warp writes them back as
// full 512-byte rows.  Q6_K units own four separate runs of 16 values: those go out as 32-byte pieces.
template <class T>
__device__ __forceinline__ void expand_units(const uint8_t* w, long rows, int K, __nv_bfloat16* out, uint4 (*stage)[9]) {
  using U = Unit<T>;
  const int upr = K / 64;
  const long total = rows * upr;
  const long rb = resident_row_bytes(T::kType, K);
  const int lane = threadIdx.x & 31;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long base = (long)blockIdx.x * blockDim.x + (threadIdx.x & ~31); base < total; base += stride) {
    const long i = base + lane;
    float v[64];
    long r = 0;
    int u = 0;
    if (i < total) {
      r = i / upr;
      u = (int)(i - r * upr);
      typename U::Regs regs;
      U::loadu(w + r * rb, u, K, regs);
      U::decodeu(regs, u, v);
    }
    if (T::kType == WT_Q6_K) {
      if (i < total) {
        __nv_bfloat16* o = out + r * K;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4* dst = reinterpret_cast<uint4*>(o + U::pos(u, 16 * g));
          dst[0] = pack8_bf16(v + 16 * g);
          dst[1] = pack8_bf16(v + 16 * g + 8);
        }
      }
    } else {
      if (i < total) {
#pragma unroll
        for (int j = 0; j < 8; ++j) stage[lane][j] = pack8_bf16(v + 8 * j);
      }
      __syncwarp();
      uint4* o = reinterpret_cast<uint4*>(out + base * 64);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int idx = j * 32 + lane, uu = idx >> 3;
        if (base + uu < total) o[idx] = stage[uu][idx & 7];
      }
      __syncwarp();
    }
  }
}

__global__ void __launch_bounds__(256) dequant_bf16_kernel(const uint8_t* w, int wtype, long rows, int K, __nv_bfloat16* out) {
  __shared__ uint4 s_stage[8][32][9];
  uint4 (*stage)[9] = s_stage[threadIdx.x >> 5];
  pdl_wait();
  pdl_launch();
  switch (wtype) {
    case WT_Q4_K: expand_units<Q4K>(w, rows, K, out, stage); break;
    case WT_Q5_K: expand_units<Q5K>(w, rows, K, out, stage); break;
    case WT_Q6_K: expand_units<Q6K>(w, rows, K, out, stage); break;
    case WT_Q8_0: expand_units<Q80>(w, rows, K, out, stage); break;
    case WT_Q8_F32: expand_units<Q8F>(w, rows, K, out, stage); break;
    case WT_NVFP4: expand_units<NvFp4>(w, rows, K, out, stage); break;
    case WT_FP8_B128: expand_units<Fp8B128>(w, rows, K, out, stage); break;
    case WT_Q2_K: expand_units<Q2K>(w, rows, K, out, stage); break;
    case WT_Q3_K: expand_units<Q3K>(w, rows, K, out, stage); break;
    case WT_Q4_0: expand_units<Q40>(w, rows, K, out, stage); break;
    case WT_Q4_1: expand_units<Q41>(w, rows, K, out, stage); break;
    case WT_Q5_0: expand_units<Q50>(w, rows, K, out, stage); break;
    case WT_Q5_1: expand_units<Q51>(w, rows, K, out, stage); break;
    default: {
      const long total = rows * (long)K;
      for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        float v;
        if (wtype == WT_F32) v = reinterpret_cast<const float*>(w)[i];
        else if (wtype == WT_F16) v = __half2float(reinterpret_cast<const __half*>(w)[i]);
        else v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
        out[i] = __float2bfloat16_rn(v);
      }
    }
  }
}

// out[t, :] = bf16(RMSNorm(x[t, :]) * gain); gain == null: plain cast
__global__ void __launch_bounds__(256) rmsnorm_bf16_kernel(const float* x, long x_stride, const float* gain, float eps, int K,
                                                          __nv_bfloat16* out, long out_stride) {
  __shared__ double red[8];
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* xr = x + (long)t * x_stride;
  float scale = 1.0f;
  if (gain) {
    float ss = 0.f;
    for (int i = tid; i < K; i += 256) { float v = xr[i]; ss += v * v; }
    double tot = warp_sum_d((double)ss);
    if ((tid & 31) == 0) red[tid >> 5] = tot;
    __syncthreads();
    double all = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) all += red[w];
    scale = 1.0f / sqrtf((float)(all / (double)K) + eps);
  }
  for (int i = tid; i < K; i += 256)
    out[(long)t * out_stride + i] = __float2bfloat16_rn(gain ? xr[i] * scale * gain[i] : xr[i]);
}

__global__ void moe_count_kernel(const int* ids, int n, int E, int* counts) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { const int e = ids[i]; if (e >= 0 && e < E) atomicAdd(counts + e, 1); }
}

// pos = offsets[e] + cursor[e]++ ; dst_row[pos] = flat slot index i; row_scale[pos] = weight
__global__ void moe_scatter_kernel(const int* ids, const float* wts, int n, int E, const int* offsets, int* cursor,
                                   int* pos_of, int* dst_row, float* row_scale) {
  pdl_wait();
  pdl_launch();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i];
  if (e < 0 || e >= E) { pos_of[i] = -1; return; }
  const int p = offsets[e] + atomicAdd(cursor + e, 1);
  pos_of[i] = p;
  dst_row[p] = i;
  row_scale[p] = wts[i];
}

// The expert-sorted plan of a micro-batch in ONE launch (one block): count the routed slots per expert, prefix-sum
// the counts into row offsets, write the grouped product's tile table, and scatter every slot to its row.
//   ids / wts [n] flat (token-major) slot lists; pos_of[i] = row of slot i (-1: expert elsewhere);
//   dst_row[p] = slot at row p (-1 in the padding rows up to `cap`); row_scale[p] = its router weight;
//   offsets[E + 1]; mtiles / n_mtiles = tiles of tile_rows rows {expert, first row, end row of the expert, 0}.
// Replaces count + tile build + scatter and three buffer clears (six launches, one of them a serial loop).
struct MTilePlan { int group, row0, row_end, pad; };
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* ids, const float* wts, int n, int E, int cap, int* offsets,
                                                        int* pos_of, int* dst_row, float* row_scale, MTilePlan* mtiles,
                                                        int* n_mtiles, int max_mtiles, int tile_rows) {
  __shared__ int s_cnt[512], s_off[513], s_toff[513], s_cur[512];
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += 1024) { s_cnt[e] = 0; s_cur[e] = 0; }
  __syncthreads();
  for (int i = tid; i < n; i += 1024) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int off = 0, toff = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = off; s_toff[e] = toff;
      off += s_cnt[e];
      toff += (s_cnt[e] + tile_rows - 1) / tile_rows;
    }
    s_off[E] = off; s_toff[E] = toff;
    *n_mtiles = toff < max_mtiles ? toff : max_mtiles;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += 1024) offsets[e] = s_off[e];
  for (int e = tid; e < E; e += 1024) {
    const int rows = s_cnt[e], off = s_off[e];
    for (int r = 0, t = s_toff[e]; r < rows; r += tile_rows, ++t)
      if (t < max_mtiles) mtiles[t] = MTilePlan{e, off + r, off + rows, 0};
  }
  for (int p = s_off[E] + tid; p < cap; p += 1024) dst_row[p] = -1;
  for (int i = tid; i < n; i += 1024) {
    const int e = ids[i];
    if (e < 0 || e >= E) { pos_of[i] = -1; continue; }
    const int p = s_off[e] + atomicAdd(&s_cur[e], 1);
    pos_of[i] = p;
    dst_row[p] = i;
    row_scale[p] = wts[i];
  }
}

// Prompt form of the per-head RMSNorm + NEOX RoPE + KV append: one block per token, a warp per head (heads w, w + 8,
// ...), the sines and cosines of the token's position computed once per lane and reused by every head.
//   q -> bf16 [n_q][T][HEAD] (scaled), k / v -> the paged f16 cache.  Same arithmetic as the decode launch.
template <int HEAD>
__global__ void __launch_bounds__(256) rope_append_prefill_kernel(const float* qkv, long qkv_stride, const float* q_gain,
                                                                  const float* k_gain, const float* inv_freq, float eps,
                                                                  float q_scale, int n_q, int n_kv, int T, const int* row_pos,
                                                                  const int* row_seq, const int* block_table, int max_pages,
                                                                  int n_pages, __half* k_cache, __half* v_cache,
                                                                  __nv_bfloat16* q_bf16, unsigned* fault, int layer) {
  constexpr int DPL = HEAD / 32;
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int seq = row_seq[t];
  if (seq < 0) return;
  const int pos = row_pos[t];
  float sn[DPL / 2], cs[DPL / 2];
#pragma unroll
  for (int j = 0; j < DPL / 2; ++j) sincosf((float)pos * inv_freq[lane + 32 * j], &sn[j], &cs[j]);
  const int pslot = pos / 64;
  const int page = (pslot < max_pages) ? block_table[(long)seq * max_pages + pslot] : -1;
  const bool page_ok = page >= 0 && page < n_pages;
  if (!page_ok && threadIdx.x == 0) raise_fault(fault, layer, FS_PAGE);
  const float* row = qkv + (long)t * qkv_stride;
  for (int head = warp; head < n_q + 2 * n_kv; head += 8) {
    const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
    float x[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) x[j] = row[(long)head * HEAD + lane + 32 * j];
    const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
    if (gain) {
      double ss = 0.0;
#pragma unroll
      for (int j = 0; j < DPL; ++j) ss += (double)(x[j] * x[j]);
      ss = warp_sum_d(ss);
      const float scale = (float)(1.0 / sqrt(ss / (double)HEAD + (double)eps));
#pragma unroll
      for (int j = 0; j < DPL; ++j) x[j] = (scale * gain[lane + 32 * j]) * x[j];
    }
    if (is_q || is_k) {
#pragma unroll
      for (int j = 0; j < DPL / 2; ++j) {
        const float x0 = x[j], x1 = x[j + DPL / 2];
        x[j] = fmaf(x0, cs[j], -(x1 * sn[j]));
        x[j + DPL / 2] = fmaf(x0, sn[j], x1 * cs[j]);
      }
    }
    if (is_q) {
      __nv_bfloat16* q = q_bf16 + ((long)head * T + t) * HEAD;
#pragma unroll
      for (int j = 0; j < DPL; ++j) q[lane + 32 * j] = __float2bfloat16_rn(x[j] * q_scale);
    } else if (page_ok) {
      const int kvh = is_k ? head - n_q : head - n_q - n_kv;
      __half* dst = (is_k ? k_cache : v_cache) + (((long)page * n_kv + kvh) * 64 + (pos % 64)) * HEAD;
#pragma unroll
      for (int j = 0; j < DPL; ++j) dst[lane + 32 * j] = __float2half_rn(x[j]);
    }
  }
}

// A_perm[p, :] = src[dst_row[p] / k, :]  (bf16 rows of K values, 16-byte vectors)
__global__ void __launch_bounds__(256) gather_rows_bf16_kernel(const __nv_bfloat16* src, long src_stride, const int* dst_row,
                                                              const int* n_rows, int k, int K, __nv_bfloat16* out) {
  pdl_wait();
  pdl_launch();
  const int p = blockIdx.x;
  if (p >= *n_rows) return;
  const int t = dst_row[p] / k;
  const uint4* s = reinterpret_cast<const uint4*>(src + (long)t * src_stride);
  uint4* o = reinterpret_cast<uint4*>(out + (long)p * K);
  for (int i = threadIdx.x; i < K / 8; i += 256) o[i] = s[i];
}

// x[t, :] = resid[t, :] + sum_j slot_out[t*k + j, :] in ascending j (rows of dropped slots are skipped)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* slot_out, const int* pos_of, int k, int H,
                                                         const float* resid, long resid_stride, float* out, long out_stride) {
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x;
  for (int i = threadIdx.x * 4; i < H; i += 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; ++j) {
      if (pos_of[t * k + j] < 0) continue;
      const float4 v = *reinterpret_cast<const float4*>(slot_out + ((long)t * k + j) * H + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (resid) {
      const float4 r = *reinterpret_cast<const float4*>(resid + (long)t * resid_stride + i);
      acc.x += r.x; acc.y += r.y; acc.z += r.z; acc.w += r.w;
    }
    *reinterpret_cast<float4*>(out + (long)t * out_stride + i) = acc;
  }
}


// Contiguous bf16 copies of one sequence's keys and values for the prompt GEMMs:
//   Kb [n_kv][T_pad][HEAD], Vt [n_kv][HEAD][T_pad]; positions >= n_keys are zero.
// One block per (cache page of 64 keys, KV head): rows are read and the key rows written whole; the values
// pass through a shared tile so that the transposed rows are written 128 contiguous bytes at a time.
__global__ void __launch_bounds__(256) kv_gather_bf16_kernel(const __half* k_cache, const __half* v_cache, const int* block_table,
                                                            int n_pages, int n_kv, int head, int n_keys, int T_pad,
                                                            __nv_bfloat16* Kb, __nv_bfloat16* Vt) {
  __shared__ __nv_bfloat16 sv[64][130];         // 65-word rows: the transposed read has no bank conflicts
  pdl_wait();
  pdl_launch();
  const int t0 = blockIdx.x * 64, kvh = blockIdx.y, tid = threadIdx.x;
  int page = t0 < n_keys ? block_table[t0 / 64] : -1;
  if (page >= n_pages) page = -1;
  const long src0 = ((long)page * n_kv + kvh) * 64 * head;
  for (int i = tid; i < 64 * head; i += 256) {
    const int tt = i / head, d = i - tt * head;
    float kv = 0.f, vv = 0.f;
    if (page >= 0 && t0 + tt < n_keys) {
      kv = __half2float(k_cache[src0 + i]);
      vv = __half2float(v_cache[src0 + i]);
    }
    Kb[((long)kvh * T_pad + t0 + tt) * head + d] = __float2bfloat16_rn(kv);
    sv[tt][d] = __float2bfloat16_rn(vv);
  }
  __syncthreads();
  for (int i = tid; i < 64 * head; i += 256) {
    const int d = i >> 6, tt = i & 63;
    Vt[((long)kvh * head + d) * T_pad + t0 + tt] = sv[tt][d];
  }
}

// P[r, :] = softmax over keys 0..pos0 + (r % Tq) of S[r, :] (rows are head-major: r = h * Tq + tq);
// masked and padded columns get exactly 0.
// One block per score row.  Thread t owns runs of eight consecutive keys (8 (t + 256 j) ..): two 16-byte loads and one
// 16-byte store per run.  Rows of up to 8,192 keys are read once into registers; longer rows re-read their scores.
// Probabilities are written (zeros past the row's last key) only as far as the values product of the row's
// 128-query tile reads them: up to the 64-key block that holds the tile's last query.
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(256) softmax_causal_kernel(const float* S, long ldS, int Tq, int pos0, int T_pad,
                                                            __nv_bfloat16* P, long ldP) {
  __shared__ float red[8];
  pdl_wait();
  pdl_launch();
  const long r = blockIdx.x;
  const int tq = (int)(r % Tq);
  const int n_valid = min(T_pad, pos0 + tq + 1);
  const int n_write = min(T_pad, (pos0 + min(tq | 127, Tq - 1) + 1 + 63) / 64 * 64);
  const float* s = S + r * ldS;
  const int tid = threadIdx.x;
  const bool cached = T_pad <= 256 * 32 && (ldS % 4) == 0 && (ldP % 8) == 0;
  float v[32];
  float mx = -INFINITY;
  if (cached) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i0 = 8 * (tid + 256 * j);
      if (i0 < n_valid) {
        const float4 a = *reinterpret_cast<const float4*>(s + i0), b = *reinterpret_cast<const float4*>(s + i0 + 4);
        const float t8[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        if (i0 + 8 <= n_valid) {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[8 * j + e] = t8[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) v[8 * j + e] = (i0 + e) < n_valid ? t8[e] : -INFINITY;
        }
        mx = fmaxf(mx, fmaxf(fmaxf(fmaxf(v[8 * j], v[8 * j + 1]), fmaxf(v[8 * j + 2], v[8 * j + 3])),
                             fmaxf(fmaxf(v[8 * j + 4], v[8 * j + 5]), fmaxf(v[8 * j + 6], v[8 * j + 7]))));
      }
    }
  } else {
    for (int i = tid; i < n_valid; i += 256) mx = fmaxf(mx, s[i]);
  }
  mx = warp_max(mx);
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  if (cached) {
    // runs past the row's last key are skipped whole; a masked key inside the last run holds -inf and
    // comes out of ex2 as exactly 0 (the row's maximum is finite: key 0 is always valid)
    const float mxl = mx * 1.4426950408889634f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (8 * (tid + 256 * j) < n_valid) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          v[8 * j + e] = exp2_approx(fmaf(v[8 * j + e], 1.4426950408889634f, -mxl));
          sum += v[8 * j + e];
        }
      }
    }
  } else {
    for (int i = tid; i < n_valid; i += 256) sum += __expf(s[i] - mx);
  }
  sum = warp_sum(sum);
  if ((tid & 31) == 0) red[tid >> 5] = sum;
  __syncthreads();
  sum = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) sum += red[w];
  const float inv = 1.0f / sum;
  __nv_bfloat16* p = P + r * ldP;
  if (cached) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i0 = 8 * (tid + 256 * j);
      if (i0 < n_write) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = i0 < n_valid ? v[8 * j + e] * inv : 0.f;
        *reinterpret_cast<uint4*>(p + i0) = pack8_bf16(o);
      }
    }
  } else {
    for (int i = tid; i < n_write; i += 256) p[i] = __float2bfloat16_rn(i < n_valid ? __expf(s[i] - mx) * inv : 0.f);
  }
}


// Split-precision rows for the prompt router: out[t] = [hi | hi | lo] with hi = bf16(xn) and
// lo = bf16(xn - hi), xn = RMSNorm(x) * gain.  Against B = [Whi | Wlo | Whi] one bf16 GEMM of
// depth 3K gives hi*Whi + hi*Wlo + lo*Whi, i.e. fp32-grade logits (the dropped lo*Wlo term is
// ~2^-16 relative) on the tensor cores -- the reference splits hi/lo the same way for its
// indexer scores (crates/gpu/src/indexer.rs:168).
__global__ void __launch_bounds__(256) rmsnorm_hilo_kernel(const float* x, long x_stride, const float* gain, float eps, int K,
                                                          __nv_bfloat16* out) {
  __shared__ double red[8];
  pdl_wait();
  pdl_launch();
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* xr = x + (long)t * x_stride;
  float ss = 0.f;
  for (int i = tid; i < K; i += 256) { float v = xr[i]; ss += v * v; }
  double tot = warp_sum_d((double)ss);
  if ((tid & 31) == 0) red[tid >> 5] = tot;
  __syncthreads();
  double all = 0.0;
#pragma unroll
  for (int w = 0; w < 8; ++w) all += red[w];
  const float scale = 1.0f / sqrtf((float)(all / (double)K) + eps);
  __nv_bfloat16* o = out + (long)t * 3 * K;
  for (int i = tid; i < K; i += 256) {
    const float v = xr[i] * scale * gain[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    o[i] = hi; o[K + i] = hi;
    o[2 * K + i] = __float2bfloat16_rn(v - __bfloat162float(hi));
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

int bl_dequant_bf16(const void* w, int wtype, long rows, int K, void* out, cudaStream_t st) {
  BL_REQUIRE(rows >= 1 && K % 64 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(resident_row_bytes(wtype, K) > 0, BL_ERR_TYPE);
  long work = rows * (K / 64);
  int grid = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
  return (int)launch(dequant_bf16_kernel, dim3(grid), dim3(256), 0, st, (const uint8_t*)w, wtype, rows, K, (__nv_bfloat16*)out);
}

int bl_rmsnorm_bf16(const float* x, long x_stride, const float* gain, float eps, int T, int K, void* out, long out_stride,
                    cudaStream_t st) {
  BL_REQUIRE(T >= 1 && K >= 1, BL_ERR_SHAPE);
  return (int)launch(rmsnorm_bf16_kernel, dim3(T), dim3(256), 0, st, x, x_stride, gain, eps, K, (__nv_bfloat16*)out, out_stride);
}

int bl_moe_count(const int* ids, int n, int E, int* counts, cudaStream_t st) {
  BL_REQUIRE(n >= 1 && E >= 1, BL_ERR_SHAPE);
  return (int)launch(moe_count_kernel, dim3((n + 255) / 256), dim3(256), 0, st, ids, n, E, counts);
}

int bl_moe_plan(const int* ids, const float* wts, int n, int E, int cap, int* offsets, int* pos_of, int* dst_row,
                float* row_scale, void* mtiles, int* n_mtiles, int max_mtiles, int tile_rows, cudaStream_t st) {
  BL_REQUIRE(n >= 1 && E >= 1 && E <= 512 && cap >= n && tile_rows >= 8, BL_ERR_SHAPE);
  return (int)launch(moe_plan_kernel, dim3(1), dim3(1024), 0, st, ids, wts, n, E, cap, offsets, pos_of, dst_row, row_scale,
                     (MTilePlan*)mtiles, n_mtiles, max_mtiles, tile_rows);
}

int bl_rope_append_prefill(const float* qkv, long qkv_stride, const float* q_gain, const float* k_gain, const float* inv_freq,
                           float eps, float q_scale, int head, int n_q, int n_kv, int T, const int* row_pos, const int* row_seq,
                           const int* block_table, int max_pages, int n_pages, void* k_cache, void* v_cache, void* q_bf16,
                           unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(head == 128 || head == 64, BL_ERR_SHAPE);
  BL_REQUIRE(T >= 1 && n_q >= 1 && n_kv >= 1 && q_bf16, BL_ERR_SHAPE);
  if (head == 128)
    return (int)launch(rope_append_prefill_kernel<128>, dim3(T), dim3(256), 0, st, qkv, qkv_stride, q_gain, k_gain, inv_freq, eps,
                       q_scale, n_q, n_kv, T, row_pos, row_seq, block_table, max_pages, n_pages, (__half*)k_cache,
                       (__half*)v_cache, (__nv_bfloat16*)q_bf16, fault, layer);
  return (int)launch(rope_append_prefill_kernel<64>, dim3(T), dim3(256), 0, st, qkv, qkv_stride, q_gain, k_gain, inv_freq, eps,
                     q_scale, n_q, n_kv, T, row_pos, row_seq, block_table, max_pages, n_pages, (__half*)k_cache,
                     (__half*)v_cache, (__nv_bfloat16*)q_bf16, fault, layer);
}

int bl_moe_scatter(const int* ids, const float* wts, int n, int E, const int* offsets, int* cursor, int* pos_of,
                   int* dst_row, float* row_scale, cudaStream_t st) {
  BL_REQUIRE(n >= 1 && E >= 1, BL_ERR_SHAPE);
  return (int)launch(moe_scatter_kernel, dim3((n + 255) / 256), dim3(256), 0, st, ids, wts, n, E, offsets, cursor, pos_of,
                     dst_row, row_scale);
}

int bl_gather_rows_bf16(const void* src, long src_stride, const int* dst_row, const int* n_rows, int max_rows, int k, int K,
                        void* out, cudaStream_t st) {
  BL_REQUIRE(max_rows >= 1 && K % 8 == 0 && src_stride % 8 == 0, BL_ERR_SHAPE);
  return (int)launch(gather_rows_bf16_kernel, dim3(max_rows), dim3(256), 0, st, (const __nv_bfloat16*)src, src_stride, dst_row,
                     n_rows, k, K, (__nv_bfloat16*)out);
}

int bl_moe_combine(const float* slot_out, const int* pos_of, int T, int k, int H, const float* resid, long resid_stride,
                   float* out, long out_stride, cudaStream_t st) {
  BL_REQUIRE(T >= 1 && H % 4 == 0, BL_ERR_SHAPE);
  return (int)launch(moe_combine_kernel, dim3(T), dim3(256), 0, st, slot_out, pos_of, k, H, resid, resid_stride, out, out_stride);
}

int bl_kv_gather_bf16(const void* k_cache, const void* v_cache, const int* block_table, int n_pages, int n_kv, int head,
                      int n_keys, int T_pad, void* Kb, void* Vt, cudaStream_t st) {
  BL_REQUIRE(head <= 128 && T_pad >= 64 && T_pad % 64 == 0 && n_keys <= T_pad, BL_ERR_SHAPE);
  return (int)launch(kv_gather_bf16_kernel, dim3(T_pad / 64, n_kv), dim3(256), 0, st, (const __half*)k_cache, (const __half*)v_cache,
                     block_table, n_pages, n_kv, head, n_keys, T_pad, (__nv_bfloat16*)Kb, (__nv_bfloat16*)Vt);
}

int bl_softmax_causal(const float* S, long ldS, long rows, int Tq, int pos0, int T_pad, void* P, long ldP, cudaStream_t st) {
  BL_REQUIRE(rows >= 1 && Tq >= 1 && T_pad >= 1, BL_ERR_SHAPE);
  return (int)launch(softmax_causal_kernel, dim3((unsigned)rows), dim3(256), 0, st, S, ldS, Tq, pos0, T_pad, (__nv_bfloat16*)P, ldP);
}

int bl_rmsnorm_hilo(const float* x, long x_stride, const float* gain, float eps, int T, int K, void* out, cudaStream_t st) {
  BL_REQUIRE(T >= 1 && K >= 1 && gain != nullptr, BL_ERR_SHAPE);
  return (int)launch(rmsnorm_hilo_kernel, dim3(T), dim3(256), 0, st, x, x_stride, gain, eps, K, (__nv_bfloat16*)out);
}

}  // extern "C"
