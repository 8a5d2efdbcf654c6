// Decode chain, shared-memory staged form: every block fetches ALL the weight rows it will use with
// bulk asynchronous copies (cp.async.bulk, completion on an mbarrier) into shared memory, and - where the
// rows do not depend on the predecessor kernel - issues those copies BEFORE griddepcontrol.wait.
//
// Why: one decode step is a chain of small dependent kernels, each bound by a DRAM round trip rather than
// by bandwidth.  Under programmatic dependent launch the next kernel's blocks start while the current one
// still runs, but only if both fit on an SM.  The staged kernels keep weights out of the register file
// (<= 85 registers per thread, one block per SM for most launches), so kernel N+1 is resident beside kernel N
// and its whole weight slice streams from HBM while kernel N computes; after the wait only an L2 read of the
// activations, the dot products out of shared memory and one store remain.  griddepcontrol.launch_dependents
// is therefore the first instruction of every kernel here.
//
//   gemv_staged        K-quant / plane rows x (RMSNorm + q8 prologue | q8 rows), residual or all-reduce push
//   attn_fused         per-head RMSNorm + NEOX RoPE + KV append + split-K flash segments; the last block of
//                      a KV head (completion ticket) merges the segments and emits q8 rows for o_proj
//   gate_up_staged     gate.x, up.x of the chosen experts (ids read from the router launch), SwiGLU, q8;
//                      also asks L2 to prefetch this block's share of the down matrices
//   down_staged        down projection of every chosen expert + router-weighted sum + residual
//
// Arithmetic (lane -> unit assignment, accumulation and butterfly order) is the same as in the
// register-streaming kernels (decode_gemv.cu, moe_decode.cu, attn_decode.cu), so both forms give the same bits.
// Reference counterparts: crates/gpu/src/arch/qwen3moe/{proj,experts}.rs (family-constant fused launches),
// crates/gpu/src/rope_neox.rs, crates/gpu/src/flash_gqa.rs; the completion ticket is the reference's own
// device-side idiom (crates/gpu/src/route_softmax.rs:33-36).
#include "staged.cuh"

namespace bl {

// =======================================================================================================
// gemv_staged
// =======================================================================================================
template <class T, int MB>
__device__ __forceinline__ void rows_staged(const GemvArgs& a, const uint8_t* sw, long rb, int nrows, const int8_t* sq,
                                            const float2* sds, const float* s_scale, float* s_out) {
  using U = Unit<T>;
  const int K = a.K, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nunits = K / 64;
  // a warp takes rows warp, warp + 8, ...: two at a time for up to two activation rows, one at a time beyond
  constexpr bool kPair = MB <= 2;
  for (int r = warp; r < nrows; r += kPair ? 16 : 8) {
    const bool two = kPair && r + 8 < nrows;
    float acc0[MB], acc1[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) { acc0[m] = 0.f; acc1[m] = 0.f; }
    for (int u = lane; u < nunits; u += 32) {
      typename U::Regs g0, g1;
      U::loadu(sw + (long)r * rb, u, K, g0);
      if constexpr (kPair) U::loadu(sw + (long)(two ? r + 8 : r) * rb, u, K, g1);
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        ActRegs act;
        StagedAct<T>::load(sq + (long)m * K, sds + (long)m * (K / 32), u, nunits, act);
        acc0[m] += ActOf<T>::dot(g0, u, act);
        if constexpr (kPair) acc1[m] += ActOf<T>::dot(g1, u, act);
      }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) { acc0[m] = warp_sum(acc0[m]); if constexpr (kPair) acc1[m] = warp_sum(acc1[m]); }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        s_out[m * a.rpb_max + r] = acc0[m] * s_scale[m];
        if (two) s_out[m * a.rpb_max + r + 8] = acc1[m] * s_scale[m];
      }
    }
  }
}

// FAM 0: K-quants and Q8_0; FAM 2: block-scaled planes and the re-laid 32-value block types
template <int MB, bool NORM, int FAM>
__global__ void __launch_bounds__(256, 2) gemv_staged_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar;
  if (a.dbg & 1) pdl_launch();
  const int K = a.K, tid = threadIdx.x;
  uint8_t* sw = smem;
  int8_t* sq = reinterpret_cast<int8_t*>(smem + a.stage_bytes);
  float2* sds = reinterpret_cast<float2*>(sq + (size_t)MB * K);
  double* red = reinterpret_cast<double*>(sds + (size_t)MB * (K / 32));
  float* s_scale = reinterpret_cast<float*>(red + MB * 8);
  float* s_out = s_scale + 8;                         // [MB][rpb_max]

  int si = 0, col0 = 0;
#pragma unroll
  for (int q = 1; q < 4; ++q)
    if (q < a.nseg && (int)blockIdx.x >= a.seg[q].blk0) si = q;
  for (int q = 0; q < si; ++q) col0 += a.seg[q].rows;
  const GemvSeg& s = a.seg[si];
  const int bi = (int)blockIdx.x - s.blk0;
  const int rpb = (s.rows + s.nblk - 1) / s.nblk;
  const int r_lo = min(s.rows, bi * rpb), r_hi = min(s.rows, r_lo + rpb);
  const int nrows = r_hi - r_lo;
  const uint32_t bytes = (uint32_t)nrows * (uint32_t)s.row_bytes;
  if (tid == 0) {
    mbar_init(&bar, 1);
    if (bytes && !(a.dbg & 4)) {                      // weights never depend on the predecessor: fetch them now
      mbar_expect_tx(&bar, bytes);
      bulk_load_chunks(sw, s.w + (long)r_lo * s.row_bytes, bytes, &bar);
    }
  }
  __syncthreads();
  pdl_wait();
  // the dependents start now: their weight copies overlap this kernel's prologue and dot products (releasing them
  // before the wait was measured slower: their blocks then sit on the SM through the whole predecessor)
  if (!(a.dbg & 1)) pdl_launch();
  if (!(a.dbg & 8)) {
  if (NORM) prologue_norm<MB, false>(a, sq, sds, nullptr, s_scale, red, staged_layout(s.wtype));
  else prologue_q8in<MB>(a, sq, sds, s_scale, staged_layout(s.wtype));
  }
  bool ok = true;
  if (bytes && !(a.dbg & 4)) ok = mbar_wait(&bar, 0, a.fault, a.layer);
  if (!(a.dbg & 2)) {
  if constexpr (FAM == 0) {
  switch (s.wtype) {
    case WT_Q4_K: rows_staged<Q4K, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q6_K: rows_staged<Q6K, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q5_K: rows_staged<Q5K, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q8_0: rows_staged<Q80, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    default: ok = false;
  }
  } else {
  switch (s.wtype) {
    case WT_NVFP4: rows_staged<NvFp4, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_FP8_B128: rows_staged<Fp8B128, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q2_K: rows_staged<Q2K, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q3_K: rows_staged<Q3K, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q4_0: rows_staged<Q40, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q4_1: rows_staged<Q41, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q5_0: rows_staged<Q50, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    case WT_Q5_1: rows_staged<Q51, MB>(a, sw, s.row_bytes, nrows, sq, sds, s_scale, s_out); break;
    default: ok = false;
  }
  }
  }
  __syncthreads();
  // coalesced epilogue: consecutive threads own consecutive output columns
  const unsigned push_epoch = a.push.n_ranks > 0 ? site_epoch(a.push.step, a.push.sites_per_step, a.push.site_index) : 0u;
  for (int i = tid; i < nrows * MB; i += 256) {
    const int m = i / nrows, c = i - m * nrows;
    if (m >= a.M) continue;
    float v = ok ? s_out[m * a.rpb_max + c] : kNaN;
    const int col = col0 + r_lo + c;
    if (a.push.n_ranks > 0) { push_store(a.push, push_epoch, (long)m * a.out_stride + col, v); continue; }
    if (a.resid) v += a.resid[(long)m * a.resid_stride + col];
    a.out[(long)m * a.out_stride + col] = v;
  }
}

// =======================================================================================================
// attn_fused: RMSNorm + RoPE + append + flash segments + ticket merge
// =======================================================================================================
constexpr int kPage = 64;
constexpr int kKeyTile = 32;
constexpr int kStages = 4;        // key / value tiles in flight per block
constexpr int kMaxPatch = 64;     // rows of one pass whose keys a block may have to take from the pass itself

struct AttnArgs {
  const float* qkv; long qkv_stride;       // [M, (n_q + 2 n_kv) * HEAD]
  const float* q_gain; const float* k_gain; const float* inv_freq;
  float eps, q_scale;
  int n_q, n_kv, M, n_seg, ctx_limit;
  const int* row_pos; const int* row_seq; const int* block_table;
  int max_pages, n_pages;
  __half* k_cache; __half* v_cache;
  float* part_ml; float* part_acc;         // [M, n_q, n_seg, 2] and [M, n_q, n_seg, HEAD]
  unsigned* tickets;                       // [M * n_kv], zero between launches (the last block resets its ticket)
  float* out; int8_t* outq; float2* outds; // attention rows [M, n_q * HEAD]: optional fp32, q8 codes, {d, s} per 32
  unsigned* fault; int layer;
  long long* probe;
  int recv_off;                            // cluster form: float offset of the merge buffer in dynamic shared memory
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One head's HEAD values held as DPL = HEAD / 32 consecutive values per lane -> q8 codes + {d, s} per 32 values.
template <int HEAD>
__device__ __forceinline__ void head_out_q8(const float (&o)[HEAD / 32], int lane, long col0, const AttnArgs& a, int m) {
  constexpr int DPL = HEAD / 32, LPB = 32 / DPL;     // lanes per 32-value block
  const long width = (long)a.n_q * HEAD;
  float amax = 0.f;
#pragma unroll
  for (int d = 0; d < DPL; ++d) amax = fmaxf(amax, fabsf(o[d]));
#pragma unroll
  for (int off = 1; off < LPB; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float dd = amax / 127.0f, inv = dd > 0.f ? 1.0f / dd : 0.f;
  int sum = 0;
  uint32_t packed = 0;
#pragma unroll
  for (int d = 0; d < DPL; ++d) {
    int q = max(-127, min(127, __float2int_rn(o[d] * inv)));
    sum += q;
    packed |= (uint32_t)(q & 0xFF) << (8 * d);
  }
#pragma unroll
  for (int off = 1; off < LPB; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const long col = col0 + lane * DPL;
  if (a.out) {
#pragma unroll
    for (int d = 0; d < DPL; ++d) a.out[(long)m * width + col + d] = o[d];
  }
  if constexpr (DPL == 4) *reinterpret_cast<uint32_t*>(a.outq + (long)m * width + col) = packed;
  else *reinterpret_cast<uint16_t*>(a.outq + (long)m * width + col) = (uint16_t)packed;
  if ((lane % LPB) == 0) a.outds[((long)m * width + col) / 32] = make_float2(dd, dd * (float)sum);
}

// grid (n_seg, n_kv, M); 256 threads = 8 warps; warp w serves q heads w, w + 8 of the KV head's group
template <int HEAD, int HPW>
__global__ void __launch_bounds__(256, 2) attn_fused_kernel(const AttnArgs a) {
  constexpr int KSTR = HEAD + 8, DPL = HEAD / 32;
  extern __shared__ __align__(128) uint8_t smem[];
  const int G = a.n_q / a.n_kv;
  float* sq = reinterpret_cast<float*>(smem);                              // [G][HEAD]
  __half* sk = reinterpret_cast<__half*>(smem + (size_t)G * HEAD * 4);     // [kStages][32][KSTR]
  __half* sv = sk + kStages * kKeyTile * KSTR;                             // [kStages][32][HEAD]
  __half* snew = sv + kStages * kKeyTile * HEAD;                           // [patch rows][2][HEAD]: keys and values of this pass
  __shared__ int s_last, s_np;
  __shared__ int s_pm[kMaxPatch], s_ppos[kMaxPatch];
  const int seg = blockIdx.x, kvh = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // positions, sequence and block table are step parameters: they do not depend on the predecessor kernel
  const int seq = a.row_seq[m];
  const int pos = a.row_pos[m];
  const int n_keys = pos + 1;
  const bool pad = seq < 0;
  const bool bad = !pad && (n_keys <= 0 || n_keys > a.ctx_limit);
  const int n_tiles = (pad || bad) ? 0 : (n_keys + kKeyTile - 1) / kKeyTile;
  const int tps = max(1, (n_tiles + a.n_seg - 1) / a.n_seg);
  const int used = (n_tiles + tps - 1) / tps;
  const int t0 = seg * tps, t1 = min(n_tiles, t0 + tps);
  if (pad || bad) {
    // padding rows and rows with a bad key count still publish rows for o_proj: zeros, or a NaN scale
    if (seg != 0) return;
    pdl_wait();
    pdl_launch();
    if (bad && tid == 0 && kvh == 0) raise_fault(a.fault, a.layer, FS_KEY_COUNT);
    const long width = (long)a.n_q * HEAD;
    for (int i = tid; i < G * HEAD; i += 256) {
      const long col = (long)kvh * G * HEAD + i;
      a.outq[(long)m * width + col] = 0;
      if (a.out) a.out[(long)m * width + col] = bad ? kNaN : 0.f;
      if ((i & 31) == 0) a.outds[((long)m * width + col) / 32] = bad ? make_float2(kNaN, 0.f) : make_float2(0.f, 0.f);
    }
    return;
  }
  if (t0 >= t1) return;                            // past the row's last key tile

  const int* bt = a.block_table + (long)seq * a.max_pages;
  auto issue_tile = [&](int t, int stage) {
    const int key0 = t * kKeyTile;
    int page = bt[key0 / kPage];
    page = (page < 0 || page >= a.n_pages) ? 0 : page;      // the append below raises the fault; stay in bounds
    const long base = (((long)page * a.n_kv + kvh) * kPage + (key0 % kPage)) * HEAD;
    constexpr int CH = HEAD / 8;
    for (int c = tid; c < kKeyTile * CH; c += 256) {
      const int r = c / CH, cc = c % CH;
      cp_async16(sk + ((size_t)stage * kKeyTile + r) * KSTR + cc * 8, a.k_cache + base + (long)r * HEAD + cc * 8);
      cp_async16(sv + ((size_t)stage * kKeyTile + r) * HEAD + cc * 8, a.v_cache + base + (long)r * HEAD + cc * 8);
    }
    cp_async_commit();
  };
  // keys of earlier positions are already in the cache: the first kStages tiles stream in while the predecessor
  // still runs (one copy group per stage, empty past the last tile, so the group count stays uniform)
  probe_mark(a.probe, 0);
#pragma unroll
  for (int st = 0; st < kStages; ++st) {
    if (t0 + st < t1) issue_tile(t0 + st, st);
    else cp_async_commit();
  }
  pdl_wait();
  pdl_launch();
  probe_mark(a.probe, 1);

  // ---- queries of this KV head's group: RMSNorm + RoPE into shared memory ---------------------------
  const float* row = a.qkv + (long)m * a.qkv_stride;
  auto norm_rope = [&](const float* src, const float* gain, bool rope, int at, float (&y)[DPL]) {
    // lane owns elements lane + 32 j; NEOX pairs are (i, i + HALF)
    float x[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) x[j] = src[lane + 32 * j];
    if (gain) {
      double ss = 0.0;
#pragma unroll
      for (int j = 0; j < DPL; ++j) ss += (double)(x[j] * x[j]);
      ss = warp_sum_d(ss);
      const float scale = (float)(1.0 / sqrt(ss / (double)HEAD + (double)a.eps));
#pragma unroll
      for (int j = 0; j < DPL; ++j) x[j] = (scale * gain[lane + 32 * j]) * x[j];
    }
    if (rope) {
#pragma unroll
      for (int j = 0; j < DPL / 2; ++j) {
        const int i = lane + 32 * j;
        float sn, cs;
        sincosf((float)at * a.inv_freq[i], &sn, &cs);
        const float x0 = x[j], x1 = x[j + DPL / 2];
        y[j] = fmaf(x0, cs, -(x1 * sn));
        y[j + DPL / 2] = fmaf(x0, sn, x1 * cs);
      }
    } else {
#pragma unroll
      for (int j = 0; j < DPL; ++j) y[j] = x[j];
    }
  };
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int hg = warp + 8 * h;
    if (hg < G) {
      float y[DPL];
      norm_rope(row + ((long)kvh * G + hg) * HEAD, a.q_gain, true, pos, y);
#pragma unroll
      for (int j = 0; j < DPL; ++j) sq[hg * HEAD + lane + 32 * j] = y[j] * a.q_scale;
    }
  }
  probe_mark(a.probe, 2);
  // ---- keys and values that this very pass appends --------------------------------------------------
  // Rows of the pass that belong to the same sequence at or before this row's position are not in the cache
  // yet (their owner blocks write them in this same launch), so a block computes the ones that fall inside its
  // key range itself and patches them into the tiles; only the row's own block stores its row to the cache.
  if (tid == 0) s_np = 0;
  __syncthreads();
  for (int mm = tid; mm < a.M; mm += 256) {
    if (a.row_seq[mm] == seq) {
      const int pp = a.row_pos[mm];
      if (pp <= pos && pp >= t0 * kKeyTile && pp < t1 * kKeyTile) {
        const int idx = atomicAdd(&s_np, 1);
        if (idx < kMaxPatch) { s_pm[idx] = mm; s_ppos[idx] = pp; }
      }
    }
  }
  __syncthreads();
  const int np = min(s_np, kMaxPatch);
  for (int it = warp; it < 2 * np; it += 8) {
    const int idx = it >> 1, mm = s_pm[idx], pp = s_ppos[idx];
    const bool is_k = (it & 1) == 0;
    float y[DPL];
    const float* src = a.qkv + (long)mm * a.qkv_stride + ((long)a.n_q + (is_k ? 0 : a.n_kv) + kvh) * HEAD;
    norm_rope(src, is_k ? a.k_gain : nullptr, is_k, pp, y);
    __half* sn = snew + ((size_t)idx * 2 + (is_k ? 0 : 1)) * HEAD;
    __half* dst = nullptr;
    if (mm == m) {
      const int pslot = pp / kPage;
      const int page = (pslot < a.max_pages) ? bt[pslot] : -1;
      if (page >= 0 && page < a.n_pages) dst = (is_k ? a.k_cache : a.v_cache) + (((long)page * a.n_kv + kvh) * kPage + (pp % kPage)) * HEAD;
      else if (lane == 0 && is_k) raise_fault(a.fault, a.layer, FS_PAGE);
    }
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const __half hv = __float2half_rn(y[j]);
      sn[lane + 32 * j] = hv;
      if (dst) dst[lane + 32 * j] = hv;
    }
  }

  probe_mark(a.probe, 3);
  float mx[HPW], l[HPW], acc[HPW][DPL];
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    mx[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }
  for (int t = t0; t < t1; ++t) {
    const int stage = (t - t0) % kStages;
    cp_async_wait<kStages - 1>();                    // the oldest group in flight (tile t) has landed
    __syncthreads();
    bool patched = false;
    for (int idx = 0; idx < np; ++idx) {
      const int r = s_ppos[idx] - t * kKeyTile;
      if (r >= 0 && r < kKeyTile) {                          // a row of this pass: the copy raced its store
        for (int i = tid; i < HEAD; i += 256) {
          sk[((size_t)stage * kKeyTile + r) * KSTR + i] = snew[(size_t)idx * 2 * HEAD + i];
          sv[((size_t)stage * kKeyTile + r) * HEAD + i] = snew[((size_t)idx * 2 + 1) * HEAD + i];
        }
        patched = true;
      }
    }
    if (patched) __syncthreads();
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
        const float tmax = warp_max(s);
        const float nm = fmaxf(mx[h], tmax);
        const float corr = (mx[h] == -INFINITY) ? 0.f : __expf(mx[h] - nm);
        const float p = (s == -INFINITY) ? 0.f : __expf(s - nm);
        l[h] = l[h] * corr + warp_sum(p);
        mx[h] = nm;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] *= corr;
        const __half* vbase = sv + (size_t)stage * kKeyTile * HEAD + lane * DPL;
        const int kmax = min(kKeyTile, n_keys - t * kKeyTile);    // masked keys are never read
#pragma unroll 4
        for (int k = 0; k < kmax; ++k) {
          const float pk = __shfl_sync(0xffffffffu, p, k);
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
    if (t + kStages < t1) issue_tile(t + kStages, stage);     // refill the stage just read
    else cp_async_commit();
  }

  probe_mark(a.probe, 4);
  if (used == 1) {
    // one segment covers the whole row: finish here, nothing to merge
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
      const int hg = warp + 8 * h;
      if (hg < G) {
        float o[DPL];
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[d] = acc[h][d] / l[h];
        head_out_q8<HEAD>(o, lane, ((long)kvh * G + hg) * HEAD, a, m);
      }
    }
    return;
  }
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int hg = warp + 8 * h;
    if (hg < G) {
      const long pidx = ((long)m * a.n_q + (long)kvh * G + hg) * a.n_seg + seg;
      if (lane == 0) { a.part_ml[pidx * 2] = mx[h]; a.part_ml[pidx * 2 + 1] = l[h]; }
#pragma unroll
      for (int d = 0; d < DPL; ++d) a.part_acc[pidx * HEAD + lane * DPL + d] = acc[h][d];
    }
  }
  // completion ticket: the block that arrives last for this (row, KV head) merges the segments
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned t = atomicAdd(a.tickets + (long)m * a.n_kv + kvh, 1u);
    s_last = (t == (unsigned)used - 1u) ? 1 : 0;
    if (s_last) a.tickets[(long)m * a.n_kv + kvh] = 0u;       // ready for the next launch (graph replay)
  }
  __syncthreads();
  probe_mark(a.probe, 5);
  if (!s_last) return;
  __threadfence();
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int hg = warp + 8 * h;
    if (hg < G) {
      const long p0 = ((long)m * a.n_q + (long)kvh * G + hg) * a.n_seg;
      // lanes fetch the segments' (max, sum) pairs side by side; the accumulators follow eight segments per
      // round trip; the sums themselves still run over the segments in ascending order
      float gm = -INFINITY;
      for (int s0 = 0; s0 < used; s0 += 32) {
        const int sg = s0 + lane;
        if (sg < used) gm = fmaxf(gm, __ldcg(a.part_ml + (p0 + sg) * 2));
      }
      gm = warp_max(gm);
      float den = 0.f, num[DPL];
#pragma unroll
      for (int d = 0; d < DPL; ++d) num[d] = 0.f;
      for (int s0 = 0; s0 < used; s0 += 32) {
        const int sg = s0 + lane;
        float ms = -INFINITY, ls = 0.f;
        if (sg < used) { const float2 v = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (p0 + sg) * 2)); ms = v.x; ls = v.y; }
        const float wl = (ms == -INFINITY) ? 0.f : __expf(ms - gm);
        const int cnt = min(32, used - s0);
        for (int k0 = 0; k0 < cnt; k0 += 8) {
          float v[8][DPL];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (k0 + k < cnt) {
              const float* src = a.part_acc + (p0 + s0 + k0 + k) * HEAD + lane * DPL;
              if constexpr (DPL == 4) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(src));
                v[k][0] = t.x; v[k][1] = t.y; v[k][2] = t.z; v[k][3] = t.w;
              } else {
                const float2 t = __ldcg(reinterpret_cast<const float2*>(src));
                v[k][0] = t.x; v[k][1] = t.y;
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (k0 + k < cnt) {
              const float wk = __shfl_sync(0xffffffffu, wl, k0 + k), lk = __shfl_sync(0xffffffffu, ls, k0 + k);
              den = fmaf(lk, wk, den);
#pragma unroll
              for (int d = 0; d < DPL; ++d) num[d] = fmaf(v[k][d], wk, num[d]);
            }
          }
        }
      }
      float o[DPL];
#pragma unroll
      for (int d = 0; d < DPL; ++d) o[d] = num[d] / den;
      head_out_q8<HEAD>(o, lane, ((long)kvh * G + hg) * HEAD, a, m);
    }
  }
}

// The same attention launch with the key segments of one (row, KV head) held by the CTAs of a thread-block cluster:
// the segments' partial results meet in distributed shared memory behind the cluster's hardware barrier instead of
// going through global memory and a completion ticket, which takes the merge's L2 round trips off the critical path.
// grid (CL, n_kv, M), cluster (CL, 1, 1); CTA c takes the c-th run of key tiles; head hg is merged by CTA hg % CL.
template <int HEAD, int HPW>
__global__ void __launch_bounds__(256, 2) attn_cluster_kernel(const AttnArgs a) {
  constexpr int KSTR = HEAD + 8, DPL = HEAD / 32;
  extern __shared__ __align__(128) uint8_t smem[];
  const int G = a.n_q / a.n_kv;
  float* sq = reinterpret_cast<float*>(smem);                              // [G][HEAD]
  __half* sk = reinterpret_cast<__half*>(smem + (size_t)G * HEAD * 4);     // [kStages][32][KSTR]
  __half* sv = sk + kStages * kKeyTile * KSTR;                             // [kStages][32][HEAD]
  __half* snew = sv + kStages * kKeyTile * HEAD;                           // [patch rows][2][HEAD]: keys and values of this pass
  __shared__ int s_np;
  __shared__ int s_pm[kMaxPatch], s_ppos[kMaxPatch];
  const int CL = (int)gridDim.x;
  const int seg = (int)cluster_ctarank(), kvh = blockIdx.y, m = blockIdx.z;
  float* s_recv = reinterpret_cast<float*>(smem) + a.recv_off;          // [heads merged here][CL][HEAD + 4]: {acc, max, sum}
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // positions, sequence and block table are step parameters: they do not depend on the predecessor kernel
  const int seq = a.row_seq[m];
  const int pos = a.row_pos[m];
  const int n_keys = pos + 1;
  const bool pad = seq < 0;
  const bool bad = !pad && (n_keys <= 0 || n_keys > a.ctx_limit);
  const int n_tiles = (pad || bad) ? 0 : (n_keys + kKeyTile - 1) / kKeyTile;
  const int tps = max(1, (n_tiles + CL - 1) / CL);
  const int t0 = min(n_tiles, seg * tps), t1 = min(n_tiles, t0 + tps);
  if (pad || bad) {
    // padding rows and rows with a bad key count still publish rows for o_proj: zeros, or a NaN scale
    if (seg != 0) return;
    pdl_wait();
    pdl_launch();
    if (bad && tid == 0 && kvh == 0) raise_fault(a.fault, a.layer, FS_KEY_COUNT);
    const long width = (long)a.n_q * HEAD;
    for (int i = tid; i < G * HEAD; i += 256) {
      const long col = (long)kvh * G * HEAD + i;
      a.outq[(long)m * width + col] = 0;
      if (a.out) a.out[(long)m * width + col] = bad ? kNaN : 0.f;
      if ((i & 31) == 0) a.outds[((long)m * width + col) / 32] = bad ? make_float2(kNaN, 0.f) : make_float2(0.f, 0.f);
    }
    return;
  }
  // a CTA past the row's last key tile still meets the cluster at its barrier, with an empty partial

  const int* bt = a.block_table + (long)seq * a.max_pages;
  auto issue_tile = [&](int t, int stage) {
    const int key0 = t * kKeyTile;
    int page = bt[key0 / kPage];
    page = (page < 0 || page >= a.n_pages) ? 0 : page;      // the append below raises the fault; stay in bounds
    const long base = (((long)page * a.n_kv + kvh) * kPage + (key0 % kPage)) * HEAD;
    constexpr int CH = HEAD / 8;
    for (int c = tid; c < kKeyTile * CH; c += 256) {
      const int r = c / CH, cc = c % CH;
      cp_async16(sk + ((size_t)stage * kKeyTile + r) * KSTR + cc * 8, a.k_cache + base + (long)r * HEAD + cc * 8);
      cp_async16(sv + ((size_t)stage * kKeyTile + r) * HEAD + cc * 8, a.v_cache + base + (long)r * HEAD + cc * 8);
    }
    cp_async_commit();
  };
  // keys of earlier positions are already in the cache: the first kStages tiles stream in while the predecessor
  // still runs (one copy group per stage, empty past the last tile, so the group count stays uniform)
  probe_mark(a.probe, 0);
#pragma unroll
  for (int st = 0; st < kStages; ++st) {
    if (t0 + st < t1) issue_tile(t0 + st, st);
    else cp_async_commit();
  }
  pdl_wait();
  pdl_launch();
  probe_mark(a.probe, 1);

  // ---- queries of this KV head's group: RMSNorm + RoPE into shared memory ---------------------------
  const float* row = a.qkv + (long)m * a.qkv_stride;
  auto norm_rope = [&](const float* src, const float* gain, bool rope, int at, float (&y)[DPL]) {
    // lane owns elements lane + 32 j; NEOX pairs are (i, i + HALF)
    float x[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) x[j] = src[lane + 32 * j];
    if (gain) {
      double ss = 0.0;
#pragma unroll
      for (int j = 0; j < DPL; ++j) ss += (double)(x[j] * x[j]);
      ss = warp_sum_d(ss);
      const float scale = (float)(1.0 / sqrt(ss / (double)HEAD + (double)a.eps));
#pragma unroll
      for (int j = 0; j < DPL; ++j) x[j] = (scale * gain[lane + 32 * j]) * x[j];
    }
    if (rope) {
#pragma unroll
      for (int j = 0; j < DPL / 2; ++j) {
        const int i = lane + 32 * j;
        float sn, cs;
        sincosf((float)at * a.inv_freq[i], &sn, &cs);
        const float x0 = x[j], x1 = x[j + DPL / 2];
        y[j] = fmaf(x0, cs, -(x1 * sn));
        y[j + DPL / 2] = fmaf(x0, sn, x1 * cs);
      }
    } else {
#pragma unroll
      for (int j = 0; j < DPL; ++j) y[j] = x[j];
    }
  };
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int hg = warp + 8 * h;
    if (hg < G) {
      float y[DPL];
      norm_rope(row + ((long)kvh * G + hg) * HEAD, a.q_gain, true, pos, y);
#pragma unroll
      for (int j = 0; j < DPL; ++j) sq[hg * HEAD + lane + 32 * j] = y[j] * a.q_scale;
    }
  }
  probe_mark(a.probe, 2);
  // ---- keys and values that this very pass appends --------------------------------------------------
  // Rows of the pass that belong to the same sequence at or before this row's position are not in the cache
  // yet (their owner blocks write them in this same launch), so a block computes the ones that fall inside its
  // key range itself and patches them into the tiles; only the row's own block stores its row to the cache.
  if (tid == 0) s_np = 0;
  __syncthreads();
  for (int mm = tid; mm < a.M; mm += 256) {
    if (a.row_seq[mm] == seq) {
      const int pp = a.row_pos[mm];
      if (pp <= pos && pp >= t0 * kKeyTile && pp < t1 * kKeyTile) {
        const int idx = atomicAdd(&s_np, 1);
        if (idx < kMaxPatch) { s_pm[idx] = mm; s_ppos[idx] = pp; }
      }
    }
  }
  __syncthreads();
  const int np = min(s_np, kMaxPatch);
  for (int it = warp; it < 2 * np; it += 8) {
    const int idx = it >> 1, mm = s_pm[idx], pp = s_ppos[idx];
    const bool is_k = (it & 1) == 0;
    float y[DPL];
    const float* src = a.qkv + (long)mm * a.qkv_stride + ((long)a.n_q + (is_k ? 0 : a.n_kv) + kvh) * HEAD;
    norm_rope(src, is_k ? a.k_gain : nullptr, is_k, pp, y);
    __half* sn = snew + ((size_t)idx * 2 + (is_k ? 0 : 1)) * HEAD;
    __half* dst = nullptr;
    if (mm == m) {
      const int pslot = pp / kPage;
      const int page = (pslot < a.max_pages) ? bt[pslot] : -1;
      if (page >= 0 && page < a.n_pages) dst = (is_k ? a.k_cache : a.v_cache) + (((long)page * a.n_kv + kvh) * kPage + (pp % kPage)) * HEAD;
      else if (lane == 0 && is_k) raise_fault(a.fault, a.layer, FS_PAGE);
    }
#pragma unroll
    for (int j = 0; j < DPL; ++j) {
      const __half hv = __float2half_rn(y[j]);
      sn[lane + 32 * j] = hv;
      if (dst) dst[lane + 32 * j] = hv;
    }
  }

  probe_mark(a.probe, 3);
  float mx[HPW], l[HPW], acc[HPW][DPL];
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    mx[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }
  for (int t = t0; t < t1; ++t) {
    const int stage = (t - t0) % kStages;
    cp_async_wait<kStages - 1>();                    // the oldest group in flight (tile t) has landed
    __syncthreads();
    bool patched = false;
    for (int idx = 0; idx < np; ++idx) {
      const int r = s_ppos[idx] - t * kKeyTile;
      if (r >= 0 && r < kKeyTile) {                          // a row of this pass: the copy raced its store
        for (int i = tid; i < HEAD; i += 256) {
          sk[((size_t)stage * kKeyTile + r) * KSTR + i] = snew[(size_t)idx * 2 * HEAD + i];
          sv[((size_t)stage * kKeyTile + r) * HEAD + i] = snew[((size_t)idx * 2 + 1) * HEAD + i];
        }
        patched = true;
      }
    }
    if (patched) __syncthreads();
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
        const float tmax = warp_max(s);
        const float nm = fmaxf(mx[h], tmax);
        const float corr = (mx[h] == -INFINITY) ? 0.f : __expf(mx[h] - nm);
        const float p = (s == -INFINITY) ? 0.f : __expf(s - nm);
        l[h] = l[h] * corr + warp_sum(p);
        mx[h] = nm;
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] *= corr;
        const __half* vbase = sv + (size_t)stage * kKeyTile * HEAD + lane * DPL;
        const int kmax = min(kKeyTile, n_keys - t * kKeyTile);    // masked keys are never read
#pragma unroll 4
        for (int k = 0; k < kmax; ++k) {
          const float pk = __shfl_sync(0xffffffffu, p, k);
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
    if (t + kStages < t1) issue_tile(t + kStages, stage);     // refill the stage just read
    else cp_async_commit();
  }

  probe_mark(a.probe, 4);
  // ---- every segment's partial of head hg goes to CTA hg % CL; the cluster barrier; that CTA merges ----
  constexpr int RS = HEAD + 4;                     // floats per partial: accumulators, max, sum, pad
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int hg = warp + 8 * h;
    if (hg < G) {
      float* slot = s_recv + ((size_t)(hg / CL) * CL + seg) * RS;
      const unsigned dst = (unsigned)(hg % CL);
      if constexpr (DPL == 4) st_peer_v4(peer_addr(slot + lane * 4, dst), acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
      else st_peer_v2(peer_addr(slot + lane * 2, dst), acc[h][0], acc[h][1]);
      if (lane == 0) st_peer_v2(peer_addr(slot + HEAD, dst), mx[h], l[h]);
    }
  }
  cluster_sync_all();
  probe_mark(a.probe, 5);
  for (int hs = warp; seg + hs * CL < G; hs += 8) {                // the heads this CTA merges, one warp each
    const int hg = seg + hs * CL;
    const float* base = s_recv + (size_t)hs * CL * RS;
    float gm = -INFINITY;
    for (int s = 0; s < CL; ++s) gm = fmaxf(gm, base[(size_t)s * RS + HEAD]);
    float den = 0.f, num[DPL];
#pragma unroll
    for (int d = 0; d < DPL; ++d) num[d] = 0.f;
    for (int s = 0; s < CL; ++s) {                               // ascending segment order, fixed
      const float ms = base[(size_t)s * RS + HEAD];
      const float w = (ms == -INFINITY) ? 0.f : __expf(ms - gm);
      den = fmaf(base[(size_t)s * RS + HEAD + 1], w, den);
#pragma unroll
      for (int d = 0; d < DPL; ++d) num[d] = fmaf(base[(size_t)s * RS + lane * DPL + d], w, num[d]);
    }
    float o[DPL];
#pragma unroll
    for (int d = 0; d < DPL; ++d) o[d] = num[d] / den;
    head_out_q8<HEAD>(o, lane, ((long)kvh * G + hg) * HEAD, a, m);
  }
}

// =======================================================================================================
// gate_up_staged
// =======================================================================================================
struct GateUpStagedArgs {
  const int8_t* xq; const float2* xds;     // [M, K] q8 rows of the normed residual
  RouteParams route;                       // route.logits != null: every block routes its row itself from the router
                                           // launch's logits (block (0, 0, m) also publishes ids / wts / heat)
  int* ids;                                // [M, n_used] chosen experts: read (route.logits == null) or written
  float* wts; unsigned* heat;
  const int* slot_map;                     // optional [E]: expert id -> resident slot (or kExpertElsewhere)
  const uint8_t* gate; const uint8_t* up; int wtype;   // stacks [E_slots, I, row_bytes]
  const uint8_t* down; long down_expert_bytes;         // optional: the down stack, for the L2 prefetch
  int K, I, E, n_used, M;
  int8_t* actq; float2* actds; float* act_f32;         // [M, n_used, I]
  unsigned* fault; int layer;
  long long* probe;
};

// grid (I / 32, n_used, M), 256 threads: a block owns 32 activation rows of one chosen expert; warp w rows 4w..4w+3
__global__ void __launch_bounds__(256, 2) gate_up_staged_kernel(const GateUpStagedArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ float s_act[32];
  __shared__ int s_e;
  __shared__ RouteWarpShared s_rw;
  const int K = a.K;
  const int chunk = blockIdx.x, j = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long rb = resident_row_bytes(a.wtype, K);
  const uint32_t half_bytes = (uint32_t)(32 * rb);
  uint8_t* sg = smem;
  uint8_t* su = smem + half_bytes;
  int8_t* sxq = reinterpret_cast<int8_t*>(smem + 2 * half_bytes);
  float2* sxds = reinterpret_cast<float2*>(sxq + K);
  probe_mark(a.probe, 0);
  if (tid == 0) mbar_init(&bar, 1);
  __syncthreads();
  pdl_wait();
  pdl_launch();
  probe_mark(a.probe, 1);
  const bool routed_here = a.route.logits != nullptr;
  const bool warp_route = routed_here && route_warp_ok(a.route);
  if (routed_here && !warp_route) {
    // general shapes (expert groups, more than 256 experts): the block-wide routine
    __shared__ RouteShared rs;
    int id; float w;
    const bool ok = route_block(a.route, m, rs, id, w);
    if (tid < 32) {
      if (tid < a.n_used) { s_rw.ids[tid] = ok ? id : -3; s_rw.wraw[tid] = w; }
    }
    __syncthreads();
  }
  if (warp == 0) {
    int e;
    if (routed_here) {
      if (warp_route) {
        int id; float w;
        const bool ok = route_warp(a.route, m, s_rw, lane, id, w);
        __syncwarp();
        if (lane < a.n_used) { s_rw.ids[lane] = ok ? id : -3; s_rw.wraw[lane] = w; }
        __syncwarp();
      }
      if (chunk == 0 && j == 0) {
        if (lane == 0 && s_rw.ids[0] == -3) raise_fault(a.fault, a.layer, FS_ROUTER);
        if (lane < a.n_used) {
          const int id = s_rw.ids[lane];
          a.ids[(long)m * a.n_used + lane] = id;
          a.wts[(long)m * a.n_used + lane] = s_rw.wraw[lane];
          if (id >= 0 && a.heat) atomicAdd(a.heat + id, 1u);
        }
      }
      e = s_rw.ids[j];
    } else {
      e = a.ids[(long)m * a.n_used + j];
    }
  if (lane == 0) {
    if (e == kExpertElsewhere) e = -1;
    else if (e < 0 || e >= a.E) { e = -2; if (chunk == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID); }
    else if (a.slot_map) { e = a.slot_map[e]; if (e < 0) e = -1; }
    if (e >= 0) {
      const long row0 = (long)e * a.I + chunk * 32;
      mbar_expect_tx(&bar, 2 * half_bytes);
      bulk_load_chunks(sg, a.gate + row0 * rb, half_bytes, &bar);
      bulk_load_chunks(su, a.up + row0 * rb, half_bytes, &bar);
      if (a.down) {
        // the down launch that follows reads expert e's matrix: this block asks L2 for its 1 / gridDim.x share
        const long share = (a.down_expert_bytes / gridDim.x) & ~15L;
        if (share > 0) bulk_prefetch_l2(a.down + (long)e * a.down_expert_bytes + (long)chunk * share, (uint32_t)share);
      }
    }
    s_e = e;
  }
  }
  probe_mark(a.probe, 2);
  {
    const int layout = staged_layout(a.wtype), nunits = K / 64;
    for (int i = tid; i < K / 16; i += 256)
      reinterpret_cast<uint4*>(sxq)[act_chunk_pos(i, nunits, layout)] = reinterpret_cast<const uint4*>(a.xq + (long)m * K)[i];
    for (int i = tid; i < K / 32; i += 256) sxds[i] = a.xds[(long)m * (K / 32) + i];
  }
  __syncthreads();
  probe_mark(a.probe, 3);
  const int e = s_e;
  const long ob = ((long)m * a.n_used + j) * a.I + chunk * 32;
  bool ok = true;
  if (e >= 0) ok = mbar_wait(&bar, 0, a.fault, a.layer);
  probe_mark(a.probe, 4);
  if (e < 0 || !ok) {
    const bool bad = e == -2 || !ok;                   // a slot served elsewhere contributes zeros; a fault NaN
    if (tid < 32) {
      a.actq[ob + tid] = 0;
      if (a.act_f32) a.act_f32[ob + tid] = bad ? kNaN : 0.f;
    }
    if (tid == 0) a.actds[ob / 32] = bad ? make_float2(kNaN, 0.f) : make_float2(0.f, 0.f);
    return;
  }
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const int r0 = warp * 4 + half * 2;
    const uint8_t* g0 = sg + (long)r0 * rb;
    const uint8_t* u0 = su + (long)r0 * rb;
    float gacc[2], uacc[2];
    switch (a.wtype) {
      case WT_Q4_K: gate_up_rows_staged<Q4K>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q5_K: gate_up_rows_staged<Q5K>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q6_K: gate_up_rows_staged<Q6K>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q8_0: gate_up_rows_staged<Q80>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_NVFP4: gate_up_rows_staged<NvFp4>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_FP8_B128: gate_up_rows_staged<Fp8B128>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q2_K: gate_up_rows_staged<Q2K>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q3_K: gate_up_rows_staged<Q3K>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q4_0: gate_up_rows_staged<Q40>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q4_1: gate_up_rows_staged<Q41>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q5_0: gate_up_rows_staged<Q50>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      case WT_Q5_1: gate_up_rows_staged<Q51>(g0, u0, rb, K, lane, sxq, sxds, gacc, uacc); break;
      default: gacc[0] = gacc[1] = kNaN; uacc[0] = uacc[1] = 0.f;
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float g = gacc[r];
        s_act[r0 + r] = (g / (1.0f + expf(-g))) * uacc[r];
      }
    }
  }
  __syncthreads();
  probe_mark(a.probe, 5);
  if (warp == 0) {
    const float v = s_act[lane];
    float d, s;
    const int8_t q = q8_lane(v, d, s);
    a.actq[ob + lane] = q;
    if (a.act_f32) a.act_f32[ob + lane] = v;
    if (lane == 0) a.actds[ob / 32] = make_float2(d, s);
  }
}

// =======================================================================================================
// down_staged
// =======================================================================================================
struct DownStagedArgs {
  const int8_t* actq; const float2* actds;  // [M, n_used, I]
  const int* ids; const float* wts;         // [M, n_used]
  const int* slot_map;
  const uint8_t* down; int dtype;           // stack [E_slots, H, row_bytes(I)]
  int I, H, E, n_used, M, rows_per_block;
  const float* resid; long resid_stride;
  const float* extra; long extra_stride;
  float* out; long out_stride;
  unsigned* fault; int layer;
  PushOut push;
  long long* probe;
};

template <class T, int UPL>
__device__ __forceinline__ float down_row_staged(const DownStagedArgs& a, const uint8_t* sw, long slot_bytes, int r, int lane,
                                                 const int8_t* sact, const float2* sads, const int* s_slot, const float* s_w) {
  using U = Unit<T>;
  const int upe = a.I / 64;
  const int total = a.n_used * upe;
  const long rb = resident_row_bytes(T::kType, a.I);
  // the rows sit in shared memory: a unit is fetched, dotted and folded into its slot's partial sum at once
  float part[kMaxTopK];
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) part[j] = 0.f;
#pragma unroll
  for (int c = 0; c < UPL; ++c) {
    const int t = lane + 32 * c;
    if (t < total) {
      const int j = t / upe, u = t - j * upe;
      if (s_slot[j] >= 0) {
        typename U::Regs regs;
        U::loadu(sw + (long)j * slot_bytes + (long)r * rb, u, a.I, regs);
        ActRegs act;
        const long ab = (long)j * a.I;
        StagedAct<T>::load(sact + ab, sads + ab / 32, u, upe, act);
        const float v = ActOf<T>::dot(regs, u, act);
#pragma unroll
        for (int q = 0; q < kMaxTopK; ++q) if (q == j) part[q] += v;
      }
    }
  }
  float y = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxTopK; ++j) {
    if (j < a.n_used) y = fmaf(s_w[j], part[j], y);
  }
  return warp_sum(y);
}

// grid (ceil(H / rows_per_block), M), 256 threads; rows_per_block <= 32: warp w owns rows w, w + 8, ...
template <int UPL, int FAM>
__global__ void __launch_bounds__(256, 2) down_staged_kernel(const DownStagedArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int s_slot[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  __shared__ float s_y[32];
  __shared__ int s_nvalid;
  const int m = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int d0 = blockIdx.x * a.rows_per_block;
  const int nrows = min(a.rows_per_block, a.H - d0);
  const long rb = resident_row_bytes(a.dtype, a.I);
  const long slot_bytes = (long)a.rows_per_block * rb;
  uint8_t* sw = smem;                                                       // [n_used][rows_per_block][rb]
  int8_t* sact = reinterpret_cast<int8_t*>(smem + (size_t)a.n_used * slot_bytes);   // [n_used][I]
  float2* sads = reinterpret_cast<float2*>(sact + (size_t)a.n_used * a.I);  // [n_used][I / 32]
  probe_mark(a.probe, 0);
  if (tid == 0) mbar_init(&bar, 1);
  __syncthreads();
  pdl_wait();
  pdl_launch();
  probe_mark(a.probe, 1);
  if (tid == 0) {
    int nvalid = 0;
    bool bad = false;
    for (int j = 0; j < a.n_used; ++j) {
      int e = a.ids[(long)m * a.n_used + j];
      if (e == kExpertElsewhere) e = -1;
      else if (e < 0 || e >= a.E) { e = -2; bad = true; }
      else if (a.slot_map) { e = a.slot_map[e]; if (e < 0) e = -1; }
      s_slot[j] = e;
      s_w[j] = a.wts[(long)m * a.n_used + j];
      nvalid += e >= 0 ? 1 : 0;
    }
    if (nvalid) {
      mbar_expect_tx(&bar, (uint32_t)(nvalid * nrows * rb));
      for (int j = 0; j < a.n_used; ++j)
        if (s_slot[j] >= 0)
          bulk_load_chunks(sw + (long)j * slot_bytes, a.down + ((long)s_slot[j] * a.H + d0) * rb, (uint32_t)(nrows * rb), &bar);
    }
    s_nvalid = bad ? -1 : nvalid;
    if (bad && blockIdx.x == 0) raise_fault(a.fault, a.layer, FS_EXPERT_ID);
  }
  {
    const long ab = (long)m * a.n_used * a.I;
    const int cps = a.I / 16, upe = a.I / 64, layout = staged_layout(a.dtype);      // chunks and units per slot row
    for (int i = tid; i < a.n_used * cps; i += 256) {
      const int j = i / cps, c = i - j * cps;
      reinterpret_cast<uint4*>(sact)[j * cps + act_chunk_pos(c, upe, layout)] = reinterpret_cast<const uint4*>(a.actq + ab)[i];
    }
    for (int i = tid; i < a.n_used * a.I / 32; i += 256) sads[i] = a.actds[ab / 32 + i];
  }
  __syncthreads();
  probe_mark(a.probe, 2);
  const int nvalid = s_nvalid;
  bool ok = nvalid >= 0;
  if (nvalid > 0) ok = mbar_wait(&bar, 0, a.fault, a.layer) && ok;
  probe_mark(a.probe, 3);
  for (int r = warp; r < nrows; r += 8) {
    float y;
    if constexpr (FAM == 0) {
    switch (a.dtype) {
      case WT_Q4_K: y = down_row_staged<Q4K, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q6_K: y = down_row_staged<Q6K, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q5_K: y = down_row_staged<Q5K, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q8_0: y = down_row_staged<Q80, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      default: y = kNaN;
    }
    } else {
    switch (a.dtype) {
      case WT_NVFP4: y = down_row_staged<NvFp4, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_FP8_B128: y = down_row_staged<Fp8B128, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q2_K: y = down_row_staged<Q2K, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q3_K: y = down_row_staged<Q3K, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q4_0: y = down_row_staged<Q40, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q4_1: y = down_row_staged<Q41, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q5_0: y = down_row_staged<Q50, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      case WT_Q5_1: y = down_row_staged<Q51, UPL>(a, sw, slot_bytes, r, lane, sact, sads, s_slot, s_w); break;
      default: y = kNaN;
    }
    }
    if (lane == 0) s_y[r] = ok ? y : kNaN;
  }
  __syncthreads();
  probe_mark(a.probe, 4);
  if (tid < nrows) {
    const int d = d0 + tid;
    float y = s_y[tid];
    if (a.extra) y += a.extra[(long)m * a.extra_stride + d];
    if (a.push.n_ranks > 0) {
      push_store(a.push, site_epoch(a.push.step, a.push.sites_per_step, a.push.site_index), (long)m * a.out_stride + d, y);
    } else {
      if (a.resid) y += a.resid[(long)m * a.resid_stride + d];
      a.out[(long)m * a.out_stride + d] = y;
    }
  }
}

int g_stage_dbg = 0;
long long* g_stage_probe = nullptr;

static bool staged_type(int t) {
  return t == WT_Q4_K || t == WT_Q5_K || t == WT_Q6_K || t == WT_Q8_0 || t == WT_NVFP4 || t == WT_FP8_B128 || t == WT_Q2_K ||
         t == WT_Q3_K || t == WT_Q4_0 || t == WT_Q4_1 || t == WT_Q5_0 || t == WT_Q5_1;
}

static int staged_fam(int t) { return (t == WT_Q4_K || t == WT_Q5_K || t == WT_Q6_K || t == WT_Q8_0) ? 0 : 2; }

constexpr size_t kStagedSmemMax = 200 * 1024;
constexpr size_t kStagedSliceMax = 100 * 1024;   // a block's weight rows (two such kernels fit one SM side by side)

template <int MB, bool NORM, int FAM>
static cudaError_t gemv_staged_launch(const GemvArgs& a, int grid, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemv_staged_kernel<MB, NORM, FAM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    attr_set = true;
  }
  return launch(gemv_staged_kernel<MB, NORM, FAM>, dim3(grid), dim3(256), smem, st, a);
}

template <bool NORM, int FAM>
static cudaError_t gemv_staged_dispatch(const GemvArgs& a, int mb, int grid, size_t smem, cudaStream_t st) {
  switch (mb) {
    case 1: return gemv_staged_launch<1, NORM, FAM>(a, grid, smem, st);
    case 2: return gemv_staged_launch<2, NORM, FAM>(a, grid, smem, st);
    case 4: return gemv_staged_launch<4, NORM, FAM>(a, grid, smem, st);
    default: return gemv_staged_launch<8, NORM, FAM>(a, grid, smem, st);
  }
}

template <int HEAD, int HPW>
static int attn_cluster_launch(const AttnArgs& a, int CL, int n_kv, int M, size_t smem, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(attn_cluster_kernel<HEAD, HPW>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    cudaFuncSetAttribute(attn_cluster_kernel<HEAD, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CL, n_kv, M);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, attn_cluster_kernel<HEAD, HPW>, a);
}

}  // namespace bl

using namespace bl;

extern "C" {

// Timing experiments on the staged GEMV (kernel_bench --dbg N): 1 = release the dependents first instead of after
// the wait, 2 = skip the dot products, 4 = skip the bulk copy, 8 = skip the activation prologue.  0 in normal use.
void bl_set_stage_debug(int flags) { bl::g_stage_dbg = flags; }
// Arms (device pointer to 16 int64 words) or disarms (null) the phase probe of the attention / expert launches.
void bl_set_stage_probe(long long* words) { bl::g_stage_probe = words; }

// Same contract as bl_gemv for quantised weight rows.  Returns BL_ERR_LIMIT (and launches nothing) when the
// weight rows of one block would not fit the shared-memory stage: the caller then uses bl_gemv.
int bl_gemv_staged(int nseg, const void* const* w, const int* rows, const int* wtypes, int K, int M,
                   int norm, const float* x, long x_stride, const float* gain, float eps,
                   const int8_t* xq, const float* xds,
                   float* out, long out_stride, const float* resid, long resid_stride,
                   const void* red_desc, const void* push_desc, unsigned* fault, int layer, int sm_count, cudaStream_t st) {
  BL_REQUIRE(nseg >= 1 && nseg <= 4, BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && M <= 8, BL_ERR_SHAPE);
  BL_REQUIRE(K > 0 && K % 256 == 0, BL_ERR_SHAPE);
  GemvArgs a = {};
  a.nseg = nseg;
  double total_bytes = 0;
  long rbs[4];
  const int fam = staged_fam(wtypes[0]);
  for (int s = 0; s < nseg; ++s) {
    BL_REQUIRE(staged_type(wtypes[s]) && staged_fam(wtypes[s]) == fam, BL_ERR_TYPE);   // one family per call
    rbs[s] = resident_row_bytes(wtypes[s], K);
    BL_REQUIRE(rbs[s] > 0 && rbs[s] % 16 == 0, BL_ERR_TYPE);
    BL_REQUIRE(((uintptr_t)w[s] & 15) == 0, BL_ERR_ALIGN);
    BL_REQUIRE(rows[s] >= 1, BL_ERR_SHAPE);
    total_bytes += (double)rows[s] * rbs[s];
  }
  const int mb = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  // one block per SM when the slices fit, two otherwise; each segment gets blocks in proportion to its bytes
  int budget = sm_count;
  if (total_bytes / budget > (double)kStagedSliceMax * 0.9) budget = 2 * sm_count;
  int grid = 0, rpb_max = 1;
  size_t slice_max = 0;
  for (int s = 0; s < nseg; ++s) {
    int nb = (int)((double)budget * ((double)rows[s] * rbs[s] / total_bytes));
    nb = nb < 1 ? 1 : nb > rows[s] ? rows[s] : nb;
    a.seg[s] = GemvSeg{(const uint8_t*)w[s], rows[s], wtypes[s], grid, nb, rbs[s]};
    grid += nb;
    const int rpb = (rows[s] + nb - 1) / nb;
    rpb_max = rpb > rpb_max ? rpb : rpb_max;
    const size_t sl = (size_t)rpb * rbs[s];
    slice_max = sl > slice_max ? sl : slice_max;
  }
  BL_REQUIRE(slice_max <= kStagedSliceMax, BL_ERR_LIMIT);
  a.stage_bytes = (int)((slice_max + 127) / 128 * 128);
  a.rpb_max = rpb_max;
  const size_t smem = (size_t)a.stage_bytes + (size_t)mb * K + (size_t)mb * (K / 32) * 8 + mb * 8 * 8 + 8 * 4 +
                      (size_t)mb * rpb_max * 4 + 16;
  BL_REQUIRE(smem <= kStagedSmemMax, BL_ERR_LIMIT);
  a.K = K; a.M = M;
  a.x = x; a.x_stride = x_stride; a.gain = gain; a.eps = eps;
  a.xq = xq; a.xds = (const float2*)xds;
  a.out = out; a.out_stride = out_stride; a.resid = resid; a.resid_stride = resid_stride;
  a.fault = fault; a.layer = layer;
  a.dbg = g_stage_dbg;
  if (red_desc) { a.red = *(const ReduceIn*)red_desc; BL_REQUIRE(norm && a.red.n_ranks <= kMaxRanks && a.red.H == K, BL_ERR_SHAPE); }
  if (push_desc) { a.push = *(const PushOut*)push_desc; BL_REQUIRE(a.push.n_ranks <= kMaxRanks, BL_ERR_SHAPE); }
  cudaError_t e;
  if (fam == 0) e = norm ? gemv_staged_dispatch<true, 0>(a, mb, grid, smem, st) : gemv_staged_dispatch<false, 0>(a, mb, grid, smem, st);
  else e = norm ? gemv_staged_dispatch<true, 2>(a, mb, grid, smem, st) : gemv_staged_dispatch<false, 2>(a, mb, grid, smem, st);
  return (int)e;
}

// Per-head RMSNorm + RoPE + KV append + flash decode + merge in one launch.  Scratch: part_ml [M*n_q*n_seg*2],
// part_acc [M*n_q*n_seg*head] floats and tickets [M*n_kv] words that are zero when the call begins (the kernel
// leaves them zero).
int bl_attn_fused(const float* qkv, long qkv_stride, const float* q_gain, const float* k_gain, const float* inv_freq,
                  float eps, float q_scale, int head, int n_q, int n_kv, int M, const int* row_pos, const int* row_seq,
                  const int* block_table, int max_pages, int n_pages, void* k_cache, void* v_cache, int n_seg,
                  int ctx_limit, float* part_ml, float* part_acc, unsigned* tickets, float* out, int8_t* outq,
                  float* outds, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(head == 128 || head == 64, BL_ERR_SHAPE);
  BL_REQUIRE(n_kv >= 1 && n_q % n_kv == 0 && n_q / n_kv <= 16, BL_ERR_SHAPE);
  BL_REQUIRE(n_seg >= 1 && M >= 1 && max_pages >= 1 && (long)ctx_limit <= (long)max_pages * kPage, BL_ERR_SHAPE);
  const int G = n_q / n_kv;
  AttnArgs a{qkv, qkv_stride, q_gain, k_gain, inv_freq, eps, q_scale, n_q, n_kv, M, n_seg, ctx_limit, row_pos, row_seq,
             block_table, max_pages, n_pages, (__half*)k_cache, (__half*)v_cache, part_ml, part_acc, tickets, out, outq,
             (float2*)outds, fault, layer, g_stage_probe, 0};
  dim3 grid(n_seg, n_kv, M);
  const int n_patch = M < kMaxPatch ? M : kMaxPatch;
  const size_t smem = (size_t)G * head * 4 + kStages * kKeyTile * (head + 8) * 2 + kStages * kKeyTile * head * 2 + (size_t)n_patch * 2 * head * 2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(attn_fused_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    cudaFuncSetAttribute(attn_fused_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    cudaFuncSetAttribute(attn_fused_kernel<64, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    cudaFuncSetAttribute(attn_fused_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    attr_set = true;
  }
  cudaError_t e;
  if (head == 128) e = G <= 8 ? launch(attn_fused_kernel<128, 1>, grid, dim3(256), smem, st, a) : launch(attn_fused_kernel<128, 2>, grid, dim3(256), smem, st, a);
  else e = G <= 8 ? launch(attn_fused_kernel<64, 1>, grid, dim3(256), smem, st, a) : launch(attn_fused_kernel<64, 2>, grid, dim3(256), smem, st, a);
  return (int)e;
}

// route_logits != null: every block routes its row from the logits (block (0, 0, m) writes ids / wts / heat);
// otherwise ids are read as given.
// bl_attn_fused with the key segments of a (row, KV head) spread over a thread-block cluster of `cluster` CTAs
// (8 or 16) that merge through distributed shared memory: no scratch, no tickets.
int bl_attn_cluster(const float* qkv, long qkv_stride, const float* q_gain, const float* k_gain, const float* inv_freq,
                    float eps, float q_scale, int head, int n_q, int n_kv, int M, const int* row_pos, const int* row_seq,
                    const int* block_table, int max_pages, int n_pages, void* k_cache, void* v_cache, int cluster,
                    int ctx_limit, float* out, int8_t* outq, float* outds, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(head == 128 || head == 64, BL_ERR_SHAPE);
  BL_REQUIRE(n_kv >= 1 && n_q % n_kv == 0 && n_q / n_kv <= 16, BL_ERR_SHAPE);
  BL_REQUIRE((cluster == 8 || cluster == 16) && M >= 1 && max_pages >= 1 && (long)ctx_limit <= (long)max_pages * kPage, BL_ERR_SHAPE);
  const int G = n_q / n_kv;
  const int n_patch = M < kMaxPatch ? M : kMaxPatch;
  size_t base = (size_t)G * head * 4 + kStages * kKeyTile * (head + 8) * 2 + kStages * kKeyTile * head * 2 + (size_t)n_patch * 2 * head * 2;
  base = (base + 15) / 16 * 16;
  const int heads_here = (G + cluster - 1) / cluster;
  const size_t smem = base + (size_t)heads_here * cluster * (head + 4) * 4;
  BL_REQUIRE(smem <= 110 * 1024, BL_ERR_LIMIT);
  AttnArgs a{qkv, qkv_stride, q_gain, k_gain, inv_freq, eps, q_scale, n_q, n_kv, M, cluster, ctx_limit, row_pos, row_seq,
             block_table, max_pages, n_pages, (__half*)k_cache, (__half*)v_cache, nullptr, nullptr, nullptr, out, outq,
             (float2*)outds, fault, layer, g_stage_probe, (int)(base / 4)};
  if (head == 128) return G <= 8 ? attn_cluster_launch<128, 1>(a, cluster, n_kv, M, smem, st) : attn_cluster_launch<128, 2>(a, cluster, n_kv, M, smem, st);
  return G <= 8 ? attn_cluster_launch<64, 1>(a, cluster, n_kv, M, smem, st) : attn_cluster_launch<64, 2>(a, cluster, n_kv, M, smem, st);
}

int bl_gate_up_staged(const int8_t* xq, const float* xds, const float* route_logits, const float* bias, int mode, int renorm,
                      float scale, int n_group, int topk_group, int* ids, float* wts, unsigned* heat, const int* slot_map,
                      const void* gate, const void* up, int wtype, const void* down, long down_expert_bytes, int K, int I, int E,
                      int n_used, int M, int8_t* actq, float* actds, float* act_f32, unsigned* fault, int layer, cudaStream_t st) {
  BL_REQUIRE(K % 256 == 0 && I % 32 == 0 && M >= 1 && n_used >= 1 && n_used <= kMaxTopK, BL_ERR_SHAPE);
  BL_REQUIRE(staged_type(wtype), BL_ERR_TYPE);
  const long rb = resident_row_bytes(wtype, K);
  BL_REQUIRE(rb > 0 && rb % 16 == 0, BL_ERR_TYPE);
  const size_t smem = (size_t)64 * rb + K + (size_t)(K / 32) * 8 + 16;
  BL_REQUIRE(smem <= kStagedSmemMax && 64 * rb < (1 << 20), BL_ERR_LIMIT);
  BL_REQUIRE(((uintptr_t)gate & 15) == 0 && ((uintptr_t)up & 15) == 0 && ((uintptr_t)down & 15) == 0 && down_expert_bytes % 16 == 0, BL_ERR_ALIGN);
  if (route_logits) {
    BL_REQUIRE(E % 4 == 0 && E <= kMaxExperts && n_group >= 1 && n_group <= 16 && E % n_group == 0 && topk_group >= 1 &&
               topk_group <= n_group && wts, BL_ERR_LIMIT);
  }
  GateUpStagedArgs a{xq, (const float2*)xds, RouteParams{route_logits, bias, E, n_used, mode, renorm, scale, n_group, topk_group},
                     ids, wts, heat, slot_map, (const uint8_t*)gate, (const uint8_t*)up, wtype,
                     (const uint8_t*)down, down_expert_bytes, K, I, E, n_used, M, actq, (float2*)actds, act_f32, fault, layer, g_stage_probe};
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gate_up_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    attr_set = true;
  }
  return (int)launch(gate_up_staged_kernel, dim3(I / 32, n_used, M), dim3(256), smem, st, a);
}

int bl_down_staged(const int8_t* actq, const float* actds, const int* ids, const float* wts, const int* slot_map,
                   const void* down, int dtype, int I, int H, int E, int n_used, int M, const float* resid,
                   long resid_stride, const float* extra, long extra_stride, float* out, long out_stride,
                   const void* push_desc, unsigned* fault, int layer, int sm_count, cudaStream_t st) {
  BL_REQUIRE(staged_type(dtype), BL_ERR_TYPE);
  BL_REQUIRE(I % 256 == 0 || ((dtype == WT_Q8_0 || dtype == WT_NVFP4 || dtype == WT_Q4_0 || dtype == WT_Q4_1 || dtype == WT_Q5_0 || dtype == WT_Q5_1) && I % 64 == 0) ||
             (dtype == WT_FP8_B128 && I % 128 == 0), BL_ERR_SHAPE);
  BL_REQUIRE(M >= 1 && n_used >= 1 && n_used <= kMaxTopK && H >= 1, BL_ERR_SHAPE);
  const long rb = resident_row_bytes(dtype, I);
  BL_REQUIRE(rb > 0 && rb % 16 == 0 && ((uintptr_t)down & 15) == 0, BL_ERR_ALIGN);
  const long total = (long)n_used * (I / 64);
  BL_REQUIRE(total <= 512, BL_ERR_LIMIT);
  // rows per block: one block per SM where the stage allows it, at most 32 rows (4 per warp)
  int rpb = (H + sm_count - 1) / sm_count;
  rpb = rpb < 8 ? 8 : rpb > 32 ? 32 : rpb;
  while (rpb > 1 && (size_t)n_used * rpb * rb > kStagedSliceMax) --rpb;
  const size_t smem = (size_t)n_used * rpb * rb + (size_t)n_used * I + (size_t)n_used * (I / 32) * 8 + 16;
  BL_REQUIRE(smem <= kStagedSmemMax && (size_t)n_used * rpb * rb < (1 << 20), BL_ERR_LIMIT);
  DownStagedArgs a{actq, (const float2*)actds, ids, wts, slot_map, (const uint8_t*)down, dtype, I, H, E, n_used, M, rpb,
                   resid, resid_stride, extra, extra_stride, out, out_stride, fault, layer, PushOut{}, g_stage_probe};
  if (push_desc) { a.push = *(const PushOut*)push_desc; BL_REQUIRE(a.push.n_ranks <= kMaxRanks && M <= kMaxRows, BL_ERR_SHAPE); }
  dim3 grid((H + rpb - 1) / rpb, M);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(down_staged_kernel<3, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    cudaFuncSetAttribute(down_staged_kernel<6, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    cudaFuncSetAttribute(down_staged_kernel<16, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    cudaFuncSetAttribute(down_staged_kernel<3, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    cudaFuncSetAttribute(down_staged_kernel<6, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    cudaFuncSetAttribute(down_staged_kernel<16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kStagedSmemMax);
    attr_set = true;
  }
  if (staged_fam(dtype) == 0) {
    if (total <= 96) return (int)launch(down_staged_kernel<3, 0>, grid, dim3(256), smem, st, a);
    if (total <= 192) return (int)launch(down_staged_kernel<6, 0>, grid, dim3(256), smem, st, a);
    return (int)launch(down_staged_kernel<16, 0>, grid, dim3(256), smem, st, a);
  }
  if (total <= 96) return (int)launch(down_staged_kernel<3, 2>, grid, dim3(256), smem, st, a);
  if (total <= 192) return (int)launch(down_staged_kernel<6, 2>, grid, dim3(256), smem, st, a);
  return (int)launch(down_staged_kernel<16, 2>, grid, dim3(256), smem, st, a);
}

}  // extern "C"
