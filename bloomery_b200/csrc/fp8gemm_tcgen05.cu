// Block-scaled FP8 grouped GEMM on tcgen05 (sm_100a only): both operands stay E4M3 all the way into the tensor cores.
//   C[t, n] = sum over 128-wide K blocks kb of  xs[t, kb] * ws[n, kb] * sum_k Xq[t, k] * Wq[g][n, k]
//   Wq: resident FP8_B128 rows (K E4M3 codes, then K / 128 f32 scales per row: the checkpoint's 128 x 128 block scale
//       repeated on each row), Xq / xs: E4M3 codes and 1 x 128 scales of the activations (fp8_rows_kernel below).
//
// The decode-batch shape: the 128 weight rows of a tile are the M side of the MMA, 32 tokens the N side.  Nothing is
// expanded: one TMA thread streams [128 rows x 128 bytes] boxes of the weight codes (128-byte swizzle) and the
// [32 tokens x 128 bytes] box of the activation codes into a ring of stages, one elected thread issues four
// tcgen05.mma kind::f8f6f4 (M 128, N 32, K 32) per stage into one of four partial accumulators in TMEM, and four
// epilogue warps (lane = weight row) read each partial back with tcgen05.ld and add it into fp32 registers with the
// block's two scales -- the promotion every 128 values that block-scaled FP8 needs for accuracy.  A pass over the
// weights is therefore bound by HBM, not by expander warps (csrc/qgemm_tcgen05.cu expands FP8 to bf16 in eight producer
// warps and reaches about a quarter of the copy bandwidth at this shape).
//   * "dual" mode runs gate and up in one main loop; the epilogue writes silu(gate) * up;
//   * the epilogue scatters and scales like the other GEMMs (dst_row / row_scale / resid).
// Every mbarrier wait is bounded by the global timer; on expiry the CTA raises status word 1, leaves its loops, frees
// its TMEM and returns.
//
// Role in the reference: none on this path (its FP8 experts run on q8 activations through mma.sync,
// crates/gpu/src/gemm/gemm32.rs); the scheme is the checkpoint's own (128 x 128 weight blocks, 1 x 128 activation
// scales, E4M3).
#include <cuda_fp8.h>

#include "tc_common.cuh"

namespace bl {

constexpr int F8_BM = 128, F8_BN = 32, F8_BK = 128;
constexpr int F8_A_BYTES = F8_BM * F8_BK;            // one matrix's stage: 128 rows x 128 bytes
constexpr int F8_B_BYTES = F8_BN * F8_BK;
constexpr int F8_THREADS = 192;                       // warp 0 TMA, warp 1 MMA + TMEM, warps 2..5 epilogue
constexpr int F8_MAX_STAGES = 8, F8_PARTS = 4;

struct F8Tile { int group, row0, row_end, pad; };   // token tile (the TileTable's rows)

struct F8Args {
  const uint8_t* w;           // [n_groups][N rows][row_bytes]
  const uint8_t* w2;
  long row_bytes, group_bytes;
  int N, K, tiles_w, stages;
  const F8Tile* tiles;
  const int* n_tiles;
  int max_tiles;
  const float* xs;            // [rows_x][K / 128] activation scales
  float* c_f32;
  __nv_bfloat16* c_bf16;
  long ldc;
  const int* dst_row;
  const float* row_scale;
  const float* resid;
  long ldr;
  unsigned* status;
};

// kind::f8f6f4 instruction descriptor: D = f32, A = B = E4M3, both K-major, M x N tile
__host__ __device__ constexpr uint32_t f8_idesc(int m, int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

template <bool DUAL>
__global__ void __launch_bounds__(F8_THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
                const __grid_constant__ CUtensorMap tma_w2, const F8Args a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * F8_A_BYTES + F8_B_BYTES;
  constexpr int B_OFF = (DUAL ? 2 : 1) * F8_A_BYTES;
  constexpr int ACC_COLS = (DUAL ? 2 : 1) * F8_BN;
  constexpr int TMEM_COLS = F8_PARTS * ACC_COLS;                     // 128 or 256 columns
  __shared__ __align__(8) uint64_t full_bar[F8_MAX_STAGES], empty_bar[F8_MAX_STAGES], part_full[F8_PARTS], part_empty[F8_PARTS];
  __shared__ __align__(8) uint64_t xs_ready, xs_done;                // the epilogue threads' own meeting points (bounded)
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int STAGES = a.stages;
  float* s_xs = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE_BYTES);     // [K / 128][32 tokens]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < F8_PARTS; ++b) { mbar_init(&part_full[b], 1); mbar_init(&part_empty[b], 4); }
    mbar_init(&xs_ready, 128); mbar_init(&xs_done, 128);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  const int n_tt = min(*a.n_tiles, a.max_tiles);
  const int total_tiles = n_tt * a.tiles_w;
  const int kblocks = a.K / F8_BK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int issued = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const F8Tile mt = a.tiles[t / a.tiles_w];
        const int n0 = (t % a.tiles_w) * F8_BM;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) break;
          uint8_t* s = smem + (size_t)stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          // rows past the matrix (and token rows past the activations) arrive as zeros and are never stored
          tma_load_3d(s, &tma_w, kb * F8_BK, n0, mt.group, &full_bar[stage]);
          if (DUAL) tma_load_3d(s + F8_A_BYTES, &tma_w2, kb * F8_BK, n0, mt.group, &full_bar[stage]);
          tma_load_2d(s + B_OFF, &tma_x, kb * F8_BK, mt.row0, &full_bar[stage]);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {
        // copies of this thread may still be landing in shared memory: the CTA must not exit under them
        unsigned long long t0 = globaltimer();
        while (issued > 0 && globaltimer() - t0 < 2000000ull) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = f8_idesc(F8_BM, F8_BN);
      int stage = 0; uint32_t phase = 0;
      uint32_t part = 0, pphase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok && !*abort_flag; t += gridDim.x) {
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&part_empty[part], pphase ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
          const uint32_t d0 = tmem_base + part * ACC_COLS;
          const uint64_t da = umma_desc(sa), db = umma_desc(sa + B_OFF);
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k) {                     // K = 32 codes = 32 bytes per instruction
            const uint64_t step = (uint64_t)(k * 32 / 16);
            umma_f8(d0, da + step, db + step, idesc, k > 0 ? 1u : 0u);
            if (DUAL) umma_f8(d0 + F8_BN, umma_desc(sa + F8_A_BYTES) + step, db + step, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          umma_commit(&part_full[part]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++part == F8_PARTS) { part = 0; pphase ^= 1; }
        }
      }
    }
  } else {
    const int q = warp & 3;                                          // TMEM lane quarter of this warp
    const int et = threadIdx.x - 64;                                 // 0 .. 127 among the epilogue threads
    uint32_t part = 0, pphase = 0;
    bool ok = true;
    int ti = 0;
    for (int t = blockIdx.x; t < total_tiles && ok && !*abort_flag; t += gridDim.x, ++ti) {
      const F8Tile mt = a.tiles[t / a.tiles_w];
      const int n = (t % a.tiles_w) * F8_BM + q * 32 + lane;         // weight row = output column of this thread
      const bool n_ok = n < a.N;
      const long wrow = (long)mt.group * a.group_bytes + (long)(n_ok ? n : a.N - 1) * a.row_bytes + a.K;
      const float* ws = reinterpret_cast<const float*>(a.w + wrow);
      const float* ws2 = DUAL ? reinterpret_cast<const float*>(a.w2 + wrow) : nullptr;
      // the row's scales, four K blocks per 16-byte load, fetched four blocks ahead of their use (the scale strip of a
      // row is padded to 16 bytes, so the last load stays inside the row)
      const float4* ws4 = reinterpret_cast<const float4*>(ws);
      const float4* ws24 = reinterpret_cast<const float4*>(ws2);
      float4 w_cur = ws4[0], w_nxt = w_cur, w2_cur = DUAL ? ws24[0] : make_float4(0.f, 0.f, 0.f, 0.f), w2_nxt = w2_cur;
      // the activation scales of this tile's 32 tokens, [kb][token]; rows past the tile scale by zero
      if (ti > 0 && !mbar_wait(&xs_done, (uint32_t)(ti - 1) & 1u, abort_flag)) break;   // the previous tile's readers are done
      for (int i = et; i < kblocks * F8_BN; i += 128) {
        const int kb = i >> 5, tok = i & 31;
        const int r = mt.row0 + tok;
        s_xs[i] = r < mt.row_end ? a.xs[(long)r * kblocks + kb] : 0.0f;
      }
      mbar_arrive(&xs_ready);
      if (!mbar_wait(&xs_ready, (uint32_t)ti & 1u, abort_flag)) break;
      float acc[F8_BN], acc2[DUAL ? F8_BN : 1];
#pragma unroll
      for (int i = 0; i < F8_BN; ++i) { acc[i] = 0.0f; if (DUAL) acc2[i] = 0.0f; }
      for (int kb = 0; kb < kblocks; ++kb) {
        const int j = kb & 3;
        if (j == 0) {
          if (kb > 0) { w_cur = w_nxt; if (DUAL) w2_cur = w2_nxt; }
          if (kb + 4 < kblocks) { w_nxt = ws4[(kb >> 2) + 1]; if (DUAL) w2_nxt = ws24[(kb >> 2) + 1]; }
        }
        const float wsc = j == 0 ? w_cur.x : j == 1 ? w_cur.y : j == 2 ? w_cur.z : w_cur.w;
        const float wsc2 = j == 0 ? w2_cur.x : j == 1 ? w2_cur.y : j == 2 ? w2_cur.z : w2_cur.w;
        if (!mbar_wait(&part_full[part], pphase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + part * ACC_COLS;
        uint32_t v[32], u[32];
        tmem_ld32(tbase, v);
        if (DUAL) tmem_ld32(tbase + F8_BN, u);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[part]);
        if (++part == F8_PARTS) { part = 0; pphase ^= 1; }
        const float4* xs4 = reinterpret_cast<const float4*>(s_xs + kb * F8_BN);
#pragma unroll
        for (int i4 = 0; i4 < F8_BN / 4; ++i4) {
          const float4 x = xs4[i4];
          const float xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = 4 * i4 + j;
            acc[i] = fmaf(__uint_as_float(v[i]) * wsc, xv[j], acc[i]);
            if (DUAL) acc2[i] = fmaf(__uint_as_float(u[i]) * wsc2, xv[j], acc2[i]);
          }
        }
      }
      if (!ok) break;
      mbar_arrive(&xs_done);
      // lane i fetches the routing of token row i of this tile; the store loop broadcasts it
      const int r_l = mt.row0 + lane;
      int orow_l = -1;
      float sc_l = 1.0f;
      if (r_l < mt.row_end) {
        orow_l = a.dst_row ? a.dst_row[r_l] : r_l;
        if (a.row_scale) sc_l = a.row_scale[r_l];
      }
#pragma unroll
      for (int i = 0; i < F8_BN; ++i) {
        const int orow = __shfl_sync(0xFFFFFFFFu, orow_l, i);
        const float sc = __shfl_sync(0xFFFFFFFFu, sc_l, i);
        if (orow < 0 || !n_ok) continue;
        float f = acc[i];
        if (DUAL) f = (f / (1.0f + __expf(-f))) * acc2[i];
        f *= sc;
        if (a.resid) f += a.resid[(long)orow * a.ldr + n];
        if (a.c_f32) a.c_f32[(long)orow * a.ldc + n] = f;
        else a.c_bf16[(long)orow * a.ldc + n] = __float2bfloat16_rn(f);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && a.status) atomicMax(a.status, 1u);
}

// One warp per (row, 128-value block): amax over the block, scale = amax / 448, E4M3 codes of x / scale (round to
// nearest even, saturating).  gain != null: the rows are RMS-normalised first (x fp32), so the norm in front of a
// product and the quantisation of its input are one launch.
struct F8RowsArgs {
  const void* x; int x_f32; long ldx; const float* gain; float eps; int M, K;
  uint8_t* codes; long ldc; float* scales;
};

__global__ void __launch_bounds__(256) fp8_rows_kernel(const F8RowsArgs a) {
  __shared__ float s_red[8];
  __shared__ float s_rms;
  pdl_wait();
  pdl_launch();
  const int m = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = a.K / 128;
  float rms = 1.0f;
  if (a.gain) {
    const float* xr = reinterpret_cast<const float*>(a.x) + (long)m * a.ldx;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < a.K; i += 256) { const float v = xr[i]; ss = fmaf(v, v, ss); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.0f;
      for (int i = 0; i < 8; ++i) tot += s_red[i];
      s_rms = rsqrtf(tot / (float)a.K + a.eps);
    }
    __syncthreads();
    rms = s_rms;
  }
  for (int kb = warp; kb < kblocks; kb += 8) {
    float v[4];
    const long base = (long)m * a.ldx + kb * 128 + 4 * lane;
    if (a.x_f32) {
      const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) + base);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
      const uint2 p = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.x) + base);
      const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&p.x), p1 = *reinterpret_cast<const __nv_bfloat162*>(&p.y);
      v[0] = __low2float(p0); v[1] = __high2float(p0); v[2] = __low2float(p1); v[3] = __high2float(p1);
    }
    if (a.gain) {
      const float4 g = *reinterpret_cast<const float4*>(a.gain + kb * 128 + 4 * lane);
      v[0] *= rms * g.x; v[1] *= rms * g.y; v[2] *= rms * g.z; v[3] *= rms * g.w;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float scale = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(a.codes + (long)m * a.ldc + kb * 128 + 4 * lane) = (uint32_t)lo | ((uint32_t)hi << 16);
    if (lane == 0) a.scales[(long)m * kblocks + kb] = scale;
  }
}

template <bool DUAL>
static int fp8_gemm_go(const CUtensorMap& mx, const F8Args& a0, int n_groups, int grid, cudaStream_t st) {
  constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * F8_A_BYTES + F8_B_BYTES;
  F8Args a = a0;
  const int xs_bytes = (a.K / F8_BK) * F8_BN * 4;
  int stages = (220 * 1024 - xs_bytes) / STAGE_BYTES;
  a.stages = stages > F8_MAX_STAGES ? F8_MAX_STAGES : stages;
  if (a.stages < 2) return BL_ERR_SHAPE;
  const size_t smem = (size_t)a.stages * STAGE_BYTES + xs_bytes + 1024;
  CUtensorMap mw, mw2;
  cuuint64_t dims[3] = {(cuuint64_t)a.row_bytes, (cuuint64_t)a.N, (cuuint64_t)n_groups};
  cuuint64_t str[2] = {(cuuint64_t)a.row_bytes, (cuuint64_t)a.group_bytes};
  cuuint32_t box[3] = {F8_BK, F8_BM, 1};
  int rc = make_map_any(&mw, a.w, 3, dims, str, box, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  mw2 = mw;
  if (DUAL) { rc = make_map_any(&mw2, a.w2, 3, dims, str, box, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_128B); if (rc) return rc; }
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(fp8_gemm_kernel<DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
    set = true;
  }
  return (int)launch(fp8_gemm_kernel<DUAL>, dim3(grid), dim3(F8_THREADS), smem, st, mx, mw, mw2, a);
}

}  // namespace bl

using namespace bl;

extern "C" {

// E4M3 codes and 1 x 128 scales of M activation rows.  x: bf16 (x_f32 = 0) or fp32 rows of ldx elements; gain != null
// (fp32 rows only): RMSNorm with that gain first.  codes [M, ldc bytes], scales [M, K / 128].
int bl_fp8_rows(const void* x, int x_f32, long ldx, const float* gain, float eps, int M, int K, void* codes, long ldc,
                float* scales, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && K >= 128 && K % 128 == 0 && ldx % 4 == 0 && ldc % 16 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)codes & 15) == 0 && ((uintptr_t)gain & 15) == 0, BL_ERR_ALIGN);
  BL_REQUIRE(gain == nullptr || x_f32, BL_ERR_TYPE);
  F8RowsArgs a{x, x_f32, ldx, gain, eps, M, K, (uint8_t*)codes, ldc, scales};
  return (int)launch(fp8_rows_kernel, dim3(M), dim3(256), 0, st, a);
}

// C[dst_row[t] or t, n] = row_scale[t] * sum_kb xs[t, kb] * ws[n, kb] * (Xq[t, kb] . Wq[g][n, kb]) (+ resid) per 32-row
// token tile of the table.  Xq [rows_x, K] E4M3 codes (ldx bytes), xs [rows_x, K / 128]; W, W2 [n_groups, N, row_bytes]
// resident FP8_B128 rows; exactly one of c_f32 / c_bf16; W2 != null: output = silu(X W^T) * (X W2^T).
int bl_fp8_gemm(const void* Xq, long ldx, long rows_x, const float* xs, const void* W, const void* W2, int n_groups, int N,
                int K, const void* tiles, const int* n_tiles, int max_tiles, int tile_rows, float* c_f32, void* c_bf16, long ldc,
                const int* dst_row, const float* row_scale, const float* resid, long ldr, unsigned* status, int sm_count,
                cudaStream_t st) {
  BL_REQUIRE(K >= 128 && K % 128 == 0 && N >= 1 && rows_x >= 1 && n_groups >= 1 && max_tiles >= 1, BL_ERR_SHAPE);
  BL_REQUIRE(tile_rows == F8_BN, BL_ERR_SHAPE);
  BL_REQUIRE(ldx % 16 == 0 && ((uintptr_t)Xq & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)W2 & 15) == 0, BL_ERR_ALIGN);
  BL_REQUIRE((c_f32 != nullptr) != (c_bf16 != nullptr), BL_ERR_SHAPE);
  const long rb = resident_row_bytes(WT_FP8_B128, K);
  BL_REQUIRE(rb > 0, BL_ERR_TYPE);
  CUtensorMap mx;
  {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows_x};
    cuuint64_t str[1] = {(cuuint64_t)ldx};
    cuuint32_t box[2] = {F8_BK, F8_BN};
    int rc = make_map_any(&mx, Xq, 2, dims, str, box, CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  F8Args a{};
  a.w = (const uint8_t*)W; a.w2 = (const uint8_t*)W2;
  a.row_bytes = rb; a.group_bytes = rb * N;
  a.N = N; a.K = K; a.tiles_w = (N + F8_BM - 1) / F8_BM;
  a.tiles = (const F8Tile*)tiles; a.n_tiles = n_tiles; a.max_tiles = max_tiles;
  a.xs = xs;
  a.c_f32 = c_f32; a.c_bf16 = (__nv_bfloat16*)c_bf16; a.ldc = ldc;
  a.dst_row = dst_row; a.row_scale = row_scale; a.resid = resid; a.ldr = ldr; a.status = status;
  const long tiles_total = (long)max_tiles * a.tiles_w;
  const int grid = (int)(tiles_total < sm_count ? tiles_total : sm_count);
  return W2 ? fp8_gemm_go<true>(mx, a, n_groups, grid, st) : fp8_gemm_go<false>(mx, a, n_groups, grid, st);
}

}  // extern "C"
