// bf16 grouped GEMM on the 5th-generation tensor cores (sm_100a only):
//   C[g][m, n] = sum_k A[m, k] * B[g][n, k]        fp32 accumulate in tensor memory
//
//   * operands staged by TMA (cp.async.bulk.tensor, 128-byte swizzle, every CTA fetches its own tiles) into
//     a 4-stage shared-memory ring; one elected thread issues tcgen05.mma (M=128, N=128,
//     K=16 per instruction) with accumulators in TMEM; four epilogue warps read them back
//     with tcgen05.ld while the next tile's main loop already runs (two TMEM buffers);
//   * persistent: one CTA per SM walks a device-resident tile table, so row counts that
//     are only known on the device (tokens per expert) never reach the host and the launch
//     is capturable in a CUDA graph;
//   * "dual" mode multiplies A with two B matrices (gate and up) in the same main loop and
//     the epilogue writes silu(gate) * up, so the SwiGLU activation never round-trips HBM;
//   * the epilogue can scatter: row r of the product goes to row dst_row[r] of the output,
//     scaled by row_scale[r] -- the expert-parallel "combine" is this store aimed at the
//     owning GPU's buffer (a peer pointer works: plain st.global over NVLink).
//
// Every wait (mbarrier phases) is bounded by the global timer; on expiry the CTA raises
// status word 1, drains what it has in flight, frees its TMEM and returns.
//
// Role of this file in the reference: the grouped tensor-core GEMM of
// crates/gpu/src/gemm/{grouped,kernels}.rs (mma.sync int8 tiles walking a route table)
// and bf16_mma_gemm in crates/gpu/src/q8f32.rs; the reference has no sm_100 path at all.
#include "tc_common.cuh"

namespace bl {

constexpr int BM = 128, BK = 64;               // BK * 2 bytes = 128 = one swizzle atom row
// Tile width: 256 columns for a plain product (one B tile of 32 KiB per stage: 48 KiB of
// operands feed 512 tensor-core cycles, which the L2 -> SM path sustains), 128 + 128 for the
// dual (gate, up) product.
constexpr int BN_SINGLE = 256, BN_DUAL = 128;
constexpr int STAGES = 4;
constexpr int TILE_A_BYTES = BM * BK * 2;      // 16 KiB
constexpr int TILE_B128_BYTES = 128 * BK * 2;  // 16 KiB per 128 B-rows

// pad: in the several-GPU form the source rank of the tile's A rows; otherwise causal limits in units of 64:
// low 16 bits = columns of the product that exist for this tile (0 = all), high 16 bits = depth blocks to run (0 = all).
struct MTile { int group, row0, row_end, pad; };
__device__ __forceinline__ bool tile_skipped(const MTile& mt, int n0) {
  const int lim = mt.pad & 0xFFFF;
  return lim != 0 && n0 >= lim * 64;
}
__device__ __forceinline__ int tile_kblocks(const MTile& mt, int kblocks) {
  const int lim = (mt.pad >> 16) & 0xFFFF;
  return lim != 0 && lim < kblocks ? lim : kblocks;
}

struct GemmArgs {
  int N, K;
  int tiles_n;
  const MTile* mtiles;        // device table of 128-row tiles
  const int* n_mtiles;        // device count
  int max_mtiles;
  int dual;                   // 1: B2 is used and the epilogue writes silu(A B^T) * (A B2^T)
  float* c_f32;               // one of c_f32 / c_bf16
  __nv_bfloat16* c_bf16;
  long ldc;
  const int* dst_row;         // optional scatter: output row of product row r (< 0 = drop)
  const float* row_scale;     // optional per-row factor
  const float* resid;         // optional addend, indexed like the output
  long ldr;
  unsigned* status;
  // distributed mode (several GPUs): rows of the output are owned by ranks in blocks of
  // rows_per_owner; a finished value is ADDED into the owner's fp32 buffer (a peer pointer:
  // red.global.add over NVLink), which is the reduce-scatter of a tensor-parallel product
  // and the combine of an expert-parallel one.  dst_div maps dst_row (a flat slot index
  // token * k + j) back to its token.
  float* own_base[8];
  int rows_per_owner;
  int n_owners;
  int dst_div;
  int src_rows;               // > 0: A is row-sharded; product row = tile's source rank * src_rows + row in the shard
  int wide_stores;            // fp32 output rows start on 32-byte boundaries: the epilogue may use 256-bit stores
};

// One tensor map of A per source rank: m-tile t reads the map of rank mtiles[t].pad, so the
// "all-gather" of a row-sharded activation is the TMA load itself (plain tile loads from the
// peer's memory, one CTA per tile, no cluster multicast).
struct AMaps { CUtensorMap m[8]; };

// ---- the kernel ------------------------------------------------------------------------
// 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..5 = epilogue
// (their warp id modulo 4 covers the four 32-lane quarters of tensor memory).
__device__ __forceinline__ void st_global_v8(float* p, const float* v) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
               "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <bool DUAL, bool DIST>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ AMaps tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ CUtensorMap tma_b2, const GemmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int BN = DUAL ? BN_DUAL : BN_SINGLE;
  constexpr int TILE_B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = TILE_A_BYTES + (DUAL ? 2 : 1) * TILE_B_BYTES;   // 48 KiB either way
  constexpr int ACC_COLS = 256;                        // TMEM columns per accumulator buffer
  constexpr int TMEM_COLS = 2 * ACC_COLS;              // two buffers: all 512 columns
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
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

  const int n_mt = min(*a.n_mtiles, a.max_mtiles);
  const int total_tiles = n_mt * a.tiles_n;
  const int kblocks = a.K / BK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int issued = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const MTile mt = a.mtiles[t / a.tiles_n];
        const int n0 = (t % a.tiles_n) * BN;
        if (!DIST && tile_skipped(mt, n0)) continue;
        const int kb_end = DIST ? kblocks : tile_kblocks(mt, kblocks);
        for (int kb = 0; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) break;
          uint8_t* sa = smem + (size_t)stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(sa, DIST ? &tma_a.m[mt.pad & 7] : &tma_a.m[0], kb * BK, mt.row0, &full_bar[stage]);
          tma_load_3d(sa + TILE_A_BYTES, &tma_b, kb * BK, n0, mt.group, &full_bar[stage]);
          if (DUAL) tma_load_3d(sa + TILE_A_BYTES + TILE_B_BYTES, &tma_b2, kb * BK, n0, mt.group, &full_bar[stage]);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {
        // our own copies may still be landing in shared memory: give the last ring of them a bounded wait
        for (int s = 0; s < STAGES && s < issued; ++s) {
          unsigned long long t0 = globaltimer();
          while (globaltimer() - t0 < 2000000ull) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(smem_u32(&full_bar[s])), "r"(0u) : "memory");
            if (ok) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const MTile mt = a.mtiles[t / a.tiles_n];
        if (!DIST && tile_skipped(mt, (t % a.tiles_n) * BN)) continue;
        const int kb_end = DIST ? kblocks : tile_kblocks(mt, kblocks);
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&acc_empty[ab], acc_phase ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + ab * ACC_COLS;
        bool ok = true;
        for (int kb = 0; kb < kb_end; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
          const uint64_t da = umma_desc(sa), db = umma_desc(sa + TILE_A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
            umma_bf16(d0, da + (uint64_t)(k * UMMA_K * 2 / 16), db + (uint64_t)(k * UMMA_K * 2 / 16), idesc, acc);
            if (DUAL) {
              const uint64_t db2 = umma_desc(sa + TILE_A_BYTES + TILE_B_BYTES);
              umma_bf16(d0 + BN, da + (uint64_t)(k * UMMA_K * 2 / 16), db2 + (uint64_t)(k * UMMA_K * 2 / 16), idesc, acc);
            }
          }
          umma_commit(&empty_bar[stage]);      // the stage is free once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[ab]);            // accumulator complete
      }
    }
  } else {
    const int q = warp & 3;                    // TMEM lane quarter of this warp
    int it = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      const MTile mt = a.mtiles[t / a.tiles_n];
      const int n0 = (t % a.tiles_n) * BN;
      if (!DIST && tile_skipped(mt, n0)) continue;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&acc_full[ab], acc_phase, abort_flag)) break;
      tc_fence_after();
      const int r = mt.row0 + q * 32 + lane;                 // product row of this thread
      const bool live = r < mt.row_end;
      long orow = r;
      if (DIST && a.src_rows > 0) orow += (long)mt.pad * a.src_rows;
      float scale = 1.0f;
      if (live && a.dst_row) orow = a.dst_row[r];
      if (live && a.row_scale) scale = a.row_scale[r];
      const bool store = live && orow >= 0;
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + ab * ACC_COLS;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tbase + c * 32, v);
        float f[32];
        if (DUAL) {
          uint32_t u[32];
          tmem_ld32(tbase + BN + c * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float g = __uint_as_float(v[i]);
            f[i] = (g / (1.0f + __expf(-g))) * __uint_as_float(u[i]);
          }
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
        }
        const int col = n0 + c * 32;
        if (store && col < a.N) {
          if (a.row_scale) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] *= scale;
          }
          if (a.resid) {
            const float* rr = a.resid + orow * a.ldr + col;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 x = *reinterpret_cast<const float4*>(rr + i);
              f[i] += x.x; f[i + 1] += x.y; f[i + 2] += x.z; f[i + 3] += x.w;
            }
          }
          if (DIST && a.n_owners > 0) {
            const long tok = a.dst_div > 1 ? orow / a.dst_div : orow;
            const int owner = (int)(tok / a.rows_per_owner);
            float* o = a.own_base[owner & 7] + (tok - (long)owner * a.rows_per_owner) * a.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; i += 4) red_add_v4(o + i, f[i], f[i + 1], f[i + 2], f[i + 3]);
          } else if (a.c_f32) {
            float* o = a.c_f32 + orow * a.ldc + col;
            if (a.wide_stores) {
              // 32-byte stores: every instruction fills whole sectors of the thread's row
#pragma unroll
              for (int i = 0; i < 32; i += 8) st_global_v8(o + i, f + i);
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
            }
          } else {
            __nv_bfloat16* o = a.c_bf16 + orow * a.ldc + col;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk;
              __nv_bfloat162 p0 = __floats2bfloat162_rn(f[i], f[i + 1]), p1 = __floats2bfloat162_rn(f[i + 2], f[i + 3]);
              __nv_bfloat162 p2 = __floats2bfloat162_rn(f[i + 4], f[i + 5]), p3 = __floats2bfloat162_rn(f[i + 6], f[i + 7]);
              pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
              pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
              *reinterpret_cast<uint4*>(o + i) = pk;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[ab]);
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

// ---- tile table ----------------------------------------------------------------------
// group_rows[g] rows for group g, laid out back to back in A (offsets = prefix sums).
// A group's B-matrix index is g / group_div (several row groups may share one B, e.g. the
// query heads of one KV head).
__global__ void build_mtiles_kernel(const int* group_rows, int n_groups, MTile* mtiles, int* n_mtiles, int max_mtiles,
                                    int* group_offset_out, int group_div, int group_stride, int base, int src_rows,
                                    int causal_pos0, int causal_kind) {
  pdl_wait();
  pdl_launch();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  // group_stride > 0: group g starts at row base + g * group_stride of A (strided groups,
  // e.g. one query chunk of every head); otherwise groups follow one another.
  int off = 0, n = 0;
  for (int g = 0; g < n_groups; ++g) {
    const int rows = group_rows[g];
    if (group_stride > 0) off = base + g * group_stride;
    if (group_offset_out) group_offset_out[g] = off;
    for (int r = 0; r < rows; r += BM) {
      // src_rows > 0: A is row-sharded over ranks in blocks of src_rows; the tile reads rank (row / src_rows)'s map
      if (n < max_mtiles) {
        if (src_rows > 0) {
          const int src = (off + r) / src_rows, lo = (off + r) - src * src_rows;
          const int end = min(off + rows, (src + 1) * src_rows) - src * src_rows;
          mtiles[n] = MTile{g / group_div, lo, end, src};
        } else {
          // causal_kind 1: the product's columns are keys, a tile of queries r..r+127 of the group needs keys up to
          // its last query's position; 2: the depth is keys.  Limits are counted in 64s.
          int pad = 0;
          if (causal_kind != 0) {
            const int last = causal_pos0 + min(r + BM, rows);          // keys 0 .. last - 1
            const int lim = min((last + 63) / 64, 0xFFFF);
            pad = causal_kind == 1 ? lim : (lim << 16);
          }
          mtiles[n] = MTile{g / group_div, off + r, off + rows, pad};
        }
      }
      ++n;
    }
    if (group_stride <= 0) off += rows;
  }
  if (group_offset_out) group_offset_out[n_groups] = off;
  *n_mtiles = n < max_mtiles ? n : max_mtiles;
}

}  // namespace bl

using namespace bl;

extern "C" {

// Fill the tile table for a grouped GEMM from per-group row counts on the device.
int bl_gemm_build_tiles(const int* group_rows, int n_groups, void* mtiles, int* n_mtiles, int max_mtiles,
                        int* group_offsets, int group_div, int group_stride, int base, cudaStream_t st) {
  BL_REQUIRE(n_groups >= 1 && max_mtiles >= 1 && group_div >= 1, BL_ERR_SHAPE);
  return (int)launch(build_mtiles_kernel, dim3(1), dim3(32), 0, st, group_rows, n_groups, (MTile*)mtiles, n_mtiles,
                     max_mtiles, group_offsets, group_div, group_stride, base, 0, 0, 0);
}

// The same with causal limits: kind 1 = columns are keys (scores), kind 2 = depth is keys (values); a group's row r is
// the query at position causal_pos0 + r.
int bl_gemm_build_tiles_causal(const int* group_rows, int n_groups, void* mtiles, int* n_mtiles, int max_mtiles,
                               int* group_offsets, int group_div, int group_stride, int base, int causal_pos0, int kind,
                               cudaStream_t st) {
  BL_REQUIRE(n_groups >= 1 && max_mtiles >= 1 && group_div >= 1 && (kind == 1 || kind == 2) && causal_pos0 >= 0, BL_ERR_SHAPE);
  return (int)launch(build_mtiles_kernel, dim3(1), dim3(32), 0, st, group_rows, n_groups, (MTile*)mtiles, n_mtiles,
                     max_mtiles, group_offsets, group_div, group_stride, base, 0, causal_pos0, kind);
}

// Tile table of a dense product whose A rows are sharded over ranks in blocks of src_rows (a multiple of 128).
int bl_gemm_build_tiles_sharded(const int* total_rows, void* mtiles, int* n_mtiles, int max_mtiles, int src_rows,
                                cudaStream_t st) {
  BL_REQUIRE(max_mtiles >= 1 && src_rows >= BM && src_rows % BM == 0, BL_ERR_SHAPE);
  return (int)launch(build_mtiles_kernel, dim3(1), dim3(32), 0, st, total_rows, 1, (MTile*)mtiles, n_mtiles, max_mtiles,
                     (int*)nullptr, 1, 0, 0, src_rows, 0, 0);
}

// C = A * B[g]^T per 128-row tile of the table.  A: [rows_a, K] bf16 (lda elements);
// B, B2: [n_groups, N, K] bf16.  Output row r -> dst_row[r] (or r), times row_scale[r],
// plus resid.  Exactly one of c_f32 / c_bf16.  status: device word, set to 1 if a wait ran out.
static int gemm_launch(const void* const* A_of_rank, int n_src, long lda, long rows_a, const void* B, const void* B2,
                       int n_groups, int N, int K, const void* mtiles, const int* n_mtiles, int max_mtiles, float* c_f32,
                       void* c_bf16, long ldc, const int* dst_row, const float* row_scale, const float* resid, long ldr,
                       float* const* own_base, int n_owners, int rows_per_owner, int dst_div, int src_rows,
                       unsigned* status, int sm_count, cudaStream_t st) {
  BL_REQUIRE(K >= BK && K % BK == 0 && N >= 32 && N % 32 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(lda % 8 == 0 && rows_a >= 1 && n_groups >= 1 && n_src >= 1 && n_src <= 8, BL_ERR_SHAPE);
  BL_REQUIRE(((uintptr_t)B & 15) == 0 && ((uintptr_t)B2 & 15) == 0, BL_ERR_ALIGN);
  const bool dist = n_src > 1 || n_owners > 0;
  if (n_owners > 0) {
    BL_REQUIRE(n_owners <= 8 && rows_per_owner >= 1 && c_f32 == nullptr && c_bf16 == nullptr && !resid && !B2, BL_ERR_SHAPE);
    for (int r = 0; r < n_owners; ++r) BL_REQUIRE(own_base[r] && ((uintptr_t)own_base[r] & 15) == 0, BL_ERR_ALIGN);
  } else {
    BL_REQUIRE((c_f32 != nullptr) != (c_bf16 != nullptr), BL_ERR_SHAPE);
  }
  BL_REQUIRE(ldc % 8 == 0 && (!resid || ldr % 4 == 0), BL_ERR_SHAPE);
  BL_REQUIRE(((uintptr_t)c_f32 & 15) == 0 && ((uintptr_t)c_bf16 & 15) == 0 && ((uintptr_t)resid & 15) == 0, BL_ERR_ALIGN);
  AMaps ma;
  CUtensorMap mb, mb2;
  for (int r = 0; r < 8; ++r) {
    const void* A = A_of_rank[r < n_src ? r : 0];
    BL_REQUIRE(A && ((uintptr_t)A & 15) == 0, BL_ERR_ALIGN);
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows_a};
    cuuint64_t str[1] = {(cuuint64_t)lda * 2};
    cuuint32_t box[2] = {BK, BM};
    int rc = make_map(&ma.m[r], A, 2, dims, str, box);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)N, (cuuint64_t)n_groups};
    cuuint64_t str[2] = {(cuuint64_t)K * 2, (cuuint64_t)K * 2 * (cuuint64_t)N};
    cuuint32_t box[3] = {BK, (cuuint32_t)(B2 ? BN_DUAL : BN_SINGLE), 1};
    int rc = make_map(&mb, B, 3, dims, str, box);
    if (rc) return rc;
    rc = make_map(&mb2, B2 ? B2 : B, 3, dims, str, box);
    if (rc) return rc;
  }
  GemmArgs a{};
  a.N = N; a.K = K;
  a.mtiles = (const MTile*)mtiles; a.n_mtiles = n_mtiles; a.max_mtiles = max_mtiles;
  a.dual = B2 ? 1 : 0;
  a.c_f32 = c_f32; a.c_bf16 = (__nv_bfloat16*)c_bf16; a.ldc = ldc;
  a.dst_row = dst_row; a.row_scale = row_scale; a.resid = resid; a.ldr = ldr; a.status = status;
  for (int r = 0; r < n_owners; ++r) a.own_base[r] = own_base[r];
  a.n_owners = n_owners; a.rows_per_owner = rows_per_owner; a.dst_div = dst_div; a.src_rows = src_rows;
  a.wide_stores = (c_f32 && ((uintptr_t)c_f32 & 31) == 0 && ldc % 8 == 0) ? 1 : 0;
  a.tiles_n = (N + (B2 ? BN_DUAL : BN_SINGLE) - 1) / (B2 ? BN_DUAL : BN_SINGLE);
  long tiles = (long)max_mtiles * a.tiles_n;
  int grid = (int)(tiles < sm_count ? tiles : sm_count);
  const size_t smem = (size_t)STAGES * (TILE_A_BYTES + 2 * TILE_B128_BYTES) + 1024;
  auto go = [&](auto kernel, bool& set) {
    if (!set) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); set = true; }
    return (int)launch(kernel, dim3(grid), dim3(192), smem, st, ma, mb, mb2, a);
  };
  static bool s00 = false, s01 = false, s10 = false, s11 = false;
  if (B2) return dist ? go(gemm_bf16_kernel<true, true>, s11) : go(gemm_bf16_kernel<true, false>, s10);
  return dist ? go(gemm_bf16_kernel<false, true>, s01) : go(gemm_bf16_kernel<false, false>, s00);
}

int bl_gemm_bf16(const void* A, long lda, long rows_a, const void* B, const void* B2, int n_groups, int N, int K,
                 const void* mtiles, const int* n_mtiles, int max_mtiles, float* c_f32, void* c_bf16, long ldc,
                 const int* dst_row, const float* row_scale, const float* resid, long ldr, unsigned* status,
                 int sm_count, cudaStream_t st) {
  const void* As[1] = {A};
  return gemm_launch(As, 1, lda, rows_a, B, B2, n_groups, N, K, mtiles, n_mtiles, max_mtiles, c_f32, c_bf16, ldc, dst_row,
                     row_scale, resid, ldr, nullptr, 0, 0, 1, 0, status, sm_count, st);
}

// The several-GPU form.  A_of_rank: one pointer per source rank (each [rows_a, K], the rank's shard; tiles pick
// their source by the table built with bl_gemm_build_tiles_sharded); n_src == 1 reads local rows only.
// own_base / n_owners / rows_per_owner: when n_owners > 0 the product is added into the owners' buffers instead
// of being stored (see GemmArgs); dst_div maps dst_row entries back to tokens.
int bl_gemm_bf16_dist(const void* const* A_of_rank, int n_src, long lda, long rows_a, const void* B, const void* B2,
                      int n_groups, int N, int K, const void* mtiles, const int* n_mtiles, int max_mtiles, float* c_f32,
                      void* c_bf16, long ldc, const int* dst_row, const float* row_scale, float* const* own_base,
                      int n_owners, int rows_per_owner, int dst_div, int src_rows, unsigned* status, int sm_count,
                      cudaStream_t st) {
  BL_REQUIRE(n_src == 1 || (src_rows >= BM && src_rows % BM == 0 && rows_a >= src_rows), BL_ERR_SHAPE);
  return gemm_launch(A_of_rank, n_src, lda, rows_a, B, B2, n_groups, N, K, mtiles, n_mtiles, max_mtiles, c_f32, c_bf16, ldc,
                     dst_row, row_scale, nullptr, 0, own_base, n_owners, rows_per_owner, dst_div < 1 ? 1 : dst_div,
                     n_src > 1 ? src_rows : 0, status, sm_count, st);
}

}  // extern "C"
