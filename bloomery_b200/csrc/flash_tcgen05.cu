// Prompt (prefill) flash attention on the 5th-generation tensor cores: scores and the output accumulator live in
// tensor memory, the probabilities go from registers to shared memory and straight back into the second product,
// and nothing of the score matrix ever reaches HBM.
//
// One CTA = one query head x 128 consecutive query positions (the 128 lanes of tensor memory).  Per 128-key tile:
//   S = Q K^T          tcgen05.mma kind::f16, M = N = 128, depth 128 (two 64-wide swizzle atoms), into TMEM
//   softmax            two threads own one query row, 64 of its 128 scores each (one tcgen05.ld pass, the scores stay
//                      in registers between the maximum and the exponentials): the halves' maxima meet through shared
//                      memory and a bounded mbarrier, running max / sum in base 2, causal mask on the diagonal tiles,
//                      probabilities as bf16 into a 128-byte-swizzled shared-memory tile (one swizzle atom per half)
//   O = O * corr       the running output is rescaled in TMEM (tcgen05.ld / tcgen05.st), each half its 64 columns, and
//                      only when the row maximum moved by more than 2^8: until then the old maximum keeps scaling the
//                      exponentials (they stay below 2^8, far inside fp32 and bf16), so most tiles skip the round trip
//   O += P V           tcgen05.mma with P as the A operand and the (dims x keys) value tile as B
// Roles: warps 0..3 and 6..9 softmax (warp id modulo 4 = TMEM lane quarter; 0..3 take score columns 0..63, 6..9
// columns 64..127), warp 4 the TMA producer (two-stage rings for keys and values), warp 5 the MMA issuer and TMEM owner.  The score accumulator is double-buffered, so the
// product of tile t + 1 runs while the softmax of tile t is still busy; the second product of tile t is issued one
// iteration late for the same reason.  Every TMA load is a plain tile load of this GPU's own memory.
//
// Inputs are what the prompt path already builds: queries bf16 [n_q][T][128] (normalised, rotated, pre-scaled),
// keys bf16 [n_kv][t_pad][128], values transposed bf16 [n_kv][128][t_pad]; output bf16 [T][n_q * 128].
// Every wait is bounded (1 s); on expiry the CTA raises the status word, frees its TMEM and returns.
//
// Reference counterpart: crates/gpu/src/flash_gqa_prefill.rs:1-80 (mma.sync m16n8k16 tiles, cp.async staging).
#include "tc_common.cuh"

namespace bl {

constexpr int FQ = 128, FKEYS = 128, FD = 128;
constexpr int FATOM = 64;                               // bf16 values per 128-byte swizzle row
constexpr int FHALF = 128 * FATOM * 2;                  // 16 KiB: 128 rows x 64 values
constexpr int FTILE = 2 * FHALF;                        // 32 KiB: a 128 x 128 bf16 tile as two swizzle atoms
constexpr int FSMEM = FTILE /*Q*/ + 2 * FTILE /*K*/ + 2 * FTILE /*V*/ + FTILE /*P*/ + 1024 /*alignment*/;
constexpr float kLog2e = 1.4426950408889634f;

struct FlashPrefillArgs {
  int T, n_q, group;          // query rows per head; heads; query heads per KV head
  int pos0;                   // position of query row 0 (keys 0 .. pos0 + T - 1 exist)
  int t_pad;                  // key rows per KV head in K = key columns per row in Vt
  __nv_bfloat16* out; long ldo;
  unsigned* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&p);
}

constexpr int FTHREADS = 320;
constexpr float kLazy = 8.0f;                           // the maximum may lag by 2^8 before the output is rescaled

__global__ void __launch_bounds__(FTHREADS, 1)
flash_prefill_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const FlashPrefillArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_full, o_done;
  __shared__ __align__(8) uint64_t mx_full[2], l_full;
  __shared__ float s_mx[2][2][FQ];                      // [score buffer][half][row]: the halves' tile maxima
  __shared__ float s_l[2][FQ];                          // [half][row]: the halves' sums at the end
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + FTILE;          // [2 stages][2 halves]
  uint8_t* sV = sK + 2 * FTILE;      // [2 stages][2 halves]
  uint8_t* sP = sV + 2 * FTILE;      // [2 halves]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;          // the tiles with the most keys start first
  const int h = blockIdx.y, kvh = h / a.group;
  const int q0 = qt * FQ;
  const int last_q = a.pos0 + min(q0 + FQ, a.T) - 1;            // position of the tile's last query
  const int n_t = last_q / FKEYS + 1;                           // key tiles 0 .. n_t - 1

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8); mbar_init(&mx_full[i], 8);
    }
    mbar_init(&p_full, 8); mbar_init(&o_done, 1); mbar_init(&l_full, 8);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_launch();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;
  const uint32_t tS0 = tmem_base, tO = tmem_base + 256;         // S[0] at column 0, S[1] at 128, O at 256

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(&q_full, FTILE);
      tma_load_2d(sQ, &tma_q, 0, h * a.T + q0, &q_full);
      tma_load_2d(sQ + FHALF, &tma_q, FATOM, h * a.T + q0, &q_full);
      for (int t = 0; t < n_t && !*abort_flag; ++t) {
        const int st = t & 1;
        const uint32_t par = (uint32_t)((t >> 1) & 1);
        if (!mbar_wait(&k_empty[st], par ^ 1, abort_flag)) break;
        mbar_expect_tx(&k_full[st], FTILE);
        tma_load_2d(sK + st * FTILE, &tma_k, 0, kvh * a.t_pad + t * FKEYS, &k_full[st]);
        tma_load_2d(sK + st * FTILE + FHALF, &tma_k, FATOM, kvh * a.t_pad + t * FKEYS, &k_full[st]);
        if (!mbar_wait(&v_empty[st], par ^ 1, abort_flag)) break;
        mbar_expect_tx(&v_full[st], FTILE);
        tma_load_2d(sV + st * FTILE, &tma_v, t * FKEYS, kvh * FD, &v_full[st]);
        tma_load_2d(sV + st * FTILE + FHALF, &tma_v, t * FKEYS + FATOM, kvh * FD, &v_full[st]);
      }
      if (*abort_flag) {
        // copies of ours may still be landing: give them a bounded moment before the block's memory goes away
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 2000000ull) { }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(FQ, FKEYS);
      const uint64_t dQ0 = umma_desc(smem_u32(sQ)), dQ1 = umma_desc(smem_u32(sQ + FHALF));
      const uint64_t dP0 = umma_desc(smem_u32(sP)), dP1 = umma_desc(smem_u32(sP + FHALF));
      auto pv = [&](int x) -> bool {
        const int sx = x & 1;
        if (!mbar_wait(&v_full[sx], (uint32_t)((x >> 1) & 1), abort_flag)) return false;
        if (!mbar_wait(&p_full, (uint32_t)(x & 1), abort_flag)) return false;
        tc_fence_after();
        const uint64_t dV0 = umma_desc(smem_u32(sV + sx * FTILE)), dV1 = umma_desc(smem_u32(sV + sx * FTILE + FHALF));
#pragma unroll
        for (int k = 0; k < FATOM / UMMA_K; ++k) umma_bf16(tO, dP0 + (uint64_t)(k * 2), dV0 + (uint64_t)(k * 2), idesc, (x > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < FATOM / UMMA_K; ++k) umma_bf16(tO, dP1 + (uint64_t)(k * 2), dV1 + (uint64_t)(k * 2), idesc, 1u);
        umma_commit(&v_empty[sx]);
        umma_commit(&o_done);
        return true;
      };
      bool ok = mbar_wait(&q_full, 0, abort_flag);
      for (int t = 0; ok && t < n_t && !*abort_flag; ++t) {
        const int b = t & 1;
        const uint32_t par = (uint32_t)((t >> 1) & 1);
        if (!mbar_wait(&k_full[b], par, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&s_empty[b], par ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint64_t dK0 = umma_desc(smem_u32(sK + b * FTILE)), dK1 = umma_desc(smem_u32(sK + b * FTILE + FHALF));
        const uint32_t tS = tS0 + b * FKEYS;
#pragma unroll
        for (int k = 0; k < FATOM / UMMA_K; ++k) umma_bf16(tS, dQ0 + (uint64_t)(k * 2), dK0 + (uint64_t)(k * 2), idesc, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < FATOM / UMMA_K; ++k) umma_bf16(tS, dQ1 + (uint64_t)(k * 2), dK1 + (uint64_t)(k * 2), idesc, 1u);
        umma_commit(&k_empty[b]);
        umma_commit(&s_full[b]);
        if (t >= 1 && !pv(t - 1)) { ok = false; break; }
      }
      if (ok && !*abort_flag) pv(n_t - 1);
    }
  } else {
    // ---- softmax: two threads per query row, 64 score columns each ---------------------------------------
    const int half = warp >= 6 ? 1 : 0;
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;
    const int qrow = q0 + r;
    const int qpos = a.pos0 + qrow;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int col0 = half * 64;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < n_t && !*abort_flag; ++t) {
      const int b = t & 1;
      const uint32_t par = (uint32_t)((t >> 1) & 1);
      if (!mbar_wait(&s_full[b], par, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int k0 = t * FKEYS + col0;
      const bool diag = t * FKEYS + FKEYS - 1 > a.pos0 + q0;    // some key of this tile lies past some query of it
      const uint32_t tS = tS0 + b * FKEYS + lane_base + col0;
      uint32_t v0[32], v1[32];
      tmem_ld32(tS, v0);
      tmem_ld32(tS + 32, v1);
      tmem_ld_wait();
      float mx = -INFINITY;
      if (diag) {                                               // only the tiles on the diagonal pay for the mask
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (k0 + i > qpos) v0[i] = 0xff800000u;               // -inf
          if (k0 + 32 + i > qpos) v1[i] = 0xff800000u;
        }
      }
      {
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;     // four chains instead of one
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          mx0 = fmaxf(mx0, __uint_as_float(v0[i])); mx1 = fmaxf(mx1, __uint_as_float(v0[i + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(v1[i])); mx3 = fmaxf(mx3, __uint_as_float(v1[i + 1]));
        }
        mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      }
      // the other half's maximum of this row
      s_mx[b][half][r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&mx_full[b]);
      if (!mbar_wait(&mx_full[b], par, abort_flag)) { ok = false; break; }
      mx = fmaxf(mx, s_mx[b][half ^ 1][r]);
      float m_new = fmaxf(m, mx);
      if (m != -INFINITY && (m_new - m) * kLog2e <= kLazy) m_new = m;     // both halves see the same numbers: same choice
      const float mb = (m_new == -INFINITY) ? 0.f : m_new * kLog2e;       // a row with no key yet keeps zeros
      const float corr = (m == -INFINITY) ? 0.f : ex2(m * kLog2e - mb);
      // the previous value product has to be complete only when some row of this warp rescales its output
      if (t > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
        if (!mbar_wait(&o_done, (uint32_t)((t - 1) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            tmem_ld32(tO + lane_base + col0 + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_st32(tO + lane_base + col0 + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      float rowsum = 0.f, rowsum1 = 0.f;
      uint8_t* prow = sP + half * FHALF + (r >> 3) * 1024 + (r & 7) * 128;     // this half's swizzle atom
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          // (s0, s1) * log2(e) - mb as one packed FMA; masked scores are -inf and 2^-inf = 0 (a row without any key
          // has mb = 0 and only -inf scores, so it needs no special case)
          uint32_t e0, e1;
          asm("{\n\t.reg .b64 rs, rk, rm, rr;\n\t"
              "mov.b64 rs, {%2, %3};\n\tmov.b64 rk, {%4, %4};\n\tmov.b64 rm, {%5, %5};\n\t"
              "fma.rn.f32x2 rr, rs, rk, rm;\n\tmov.b64 {%0, %1}, rr;\n\t}"
              : "=r"(e0), "=r"(e1) : "r"(c ? v1[i] : v0[i]), "r"(c ? v1[i + 1] : v0[i + 1]), "f"(kLog2e), "f"(-mb));
          const float p0 = ex2(__uint_as_float(e0)), p1 = ex2(__uint_as_float(e1));
          rowsum += p0; rowsum1 += p1;
          pk[i >> 1] = pack_bf16(p0, p1);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int chunk = (c * 4 + j) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
      }
      l = l * corr + (rowsum + rowsum1);
      m = m_new;
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[b]); mbar_arrive(&p_full); }
    }
    if (ok && !*abort_flag && mbar_wait(&o_done, (uint32_t)((n_t - 1) & 1), abort_flag)) {
      tc_fence_after();
      s_l[half][r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&l_full);
      if (mbar_wait(&l_full, 0, abort_flag)) {
        const float lt = s_l[0][r] + s_l[1][r];
        const float inv = lt > 0.f ? 1.0f / lt : 0.f;
        __nv_bfloat16* orow = a.out + (long)qrow * a.ldo + (long)h * FD + col0;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld32(tO + lane_base + col0 + c * 32, v);
          tmem_ld_wait();
          if (qrow < a.T) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 pk;
              pk.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
              pk.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
              pk.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
              pk.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + i) = pk;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  if (threadIdx.x == 0 && s_abort && a.status) atomicMax(a.status, 1u);
}

}  // namespace bl

using namespace bl;

extern "C" {

// Causal attention of T query rows per head (positions pos0 .. pos0 + T - 1) over keys 0 .. pos0 + T - 1.
//   q  bf16 [n_q][T][128]   k  bf16 [n_kv][t_pad][128]   vt  bf16 [n_kv][128][t_pad]   out  bf16 [T][ldo >= n_q * 128]
// t_pad is a multiple of 128 that covers the keys; value columns past the last key must be finite (zero).
int bl_flash_prefill(const void* q, const void* k, const void* vt, void* out, long ldo, int T, int n_q, int n_kv, int pos0,
                     int t_pad, unsigned* status, cudaStream_t st) {
  BL_REQUIRE(T >= 1 && n_q >= 1 && n_kv >= 1 && n_q % n_kv == 0 && pos0 >= 0, BL_ERR_SHAPE);
  BL_REQUIRE(t_pad % 128 == 0 && t_pad >= pos0 + T && ldo >= (long)n_q * FD && ldo % 8 == 0, BL_ERR_SHAPE);
  BL_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)vt | (uintptr_t)out) & 15) == 0, BL_ERR_ALIGN);
  CUtensorMap mq, mk, mv;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)FD, (cuuint64_t)n_q * T};
    const cuuint64_t strides[1] = {(cuuint64_t)FD * 2};
    const cuuint32_t box[2] = {FATOM, FQ};
    int rc = make_map(&mq, q, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)FD, (cuuint64_t)n_kv * t_pad};
    const cuuint64_t strides[1] = {(cuuint64_t)FD * 2};
    const cuuint32_t box[2] = {FATOM, FKEYS};
    int rc = make_map(&mk, k, 2, dims, strides, box);
    if (rc) return rc;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)t_pad, (cuuint64_t)n_kv * FD};
    const cuuint64_t strides[1] = {(cuuint64_t)t_pad * 2};
    const cuuint32_t box[2] = {FATOM, FD};
    int rc = make_map(&mv, vt, 2, dims, strides, box);
    if (rc) return rc;
  }
  FlashPrefillArgs a{T, n_q, n_q / n_kv, pos0, t_pad, (__nv_bfloat16*)out, ldo, status};
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(flash_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FSMEM);
    attr_set = true;
  }
  dim3 grid((T + FQ - 1) / FQ, n_q);
  return (int)launch(flash_prefill_kernel, grid, dim3(FTHREADS), (size_t)FSMEM, st, mq, mk, mv, a);
}

}  // extern "C"
