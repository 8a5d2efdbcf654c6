// Grouped GEMM on tcgen05 whose weight operand stays block-quantised in HBM (sm_100a only):
//   C[t, n] = sum_k X[t, k] * W[g][n, k]          W resident Q4_K / Q5_K / Q6_K / Q8_0, X bf16, fp32 accumulate
//
// The product is issued transposed: the 128 weight rows of a tile are the M side of the MMA and the tokens the N side
// (16 .. 128 per tile), so a decode batch of a few rows per expert pays for the tokens it has instead of a 128-row
// tile, and a prompt tile expands each weight once for 128 tokens.
//
//   * weights: eight producer warps decode 64-value units in registers and store bf16 into the 128-byte-swizzled A
//     stage (generic-proxy stores, fence.proxy.async, mbarrier arrive) -- the bf16 form of a weight never exists in
//     HBM.  The quantised super-blocks of the tile's 128 rows reach the producers through a ring of raw TMA boxes
//     ([128 rows x one super-block] of bytes, several in flight per SM, which is what a pass bound by weight
//     streaming needs), or, where the ring does not fit beside the operand stages (gate+up at 128 tokens, Q8_0),
//     by register loads one stage ahead;
//   * tokens: one TMA thread loads [tokens x 64] bf16 boxes into the B stage of the same ring;
//   * one elected thread issues tcgen05.mma (M = 128, N = tokens, K = 16) into TMEM, two accumulator buffers, so four
//     epilogue warps read tile i back with tcgen05.ld while tile i + 1 accumulates;
//   * "dual" mode runs gate and up in one main loop and the epilogue writes silu(gate) * up;
//   * the epilogue scatters and scales like the bf16 GEMM (dst_row / row_scale / resid): lane = weight row, so one
//     token's 32 outputs of a warp are one contiguous 128-byte (fp32) or 64-byte (bf16) store.
//
// Every mbarrier wait is bounded by the global timer; on expiry the CTA raises status word 1, leaves its loops,
// frees its TMEM and returns.
//
// Role in the reference: the int8 mma.sync grouped GEMMs that read quantised experts directly
// (crates/gpu/src/gemm/q4k_sel.rs, q6k_sel.rs, kernels.rs); there the activations are quantised to q8 and the
// product runs on mma.sync -- here the weights are expanded in flight and the product runs on tcgen05.
#define BL_UNITS_GENERIC_LD 1      // weight units are also read out of shared memory here: plain loads
#include "tc_common.cuh"

namespace bl {

constexpr int QBM = 128;                  // weight rows per tile (MMA M)
constexpr int QBK = 128;                  // depth per stage: two swizzle atoms of 64 values
constexpr int QATOM_A = QBM * 128;        // 16 KiB: 128 rows of 128 bytes
constexpr int QPRODUCERS = 256;           // threads that expand weights: (row, half of the stage's depth)
constexpr int QTHREADS = 192 + QPRODUCERS;

struct QTile { int group, row0, row_end, pad; };   // token tile: rows row0 .. of X use weight matrix `group`

struct QGemmArgs {
  const uint8_t* w;           // [n_groups][N rows][row_bytes]
  const uint8_t* w2;          // dual: the second matrix (same type and shape)
  long group_bytes, row_bytes;
  int N, K;
  int tiles_w;                // ceil(N / 128)
  const QTile* tiles;
  const int* n_tiles;
  int max_tiles;
  float* c_f32;
  __nv_bfloat16* c_bf16;
  long ldc;
  const int* dst_row;         // optional scatter of token rows (< 0 = drop)
  const float* row_scale;     // optional per-token factor
  const float* resid;         // optional addend, indexed like the output
  long ldr;
  unsigned* status;
};

__device__ __forceinline__ uint4 q_pack8(const float* v) {
  uint4 o;
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&a); o.y = *reinterpret_cast<uint32_t*>(&b);
  o.z = *reinterpret_cast<uint32_t*>(&c); o.w = *reinterpret_cast<uint32_t*>(&d);
  return o;
}

// Unit u (64 values of row `row`) of stage kb into the swizzled A stage at `sa`: value position p of the stage lives in
// atom p / 64, row `row`, 16-byte chunk ((p % 64) / 8) ^ (row % 8).
template <class T>
__device__ __forceinline__ void expand_unit(const typename Unit<T>::Regs& regs, int u, int kb, int row, uint8_t* sa) {
  float v[64];
  Unit<T>::decodeu(regs, u, v);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int p = Unit<T>::pos(u, 8 * j) - QBK * kb;
    const int atom = p >> 6, ch = (p & 63) >> 3;
    *reinterpret_cast<uint4*>(sa + atom * QATOM_A + row * 128 + ((ch ^ (row & 7)) << 4)) = q_pack8(v + 8 * j);
  }
}

// ---- fast expanders ---------------------------------------------------------------------
// Integer-to-float conversions run at a quarter of the FMA rate, so the K-quant expanders avoid them.
//   exact form (token tiles of 128, i.e. prompts): a code byte q (< 128) dropped into mantissa bits 16..22 of 1.0f
//   reads as X = 1 + q / 128, and the block's affine map v = s * q + o becomes one FMA
//   v = (128 s) * X + (o - 128 s) on a packed pair (fma.rn.f32x2), rounded to bf16 once.  The result equals the fp32
//   decode to within an fp32 rounding of the offset.
//   short form (token tiles of 32 / 64, i.e. decode batches, where the expanders are the bottleneck): two code bytes
//   become the bf16 pair (128 + q0, 128 + q1) with one byte permute, a packed bf16 subtract gives (q0, q1) exactly and
//   a packed bf16 FMA gives s * q + o with s and o rounded to bf16: 1.5 instructions per value, at most about one
//   more bf16 ulp of error per weight than the exact form.
// FastUnit<T>::codes yields the unit's 64 code bytes in value order (16 words; word w belongs to group w / 4) and the
// (scale, offset) pair of each of the four groups of 16 values.
template <class T> struct FastUnit { static constexpr bool kHas = false; };

template <> struct FastUnit<Q4K> {
  static constexpr bool kHas = true;
  static __device__ __forceinline__ void codes(const Q4K::Regs& r, int u, uint32_t* cw, float* s, float* o) {
    const int j = u & 3;
    const uint32_t w[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) { cw[i] = w[i] & 0x0F0F0F0Fu; cw[8 + i] = (w[i] >> 4) & 0x0F0F0F0Fu; }
    int sc0, mn0, sc1, mn1;
    Q4K::scale_min(r, 2 * j, sc0, mn0);
    Q4K::scale_min(r, 2 * j + 1, sc1, mn1);
    const float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF)), dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    s[0] = s[1] = d * sc0; o[0] = o[1] = -(dmin * mn0);
    s[2] = s[3] = d * sc1; o[2] = o[3] = -(dmin * mn1);
  }
};
template <> struct FastUnit<Q5K> {
  static constexpr bool kHas = true;
  static __device__ __forceinline__ void codes(const Q5K::Regs& r, int u, uint32_t* cw, float* s, float* o) {
    const int j = u & 3;
    Q5K::codes(r, u, cw, cw + 8);
    Q4K::Regs t; t.s0 = r.s0; t.s1 = r.s1; t.s2 = r.s2;
    int sc0, mn0, sc1, mn1;
    Q4K::scale_min(t, 2 * j, sc0, mn0);
    Q4K::scale_min(t, 2 * j + 1, sc1, mn1);
    const float d = half_bits_to_float((uint16_t)(r.dm & 0xFFFF)), dmin = half_bits_to_float((uint16_t)(r.dm >> 16));
    s[0] = s[1] = d * sc0; o[0] = o[1] = -(dmin * mn0);
    s[2] = s[3] = d * sc1; o[2] = o[3] = -(dmin * mn1);
  }
};
template <> struct FastUnit<Q6K> {
  static constexpr bool kHas = true;
  static __device__ __forceinline__ void codes(const Q6K::Regs& r, int u, uint32_t* cw, float* s, float* o) {
    const int n = (u >> 1) & 1, h = u & 1;
    uint32_t c[4][4];
    Q6K::codes(r, c);
    const float d = half_bits_to_float((uint16_t)r.d);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
#pragma unroll
      for (int i = 0; i < 4; ++i) cw[4 * g + i] = c[g][i];
      s[g] = d * (float)Q6K::scale(r, 8 * n + 2 * g + h);
      o[g] = -32.0f * s[g];
    }
  }
};

// bf16x2 of (a * x0 + c, a * x1 + c) with one packed FMA
__device__ __forceinline__ uint32_t fma2_bf16(uint32_t x0, uint32_t x1, float a, float c) {
  uint32_t lo, hi;
  asm("{\n\t.reg .b64 ra, rx, rc, rr;\n\t"
      "mov.b64 ra, {%2, %2};\n\tmov.b64 rx, {%3, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rr, ra, rx, rc;\n\tmov.b64 {%0, %1}, rr;\n\t}"
      : "=r"(lo), "=r"(hi) : "f"(a), "r"(x0), "r"(x1), "f"(c));
  __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ uint4 fast8(uint32_t w0, uint32_t w1, float a, float c) {
  w0 |= 0x80808080u; w1 |= 0x80808080u;
  uint4 out;
  out.x = fma2_bf16(__byte_perm(w0, 0x3F000000u, 0x7044), __byte_perm(w0, 0x3F000000u, 0x7144), a, c);
  out.y = fma2_bf16(__byte_perm(w0, 0x3F000000u, 0x7244), __byte_perm(w0, 0x3F000000u, 0x7344), a, c);
  out.z = fma2_bf16(__byte_perm(w1, 0x3F000000u, 0x7044), __byte_perm(w1, 0x3F000000u, 0x7144), a, c);
  out.w = fma2_bf16(__byte_perm(w1, 0x3F000000u, 0x7244), __byte_perm(w1, 0x3F000000u, 0x7344), a, c);
  return out;
}

// bf16x2 FMA / subtract on raw register pairs
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf2_dup(float v) {
  __nv_bfloat162 p = __float2bfloat162_rn(v);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ uint4 short8(uint32_t w0, uint32_t w1, uint32_t s2, uint32_t o2) {
  constexpr uint32_t k128 = 0x43004300u;                       // (128, 128) in bf16
  uint4 out;
  out.x = bf2_fma(bf2_sub(__byte_perm(w0, k128, 0x5150), k128), s2, o2);   // bytes (low to high): q0, 0x43, q1, 0x43
  out.y = bf2_fma(bf2_sub(__byte_perm(w0, k128, 0x5352), k128), s2, o2);
  out.z = bf2_fma(bf2_sub(__byte_perm(w1, k128, 0x5150), k128), s2, o2);
  out.w = bf2_fma(bf2_sub(__byte_perm(w1, k128, 0x5352), k128), s2, o2);
  return out;
}

template <class T, bool SHORT>
__device__ __forceinline__ void expand_unit_fast(const typename Unit<T>::Regs& regs, int u, int kb, int row, uint8_t* sa) {
  uint32_t cw[16];
  float s[4], o[4];
  FastUnit<T>::codes(regs, u, cw, s, o);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int g = j >> 1;
    const int p = Unit<T>::pos(u, 8 * j) - QBK * kb;
    const int atom = p >> 6, ch = (p & 63) >> 3;
    uint4* dst = reinterpret_cast<uint4*>(sa + atom * QATOM_A + row * 128 + ((ch ^ (row & 7)) << 4));
    if (SHORT) {
      *dst = short8(cw[2 * j], cw[2 * j + 1], bf2_dup(s[g]), bf2_dup(o[g]));
    } else {
      const float a = 128.0f * s[g], c = o[g] - a;
      *dst = fast8(cw[2 * j], cw[2 * j + 1], a, c);
    }
  }
}
// ---- float-coded types ---------------------------------------------------------------------
// ChunkUnit<T>::chunk(regs, j) yields values 8j .. 8j+7 of the unit as eight bf16, never holding the unit's 64 floats.
//   FP8 (E4M3 codes, one f32 scale per 128 values): the hardware converter takes two codes to an f16 pair; the pair
//   widens to f32, takes the block scale and is rounded to bf16 once.
//   NVFP4 (E2M1 codes, E4M3 scale per 16 values, f32 tensor scale): a code's magnitude is one of eight values, so two
//   byte permutes with the code nibbles as selectors look up the low and the high byte of bf16(2 * magnitude) for four
//   codes at once; the sign bits are gathered with two more permutes, and a packed bf16 multiply applies the group
//   scale (rounded to bf16: the code values have two significant bits, so the product is exact in bf16 but for that
//   rounding of the scale).
template <class T> struct ChunkUnit { static constexpr bool kHas = false; };

template <> struct ChunkUnit<Fp8B128> {
  static constexpr bool kHas = true;
  struct Pre { float sc; };
  static __device__ __forceinline__ Pre pre(const Fp8B128::Regs& r) { return Pre{r.sc}; }
  static __device__ __forceinline__ uint4 chunk(const Fp8B128::Regs& r, const Pre& pr, int j) {
    const u32x4& q = r.q[j >> 1];
    const uint32_t w0 = (j & 1) ? q.z : q.x, w1 = (j & 1) ? q.w : q.y;
    float f[8];
    e4m3x4_to_float(w0, f);
    e4m3x4_to_float(w1, f + 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= pr.sc;
    return q_pack8(f);
  }
};

template <> struct ChunkUnit<NvFp4> {
  static constexpr bool kHas = true;
  struct Pre { uint32_t s2[4]; };
  static __device__ __forceinline__ Pre pre(const NvFp4::Regs& r) {
    float sc[4];
    e4m3x4_to_float(r.sc, sc);
    Pre pr;
#pragma unroll
    for (int g = 0; g < 4; ++g) pr.s2[g] = bf2_dup(sc[g] * r.g * 0.5f);   // the table below holds 2 * magnitude
    return pr;
  }
  static __device__ __forceinline__ uint4 chunk(const NvFp4::Regs& r, const Pre& pr, int j) {
    const uint32_t w = j == 0 ? r.q0.x : j == 1 ? r.q0.y : j == 2 ? r.q0.z : j == 3 ? r.q0.w
                     : j == 4 ? r.q1.x : j == 5 ? r.q1.y : j == 6 ? r.q1.z : r.q1.w;
    const uint32_t sel = w & 0x77777777u;
    const uint32_t sodd = w & 0x80808080u, seven = (w << 4) & 0x80808080u;   // signs of the odd / the even codes
    const uint32_t s2 = pr.s2[j >> 1];
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t c = h ? sel >> 16 : sel;
      const uint32_t lo4 = __byte_perm(0x40008000u, 0x4000C080u, c);
      const uint32_t hi4 = __byte_perm(0x40403F00u, 0x41414040u, c) | __byte_perm(seven, sodd, h ? 0x7362 : 0x5140);
      o[2 * h] = bf2_fma(__byte_perm(lo4, hi4, 0x5140), s2, 0u);
      o[2 * h + 1] = bf2_fma(__byte_perm(lo4, hi4, 0x7362), s2, 0u);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
  }
};

template <class T>
__device__ __forceinline__ void expand_unit_chunks(const typename Unit<T>::Regs& regs, int u, int kb, int row, uint8_t* sa) {
  const typename ChunkUnit<T>::Pre pr = ChunkUnit<T>::pre(regs);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int p = Unit<T>::pos(u, 8 * j) - QBK * kb;
    const int atom = p >> 6, ch = (p & 63) >> 3;
    *reinterpret_cast<uint4*>(sa + atom * QATOM_A + row * 128 + ((ch ^ (row & 7)) << 4)) = ChunkUnit<T>::chunk(regs, pr, j);
  }
}

template <class T, bool SHORT>
__device__ __forceinline__ void expand_any(const typename Unit<T>::Regs& regs, int u, int kb, int row, uint8_t* sa) {
  if constexpr (FastUnit<T>::kHas) expand_unit_fast<T, SHORT>(regs, u, kb, row, sa);
  else if constexpr (ChunkUnit<T>::kHas) expand_unit_chunks<T>(regs, u, kb, row, sa);
  else expand_unit<T>(regs, u, kb, row, sa);
}

__host__ __device__ constexpr int q_stages(bool dual, int bn) {
  const int stage = (dual ? 2 : 1) * 2 * QATOM_A + 2 * bn * 128;
  const int n = (220 * 1024) / stage;
  return n > 4 ? 4 : n;
}
// Raw ring: slots of [matrices][128 rows][super-block bytes]; 0 slots = the register-load path.
template <class T> struct SbBytes { static constexpr int v = 0; };
template <> struct SbBytes<Q4K> { static constexpr int v = Q4K::kSbBytes; };
template <> struct SbBytes<Q5K> { static constexpr int v = Q5K::kSbBytes; };
template <> struct SbBytes<Q6K> { static constexpr int v = Q6K::kSbBytes; };
__host__ __device__ constexpr int q_raw_slots(int sb_bytes, bool dual, int bn) {
  if (sb_bytes == 0) return 0;
  const int stage = (dual ? 2 : 1) * 2 * QATOM_A + 2 * bn * 128;
  const int raw = (dual ? 2 : 1) * QBM * sb_bytes;
  const int n = (220 * 1024 - 2 * stage) / raw;
  const int cap = dual ? 2 : 4;                                    // super-blocks in flight per SM; the rest goes to stages
  return n > cap ? cap : (n < 0 ? 0 : n);
}
__host__ __device__ constexpr int q_stages_raw(int sb_bytes, bool dual, int bn) {
  const int stage = (dual ? 2 : 1) * 2 * QATOM_A + 2 * bn * 128;
  const int raw = (dual ? 2 : 1) * QBM * sb_bytes;
  const int n = (220 * 1024 - q_raw_slots(sb_bytes, dual, bn) * raw) / stage;
  return n > 4 ? 4 : n;
}
__host__ __device__ constexpr int q_tmem_cols(bool dual, int bn) {
  const int need = 2 * (dual ? 2 : 1) * bn;
  return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}

// 448 threads: warp 0 = TMA producer of the token tiles, warp 1 = MMA issuer and TMEM owner, warps 2..5 = epilogue
// (warp id modulo 4 = TMEM lane quarter), warps 6..13 = weight expanders.
template <class T, bool DUAL, int BN>
__global__ void __launch_bounds__(QTHREADS, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tma_x, const __grid_constant__ CUtensorMap tma_w,
             const __grid_constant__ CUtensorMap tma_w2, const QGemmArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int SB = SbBytes<T>::v;
  constexpr int RS = q_raw_slots(SB, DUAL, BN);                      // raw ring slots (0: register loads)
  constexpr int RAW_MAT = QBM * SB;                                  // one matrix's 128 super-blocks
  constexpr int RAW_SLOT = (DUAL ? 2 : 1) * RAW_MAT;
  constexpr int STAGES = RS > 0 ? q_stages_raw(SB, DUAL, BN) : q_stages(DUAL, BN);
  constexpr int A_BYTES = 2 * QATOM_A;
  constexpr int B_ATOM = BN * 128;
  constexpr int STAGE_BYTES = (DUAL ? 2 : 1) * A_BYTES + 2 * B_ATOM;
  constexpr int B_OFF = (DUAL ? 2 : 1) * A_BYTES;
  constexpr int ACC_COLS = (DUAL ? 2 : 1) * BN;
  constexpr int TMEM_COLS = q_tmem_cols(DUAL, BN);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ __align__(8) uint64_t raw_full[RS > 0 ? RS : 1], raw_empty[RS > 0 ? RS : 1];
  uint8_t* const raw_ring = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023) + (size_t)STAGES * STAGE_BYTES;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1 + QPRODUCERS / 32); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    for (int r = 0; r < RS; ++r) { mbar_init(&raw_full[r], 1); mbar_init(&raw_empty[r], QPRODUCERS / 32); }
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
  const int kblocks = a.K / QBK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int rslot = 0; uint32_t rphase = 0;
      int issued = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const QTile mt = a.tiles[t / a.tiles_w];
        const int n0 = (t % a.tiles_w) * QBM;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (RS > 0 && (kb & 1) == 0) {
            // the super-block of stages kb and kb + 1: rows n0 .. n0 + 127 of the group's matrix (rows past the
            // matrix arrive as zeros and are never stored)
            if (!mbar_wait(&raw_empty[rslot], rphase ^ 1, abort_flag)) break;
            uint8_t* dst = raw_ring + (size_t)rslot * RAW_SLOT;
            mbar_expect_tx(&raw_full[rslot], RAW_SLOT);
            tma_load_3d(dst, &tma_w, (kb >> 1) * SB, n0, mt.group, &raw_full[rslot]);
            if (DUAL) tma_load_3d(dst + RAW_MAT, &tma_w2, (kb >> 1) * SB, n0, mt.group, &raw_full[rslot]);
            if (++rslot == RS) { rslot = 0; rphase ^= 1; }
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) break;
          uint8_t* sb = smem + (size_t)stage * STAGE_BYTES + B_OFF;
          mbar_expect_tx(&full_bar[stage], 2 * B_ATOM);
          tma_load_2d(sb, &tma_x, kb * QBK, mt.row0, &full_bar[stage]);
          tma_load_2d(sb + B_ATOM, &tma_x, kb * QBK + 64, mt.row0, &full_bar[stage]);
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
      constexpr uint32_t idesc = umma_idesc(QBM, BN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&acc_empty[ab], acc_phase ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + ab * ACC_COLS;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * STAGE_BYTES);
#pragma unroll
          for (int atom = 0; atom < 2; ++atom) {
            const uint64_t da = umma_desc(sa + atom * QATOM_A), db = umma_desc(sa + B_OFF + atom * B_ATOM);
#pragma unroll
            for (int k = 0; k < 64 / UMMA_K; ++k) {
              const uint32_t acc = (kb > 0 || atom > 0 || k > 0) ? 1u : 0u;
              const uint64_t step = (uint64_t)(k * UMMA_K * 2 / 16);
              umma_bf16(d0, da + step, db + step, idesc, acc);
              if (DUAL) umma_bf16(d0 + BN, umma_desc(sa + A_BYTES + atom * QATOM_A) + step, db + step, idesc, acc);
            }
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[ab]);
      }
    }
  } else if (warp < 6) {
    const int q = warp & 3;
    int it = 0;
    for (int t = blockIdx.x; t < total_tiles && !*abort_flag; t += gridDim.x) {
      const QTile mt = a.tiles[t / a.tiles_w];
      const int n = (t % a.tiles_w) * QBM + q * 32 + lane;         // weight row = output column of this thread
      const bool n_ok = n < a.N;
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&acc_full[ab], acc_phase, abort_flag)) break;
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + ab * ACC_COLS;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (mt.row0 + c * 32 >= mt.row_end) break;
        uint32_t v[32], u[32];
        tmem_ld32(tbase + c * 32, v);
        if (DUAL) tmem_ld32(tbase + BN + c * 32, u);
        tmem_ld_wait();
        // lane i fetches the routing of token row i of this chunk; the store loop broadcasts it
        const int r_l = mt.row0 + c * 32 + lane;
        int orow_l = -1;
        float sc_l = 1.0f;
        if (r_l < mt.row_end) {
          orow_l = a.dst_row ? a.dst_row[r_l] : r_l;
          if (a.row_scale) sc_l = a.row_scale[r_l];
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int orow = __shfl_sync(0xFFFFFFFFu, orow_l, i);
          const float sc = __shfl_sync(0xFFFFFFFFu, sc_l, i);
          if (orow < 0 || !n_ok) continue;
          float f = __uint_as_float(v[i]);
          if (DUAL) f = (f / (1.0f + __expf(-f))) * __uint_as_float(u[i]);
          f *= sc;
          if (a.resid) f += a.resid[(long)orow * a.ldr + n];
          if (a.c_f32) a.c_f32[(long)orow * a.ldc + n] = f;
          else a.c_bf16[(long)orow * a.ldc + n] = __float2bfloat16_rn(f);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[ab]);
    }
  } else {
    // Producer thread = (weight row, part): in dual mode the part is the matrix (gate / up) and the thread expands both
    // units of the stage; otherwise the part is the unit.  The blocks of stage kb + 1 are fetched into a second register
    // set before stage kb is decoded, so a load has a whole decode (and the wait for the ring) to land.
    using U = Unit<T>;
    constexpr int NU = DUAL ? 2 : 1;
    const int pt = threadIdx.x - 192;
    const int row = pt & 127, part = pt >> 7;
    int stage = 0; uint32_t phase = 0;
    bool ok = true;
    auto fetch = [&](const uint8_t* wrow, int kb, typename U::Regs (&r)[NU]) {
#pragma unroll
      for (int i = 0; i < NU; ++i) U::loadu(wrow, 2 * kb + (DUAL ? i : part), a.K, r[i]);
    };
    auto emit = [&](int kb, const typename U::Regs (&r)[NU]) {
      if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; return; }
      tc_fence_after();
      uint8_t* sa = smem + (size_t)stage * STAGE_BYTES + (DUAL ? part * A_BYTES : 0);
#pragma unroll
      for (int i = 0; i < NU; ++i) expand_any<T, (BN < 128)>(r[i], 2 * kb + (DUAL ? i : part), kb, row, sa);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[stage]);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    };
    if constexpr (RS > 0) {
      // raw ring: the tile's super-blocks arrive by TMA; a thread reads its row's units out of shared memory
      int rslot = 0; uint32_t rphase = 0;
      for (int t = blockIdx.x; t < total_tiles && ok && !*abort_flag; t += gridDim.x) {
        for (int sbi = 0; sbi < kblocks / 2 && ok; ++sbi) {
          if (!mbar_wait(&raw_full[rslot], rphase, abort_flag)) { ok = false; break; }
          const uint8_t* rawrow = raw_ring + (size_t)rslot * RAW_SLOT + (DUAL ? part * RAW_MAT : 0) + row * SB - (long)sbi * SB;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int kb = 2 * sbi + half;
            typename U::Regs r[NU];
            fetch(rawrow, kb, r);
            emit(kb, r);
            if (!ok) break;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&raw_empty[rslot]);
          if (++rslot == RS) { rslot = 0; rphase ^= 1; }
        }
      }
    } else
    for (int t = blockIdx.x; t < total_tiles && ok && !*abort_flag; t += gridDim.x) {
      const QTile mt = a.tiles[t / a.tiles_w];
      int n = (t % a.tiles_w) * QBM + row;
      n = n < a.N ? n : a.N - 1;                                   // rows past the matrix repeat the last one (never stored)
      const uint8_t* wrow = (DUAL && part ? a.w2 : a.w) + (long)mt.group * a.group_bytes + (long)n * a.row_bytes;
      typename U::Regs ra[NU], rb[NU];
      fetch(wrow, 0, ra);
      for (int kb = 0; kb < kblocks && ok; kb += 2) {
        if (kb + 1 < kblocks) fetch(wrow, kb + 1, rb);
        emit(kb, ra);
        if (!ok) break;
        if (kb + 2 < kblocks) fetch(wrow, kb + 2, ra);
        if (kb + 1 < kblocks) emit(kb + 1, rb);
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

template <class T, bool DUAL, int BN>
static int qgemm_go(const CUtensorMap& mx, const QGemmArgs& a, int n_groups, int grid, cudaStream_t st) {
  constexpr int SB = SbBytes<T>::v;
  constexpr int RS = q_raw_slots(SB, DUAL, BN);
  constexpr int STAGES = RS > 0 ? q_stages_raw(SB, DUAL, BN) : q_stages(DUAL, BN);
  constexpr size_t smem = (size_t)STAGES * ((DUAL ? 2 : 1) * 2 * QATOM_A + 2 * BN * 128) + (size_t)RS * (DUAL ? 2 : 1) * QBM * SB + 1024;
  CUtensorMap mw = mx, mw2 = mx;
  if (RS > 0) {
    cuuint64_t dims[3] = {(cuuint64_t)a.row_bytes, (cuuint64_t)a.N, (cuuint64_t)n_groups};
    cuuint64_t str[2] = {(cuuint64_t)a.row_bytes, (cuuint64_t)a.group_bytes};
    cuuint32_t box[3] = {(cuuint32_t)SB, QBM, 1};
    int rc = make_map_u8(&mw, a.w, 3, dims, str, box);
    if (rc) return rc;
    if (DUAL) { rc = make_map_u8(&mw2, a.w2, 3, dims, str, box); if (rc) return rc; }
  }
  static bool set = false;
  if (!set) {
    cudaFuncSetAttribute(qgemm_kernel<T, DUAL, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    set = true;
  }
  return (int)launch(qgemm_kernel<T, DUAL, BN>, dim3(grid), dim3(QTHREADS), smem, st, mx, mw, mw2, a);
}

template <class T>
static int qgemm_pick(bool dual, int bn, const CUtensorMap& mx, const QGemmArgs& a, int n_groups, int grid, cudaStream_t st) {
  if (dual) {
    if (bn == 128) return qgemm_go<T, true, 128>(mx, a, n_groups, grid, st);
    if (bn == 64) return qgemm_go<T, true, 64>(mx, a, n_groups, grid, st);
    if (bn == 32) return qgemm_go<T, true, 32>(mx, a, n_groups, grid, st);
  } else {
    if (bn == 128) return qgemm_go<T, false, 128>(mx, a, n_groups, grid, st);
    if (bn == 64) return qgemm_go<T, false, 64>(mx, a, n_groups, grid, st);
    if (bn == 32) return qgemm_go<T, false, 32>(mx, a, n_groups, grid, st);
  }
  return BL_ERR_SHAPE;
}

}  // namespace bl

using namespace bl;

extern "C" {

// 1 when bl_qgemm has a kernel for this weight type
int bl_qgemm_supports(int wtype) {
  return wtype == WT_Q4_K || wtype == WT_Q5_K || wtype == WT_Q6_K || wtype == WT_Q8_0 || wtype == WT_FP8_B128 || wtype == WT_NVFP4 ||
         wtype == WT_Q8_F32;
}

// C[dst_row[t] or t, n] = row_scale[t] * sum_k X[t, k] W[g][n, k] (+ resid), per token tile of the table.
//   X [rows_x, K] bf16 (ldx elements); W, W2 [n_groups, N, row_bytes] resident blocks of type wtype;
//   tiles: {group, row0, row_end, -} token tiles of at most tile_rows (32, 64 or 128) rows; exactly one of c_f32 / c_bf16;
//   W2 != null: output = silu(X W^T) * (X W2^T).  status: device word, set to 1 when a wait ran out.
int bl_qgemm(const void* X, long ldx, long rows_x, const void* W, const void* W2, int wtype, int n_groups, int N, int K,
             const void* tiles, const int* n_tiles, int max_tiles, int tile_rows, float* c_f32, void* c_bf16, long ldc,
             const int* dst_row, const float* row_scale, const float* resid, long ldr, unsigned* status, int sm_count,
             cudaStream_t st) {
  BL_REQUIRE(K >= 256 && K % 256 == 0 && N >= 1 && rows_x >= 1 && n_groups >= 1 && max_tiles >= 1, BL_ERR_SHAPE);
  BL_REQUIRE(tile_rows == 32 || tile_rows == 64 || tile_rows == 128, BL_ERR_SHAPE);
  BL_REQUIRE(ldx % 8 == 0 && ((uintptr_t)X & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)W2 & 15) == 0, BL_ERR_ALIGN);
  BL_REQUIRE((c_f32 != nullptr) != (c_bf16 != nullptr), BL_ERR_SHAPE);
  const long rb = resident_row_bytes(wtype, K);
  BL_REQUIRE(rb > 0 && bl_qgemm_supports(wtype), BL_ERR_TYPE);
  CUtensorMap mx;
  {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows_x};
    cuuint64_t str[1] = {(cuuint64_t)ldx * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)tile_rows};
    int rc = make_map(&mx, X, 2, dims, str, box);
    if (rc) return rc;
  }
  QGemmArgs a{};
  a.w = (const uint8_t*)W; a.w2 = (const uint8_t*)W2;
  a.row_bytes = rb; a.group_bytes = rb * N;
  a.N = N; a.K = K; a.tiles_w = (N + QBM - 1) / QBM;
  a.tiles = (const QTile*)tiles; a.n_tiles = n_tiles; a.max_tiles = max_tiles;
  a.c_f32 = c_f32; a.c_bf16 = (__nv_bfloat16*)c_bf16; a.ldc = ldc;
  a.dst_row = dst_row; a.row_scale = row_scale; a.resid = resid; a.ldr = ldr; a.status = status;
  const long tiles_total = (long)max_tiles * a.tiles_w;
  const int grid = (int)(tiles_total < sm_count ? tiles_total : sm_count);
  const bool dual = W2 != nullptr;
  switch (wtype) {
    case WT_Q4_K: return qgemm_pick<Q4K>(dual, tile_rows, mx, a, n_groups, grid, st);
    case WT_Q5_K: return qgemm_pick<Q5K>(dual, tile_rows, mx, a, n_groups, grid, st);
    case WT_Q6_K: return qgemm_pick<Q6K>(dual, tile_rows, mx, a, n_groups, grid, st);
    case WT_Q8_0: return qgemm_pick<Q80>(dual, tile_rows, mx, a, n_groups, grid, st);
    case WT_FP8_B128: return qgemm_pick<Fp8B128>(dual, tile_rows, mx, a, n_groups, grid, st);
    case WT_NVFP4: return qgemm_pick<NvFp4>(dual, tile_rows, mx, a, n_groups, grid, st);
    case WT_Q8_F32: return qgemm_pick<Q8F>(dual, tile_rows, mx, a, n_groups, grid, st);
  }
  return BL_ERR_TYPE;
}

}  // extern "C"
