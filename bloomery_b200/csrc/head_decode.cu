// Token embedding gather, arg-max head and small utilities of the decode chain.
//
// embed_rows decodes one quantised row of the embedding table per token
// (crates/gpu/src/elem.rs embed_rows{,_q4k,_q6k,...} in the reference).  argmax_rows
// follows the greedy tie rule of crates/sampler/src/lib.rs:434-459 (strictly greater
// wins, equal wins at the lower id, NaN never wins, an all-NaN row gives id 0) and copies
// the fault word beside the tokens so one small read returns both
// (crates/gpu/src/elem.rs argmax_rows_fault).
#include "common.cuh"

namespace bl {

struct EmbedArgs {
  const int* tokens; int M;
  const uint8_t* table; int wtype; int K; int vocab;
  float* out; long out_stride;
  unsigned* fault;
  unsigned* step;       // optional: pass counter, bumped once per launch (epochs of the fused reductions)
};

template <class T>
__device__ __forceinline__ void embed_row_q(const uint8_t* row, int K, float* out, int tid, int nthr) {
  using U = Unit<T>;
  for (int u = tid; u < K / 64; u += nthr) {
    typename U::Regs r;
    U::loadu(row, u, K, r);
    float v[64];
    U::decodeu(r, u, v);
#pragma unroll
    for (int e = 0; e < 64; ++e) out[U::pos(u, e)] = v[e];
  }
}

__global__ void __launch_bounds__(128) embed_rows_kernel(const EmbedArgs a) {
  const int m = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  if (a.step && m == 0 && tid == 0) *a.step = *a.step + 1u;
  const int tok = a.tokens[m];
  float* out = a.out + (long)m * a.out_stride;
  if (tok < 0 || tok >= a.vocab) {
    if (tid == 0) raise_fault(a.fault, 0, FS_TOKEN_ID);
    for (int i = tid; i < a.K; i += 128) out[i] = __int_as_float(0x7fc00000);
    return;
  }
  const uint8_t* row = a.table + (long)tok * resident_row_bytes(a.wtype, a.K);
  switch (a.wtype) {
    case WT_Q4_K: embed_row_q<Q4K>(row, a.K, out, tid, 128); break;
    case WT_Q5_K: embed_row_q<Q5K>(row, a.K, out, tid, 128); break;
    case WT_Q6_K: embed_row_q<Q6K>(row, a.K, out, tid, 128); break;
    case WT_Q8_0: embed_row_q<Q80>(row, a.K, out, tid, 128); break;
    case WT_Q8_F32: embed_row_q<Q8F>(row, a.K, out, tid, 128); break;
    case WT_NVFP4: embed_row_q<NvFp4>(row, a.K, out, tid, 128); break;
    case WT_FP8_B128: embed_row_q<Fp8B128>(row, a.K, out, tid, 128); break;
    case WT_Q2_K: embed_row_q<Q2K>(row, a.K, out, tid, 128); break;
    case WT_Q3_K: embed_row_q<Q3K>(row, a.K, out, tid, 128); break;
    case WT_Q4_0: embed_row_q<Q40>(row, a.K, out, tid, 128); break;
    case WT_Q4_1: embed_row_q<Q41>(row, a.K, out, tid, 128); break;
    case WT_Q5_0: embed_row_q<Q50>(row, a.K, out, tid, 128); break;
    case WT_Q5_1: embed_row_q<Q51>(row, a.K, out, tid, 128); break;
    case WT_F32: for (int i = tid; i < a.K; i += 128) out[i] = reinterpret_cast<const float*>(row)[i]; break;
    case WT_F16: for (int i = tid; i < a.K; i += 128) out[i] = __half2float(reinterpret_cast<const __half*>(row)[i]); break;
    case WT_BF16: for (int i = tid; i < a.K; i += 128) out[i] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(row)[i]); break;
    default: for (int i = tid; i < a.K; i += 128) out[i] = __int_as_float(0x7fc00000);
  }
}

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  // NaN compares false everywhere, so it never wins
  return v > bv || (v == bv && i < bi);
}

struct ArgmaxArgs {
  const float* logits; long stride; int V; int M;
  float* part_v; int* part_i;      // [M, nblk]
  unsigned* counter;
  int* tokens_out;                 // [M] + 1 word: fault copy
  float* best_val;                 // optional [M]
  const unsigned* fault;
};

// grid (nblk, M), 256 threads
__global__ void __launch_bounds__(256) argmax_rows_kernel(const ArgmaxArgs a) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ unsigned s_ticket;
  const int b = blockIdx.x, nblk = gridDim.x, m = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_launch();
  const float* row = a.logits + (long)m * a.stride;
  float bv = -INFINITY; int bi = 0x7fffffff;
  for (int i = b * 256 + tid; i < a.V; i += nblk * 256) {
    float v = row[i];
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < 8; ++w) if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    a.part_v[(long)m * nblk + b] = bv;
    a.part_i[(long)m * nblk + b] = bi;
    __threadfence();
    s_ticket = atomicAdd(a.counter, 1u);
  }
  __syncthreads();
  if (s_ticket != (unsigned)(nblk * a.M) - 1) return;
  __threadfence();
  if (tid == 0) *a.counter = 0u;
  for (int mm = warp; mm < a.M; mm += 8) {
    float v = -INFINITY; int id = 0x7fffffff;
    for (int i = lane; i < nblk; i += 32) {
      float pv = __ldcg(a.part_v + (long)mm * nblk + i);
      int pi = __ldcg(a.part_i + (long)mm * nblk + i);
      if (better(pv, pi, v, id)) { v = pv; id = pi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, v, o);
      int oi = __shfl_xor_sync(0xffffffffu, id, o);
      if (better(ov, oi, v, id)) { v = ov; id = oi; }
    }
    if (lane == 0) {
      a.tokens_out[mm] = (id == 0x7fffffff) ? 0 : id;
      if (a.best_val) a.best_val[mm] = v;
    }
  }
  if (tid == 0) a.tokens_out[a.M] = a.fault ? (int)*a.fault : -1;
}

__global__ void fill_u32_kernel(unsigned* p, unsigned v, int n) {
  pdl_wait();
  pdl_launch();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

// advance per-row positions after a step and feed the chosen token back (chained decode)
// and log the picks into a device-side history ring so a chain of replays is read once
__global__ void advance_rows_kernel(int* tokens, int* row_pos, const int* row_seq, const int* chosen, int M,
                                    int* hist, int hist_cap, int* hist_count) {
  pdl_wait();
  pdl_launch();
  int m = threadIdx.x;
  int slot = hist ? *hist_count : 0;
  if (m < M && row_seq[m] >= 0) { tokens[m] = chosen[m]; row_pos[m] += 1; }
  if (hist && m < M && slot < hist_cap) hist[(long)slot * M + m] = chosen[m];
  __syncthreads();
  if (hist && m == 0) *hist_count = slot + 1;
}


// SwiGLU of a dense FFN: gu holds [gate | up] rows of width I each; result goes out as q8
// (and optionally fp32) for the down projection.  grid (I/32, M), one warp per 32 values.
__global__ void __launch_bounds__(32) swiglu_q8_kernel(const float* gu, long gu_stride, int I, int8_t* actq,
                                                      float2* actds, float* act_f32) {
  pdl_wait();
  pdl_launch();
  const int c = blockIdx.x, m = blockIdx.y, lane = threadIdx.x;
  const float g = gu[(long)m * gu_stride + c * 32 + lane];
  const float u = gu[(long)m * gu_stride + I + c * 32 + lane];
  const float v = (g / (1.0f + expf(-g))) * u;
  float d, s;
  int8_t q = q8_lane(v, d, s);
  actq[(long)m * I + c * 32 + lane] = q;
  if (act_f32) act_f32[(long)m * I + c * 32 + lane] = v;
  if (lane == 0) actds[((long)m * I) / 32 + c] = make_float2(d, s);
}


// Input of the multi-token-prediction layer: row m = [ RMSNorm(e[m]) * enorm | RMSNorm(h[src[m]]) * hnorm ],
// quantised to q8 for the eh_proj product (K = 2H).  e = embedding of the token that follows position m,
// h = the trunk's final hidden state of the row it was computed in (src maps draft rows to pass rows).
// grid (M), 256 threads; dynamic shared memory: nothing (red is static)
__global__ void __launch_bounds__(256) mtp_prep_kernel(const float* e, long e_stride, const float* h, long h_stride,
                                                       const int* src, const float* enorm, const float* hnorm, float eps,
                                                       int H, int8_t* xq, float2* xds) {
  __shared__ __align__(8) float red[64];
  const int m = blockIdx.x;
  pdl_wait();
  pdl_launch();
  const int sm = src ? src[m] : m;
  block_rmsnorm_q8(e + (long)m * e_stride, enorm, H, eps, xq + (long)m * 2 * H, xds + (long)m * (2 * H / 32), red, nullptr);
  block_rmsnorm_q8(h + (long)sm * h_stride, hnorm, H, eps, xq + (long)m * 2 * H + H, xds + (long)m * (2 * H / 32) + H / 32, red, nullptr);
}

}  // namespace bl

using namespace bl;

extern "C" {

int bl_embed_rows(const int* tokens, int M, const void* table, int wtype, int K, int vocab, float* out, long out_stride,
                  unsigned* fault, unsigned* step, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && K % 64 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(resident_row_bytes(wtype, K) > 0, BL_ERR_TYPE);
  EmbedArgs a{tokens, M, (const uint8_t*)table, wtype, K, vocab, out, out_stride, fault, step};
  return (int)launch(embed_rows_kernel, dim3(M), dim3(128), 0, st, a);
}

// scratch: part_v/part_i of M*nblk entries each; counter one zeroed word
int bl_argmax_rows(const float* logits, long stride, int V, int M, int nblk, float* part_v, int* part_i,
                   unsigned* counter, int* tokens_out, float* best_val, const unsigned* fault, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && V >= 1 && nblk >= 1, BL_ERR_SHAPE);
  ArgmaxArgs a{logits, stride, V, M, part_v, part_i, counter, tokens_out, best_val, fault};
  return (int)launch(argmax_rows_kernel, dim3(nblk, M), dim3(256), 0, st, a);
}

int bl_fill_u32(unsigned* p, unsigned v, int n, cudaStream_t st) {
  return (int)launch(fill_u32_kernel, dim3((n + 255) / 256), dim3(256), 0, st, p, v, n);
}

int bl_advance_rows(int* tokens, int* row_pos, const int* row_seq, const int* chosen, int M, int* hist, int hist_cap,
                    int* hist_count, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && M <= 1024, BL_ERR_SHAPE);
  return (int)launch(advance_rows_kernel, dim3(1), dim3(1024), 0, st, tokens, row_pos, row_seq, chosen, M, hist,
                     hist_cap, hist_count);
}

int bl_swiglu_q8(const float* gu, long gu_stride, int I, int M, int8_t* actq, float* actds, float* act_f32,
                 cudaStream_t st) {
  BL_REQUIRE(I % 32 == 0 && M >= 1, BL_ERR_SHAPE);
  return (int)launch(swiglu_q8_kernel, dim3(I / 32, M), dim3(32), 0, st, gu, gu_stride, I, actq, (float2*)actds, act_f32);
}

int bl_mtp_prep(const float* e, long e_stride, const float* h, long h_stride, const int* src, const float* enorm,
                const float* hnorm, float eps, int H, int M, int8_t* xq, float* xds, cudaStream_t st) {
  BL_REQUIRE(H % 32 == 0 && M >= 1 && enorm && hnorm, BL_ERR_SHAPE);
  return (int)launch(mtp_prep_kernel, dim3(M), dim3(256), 0, st, e, e_stride, h, h_stride, src, enorm, hnorm, eps, H, xq,
                     (float2*)xds);
}

const char* bl_error_string(int code) {
  if (code == 0) return "ok";
  if (code == BL_ERR_SHAPE) return "launch contract: bad shape";
  if (code == BL_ERR_TYPE) return "launch contract: unsupported weight type";
  if (code == BL_ERR_ALIGN) return "launch contract: pointer not 16-byte aligned";
  if (code == BL_ERR_LIMIT) return "launch contract: size beyond the kernel's limit";
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  return "unknown";
}

}  // extern "C"
