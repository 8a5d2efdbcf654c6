// Shared device helpers: fault word, programmatic dependent launch, reductions,
// the block-level q8 activation quantiser and the launch wrapper.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math.h>

#include "quant_units.cuh"

namespace bl {

// ------------------------------------------------------------------------------------
// Fault word.  One u32 per engine, 0xFFFFFFFF = clean.  A kernel that meets bad data
// keeps every access defined, writes NaN (never a plausible value) and lowers the word
// to (layer << 8) | site with atomicMin, so the first site in layer order wins and the
// word is sticky until the host resets it.  Same idea as crates/gpu/src/fault.rs:1-46
// in the reference; nothing here ever traps.
// ------------------------------------------------------------------------------------
enum FaultSite : unsigned {
  FS_TOKEN_ID = 1,
  FS_NONFINITE_ACT = 2,
  FS_ROUTER = 3,
  FS_EXPERT_ID = 4,
  FS_KEY_COUNT = 5,
  FS_PAGE = 6,
  FS_WAIT_TIMEOUT = 7,
  FS_SAMPLER = 8,
};

__device__ __forceinline__ void raise_fault(unsigned* fault, int layer, unsigned site) {
  if (fault) atomicMin(fault, ((unsigned)layer << 8) | site);
}

// Expert id sentinel: a routed slot that another tier serves (host RAM leg, a peer).
// Kernels skip it silently; any other id >= n_expert is a fault.
constexpr int kExpertElsewhere = -1;

// ------------------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the decode chain loads what does not
// depend on its predecessor (weights) first, then waits for the predecessor's memory.
// Each kernel calls pdl_wait() exactly once before reading or writing activations, which
// keeps the chain transitively ordered.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Quantise 32 consecutive values held one per lane.  Returns the code; lane 0 gets {d, s}.
__device__ __forceinline__ int8_t q8_lane(float v, float& d_out, float& s_out) {
  float amax = warp_max(fabsf(v));
  float d = amax / 127.0f;
  float inv = d > 0.f ? 1.0f / d : 0.f;
  int q = __float2int_rn(v * inv);
  q = max(-127, min(127, q));
  int sum = q;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  d_out = d;
  s_out = d * (float)sum;
  return (int8_t)q;
}

// RMS-normalise `x` (fp32, K values) with `gain`, quantise to q8 into shared memory.
// All threads of the block take part; K % 32 == 0.  `red` is >= 32 floats of scratch.
// Sum of squares is accumulated in fp32 per thread and in double across the block, in
// a fixed order, so reruns are bit-identical.
__device__ __forceinline__ void block_rmsnorm_q8(const float* __restrict__ x, const float* __restrict__ gain,
                                                 int K, float eps, int8_t* sq, float2* sds, float* red,
                                                 float* normed_out /* optional global/shared fp32 */) {
  const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = nthr >> 5;
  float ss = 0.f;
  for (int i = tid; i < K; i += nthr) { float v = x[i]; ss += v * v; }
  double tot = warp_sum_d((double)ss);
  double* redd = reinterpret_cast<double*>(red);
  __syncthreads();
  if (lane == 0) redd[warp] = tot;
  __syncthreads();
  double all = 0.0;
  for (int w = 0; w < nwarp; ++w) all += redd[w];
  float scale = (float)(1.0 / sqrt(all / (double)K + (double)eps));
  for (int b = warp; b < K / 32; b += nwarp) {
    int i = b * 32 + lane;
    float v = x[i] * scale * gain[i];
    if (normed_out) normed_out[i] = v;
    float d, s;
    int8_t q = q8_lane(v, d, s);
    sq[i] = q;
    if (lane == 0) sds[b] = make_float2(d, s);
  }
  __syncthreads();
}


// ------------------------------------------------------------------------------------
// Fused all-reduce of the residual-stream update across GPUs (tensor-parallel attention
// output, expert-parallel MoE output), split into a producer half and a consumer half
// that live inside the compute kernels:
//
//   producer  the kernel that computes a partial [M, H] update (o_proj GEMV over this
//             rank's heads; down-projection + combine over this rank's experts) stores
//             it in its own receive slot; the last block to finish copies the rows into
//             slot `my_rank` of every peer's receive buffer with 16-byte stores over
//             NVLink, fences system-wide and then stores the site's sequence number into
//             flag `my_rank` on every peer (st.release.sys).
//   consumer  the next kernel's prologue (router / QKV / head GEMV) waits until all N
//             flags reached the local sequence number, adds the N partial rows to the
//             residual in rank order (bit-identical on every rank) and carries on; block 0
//             also stores the new residual rows.
//
// Two sites (attention, MoE) alternate, each with its own buffers; a rank can only reach a
// site's next producer after every rank consumed the previous one, so one buffer per site
// suffices.  The wait is bounded (1 s on the global timer): on expiry the kernel raises
// FS_WAIT_TIMEOUT in the fault word and continues, it never hangs.  The reference makes the
// same reduction as "all-gather of f32 row spans + every rank sums parts in rank order"
// through host-mapped pages (crates/gpu/src/host/link/gather.rs:1-27).
// ------------------------------------------------------------------------------------
constexpr int kMaxRanks = 8;
constexpr int kMaxRows = 8;

struct PushOut {
  float* local;                 // this rank's slot of its own receive buffer: [kMaxRows][H]
  float* peer_recv[kMaxRanks];  // slot `my_rank` of every rank's receive buffer (own entry == local)
  unsigned* peer_flag[kMaxRanks];
  unsigned* seq;                // local sequence number of this site
  unsigned* ticket;             // block-completion ticket, zero at rest
  int n_ranks, my_rank, n_floats;
};

struct ReduceIn {
  const float* recv;            // [n_ranks][kMaxRows][H]
  const unsigned* flags;        // [n_ranks]
  const unsigned* seq;          // local sequence number of the site to consume
  float* x_out;                 // residual rows to update (block 0 stores them), may equal the input
  long x_out_stride;
  int n_ranks, H;
  unsigned* fault;
  int layer;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Every thread of every block calls this after its stores to p.local.
__device__ __forceinline__ void push_finish(const PushOut& p) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.ticket, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) *p.ticket = 0u;
  const int n4 = p.n_floats / 4;
  for (int r = 0; r < p.n_ranks; ++r) {
    if (r == p.my_rank) continue;
    float4* dst = reinterpret_cast<float4*>(p.peer_recv[r]);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = __ldcg(reinterpret_cast<const float4*>(p.local) + i);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.n_ranks) {
    const unsigned e = *p.seq + 1u;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flag[threadIdx.x]), "r"(e) : "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) *p.seq = *p.seq + 1u;
}

// Wait for every rank's flag (bounded); true when all arrived.  Called by all threads of a block.
__device__ __forceinline__ bool reduce_wait(const ReduceIn& r) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < r.n_ranks) {
    const unsigned want = *r.seq;
    const unsigned* f = r.flags + threadIdx.x;
    unsigned long long t0 = 0;
    for (unsigned it = 0;; ++it) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int)(v - want) >= 0) break;
      if ((it & 255) == 255) {
        const unsigned long long now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 1000000000ull) { s_ok = 0; raise_fault(r.fault, r.layer, FS_WAIT_TIMEOUT); break; }
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// Residual value (row m, column i) after the reduction: x + sum over ranks in rank order.
__device__ __forceinline__ float reduce_value(const ReduceIn& r, const float* x_row, int m, int i) {
  float v = x_row[i];
  for (int k = 0; k < r.n_ranks; ++k) v += __ldcg(r.recv + ((long)k * kMaxRows + m) * r.H + i);
  return v;
}
__device__ __forceinline__ float4 reduce_value4(const ReduceIn& r, const float* x_row, int m, int i) {
  float4 v = *reinterpret_cast<const float4*>(x_row + i);
  for (int k = 0; k < r.n_ranks; ++k) {
    const float4 p = __ldcg(reinterpret_cast<const float4*>(r.recv + ((long)k * kMaxRows + m) * r.H + i));
    v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
  }
  return v;
}

// ------------------------------------------------------------------------------------
// Launch wrapper: programmatic stream serialisation is an attribute of the *dependent*
// launch.  It is legal under stream capture (the edge becomes a programmatic graph edge).
// ------------------------------------------------------------------------------------
extern int g_use_pdl;  // set by bl_set_pdl(); default on

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Host-side launch contract: a failed check returns a negative code and launches nothing.
#define BL_REQUIRE(cond, code) \
  do { if (!(cond)) return (code); } while (0)

constexpr int BL_ERR_SHAPE = -2;
constexpr int BL_ERR_TYPE = -3;
constexpr int BL_ERR_ALIGN = -4;
constexpr int BL_ERR_LIMIT = -5;

}  // namespace bl
