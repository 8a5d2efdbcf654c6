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
// that live inside the compute kernels.  The transport is flag-in-data: every element
// travels as one 8-byte store {value bits, epoch}, which the hardware writes atomically,
// so neither fences nor completion tickets nor separate flags are needed and the latency
// is one NVLink write.
//
//   producer  the kernel that computes a partial [M, H] update (o_proj GEMV over this
//             rank's heads; down-projection + combine over this rank's experts) stores
//             each finished value, tagged with the site's epoch, into slot `my_rank` of
//             every rank's receive buffer (plain st.global.v2 through the peer mapping).
//   consumer  the next kernel's prologue (router / QKV / head GEMV) reads, for every
//             element, the N tagged values, spinning on a slot until its tag equals the
//             epoch, and adds them to the residual in rank order (bit-identical on every
//             rank); block 0 also stores the new residual rows.
//
// The epoch of a site is  step * sites_per_step + site_index + 1, where `step` is a device
// word that the first kernel of every pass increments; all ranks run the same passes, so
// they agree on it without talking.  Two buffers (attention site, MoE site) alternate: a
// rank reaches a site's next producer only after every rank consumed the previous one.
// Waits are bounded (1 s on the global timer, shared per block): on expiry the kernel
// raises FS_WAIT_TIMEOUT in the fault word, yields NaN and continues; it never hangs.
// The reference makes the same reduction as "all-gather of f32 row spans + every rank sums
// parts in rank order" through host-mapped pages (crates/gpu/src/host/link/gather.rs:1-27).
// ------------------------------------------------------------------------------------
constexpr int kMaxRanks = 8;
constexpr int kMaxRows = 8;

struct PushOut {
  uint2* peer_recv[kMaxRanks];  // slot `my_rank` of every rank's receive buffer: [kMaxRows][H] of {bits, epoch}
  const unsigned* step;         // device word: passes started so far
  unsigned sites_per_step, site_index;
  int n_ranks, my_rank;
};

struct ReduceIn {
  const uint2* recv;            // [n_ranks][kMaxRows][H] of {bits, epoch}
  const unsigned* step;
  unsigned sites_per_step, site_index;
  float* x_out;                 // residual rows to update (block 0 stores them); never the input buffer
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

__device__ __forceinline__ unsigned site_epoch(const unsigned* step, unsigned sites_per_step, unsigned site_index) {
  return *step * sites_per_step + site_index + 1u;
}

// One value of the partial update, tagged and stored into every rank's slot (own copy included).
__device__ __forceinline__ void push_store(const PushOut& p, unsigned epoch, long idx, float v) {
  const uint2 w = make_uint2(__float_as_uint(v), epoch);
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < p.n_ranks) {
      asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p.peer_recv[r] + idx), "r"(w.x), "r"(w.y) : "memory");
    }
}

// Per-block state of the consumer's bounded waits.
struct ReduceWait {
  unsigned epoch;
  unsigned long long t0;
  volatile int* gave_up;    // shared by the block
};

__device__ __forceinline__ uint4 ld_volatile_v4(const uint2* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Bounded re-poll bookkeeping shared by the batched readers below; true = keep polling.
__device__ __forceinline__ bool reduce_again(const ReduceIn& r, ReduceWait& w, unsigned it) {
  if ((it & 31) != 31) return true;
  if (*w.gave_up) return false;
  const unsigned long long now = global_timer_ns();
  if (w.t0 == 0) { w.t0 = now; return true; }
  if (now - w.t0 > 1000000000ull) { *w.gave_up = 1; raise_fault(r.fault, r.layer, FS_WAIT_TIMEOUT); return false; }
  return true;
}

// acc[0..8) += the eight values (row m, columns i0..i0+7) of every rank, in rank order.
// Two ranks' slots are fetched per round trip (eight 16-byte loads in flight), checked, and
// only re-fetched if a tag is still old; values are added strictly in rank order so every
// rank computes bit-identical sums.
__device__ __forceinline__ void reduce_sum8(const ReduceIn& r, ReduceWait& w, int m, int i0, float (&acc)[8]) {
  for (int k0 = 0; k0 < r.n_ranks; k0 += 2) {
    const int n = min(2, r.n_ranks - k0);
    uint4 b[2][4];
    bool ok = false;
    for (unsigned it = 0; !ok; ++it) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (j < n) {
          const uint2* s = r.recv + ((long)(k0 + j) * kMaxRows + m) * r.H + i0;
#pragma unroll
          for (int q = 0; q < 4; ++q) b[j][q] = ld_volatile_v4(s + 2 * q);
        }
      ok = true;
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (j < n) {
#pragma unroll
          for (int q = 0; q < 4; ++q) ok = ok && b[j][q].y == w.epoch && b[j][q].w == w.epoch;
        }
      if (!ok && !reduce_again(r, w, it)) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = __int_as_float(0x7fc00000);
        return;
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
      if (j < n) {
#pragma unroll
        for (int q = 0; q < 4; ++q) { acc[2 * q] += __uint_as_float(b[j][q].x); acc[2 * q + 1] += __uint_as_float(b[j][q].z); }
      }
  }
}

// One column (row m, column i): every rank's slot is fetched before any tag is checked.
__device__ __forceinline__ float reduce_value(const ReduceIn& r, ReduceWait& w, const float* x_row, int m, int i) {
  float v = x_row[i];
  uint2 b[kMaxRanks];
  bool ok = false;
  for (unsigned it = 0; !ok; ++it) {
#pragma unroll
    for (int k = 0; k < kMaxRanks; ++k)
      if (k < r.n_ranks) {
        const uint2* s = r.recv + ((long)k * kMaxRows + m) * r.H + i;
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(b[k].x), "=r"(b[k].y) : "l"(s) : "memory");
      }
    ok = true;
#pragma unroll
    for (int k = 0; k < kMaxRanks; ++k)
      if (k < r.n_ranks) ok = ok && b[k].y == w.epoch;
    if (!ok && !reduce_again(r, w, it)) return __int_as_float(0x7fc00000);
  }
#pragma unroll
  for (int k = 0; k < kMaxRanks; ++k)
    if (k < r.n_ranks) v += __uint_as_float(b[k].x);
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
