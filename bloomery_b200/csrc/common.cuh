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
