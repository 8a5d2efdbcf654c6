// Card side of the host expert tier: routed slots whose expert is not resident in HBM are
// handed to the CPU leg through one host-mapped pinned page, inside the captured graph.
//
//   handoff  (1 block)  marks which routed slots are cold (slot_map[id] < 0); when there is
//                       at least one it writes ids / weights / the q8 activation rows into the
//                       page, fences system-wide and bumps the page's `go` word;
//   ... the card computes its resident experts meanwhile ...
//   wait     (1 block)  when something was handed off, polls the page's `done` word with a
//                       bound (2 s on the global timer), then copies the host's rows into a
//                       device buffer that the down+combine launch adds; otherwise zeros it.
//
// One writer per word: the card writes `go`, layer, counts and inputs; the host writes `done`
// and the output rows.  On expiry the wait raises FS_WAIT_TIMEOUT and yields NaN rows; it
// never hangs.  Same protocol as the reference's router -> handoff -> go -> [card experts]
// -> wait -> add (crates/gpu/src/host/mod.rs:12-39), with kernels instead of stream memops.
#include "common.cuh"

namespace bl {

struct HandoffArgs {
  const int* ids; const float* wts;          // [M, n_used] routed
  const int* slot_map;                       // [E] -> resident slot or < 0
  const int8_t* xq; const float2* xds;       // [M, K] q8 rows
  int M, n_used, K, E, layer, max_rows;
  volatile uint32_t* page;                   // host-mapped
  unsigned* seq;                             // device: hand-offs made so far
  int* pending;                              // device: 1 when this layer handed something off
  unsigned* cold_total;                      // device counter (statistics)
};

__device__ __forceinline__ long page_off_ids() { return 16; }
__device__ __forceinline__ long page_off_wts(int max_rows) { return 16 + (long)max_rows * 16; }
__device__ __forceinline__ long page_off_xq(int max_rows) { return page_off_wts(max_rows) + (long)max_rows * 16; }
__device__ __forceinline__ long page_off_xds(int max_rows, int K) { return page_off_xq(max_rows) + ((long)max_rows * K + 3) / 4; }
__device__ __forceinline__ long page_off_out(int max_rows, int K) { return page_off_xds(max_rows, K) + (long)max_rows * (K / 32) * 2; }

__global__ void __launch_bounds__(256) host_handoff_kernel(const HandoffArgs a) {
  __shared__ int s_cold;
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x;
  if (tid == 0) s_cold = 0;
  __syncthreads();
  const int n = a.M * a.n_used;
  volatile int* p_ids = (volatile int*)(a.page + page_off_ids());
  volatile float* p_wts = (volatile float*)(a.page + page_off_wts(a.max_rows));
  if (tid < n) {
    const int id = a.ids[tid];
    const bool cold = id >= 0 && id < a.E && a.slot_map[id] < 0;
    p_ids[tid] = cold ? id : -1;
    p_wts[tid] = a.wts[tid];
    if (cold) atomicAdd(&s_cold, 1);
  }
  __syncthreads();
  const int n_cold = s_cold;
  if (n_cold == 0) {
    if (tid == 0) *a.pending = 0;
    return;
  }
  volatile uint32_t* p_xq = a.page + page_off_xq(a.max_rows);
  const uint32_t* xq32 = reinterpret_cast<const uint32_t*>(a.xq);
  for (int i = tid; i < a.M * a.K / 4; i += 256) p_xq[i] = xq32[i];
  volatile float2* p_xds = (volatile float2*)(a.page + page_off_xds(a.max_rows, a.K));
  for (int i = tid; i < a.M * (a.K / 32); i += 256) { float2 v = a.xds[i]; p_xds[i].x = v.x; p_xds[i].y = v.y; }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    a.page[2] = (uint32_t)a.layer; a.page[3] = (uint32_t)a.M; a.page[4] = (uint32_t)n_cold;
    __threadfence_system();
    const unsigned s = *a.seq + 1u;
    *a.seq = s;
    a.page[0] = s;                                  // go
    *a.pending = 1;
    if (a.cold_total) atomicAdd(a.cold_total, (unsigned)n_cold);
  }
}

struct HostWaitArgs {
  volatile uint32_t* page;
  const unsigned* seq;
  const int* pending;
  float* extra;            // [M, K] device rows the combine adds
  int M, K, max_rows;
  unsigned* fault; int layer;
  unsigned long long* wait_ns;   // statistics: time spent waiting for the host
};

__global__ void __launch_bounds__(256) host_wait_kernel(const HostWaitArgs a) {
  __shared__ int s_ok;
  pdl_wait();
  pdl_launch();
  const int tid = threadIdx.x;
  const int n = a.M * a.K;
  if (!*a.pending) {
    for (int i = tid; i < n; i += 256) a.extra[i] = 0.f;
    return;
  }
  if (tid == 0) {
    const unsigned want = *a.seq;
    const unsigned long long t0 = global_timer_ns();
    int ok = 1;
    for (unsigned it = 0;; ++it) {
      const unsigned d = a.page[1];
      if ((int)(d - want) >= 0) break;
      if ((it & 63) == 63 && global_timer_ns() - t0 > 2000000000ull) { ok = 0; raise_fault(a.fault, a.layer, FS_WAIT_TIMEOUT); break; }
    }
    __threadfence_system();
    s_ok = ok;
    if (a.wait_ns) atomicAdd(a.wait_ns, global_timer_ns() - t0);
  }
  __syncthreads();
  volatile const float* out = (volatile const float*)(a.page + page_off_out(a.max_rows, a.K));
  for (int i = tid; i < n; i += 256) a.extra[i] = s_ok ? out[i] : __int_as_float(0x7fc00000);
}

}  // namespace bl

using namespace bl;

extern "C" {

int bl_host_handoff(const int* ids, const float* wts, const int* slot_map, const int8_t* xq, const float* xds, int M,
                    int n_used, int K, int E, int layer, int max_rows, void* page, unsigned* seq, int* pending,
                    unsigned* cold_total, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && M <= max_rows && max_rows <= 8 && M * n_used <= 256 && n_used <= 16 && K % 32 == 0, BL_ERR_SHAPE);
  HandoffArgs a{ids, wts, slot_map, xq, (const float2*)xds, M, n_used, K, E, layer, max_rows, (volatile uint32_t*)page, seq,
                pending, cold_total};
  return (int)launch(host_handoff_kernel, dim3(1), dim3(256), 0, st, a);
}

int bl_host_wait(void* page, const unsigned* seq, const int* pending, float* extra, int M, int K, int max_rows,
                 unsigned* fault, int layer, unsigned long long* wait_ns, cudaStream_t st) {
  BL_REQUIRE(M >= 1 && M <= max_rows && max_rows <= 8, BL_ERR_SHAPE);
  HostWaitArgs a{(volatile uint32_t*)page, seq, pending, extra, M, K, max_rows, fault, layer, wait_ns};
  return (int)launch(host_wait_kernel, dim3(1), dim3(256), 0, st, a);
}

}  // extern "C"
