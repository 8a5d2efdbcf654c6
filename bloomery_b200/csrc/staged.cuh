// Helpers of the kernels that keep weight rows in shared memory: bulk asynchronous copies completing on an
// mbarrier, the bounded wait, the conflict-free activation loaders and the two-row gate / up product.
// A translation unit that includes this header reads weight units out of shared memory, so the units' 16-byte
// loads must be plain loads (BL_UNITS_GENERIC_LD) rather than read-only-cache loads.
#pragma once
#define BL_UNITS_GENERIC_LD 1
#include "gemv_common.cuh"
#include "route.cuh"

namespace bl {

// ---- bulk copy + mbarrier -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> shared, both 16-byte aligned, size a multiple of 16; completes `bytes` on the barrier
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_load_chunks(uint8_t* dst, const uint8_t* src, uint32_t bytes, uint64_t* bar) {
  constexpr uint32_t kChunk = 32 * 1024;
  for (uint32_t o = 0; o < bytes; o += kChunk) bulk_load(dst + o, src + o, min(kChunk, bytes - o), bar);
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Bounded wait (1 s on the global timer) for phase `parity`.  On expiry: fault site "device wait ran out",
// false is returned and the caller writes NaN; the kernel still returns.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned* fault, int layer) {
  const uint32_t addr = smem_u32(bar);
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    if ((it & 255) == 255) {
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > 1000000000ull) { raise_fault(fault, layer, FS_WAIT_TIMEOUT); return false; }
    }
  }
}

constexpr float kNaN = __builtin_nanf("");

// Phase probe (kernel_bench --probe): when armed, thread 0 of block (0, 0, 0) stores the SM cycle counter at the
// kernel's phase boundaries, which shows where a launch's microseconds go without a profiler.  Null in normal use.
__device__ __forceinline__ void probe_mark(long long* probe, int i) {
  if (probe && threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) probe[i] = clock64();
}


template <class T>
__device__ __forceinline__ void gate_up_rows_staged(const uint8_t* g0, const uint8_t* u0, long rb, int K, int lane,
                                                    const int8_t* xq, const float2* xds, float (&gacc)[2], float (&uacc)[2]) {
  using U = Unit<T>;
  const int nunits = K / 64;
#pragma unroll
  for (int r = 0; r < 2; ++r) { gacc[r] = 0.f; uacc[r] = 0.f; }
  for (int u = lane; u < nunits; u += 32) {
    typename U::Regs rg[2], ru[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) { U::loadu(g0 + r * rb, u, K, rg[r]); U::loadu(u0 + r * rb, u, K, ru[r]); }
    ActRegs act;
    StagedAct<T>::load(xq, xds, u, nunits, act);
#pragma unroll
    for (int r = 0; r < 2; ++r) { gacc[r] += ActOf<T>::dot(rg[r], u, act); uacc[r] += ActOf<T>::dot(ru[r], u, act); }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) { gacc[r] = warp_sum(gacc[r]); uacc[r] = warp_sum(uacc[r]); }
}


// ---- thread-block clusters: rank, hardware barrier, distributed shared memory ------------------------
__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (a shared-memory address of this CTA) in the CTA of rank `rank` of the cluster
__device__ __forceinline__ uint32_t peer_addr(const void* local, unsigned rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(local)), "r"(rank));
  return out;
}
__device__ __forceinline__ void st_peer_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void st_peer_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void st_peer_v2(uint32_t addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}

}  // namespace bl
