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

// Activation registers of weight unit u out of a shared-memory row in layout 1 / 2 (act_chunk_pos): every load of
// a warp touches 32 consecutive 16-byte chunks, so none meets a bank conflict.  `sds` stays linear.
template <class T> struct StagedAct {
  static constexpr int kLayout = 1;
  static __device__ __forceinline__ void load(const int8_t* sq, const float2* sds, int u, int nunits, ActRegs& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(sq + ((long)(i * nunits + u) << 4));
      a.q[4 * i] = v.x; a.q[4 * i + 1] = v.y; a.q[4 * i + 2] = v.z; a.q[4 * i + 3] = v.w;
    }
    const float4 ds = *reinterpret_cast<const float4*>(sds + 2 * u);
    a.d[0] = ds.x; a.s[0] = ds.y; a.d[1] = ds.z; a.s[1] = ds.w;
  }
};
template <> struct StagedAct<Q6K> {
  static constexpr int kLayout = 2;
  static __device__ __forceinline__ void load(const int8_t* sq, const float2* sds, int u, int nunits, ActRegs& a) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 v = *reinterpret_cast<const uint4*>(sq + ((long)(g * nunits + u) << 4));
      a.q[4 * g] = v.x; a.q[4 * g + 1] = v.y; a.q[4 * g + 2] = v.z; a.q[4 * g + 3] = v.w;
    }
    const int sb = u >> 2, n = (u >> 1) & 1;
    const float4 d01 = *reinterpret_cast<const float4*>(sds + 8 * sb + 4 * n);
    const float4 d23 = *reinterpret_cast<const float4*>(sds + 8 * sb + 4 * n + 2);
    a.d[0] = d01.x; a.d[1] = d01.z; a.d[2] = d23.x; a.d[3] = d23.z;
  }
};
__host__ __device__ inline int staged_layout(int wtype) { return wtype == WT_Q6_K ? 2 : 1; }

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


}  // namespace bl
