// Pieces of the several-GPU prompt path that are not the GEMM itself:
//   rank_barrier      every rank tells every peer "my phase e is done" (one 4-byte store into the
//                     peer's flag row) and waits, bounded, until all peers said the same
//   gather_rows_peer  the expert-parallel dispatch as a pull: row p of the expert-sorted A matrix is
//                     copied from the rank that owns its token (plain 16-byte loads over NVLink)
//   zero / count helpers on routing tables that span all ranks' tokens
//   push_rows / rank_barrier_step / sum_ranks  a deterministic all-reduce of fp32 rows for captured passes (the batched
//                     decode over ranks): every rank stores its partial rows into slot `rank` of every peer's gather
//                     buffer, a barrier whose epoch comes from a device-side pass counter (so a CUDA graph can replay
//                     it) orders writers and readers, and every rank adds the slots in rank order -- the same bits
//                     on every rank, which replicated activations need
//
// Each rank runs these as ordinary launches on its own GPU; two ranks never share a GPU (tests that
// emulate ranks on one GPU skip the barrier: stream order already separates the phases there).
#include "common.cuh"

namespace bl {

struct BarrierArgs {
  unsigned* peer_flags[8];   // peer r's flag row: n_ranks words, word i written by rank i
  unsigned* my_flags;
  unsigned epoch;
  int n_ranks, my_rank;
  unsigned* status;          // set to 1 when the wait ran out
};

__global__ void rank_barrier_kernel(const BarrierArgs a) {
  const int r = threadIdx.x;
  pdl_wait();                                               // everything enqueued before the barrier has finished
  pdl_launch();
  if (r >= a.n_ranks) return;
  __threadfence_system();                                   // this rank's earlier kernels' writes come first
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[r] + a.my_rank), "r"(a.epoch) : "memory");
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (unsigned it = 0;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.my_flags + r) : "memory");
    if ((int)(v - a.epoch) >= 0) break;
    if ((it & 255) == 255) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > 2000000000ull) { if (a.status) atomicMax(a.status, 1u); break; }
    }
  }
  __threadfence_system();
}

struct PeerGatherArgs {
  const __nv_bfloat16* src[8];   // rank r's shard [rows_per_rank, K]
  long src_stride;
  int rows_per_rank;
  const int* dst_row;            // flat slot index (token * k + j) of sorted row p
  const int* n_rows;
  int k, K;
  __nv_bfloat16* out;
};

__global__ void __launch_bounds__(256) gather_rows_peer_kernel(const PeerGatherArgs a) {
  const int p = blockIdx.x;
  pdl_wait();
  pdl_launch();
  if (p >= *a.n_rows) return;
  const int t = a.dst_row[p] / a.k;
  const int owner = t / a.rows_per_rank;
  const uint4* s = reinterpret_cast<const uint4*>(a.src[owner & 7] + (long)(t - owner * a.rows_per_rank) * a.src_stride);
  uint4* o = reinterpret_cast<uint4*>(a.out + (long)p * a.K);
  for (int i = threadIdx.x; i < a.K / 8; i += 256) o[i] = s[i];
}

// ids of all tokens -> this rank's expert numbering (others become -1)
__global__ void localize_ids_kernel(const int* ids, int n, int e_lo, int e_hi, int* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  pdl_launch();
  if (i < n) { const int e = ids[i]; out[i] = (e >= e_lo && e < e_hi) ? e - e_lo : -1; }
}

// plain copy of n 16-byte words (either side may be a peer pointer)
__global__ void __launch_bounds__(256) copy16_kernel(const uint4* src, uint4* dst, long n) {
  pdl_wait();
  pdl_launch();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) dst[i] = src[i];
}

// the same barrier with its epoch taken from a pass counter on the device: epoch = *step * sites_per_step + site + 1
struct StepBarrierArgs {
  unsigned* peer_flags[8];
  unsigned* my_flags;
  const unsigned* step;
  unsigned sites_per_step, site;
  int n_ranks, my_rank;
  unsigned* status;
};

__global__ void rank_barrier_step_kernel(const StepBarrierArgs a) {
  const int r = threadIdx.x;
  pdl_wait();
  pdl_launch();
  if (r >= a.n_ranks) return;
  const unsigned epoch = *a.step * a.sites_per_step + a.site + 1u;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer_flags[r] + a.my_rank), "r"(epoch) : "memory");
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (unsigned it = 0;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.my_flags + r) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if ((it & 255) == 255) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (now - t0 > 2000000000ull) { if (a.status) atomicMax(a.status, 1u); break; }
    }
  }
  __threadfence_system();
}

// n 16-byte words of src into dst[r] for every rank r (blockIdx.y = r); plain stores, peer pointers included
struct PushArgs { const uint4* src; uint4* dst[8]; long n; };
__global__ void __launch_bounds__(256) push_rows_kernel(const PushArgs a) {
  pdl_wait();
  pdl_launch();
  uint4* d = a.dst[blockIdx.y];
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (long)gridDim.x * blockDim.x) d[i] = a.src[i];
}

// x[i] += g[0][i] + g[1][i] + ... in rank order (g = [n_ranks][slot_stride] floats)
__global__ void __launch_bounds__(256) sum_ranks_kernel(const float4* g, long slot_stride4, int n_ranks, float4* x, long n4) {
  pdl_wait();
  pdl_launch();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 acc = g[i];
    for (int r = 1; r < n_ranks; ++r) {
      const float4 v = g[(long)r * slot_stride4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float4 o = x[i];
    o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
    x[i] = o;
  }
}

}  // namespace bl

using namespace bl;

extern "C" {

int bl_rank_barrier(void* const* peer_flags, void* my_flags, unsigned epoch, int n_ranks, int my_rank, unsigned* status,
                    cudaStream_t st) {
  BL_REQUIRE(n_ranks >= 1 && n_ranks <= 8 && my_rank >= 0 && my_rank < n_ranks, BL_ERR_SHAPE);
  BarrierArgs a{};
  for (int r = 0; r < n_ranks; ++r) a.peer_flags[r] = (unsigned*)peer_flags[r];
  a.my_flags = (unsigned*)my_flags; a.epoch = epoch; a.n_ranks = n_ranks; a.my_rank = my_rank; a.status = status;
  return (int)launch(rank_barrier_kernel, dim3(1), dim3(32), 0, st, a);
}

int bl_gather_rows_peer(void* const* src_of_rank, int n_ranks, long src_stride, int rows_per_rank, const int* dst_row,
                        const int* n_rows, int max_rows, int k, int K, void* out, cudaStream_t st) {
  BL_REQUIRE(max_rows >= 1 && K % 8 == 0 && src_stride % 8 == 0 && n_ranks >= 1 && n_ranks <= 8 && rows_per_rank >= 1, BL_ERR_SHAPE);
  PeerGatherArgs a{};
  for (int r = 0; r < 8; ++r) a.src[r] = (const __nv_bfloat16*)src_of_rank[r < n_ranks ? r : 0];
  a.src_stride = src_stride; a.rows_per_rank = rows_per_rank; a.dst_row = dst_row; a.n_rows = n_rows; a.k = k; a.K = K;
  a.out = (__nv_bfloat16*)out;
  return (int)launch(gather_rows_peer_kernel, dim3(max_rows), dim3(256), 0, st, a);
}

int bl_rank_barrier_step(void* const* peer_flags, void* my_flags, const unsigned* step, unsigned sites_per_step,
                         unsigned site, int n_ranks, int my_rank, unsigned* status, cudaStream_t st) {
  BL_REQUIRE(n_ranks >= 1 && n_ranks <= 8 && my_rank >= 0 && my_rank < n_ranks && step != nullptr && site < sites_per_step,
             BL_ERR_SHAPE);
  StepBarrierArgs a{};
  for (int r = 0; r < n_ranks; ++r) a.peer_flags[r] = (unsigned*)peer_flags[r];
  a.my_flags = (unsigned*)my_flags; a.step = step; a.sites_per_step = sites_per_step; a.site = site;
  a.n_ranks = n_ranks; a.my_rank = my_rank; a.status = status;
  return (int)launch(rank_barrier_step_kernel, dim3(1), dim3(32), 0, st, a);
}

int bl_push_rows(const void* src, void* const* dst_of_rank, int n_ranks, long n_bytes, cudaStream_t st) {
  BL_REQUIRE(n_ranks >= 1 && n_ranks <= 8 && n_bytes >= 16 && n_bytes % 16 == 0 && ((uintptr_t)src & 15) == 0, BL_ERR_SHAPE);
  PushArgs a{};
  a.src = (const uint4*)src; a.n = n_bytes / 16;
  for (int r = 0; r < n_ranks; ++r) { BL_REQUIRE(((uintptr_t)dst_of_rank[r] & 15) == 0, BL_ERR_ALIGN); a.dst[r] = (uint4*)dst_of_rank[r]; }
  const long per = (a.n + 255) / 256;
  return (int)launch(push_rows_kernel, dim3((unsigned)(per < 64 ? per : 64), n_ranks), dim3(256), 0, st, a);
}

int bl_sum_ranks(const float* gathered, long slot_stride, int n_ranks, float* x, long n, cudaStream_t st) {
  BL_REQUIRE(n_ranks >= 1 && n_ranks <= 8 && n >= 4 && n % 4 == 0 && slot_stride % 4 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(((uintptr_t)gathered & 15) == 0 && ((uintptr_t)x & 15) == 0, BL_ERR_ALIGN);
  const long n4 = n / 4, per = (n4 + 255) / 256;
  return (int)launch(sum_ranks_kernel, dim3((unsigned)(per < 296 ? per : 296)), dim3(256), 0, st, (const float4*)gathered,
                     slot_stride / 4, n_ranks, (float4*)x, n4);
}

int bl_copy_bytes(const void* src, void* dst, long n_bytes, cudaStream_t st) {
  BL_REQUIRE(n_bytes >= 16 && n_bytes % 16 == 0, BL_ERR_SHAPE);
  BL_REQUIRE(((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0, BL_ERR_ALIGN);
  const long n = n_bytes / 16;
  const int grid = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  return (int)launch(copy16_kernel, dim3(grid), dim3(256), 0, st, (const uint4*)src, (uint4*)dst, n);
}

int bl_localize_ids(const int* ids, int n, int e_lo, int e_hi, int* out, cudaStream_t st) {
  BL_REQUIRE(n >= 1, BL_ERR_SHAPE);
  return (int)launch(localize_ids_kernel, dim3((n + 255) / 256), dim3(256), 0, st, ids, n, e_lo, e_hi, out);
}

}  // extern "C"
