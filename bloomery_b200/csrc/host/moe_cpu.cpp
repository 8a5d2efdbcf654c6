// CPU expert leg: gate·x, up·x, SwiGLU, q8, down, router-weighted sum for the routed slots
// the card does not hold, on the resident worker pool.  It reads the same resident block
// layouts and runs the same unit dots as the card kernels (quant_units.cuh), so a slot
// served here and a slot served on the card agree to rounding.
//
// Two entry points:
//   blh_moe_experts      one call for M rows (the CPU engine and the prompt batch port)
//   blh_host_tier_*      a service thread that answers hand-offs written by the card into
//                        a host-mapped pinned page: the card bumps `go`, the thread computes
//                        and bumps `done`; both sides only ever wait with a bound.
// Counterparts in the reference: HostLayer::experts_step_union_into
// (crates/model/src/moe.rs:3476) and the host tier protocol router -> handoff -> go ->
// [card experts] -> wait -> add (crates/gpu/src/host/mod.rs:12-65).
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../quant_units.cuh"
#include "pool.h"

using namespace bl;

namespace {

float dot_any(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  auto run = [&](auto tag) {
    using T = decltype(tag);
    using U = Unit<T>;
    float acc = 0.f;
    for (int u = 0; u < K / 64; ++u) {
      typename U::Regs r;
      U::loadu(row, u, K, r);
      acc += U::dotu(r, u, reinterpret_cast<const uint32_t*>(xq), reinterpret_cast<const F2*>(xds));
    }
    return acc;
  };
  switch (wtype) {
    case WT_Q4_K: return run(Q4K{});
    case WT_Q5_K: return run(Q5K{});
    case WT_Q6_K: return run(Q6K{});
    case WT_Q8_0: return run(Q80{});
    case WT_NVFP4: return run(NvFp4{});
    case WT_FP8_B128: return run(Fp8B128{});
    case WT_Q2_K: return run(Q2K{});
    case WT_Q3_K: return run(Q3K{});
    case WT_Q4_0: return run(Q40{});
    case WT_Q4_1: return run(Q41{});
    case WT_Q5_0: return run(Q50{});
    case WT_Q5_1: return run(Q51{});
  }
  return NAN;
}

void quantize_q8(const float* x, int n, int8_t* q, float* ds) {
  for (int b = 0; b < n / 32; ++b) {
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(x[b * 32 + i]));
    const float d = amax / 127.0f, inv = d > 0.f ? 1.0f / d : 0.f;
    int sum = 0;
    for (int i = 0; i < 32; ++i) {
      int v = (int)std::nearbyintf(x[b * 32 + i] * inv);
      v = v < -127 ? -127 : v > 127 ? 127 : v;
      q[b * 32 + i] = (int8_t)v;
      sum += v;
    }
    ds[2 * b] = d;
    ds[2 * b + 1] = d * (float)sum;
  }
}

struct Stacks {
  const uint8_t* gate; const uint8_t* up; const uint8_t* down;
  int gtype, dtype, E, K, I;
};

// out[m, :] = sum over slots j with ids[m, j] >= 0 of w * down_e(silu(gate_e x) * up_e x)
void moe_rows(const Stacks& s, int M, int n_used, const int* ids, const float* wts, const int8_t* xq, const float* xds,
              float* out, float* act_scratch /* [M * n_used * I] */, int8_t* actq /* same count */, float* actds) {
  const long grb = resident_row_bytes(s.gtype, s.K), drb = resident_row_bytes(s.dtype, s.I);
  const int slots = M * n_used;
  // phase 1: activations, parallel over (slot, 32-row chunks)
  const int chunks = s.I / 32;
  blh::Pool::instance().parallel_for(slots * chunks, 4, [&](int b, int e) {
    for (int t = b; t < e; ++t) {
      const int slot = t / chunks, c = t - slot * chunks;
      const int m = slot / n_used;
      const int ex = ids[slot];
      float* a = act_scratch + (long)slot * s.I + c * 32;
      if (ex < 0 || ex >= s.E) { std::memset(a, 0, 32 * sizeof(float)); continue; }
      for (int r = 0; r < 32; ++r) {
        const long row = (long)ex * s.I + c * 32 + r;
        const float g = dot_any(s.gtype, s.gate + row * grb, s.K, xq + (long)m * s.K, xds + (long)m * (s.K / 32) * 2);
        const float u = dot_any(s.gtype, s.up + row * grb, s.K, xq + (long)m * s.K, xds + (long)m * (s.K / 32) * 2);
        a[r] = (g / (1.0f + std::exp(-g))) * u;
      }
      quantize_q8(a, 32, actq + (long)slot * s.I + c * 32, actds + ((long)slot * (s.I / 32) + c) * 2);
    }
  });
  // phase 2: down + weighted sum in ascending slot order, parallel over output rows
  blh::Pool::instance().parallel_for(M * s.K, 64, [&](int b, int e) {
    for (int t = b; t < e; ++t) {
      const int m = t / s.K, d = t - m * s.K;
      float y = 0.f;
      for (int j = 0; j < n_used; ++j) {
        const int slot = m * n_used + j;
        const int ex = ids[slot];
        if (ex < 0 || ex >= s.E) continue;
        const float v = dot_any(s.dtype, s.down + ((long)ex * s.K + d) * drb, s.I, actq + (long)slot * s.I,
                                actds + (long)slot * (s.I / 32) * 2);
        y = std::fmaf(wts[slot], v, y);
      }
      out[t] = y;
    }
  });
}

// ---- service thread ------------------------------------------------------------------------
// Page layout (host-mapped pinned memory, 4-byte words unless noted):
//   [0] go       card -> host: sequence number of the hand-off
//   [1] done     host -> card: sequence number answered
//   [2] layer    [3] M    [4] n_cold (0: nothing to do, host answers at once)
//   [16 ...)     ids  [MAX_ROWS * MAX_USED] int32   (resident slots are written as -1)
//   then wts  [MAX_ROWS * MAX_USED] float, xq [MAX_ROWS * K] int8, xds [MAX_ROWS * K/32 * 2] float,
//   out [MAX_ROWS * K] float
struct Tier {
  std::vector<Stacks> layers;
  volatile uint32_t* page = nullptr;
  int K = 0, I = 0, n_used = 0, max_rows = 8;
  std::thread thr;
  std::atomic<bool> quit{false};
  std::atomic<uint64_t> served{0}, cold_slots{0};
  std::atomic<uint64_t> busy_ns{0};
  std::vector<float> act; std::vector<int8_t> actq; std::vector<float> actds;
  long off_ids() const { return 16; }
  long off_wts() const { return off_ids() + (long)max_rows * 16; }
  long off_xq() const { return off_wts() + (long)max_rows * 16; }                     // in words
  long off_xds() const { return off_xq() + ((long)max_rows * K + 3) / 4; }
  long off_out() const { return off_xds() + (long)max_rows * (K / 32) * 2; }
  long words() const { return off_out() + (long)max_rows * K; }
  void loop() {
    uint32_t seen = page[0];
    int idle = 0;
    while (!quit.load(std::memory_order_relaxed)) {
      const uint32_t go = page[0];
      if (go == seen) {
        if (++idle > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
        else __builtin_ia32_pause();
        continue;
      }
      idle = 0;
      std::atomic_thread_fence(std::memory_order_acquire);
      const auto t0 = std::chrono::steady_clock::now();
      const int layer = (int)page[2], M = (int)page[3], n_cold = (int)page[4];
      float* out = (float*)(page + off_out());
      if (n_cold > 0 && layer >= 0 && layer < (int)layers.size() && M >= 1 && M <= max_rows && layers[layer].gate) {
        moe_rows(layers[layer], M, n_used, (const int*)(page + off_ids()), (const float*)(page + off_wts()),
                 (const int8_t*)(page + off_xq()), (const float*)(page + off_xds()), out, act.data(), actq.data(), actds.data());
        cold_slots += n_cold;
      } else {
        std::memset(out, 0, sizeof(float) * (size_t)max_rows * K);
      }
      std::atomic_thread_fence(std::memory_order_release);
      page[1] = go;
      seen = go;
      served++;
      busy_ns += (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
    }
  }
};

}  // namespace

extern "C" {

int blh_moe_experts(int M, int K, int I, int E, int n_used, const int* ids, const float* wts, const int8_t* xq,
                    const float* xds, const uint8_t* gate, const uint8_t* up, const uint8_t* down, int gtype, int dtype,
                    float* out) {
  if (K % 256 || I % 256 || resident_row_bytes(gtype, K) <= 0 || resident_row_bytes(dtype, I) <= 0) return -1;
  Stacks s{gate, up, down, gtype, dtype, E, K, I};
  std::vector<float> act((size_t)M * n_used * I);
  std::vector<int8_t> actq((size_t)M * n_used * I);
  std::vector<float> actds((size_t)M * n_used * (I / 32) * 2);
  moe_rows(s, M, n_used, ids, wts, xq, xds, out, act.data(), actq.data(), actds.data());
  return 0;
}

long blh_host_tier_page_words(int K, int max_rows) {
  Tier t; t.K = K; t.max_rows = max_rows;
  return t.words();
}

void* blh_host_tier_create(int n_layers, int K, int I, int n_used, int max_rows, void* page) {
  if (max_rows > 8 || n_used > 16) return nullptr;
  Tier* t = new Tier();
  t->layers.resize(n_layers, Stacks{nullptr, nullptr, nullptr, 0, 0, 0, K, I});
  t->K = K; t->I = I; t->n_used = n_used; t->max_rows = max_rows;
  t->page = (volatile uint32_t*)page;
  t->act.resize((size_t)max_rows * n_used * I);
  t->actq.resize((size_t)max_rows * n_used * I);
  t->actds.resize((size_t)max_rows * n_used * (I / 32) * 2);
  return t;
}

void blh_host_tier_set_layer(void* h, int layer, const uint8_t* gate, const uint8_t* up, const uint8_t* down, int gtype,
                             int dtype, int E) {
  Tier* t = (Tier*)h;
  t->layers[layer] = Stacks{gate, up, down, gtype, dtype, E, t->K, t->I};
}

void blh_host_tier_start(void* h) {
  Tier* t = (Tier*)h;
  t->quit = false;
  t->thr = std::thread([t] { t->loop(); });
}

void blh_host_tier_stop(void* h) {
  Tier* t = (Tier*)h;
  t->quit = true;
  if (t->thr.joinable()) t->thr.join();
}

void blh_host_tier_stats(void* h, uint64_t* served, uint64_t* cold_slots, uint64_t* busy_ns) {
  Tier* t = (Tier*)h;
  *served = t->served; *cold_slots = t->cold_slots; *busy_ns = t->busy_ns;
}

void blh_host_tier_destroy(void* h) {
  blh_host_tier_stop(h);
  delete (Tier*)h;
}

}  // extern "C"
