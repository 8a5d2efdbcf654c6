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
#include <algorithm>
#include <thread>
#include <utility>
#include <vector>

#include <fcntl.h>
#include <stdlib.h>
#include <unistd.h>

#include "../quant_units.cuh"
#include "pool.h"
#include "qdot_avx2.h"
#include "qdot_vnni.h"

using namespace bl;

namespace {

float dot_any(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds) {
  float fast;
  if (blh::row_dot_vnni(wtype, row, K, xq, xds, &fast)) return fast;        // AVX-512 VNNI where the CPU has it
  if (blh::row_dot_fast(wtype, row, K, xq, xds, &fast)) return fast;        // AVX2 paths of the Q4_K_M mix
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
    case WT_Q8_F32: return run(Q8F{});
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
  // Arena form (experts paged from a drive): expert e lives in slot slot_of[e] (< 0: not loaded) and the parts of
  // consecutive slots are gstride / dstride bytes apart (0 = experts back to back, slot = expert id).
  const int* slot_of = nullptr;
  long gstride = 0, dstride = 0;
};

// out[m, :] = sum over slots j with ids[m, j] >= 0 of w * down_e(silu(gate_e x) * up_e x)
void moe_rows(const Stacks& s, int M, int n_used, const int* ids, const float* wts, const int8_t* xq, const float* xds,
              float* out, float* act_scratch /* [M * n_used * I] */, int8_t* actq /* same count */, float* actds) {
  const long grb = resident_row_bytes(s.gtype, s.K), drb = resident_row_bytes(s.dtype, s.I);
  const long gstr = s.gstride ? s.gstride : (long)s.I * grb, dstr = s.dstride ? s.dstride : (long)s.K * drb;
  auto where = [&](int ex) { return ex < 0 || ex >= s.E ? -1 : (s.slot_of ? s.slot_of[ex] : ex); };
  const int slots = M * n_used;
  // phase 1: activations, parallel over (slot, 32-row chunks)
  const int chunks = s.I / 32;
  blh::Pool::instance().parallel_for(slots * chunks, 4, [&](int b, int e) {
    for (int t = b; t < e; ++t) {
      const int slot = t / chunks, c = t - slot * chunks;
      const int m = slot / n_used;
      const int ex = where(ids[slot]);
      float* a = act_scratch + (long)slot * s.I + c * 32;
      if (ex < 0) { std::memset(a, 0, 32 * sizeof(float)); continue; }
      for (int r = 0; r < 32; ++r) {
        const long row = (long)ex * gstr + (long)(c * 32 + r) * grb;
        const float g = dot_any(s.gtype, s.gate + row, s.K, xq + (long)m * s.K, xds + (long)m * (s.K / 32) * 2);
        const float u = dot_any(s.gtype, s.up + row, s.K, xq + (long)m * s.K, xds + (long)m * (s.K / 32) * 2);
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
        const int ex = where(ids[slot]);
        if (ex < 0) continue;
        const float v = dot_any(s.dtype, s.down + (long)ex * dstr + (long)d * drb, s.I, actq + (long)slot * s.I,
                                actds + (long)slot * (s.I / 32) * 2);
        y = std::fmaf(wts[slot], v, y);
      }
      out[t] = y;
    }
  });
}


// ---- experts paged from a drive ---------------------------------------------------------------
// A side file holds every routed expert in its resident layout, one 4096-aligned blob per (layer, expert):
// [gate rows | up rows | down rows], each part padded to 4096.  A RAM arena keeps n_slots experts per layer;
// a routed expert that is not in the arena is read with O_DIRECT by reader threads into the slot of the
// least recently used expert that the current call does not need (pinned experts never leave).
// Counterpart of the reference's NVMe expert tier (crates/gpu/src/host/nvtier.rs: RAM arena of expert
// slots filled by O_DIRECT reads on dedicated reader threads, LRU / heat eviction, pins; crates/engram/src/direct.rs).
struct NvLayer {
  long file_off = 0;                 // blob of expert 0
  int dtype = 0;                     // the down projection's type may differ from layer to layer (Q4_K_M mixes)
  long dpart = 0, blob = 0;
  uint8_t* arena = nullptr;          // n_slots blobs
  std::vector<int> slot_of, expert_in;
  std::vector<uint64_t> last_use;
  std::vector<uint8_t> pinned;
};

struct NvTier {
  int fd = -1;
  bool direct = false;
  int n_layers = 0, E = 0, n_slots = 0, K = 0, I = 0, gtype = 0, dtype = 0, n_readers = 4;
  long gpart = 0;                               // padded gate / up part size (blob sizes are per layer)
  std::vector<NvLayer> layers;
  uint64_t tick = 0;
  std::atomic<uint64_t> hits{0}, misses{0}, evictions{0}, bytes_read{0}, read_ns{0}, failed{0};

  bool read_all(const std::vector<std::pair<long, uint8_t*>>& reqs, long blob) {
    // every request is one blob; split the list over reader threads, each issuing aligned preads
    std::atomic<size_t> cursor{0};
    std::atomic<bool> ok{true};
    auto work = [&] {
      for (;;) {
        const size_t i = cursor.fetch_add(1);
        if (i >= reqs.size()) return;
        long done = 0;
        while (done < blob) {
          const ssize_t n = pread(fd, reqs[i].second + done, (size_t)(blob - done), reqs[i].first + done);
          if (n <= 0) { ok = false; break; }
          done += n;
        }
      }
    };
    const auto t0 = std::chrono::steady_clock::now();
    const int nt = (int)std::min<size_t>(n_readers, reqs.size());
    std::vector<std::thread> ths;
    for (int t = 1; t < nt; ++t) ths.emplace_back(work);
    work();
    for (auto& t : ths) t.join();
    read_ns += (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count();
    bytes_read += (uint64_t)reqs.size() * (uint64_t)blob;
    return ok;
  }

  // make every expert of ids[] (>= 0) of `layer` present: 0 done, 1 the call needs more experts than there are
  // free slots (the caller may split it), 2 a read failed
  int ensure(int layer, const int* ids, int n) {
    NvLayer& L = layers[layer];
    ++tick;
    std::vector<int> need;
    for (int i = 0; i < n; ++i) {
      const int e = ids[i];
      if (e < 0 || e >= E) continue;
      const int s = L.slot_of[e];
      if (s >= 0) { if (L.last_use[s] != tick) { L.last_use[s] = tick; ++hits; } continue; }
      if (std::find(need.begin(), need.end(), e) == need.end()) need.push_back(e);
    }
    if (need.empty()) return 0;
    {
      int room = 0;
      for (int s = 0; s < n_slots; ++s) room += (!L.pinned[s] && L.last_use[s] != tick) ? 1 : 0;
      if ((int)need.size() > room) return 1;        // nothing was evicted yet
    }
    std::vector<std::pair<long, uint8_t*>> reqs;
    std::vector<std::pair<int, int>> placed;           // (expert, slot)
    for (int e : need) {
      int victim = -1;
      uint64_t oldest = ~0ull;
      for (int s = 0; s < n_slots; ++s) {
        if (L.pinned[s] || L.last_use[s] == tick) continue;       // in use by this very call
        if (L.expert_in[s] < 0) { victim = s; break; }
        if (L.last_use[s] < oldest) { oldest = L.last_use[s]; victim = s; }
      }
      if (victim < 0) { ++failed; return 2; }
      if (L.expert_in[victim] >= 0) { L.slot_of[L.expert_in[victim]] = -1; ++evictions; }
      L.expert_in[victim] = e;
      L.last_use[victim] = tick;
      placed.emplace_back(e, victim);
      reqs.emplace_back(L.file_off + (long)e * L.blob, L.arena + (long)victim * L.blob);
      ++misses;
    }
    if (!read_all(reqs, L.blob)) {
      for (auto& p : placed) { L.expert_in[p.second] = -1; L.last_use[p.second] = 0; }
      ++failed;
      return 2;
    }
    for (auto& p : placed) L.slot_of[p.first] = p.second;
    return 0;
  }

  // the expert leg of M rows from the arena; rows are served one at a time when together they need more experts
  // than the arena has slots.  false: a read failed or one row alone does not fit.
  bool serve(int layer, int M, int n_used, const int* ids, const float* wts, const int8_t* xq, const float* xds, float* out,
             float* act, int8_t* actq, float* actds) {
    const int rc = ensure(layer, ids, M * n_used);
    if (rc == 0) { moe_rows(stacks(layer), M, n_used, ids, wts, xq, xds, out, act, actq, actds); return true; }
    if (rc == 2 || M == 1) { ++failed; return false; }
    for (int m = 0; m < M; ++m) {
      if (ensure(layer, ids + (long)m * n_used, n_used) != 0) { ++failed; return false; }
      moe_rows(stacks(layer), 1, n_used, ids + (long)m * n_used, wts + (long)m * n_used, xq + (long)m * K,
               xds + (long)m * (K / 32) * 2, out + (long)m * K, act, actq, actds);
    }
    return true;
  }

  Stacks stacks(int layer) const {
    const NvLayer& L = layers[layer];
    Stacks s{L.arena, L.arena + gpart, L.arena + 2 * gpart, gtype, L.dtype, E, K, I};
    s.slot_of = L.slot_of.data();
    s.gstride = L.blob; s.dstride = L.blob;
    return s;
  }
};

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
  NvTier* nv = nullptr;                // when set, cold experts come from the drive-backed arena
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
      if (n_cold > 0 && nv && layer >= 0 && layer < nv->n_layers && M >= 1 && M <= max_rows) {
        const int* ids = (const int*)(page + off_ids());
        if (!nv->serve(layer, M, n_used, ids, (const float*)(page + off_wts()), (const int8_t*)(page + off_xq()),
                       (const float*)(page + off_xds()), out, act.data(), actq.data(), actds.data())) {
          for (long i = 0; i < (long)max_rows * K; ++i) out[i] = std::nanf("");       // a failed read must not pass as zeros
        }
        cold_slots += n_cold;
      } else if (n_cold > 0 && layer >= 0 && layer < (int)layers.size() && M >= 1 && M <= max_rows && layers[layer].gate) {
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

namespace blh {
// the fastest dot this CPU has for a resident row against q8 activations (VNNI, AVX2, scalar), for the other host files
float dot_row(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds) { return dot_any(wtype, row, K, xq, xds); }
}  // namespace blh

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

// ---- drive-backed expert arena ---------------------------------------------------------------------
void blh_nv_close(void* h);

long blh_nv_part_bytes(int wtype, int rows, int K) {
  const long rb = resident_row_bytes(wtype, K);
  return rb <= 0 ? -1 : ((long)rows * rb + 4095) / 4096 * 4096;
}

// file: the side file; layer_off[l]: offset of layer l's expert 0 blob (4096-aligned).  Returns null on failure.
void* blh_nv_open(const char* file, int n_layers, const long* layer_off, const int* layer_dtype, int E, int n_slots, int K,
                  int I, int gtype, int n_readers) {
  if (n_slots < 1 || n_slots > E || K % 256 || I % 256) return nullptr;
  NvTier* t = new NvTier();
  t->fd = open(file, O_RDONLY | O_DIRECT);
  t->direct = t->fd >= 0;
  if (t->fd < 0) t->fd = open(file, O_RDONLY);          // file systems without direct I/O (tmpfs): page-cache reads
  if (t->fd < 0) { delete t; return nullptr; }
  t->n_layers = n_layers; t->E = E; t->n_slots = n_slots; t->K = K; t->I = I; t->gtype = gtype;
  t->n_readers = n_readers < 1 ? 1 : n_readers;
  t->gpart = blh_nv_part_bytes(gtype, I, K);
  if (t->gpart <= 0) { close(t->fd); delete t; return nullptr; }
  t->layers.resize(n_layers);
  for (int l = 0; l < n_layers; ++l) {
    NvLayer& L = t->layers[l];
    L.file_off = layer_off[l];
    L.dtype = layer_dtype[l];
    L.dpart = blh_nv_part_bytes(L.dtype, K, I);
    if (L.dpart <= 0) { blh_nv_close(t); return nullptr; }
    L.blob = 2 * t->gpart + L.dpart;
    void* mem = nullptr;
    if (posix_memalign(&mem, 4096, (size_t)n_slots * (size_t)L.blob) != 0) { blh_nv_close(t); return nullptr; }
    L.arena = (uint8_t*)mem;
    L.slot_of.assign(E, -1);
    L.expert_in.assign(n_slots, -1);
    L.last_use.assign(n_slots, 0);
    L.pinned.assign(n_slots, 0);
  }
  return t;
}

void blh_nv_close(void* h) {
  NvTier* t = (NvTier*)h;
  if (!t) return;
  for (auto& L : t->layers) free(L.arena);
  if (t->fd >= 0) close(t->fd);
  delete t;
}

// pin (1) or unpin (0) an expert: a pinned expert is loaded now and never evicted
int blh_nv_pin(void* h, int layer, int expert, int on) {
  NvTier* t = (NvTier*)h;
  if (layer < 0 || layer >= t->n_layers || expert < 0 || expert >= t->E) return -1;
  if (on && t->ensure(layer, &expert, 1) != 0) return -2;
  const int s = t->layers[layer].slot_of[expert];
  if (s >= 0) t->layers[layer].pinned[s] = on ? 1 : 0;
  return 0;
}

// the expert leg over the arena in one call (tests, the CPU engine): ensure, then compute
int blh_nv_moe_experts(void* h, int layer, int M, int n_used, const int* ids, const float* wts, const int8_t* xq,
                       const float* xds, float* out) {
  NvTier* t = (NvTier*)h;
  if (layer < 0 || layer >= t->n_layers) return -1;
  std::vector<float> act((size_t)M * n_used * t->I);
  std::vector<int8_t> actq((size_t)M * n_used * t->I);
  std::vector<float> actds((size_t)M * n_used * (t->I / 32) * 2);
  return t->serve(layer, M, n_used, ids, wts, xq, xds, out, act.data(), actq.data(), actds.data()) ? 0 : -2;
}

// hits, misses, evictions, bytes read, nanoseconds reading, failures, direct I/O in use
void blh_nv_stats(void* h, uint64_t* out7) {
  NvTier* t = (NvTier*)h;
  out7[0] = t->hits; out7[1] = t->misses; out7[2] = t->evictions; out7[3] = t->bytes_read; out7[4] = t->read_ns;
  out7[5] = t->failed; out7[6] = t->direct ? 1 : 0;
}

int blh_nv_resident(void* h, int layer, int* experts_out) {
  NvTier* t = (NvTier*)h;
  int n = 0;
  for (int s = 0; s < t->n_slots; ++s)
    if (t->layers[layer].expert_in[s] >= 0 && t->layers[layer].slot_of[t->layers[layer].expert_in[s]] == s)
      experts_out[n++] = t->layers[layer].expert_in[s];
  return n;
}

// serve the host tier's cold experts from the arena instead of RAM-resident stacks
void blh_host_tier_set_nv(void* h, void* nv) { ((Tier*)h)->nv = (NvTier*)nv; }

void blh_host_tier_destroy(void* h) {
  blh_host_tier_stop(h);
  delete (Tier*)h;
}

}  // extern "C"
