// A whole decode step of a grouped-query-attention mixture-of-experts model on the host, in one native call:
// embedding row, per layer RMSNorm -> q8 -> Q/K/V rows, per-head norm and rotary, f16-rounded K/V appended to the
// sequence's cache, attention over the cached positions, o rows, router (softmax top-k, renormalised), the chosen
// experts through the expert leg, and the head.  Every matrix stays in its resident quantised rows; every product is a
// quantised row dot against q8 activations (the CPU's VNNI / AVX2 / scalar path), so the arithmetic is the CPU
// oracle's (models/cpu_ref.py) up to the order of fp32 sums.  Rows of one matrix and heads of one attention are
// spread over the resident worker pool.
// Counterpart of the reference's host model crate (crates/models: the CPU engine whose trunk and experts both run
// native, `docs/architecture.md` "host path").
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "../quant_units.cuh"
#include "pool.h"

using namespace bl;

namespace blh {
float dot_row(int wtype, const uint8_t* row, int K, const int8_t* xq, const float* xds);
}

extern "C" {
void blh_act_q8(const float* x, int M, int K, int8_t* codes, float* ds);
int blh_decode_rows(int wtype, const uint8_t* w, int rows, int K, float* out);
int blh_moe_experts(int M, int K, int I, int E, int n_used, const int* ids, const float* wts, const int8_t* xq,
                    const float* xds, const uint8_t* gate, const uint8_t* up, const uint8_t* down, int gtype, int dtype,
                    float* out);
}

namespace {

struct Mat { const uint8_t* w = nullptr; int type = 0, rows = 0, K = 0; };

struct HostLayer {
  Mat q, k, v, o;
  const float *attn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *ffn_norm = nullptr;
  const float* router = nullptr;                       // [n_expert][hidden] f32
  const uint8_t *gate = nullptr, *up = nullptr, *down = nullptr;
  int gtype = 0, dtype = 0;
};

struct HostModel {
  int n_layer, hidden, n_q, n_kv, head, vocab, n_expert, n_used, inter, ctx, renorm;
  float eps, router_scale;
  std::vector<HostLayer> layers;
  Mat embd, out;
  const float* out_norm = nullptr;
  std::vector<float> inv_freq;                         // head / 2
  std::vector<float> kc, vc;                           // [layer][ctx][n_kv * head], values rounded through f16
  // scratch of one step
  std::vector<float> x, h, qkv, att, y, logits_r, scores;
  std::vector<int8_t> q8;
  std::vector<float> ds;
};

// float -> nearest f16 -> float (round to nearest even), what a cache of halves keeps
inline float through_half(float f) {
  uint32_t b;
  std::memcpy(&b, &f, 4);
  const uint32_t sign = b & 0x80000000u;
  uint32_t x = b & 0x7FFFFFFFu;
  if (x >= 0x7F800000u) return f;                                            // inf / nan
  if (x < 0x38800000u) {                                                     // below the smallest normal half: steps of 2^-24
    const float q = std::nearbyintf(std::fabs(f) * 16777216.0f) / 16777216.0f;
    return sign ? -q : q;
  }
  x += 0xFFFu + ((x >> 13) & 1u);
  x &= ~0x1FFFu;
  if (x >= 0x47800000u) x = 0x7F800000u;
  x |= sign;
  float out;
  std::memcpy(&out, &x, 4);
  return out;
}

void rms_norm(const float* x, const float* gain, float eps, int n, float* out) {
  double ss = 0.0;
  for (int i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
  const float scale = (float)(1.0 / std::sqrt(ss / n + (double)eps));
  for (int i = 0; i < n; ++i) out[i] = x[i] * scale * gain[i];
}

void gemv(const Mat& m, const int8_t* xq, const float* xds, float* out) {
  const long rb = resident_row_bytes(m.type, m.K);
  blh::Pool::instance().parallel_for(m.rows, 32, [&](int r0, int r1) {
    for (int r = r0; r < r1; ++r) out[r] = blh::dot_row(m.type, m.w + (long)r * rb, m.K, xq, xds);
  });
}

void quantise(HostModel& M, const float* x, int K) {
  M.q8.resize(K);
  M.ds.resize((size_t)(K / 32) * 2);
  blh_act_q8(x, 1, K, M.q8.data(), M.ds.data());
}

}  // namespace

extern "C" {

void* blh_model_create(int n_layer, int hidden, int n_q, int n_kv, int head, int vocab, int n_expert, int n_used, int inter,
                       int ctx, float eps, int renorm, float router_scale, const float* inv_freq) {
  if (n_layer < 1 || hidden % 256 || head % 2 || n_q % n_kv || ctx < 1 || n_used < 1 || n_used > n_expert) return nullptr;
  auto* M = new HostModel();
  M->n_layer = n_layer; M->hidden = hidden; M->n_q = n_q; M->n_kv = n_kv; M->head = head; M->vocab = vocab;
  M->n_expert = n_expert; M->n_used = n_used; M->inter = inter; M->ctx = ctx; M->eps = eps; M->renorm = renorm;
  M->router_scale = router_scale;
  M->layers.resize(n_layer);
  M->inv_freq.assign(inv_freq, inv_freq + head / 2);
  M->kc.assign((size_t)n_layer * ctx * n_kv * head, 0.f);
  M->vc.assign((size_t)n_layer * ctx * n_kv * head, 0.f);
  M->x.resize(hidden); M->h.resize(hidden); M->y.resize(hidden);
  M->qkv.resize((size_t)(n_q + 2 * n_kv) * head);
  M->att.resize((size_t)n_q * head);
  M->logits_r.resize(n_expert);
  M->scores.resize((size_t)n_q * ctx);
  return M;
}

void blh_model_destroy(void* h) { delete (HostModel*)h; }

void blh_model_set_io(void* h, const uint8_t* embd, int embd_type, const uint8_t* out, int out_type, const float* out_norm) {
  auto* M = (HostModel*)h;
  M->embd = Mat{embd, embd_type, M->vocab, M->hidden};
  M->out = Mat{out, out_type, M->vocab, M->hidden};
  M->out_norm = out_norm;
}

void blh_model_set_layer(void* h, int il, const uint8_t* q, int tq, const uint8_t* k, int tk, const uint8_t* v, int tv,
                         const uint8_t* o, int to, const float* attn_norm, const float* q_norm, const float* k_norm,
                         const float* ffn_norm, const float* router, const uint8_t* gate, const uint8_t* up,
                         const uint8_t* down, int gtype, int dtype) {
  auto* M = (HostModel*)h;
  HostLayer& L = M->layers[il];
  L.q = Mat{q, tq, M->n_q * M->head, M->hidden};
  L.k = Mat{k, tk, M->n_kv * M->head, M->hidden};
  L.v = Mat{v, tv, M->n_kv * M->head, M->hidden};
  L.o = Mat{o, to, M->hidden, M->n_q * M->head};
  L.attn_norm = attn_norm; L.q_norm = q_norm; L.k_norm = k_norm; L.ffn_norm = ffn_norm; L.router = router;
  L.gate = gate; L.up = up; L.down = down; L.gtype = gtype; L.dtype = dtype;
}

// The first n positions of the sequence's cache, out to / in from [layer][n][n_kv * head] floats (snapshots, shared
// prefixes, slot files).  0 on success.
int blh_model_kv_get(void* h, int n, float* k, float* v) {
  auto* M = (HostModel*)h;
  if (n < 0 || n > M->ctx) return -1;
  const size_t w = (size_t)M->n_kv * M->head;
  for (int il = 0; il < M->n_layer; ++il) {
    std::memcpy(k + (size_t)il * n * w, M->kc.data() + (size_t)il * M->ctx * w, (size_t)n * w * sizeof(float));
    std::memcpy(v + (size_t)il * n * w, M->vc.data() + (size_t)il * M->ctx * w, (size_t)n * w * sizeof(float));
  }
  return 0;
}

int blh_model_kv_set(void* h, int n, const float* k, const float* v) {
  auto* M = (HostModel*)h;
  if (n < 0 || n > M->ctx) return -1;
  const size_t w = (size_t)M->n_kv * M->head;
  for (int il = 0; il < M->n_layer; ++il) {
    std::memcpy(M->kc.data() + (size_t)il * M->ctx * w, k + (size_t)il * n * w, (size_t)n * w * sizeof(float));
    std::memcpy(M->vc.data() + (size_t)il * M->ctx * w, v + (size_t)il * n * w, (size_t)n * w * sizeof(float));
  }
  return 0;
}

// One token at position pos (0 <= pos < ctx; the positions before it hold this sequence's earlier tokens).
// logits == null skips the head (prompt positions whose next token is known).  0 on success.
int blh_model_step(void* h, int token, int pos, float* logits) {
  auto* Mp = (HostModel*)h;
  HostModel& M = *Mp;
  if (token < 0 || token >= M.vocab || pos < 0 || pos >= M.ctx) return -1;
  const int H = M.hidden, D = M.head, nq = M.n_q, nkv = M.n_kv, G = nq / nkv, half = D / 2;
  if (blh_decode_rows(M.embd.type, M.embd.w + (long)token * resident_row_bytes(M.embd.type, H), 1, H, M.x.data())) return -2;
  const float inv_sqrt_d = 1.0f / std::sqrt((float)D);
  for (int il = 0; il < M.n_layer; ++il) {
    const HostLayer& L = M.layers[il];
    rms_norm(M.x.data(), L.attn_norm, M.eps, H, M.h.data());
    quantise(M, M.h.data(), H);
    float* q = M.qkv.data();
    float* k = q + (long)nq * D;
    float* v = k + (long)nkv * D;
    gemv(L.q, M.q8.data(), M.ds.data(), q);
    gemv(L.k, M.q8.data(), M.ds.data(), k);
    gemv(L.v, M.q8.data(), M.ds.data(), v);
    // per-head norm, rotary over pairs (i, i + D/2), keys and values through f16 into the cache
    float* kc = M.kc.data() + ((size_t)il * M.ctx + pos) * nkv * D;
    float* vc = M.vc.data() + ((size_t)il * M.ctx + pos) * nkv * D;
    auto rotate = [&](float* x) {
      for (int i = 0; i < half; ++i) {
        const float ang = (float)pos * M.inv_freq[i];
        const float c = std::cos(ang), s = std::sin(ang);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * c - x1 * s;
        x[i + half] = x0 * s + x1 * c;
      }
    };
    for (int hh = 0; hh < nq; ++hh) {
      if (L.q_norm) rms_norm(q + (long)hh * D, L.q_norm, M.eps, D, q + (long)hh * D);
      rotate(q + (long)hh * D);
    }
    for (int hh = 0; hh < nkv; ++hh) {
      if (L.k_norm) rms_norm(k + (long)hh * D, L.k_norm, M.eps, D, k + (long)hh * D);
      rotate(k + (long)hh * D);
      for (int i = 0; i < D; ++i) {
        kc[(long)hh * D + i] = through_half(k[(long)hh * D + i]);
        vc[(long)hh * D + i] = through_half(v[(long)hh * D + i]);
      }
    }
    // attention of every query head over positions 0 .. pos
    const float* kl = M.kc.data() + (size_t)il * M.ctx * nkv * D;
    const float* vl = M.vc.data() + (size_t)il * M.ctx * nkv * D;
    blh::Pool::instance().parallel_for(nq, 1, [&](int h0, int h1) {
      for (int hh = h0; hh < h1; ++hh) {
        const int kvh = hh / G;
        const float* qh = q + (long)hh * D;
        float* sc = M.scores.data() + (size_t)hh * M.ctx;
        float mx = -INFINITY;
        for (int s = 0; s <= pos; ++s) {
          const float* ks = kl + ((size_t)s * nkv + kvh) * D;
          float acc = 0.f;
          for (int i = 0; i < D; ++i) acc += qh[i] * ks[i];
          sc[s] = acc * inv_sqrt_d;
          mx = std::fmax(mx, sc[s]);
        }
        float sum = 0.f;
        for (int s = 0; s <= pos; ++s) { sc[s] = std::exp(sc[s] - mx); sum += sc[s]; }
        const float inv = 1.0f / sum;
        float* out = M.att.data() + (long)hh * D;
        for (int i = 0; i < D; ++i) out[i] = 0.f;
        for (int s = 0; s <= pos; ++s) {
          const float p = sc[s] * inv;
          const float* vs = vl + ((size_t)s * nkv + kvh) * D;
          for (int i = 0; i < D; ++i) out[i] += p * vs[i];
        }
      }
    });
    quantise(M, M.att.data(), nq * D);
    gemv(L.o, M.q8.data(), M.ds.data(), M.y.data());
    for (int i = 0; i < H; ++i) M.x[i] += M.y[i];
    // router on the normed row in fp32, softmax over all experts, top-k (ties to the smaller id), renormalised
    rms_norm(M.x.data(), L.ffn_norm, M.eps, H, M.h.data());
    const int E = M.n_expert, kk = M.n_used;
    blh::Pool::instance().parallel_for(E, 8, [&](int e0, int e1) {
      for (int e = e0; e < e1; ++e) {
        const float* wr = L.router + (long)e * H;
        float acc = 0.f;
        for (int i = 0; i < H; ++i) acc += M.h[i] * wr[i];
        M.logits_r[e] = acc;
      }
    });
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = std::fmax(mx, M.logits_r[e]);
    float sum = 0.f;
    std::vector<float> probs(E);
    for (int e = 0; e < E; ++e) { probs[e] = std::exp(M.logits_r[e] - mx); sum += probs[e]; }
    for (int e = 0; e < E; ++e) probs[e] /= sum;
    std::vector<int> order(E);
    for (int e = 0; e < E; ++e) order[e] = e;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return probs[a] > probs[b]; });
    std::vector<int> ids(kk);
    std::vector<float> wts(kk);
    double wsum = 0.0;
    for (int j = 0; j < kk; ++j) { ids[j] = order[j]; wts[j] = probs[order[j]]; wsum += (double)wts[j]; }
    for (int j = 0; j < kk; ++j) wts[j] = (M.renorm ? wts[j] / (float)wsum : wts[j]) * M.router_scale;
    quantise(M, M.h.data(), H);
    if (blh_moe_experts(1, H, M.inter, E, kk, ids.data(), wts.data(), M.q8.data(), M.ds.data(), L.gate, L.up, L.down, L.gtype,
                        L.dtype, M.y.data())) return -3;
    for (int i = 0; i < H; ++i) M.x[i] += M.y[i];
  }
  if (!logits) return 0;
  rms_norm(M.x.data(), M.out_norm, M.eps, H, M.h.data());
  quantise(M, M.h.data(), H);
  gemv(M.out, M.q8.data(), M.ds.data(), logits);
  return 0;
}

}  // extern "C"
