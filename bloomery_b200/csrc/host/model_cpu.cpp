// A whole decode step of a mixture-of-experts model on the host, in one native call: embedding row, per layer
// RMSNorm -> q8 -> the attention rows (grouped-query: Q/K/V, per-head norm, rotary over half-split pairs; latent:
// q_a / q_b and kv_a rows, rotary over interleaved pairs, the absorbed form over the cached latent), the f16-rounded
// cache row appended, attention over the cached positions, o rows, then a dense SwiGLU layer or the router (softmax,
// or sigmoid with selection bias and groups; top-k, renormalised), the chosen experts through the expert leg, the
// shared expert, and the head.  Every matrix stays in its resident quantised rows; every product is a
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

// slots of blh_model_set_mat / blh_model_set_vec
enum MatSlot { M_Q = 0, M_K, M_V, M_O, M_QA, M_QB, M_KVA, M_GATE, M_UP, M_DOWN, M_SH_GATE, M_SH_UP, M_SH_DOWN, M_COUNT };
enum VecSlot { V_ATTN_NORM = 0, V_Q_NORM, V_K_NORM, V_FFN_NORM, V_ROUTER, V_ROUTER_BIAS, V_QA_NORM, V_KVA_NORM, V_KB, V_VB, V_COUNT };

struct HostLayer {
  Mat m[M_COUNT];
  const float* v[V_COUNT] = {};
  const uint8_t *gate = nullptr, *up = nullptr, *down = nullptr;     // routed stacks
  int gtype = 0, dtype = 0;
};

struct HostModel {
  int n_layer, hidden, n_q, n_kv, head, vocab, n_expert, n_used, inter, ctx, renorm;
  float eps, router_scale;
  // latent attention, dense layers, shared expert, router rule (blh_model_set_arch)
  int mla = 0, q_lora = 0, kv_lora = 0, rope_dim = 0, nope = 0, v_dim = 0, first_dense = 0, dense_inter = 0, shared_inter = 0;
  int sigmoid = 0, n_group = 1, topk_group = 1;
  float attn_scale = 0.f;
  int kw = 0, vw = 0, att_w = 0;                       // cache row widths, attention output width
  std::vector<HostLayer> layers;
  Mat embd, out;
  const float* out_norm = nullptr;
  std::vector<float> inv_freq;
  std::vector<float> kc, vc;                           // [layer][ctx][kw] / [layer][ctx][vw], values rounded through f16
  std::vector<float> x, h, qkv, qfull, qlat, att, y, logits_r, scores, act, olat;
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

// y = down(q8(silu(gate x) * up x)) for the q8 row already in M.q8 / M.ds (a dense layer or the shared expert)
void swiglu_ffn(HostModel& M, const Mat& gate, const Mat& up, const Mat& down, float* y) {
  const int I = gate.rows;
  M.act.resize((size_t)2 * I);
  float* g = M.act.data();
  float* u = g + I;
  gemv(gate, M.q8.data(), M.ds.data(), g);
  gemv(up, M.q8.data(), M.ds.data(), u);
  for (int i = 0; i < I; ++i) g[i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
  std::vector<int8_t> aq(I);
  std::vector<float> ads((size_t)(I / 32) * 2);
  blh_act_q8(g, 1, I, aq.data(), ads.data());
  gemv(down, aq.data(), ads.data(), y);
}

void attention_gqa(HostModel& M, const HostLayer& L, int il, int pos) {
  const int D = M.head, nq = M.n_q, nkv = M.n_kv, G = nq / nkv, half = D / 2;
  const float inv_sqrt_d = 1.0f / std::sqrt((float)D);
  float* q = M.qkv.data();
  float* k = q + (long)nq * D;
  float* v = k + (long)nkv * D;
  gemv(L.m[M_Q], M.q8.data(), M.ds.data(), q);
  gemv(L.m[M_K], M.q8.data(), M.ds.data(), k);
  gemv(L.m[M_V], M.q8.data(), M.ds.data(), v);
  float* kc = M.kc.data() + ((size_t)il * M.ctx + pos) * M.kw;
  float* vc = M.vc.data() + ((size_t)il * M.ctx + pos) * M.vw;
  auto rotate = [&](float* x) {                         // pairs (i, i + D/2)
    for (int i = 0; i < half; ++i) {
      const float ang = (float)pos * M.inv_freq[i];
      const float c = std::cos(ang), s = std::sin(ang);
      const float x0 = x[i], x1 = x[i + half];
      x[i] = x0 * c - x1 * s;
      x[i + half] = x0 * s + x1 * c;
    }
  };
  for (int hh = 0; hh < nq; ++hh) {
    if (L.v[V_Q_NORM]) rms_norm(q + (long)hh * D, L.v[V_Q_NORM], M.eps, D, q + (long)hh * D);
    rotate(q + (long)hh * D);
  }
  for (int hh = 0; hh < nkv; ++hh) {
    if (L.v[V_K_NORM]) rms_norm(k + (long)hh * D, L.v[V_K_NORM], M.eps, D, k + (long)hh * D);
    rotate(k + (long)hh * D);
    for (int i = 0; i < D; ++i) {
      kc[(long)hh * D + i] = through_half(k[(long)hh * D + i]);
      vc[(long)hh * D + i] = through_half(v[(long)hh * D + i]);
    }
  }
  const float* kl = M.kc.data() + (size_t)il * M.ctx * M.kw;
  const float* vl = M.vc.data() + (size_t)il * M.ctx * M.vw;
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
}

// Latent attention in the absorbed form: the query's no-rotary part is carried into the latent space through k_b, the
// scores run against the cached latent and the shared rotary key, the weighted latent sum goes through v_b.
void attention_mla(HostModel& M, const HostLayer& L, int il, int pos) {
  const int nq = M.n_q, C = M.kv_lora, R = M.rope_dim, NP = M.nope, VD = M.v_dim, QK = NP + R;
  float* q = M.qfull.data();
  if (M.q_lora) {
    float* qa = M.qkv.data();
    gemv(L.m[M_QA], M.q8.data(), M.ds.data(), qa);
    std::vector<float> qn(M.q_lora);
    rms_norm(qa, L.v[V_QA_NORM], M.eps, M.q_lora, qn.data());
    std::vector<int8_t> aq(M.q_lora);
    std::vector<float> ads((size_t)(M.q_lora / 32) * 2);
    blh_act_q8(qn.data(), 1, M.q_lora, aq.data(), ads.data());
    gemv(L.m[M_QB], aq.data(), ads.data(), q);
  } else {
    gemv(L.m[M_Q], M.q8.data(), M.ds.data(), q);
  }
  std::vector<float> kva(C + R);
  gemv(L.m[M_KVA], M.q8.data(), M.ds.data(), kva.data());
  float* row = M.kc.data() + ((size_t)il * M.ctx + pos) * M.kw;
  rms_norm(kva.data(), L.v[V_KVA_NORM], M.eps, C, row);
  auto rotate = [&](float* x) {                         // interleaved pairs (2i, 2i + 1)
    for (int i = 0; i < R / 2; ++i) {
      const float ang = (float)pos * M.inv_freq[i];
      const float c = std::cos(ang), s = std::sin(ang);
      const float x0 = x[2 * i], x1 = x[2 * i + 1];
      x[2 * i] = x0 * c - x1 * s;
      x[2 * i + 1] = x0 * s + x1 * c;
    }
  };
  rotate(kva.data() + C);
  for (int i = 0; i < R; ++i) row[C + i] = kva[C + i];
  for (int i = 0; i < C + R; ++i) row[i] = through_half(row[i]);
  const float* cache = M.kc.data() + (size_t)il * M.ctx * M.kw;
  blh::Pool::instance().parallel_for(nq, 1, [&](int h0, int h1) {
    for (int hh = h0; hh < h1; ++hh) {
      float* qh = q + (long)hh * QK;
      rotate(qh + NP);
      // q_lat[c] = sum_n q_nope[n] * k_b[h][n][c]
      float* ql = M.qlat.data() + (long)hh * C;
      const float* kb = L.v[V_KB] + (size_t)hh * NP * C;
      for (int c = 0; c < C; ++c) ql[c] = 0.f;
      for (int n = 0; n < NP; ++n) {
        const float qn = qh[n];
        const float* kr = kb + (size_t)n * C;
        for (int c = 0; c < C; ++c) ql[c] += qn * kr[c];
      }
      float* sc = M.scores.data() + (size_t)hh * M.ctx;
      float mx = -INFINITY;
      for (int s = 0; s <= pos; ++s) {
        const float* rs = cache + (size_t)s * M.kw;
        float acc = 0.f;
        for (int c = 0; c < C; ++c) acc += ql[c] * rs[c];
        for (int r = 0; r < R; ++r) acc += qh[NP + r] * rs[C + r];
        sc[s] = acc * M.attn_scale;
        mx = std::fmax(mx, sc[s]);
      }
      float sum = 0.f;
      for (int s = 0; s <= pos; ++s) { sc[s] = std::exp(sc[s] - mx); sum += sc[s]; }
      const float inv = 1.0f / sum;
      float* ol = M.olat.data() + (long)hh * C;
      for (int c = 0; c < C; ++c) ol[c] = 0.f;
      for (int s = 0; s <= pos; ++s) {
        const float p = sc[s] * inv;
        const float* rs = cache + (size_t)s * M.kw;
        for (int c = 0; c < C; ++c) ol[c] += p * rs[c];
      }
      const float* vb = L.v[V_VB] + (size_t)hh * VD * C;
      float* out = M.att.data() + (long)hh * VD;
      for (int v = 0; v < VD; ++v) {
        float acc = 0.f;
        const float* vr = vb + (size_t)v * C;
        for (int c = 0; c < C; ++c) acc += vr[c] * ol[c];
        out[v] = acc;
      }
    }
  });
}

// ids / weights of the row's experts from the router logits: softmax over all experts, or sigmoid with a selection bias
// and a group limit; the k largest choices (ties to the smaller id); weights renormalised over the chosen ones.
void route(const HostModel& M, const HostLayer& L, const float* logits, int* ids, float* wts) {
  const int E = M.n_expert, kk = M.n_used;
  std::vector<float> probs(E), choice(E);
  if (!M.sigmoid) {
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) mx = std::fmax(mx, logits[e]);
    float sum = 0.f;
    for (int e = 0; e < E; ++e) { probs[e] = std::exp(logits[e] - mx); sum += probs[e]; }
    for (int e = 0; e < E; ++e) { probs[e] /= sum; choice[e] = probs[e]; }
  } else {
    for (int e = 0; e < E; ++e) {
      probs[e] = 1.0f / (1.0f + std::exp(-logits[e]));
      choice[e] = probs[e] + (L.v[V_ROUTER_BIAS] ? L.v[V_ROUTER_BIAS][e] : 0.0f);
    }
  }
  if (M.n_group > 1) {
    const int per = E / M.n_group;
    std::vector<float> gs(M.n_group);
    for (int g = 0; g < M.n_group; ++g) {              // a group's score: its two largest choices
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < per; ++i) {
        const float c = choice[g * per + i];
        if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
      }
      gs[g] = a + b;
    }
    std::vector<int> go(M.n_group);
    for (int g = 0; g < M.n_group; ++g) go[g] = g;
    std::stable_sort(go.begin(), go.end(), [&](int a, int b) { return gs[a] > gs[b]; });
    std::vector<char> keep(M.n_group, 0);
    for (int j = 0; j < M.topk_group; ++j) keep[go[j]] = 1;
    for (int e = 0; e < E; ++e) if (!keep[e / per]) choice[e] = -INFINITY;
  }
  std::vector<int> order(E);
  for (int e = 0; e < E; ++e) order[e] = e;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return choice[a] > choice[b]; });
  double wsum = 0.0;
  for (int j = 0; j < kk; ++j) { ids[j] = order[j]; wts[j] = probs[order[j]]; wsum += (double)wts[j]; }
  for (int j = 0; j < kk; ++j) wts[j] = (M.renorm ? wts[j] / (float)wsum : wts[j]) * M.router_scale;
}

}  // namespace

extern "C" {

void* blh_model_create(int n_layer, int hidden, int n_q, int n_kv, int head, int vocab, int n_expert, int n_used, int inter,
                       int ctx, float eps, int renorm, float router_scale, const float* inv_freq, int n_freq) {
  if (n_layer < 1 || hidden % 256 || n_q < 1 || ctx < 1 || n_used < 0 || n_used > n_expert || n_freq < 1) return nullptr;
  auto* M = new HostModel();
  M->n_layer = n_layer; M->hidden = hidden; M->n_q = n_q; M->n_kv = n_kv; M->head = head; M->vocab = vocab;
  M->n_expert = n_expert; M->n_used = n_used; M->inter = inter; M->ctx = ctx; M->eps = eps; M->renorm = renorm;
  M->router_scale = router_scale;
  M->layers.resize(n_layer);
  M->inv_freq.assign(inv_freq, inv_freq + n_freq);
  return M;
}

// Attention kind and layer plan; sizes the caches and the scratch.  Call once, after blh_model_create.
int blh_model_set_arch(void* h, int mla, int q_lora, int kv_lora, int rope_dim, int nope, int v_dim, float attn_scale,
                       int first_dense, int dense_inter, int shared_inter, int sigmoid, int n_group, int topk_group) {
  auto* M = (HostModel*)h;
  M->mla = mla; M->q_lora = q_lora; M->kv_lora = kv_lora; M->rope_dim = rope_dim; M->nope = nope; M->v_dim = v_dim;
  M->attn_scale = attn_scale; M->first_dense = first_dense; M->dense_inter = dense_inter; M->shared_inter = shared_inter;
  M->sigmoid = sigmoid; M->n_group = n_group < 1 ? 1 : n_group; M->topk_group = topk_group < 1 ? 1 : topk_group;
  if (mla) {
    if (kv_lora % 32 || rope_dim % 2 || (q_lora && q_lora % 256) || (int)M->inv_freq.size() < rope_dim / 2) return -1;
    M->kw = kv_lora + rope_dim; M->vw = 0; M->att_w = M->n_q * v_dim;
  } else {
    if (M->head % 2 || M->n_kv < 1 || M->n_q % M->n_kv || (int)M->inv_freq.size() < M->head / 2) return -1;
    M->kw = M->n_kv * M->head; M->vw = M->kw; M->att_w = M->n_q * M->head;
  }
  if (M->att_w % 32 || (M->n_expert && M->n_expert % M->n_group) || M->topk_group > M->n_group) return -1;
  const int H = M->hidden;
  M->kc.assign((size_t)M->n_layer * M->ctx * M->kw, 0.f);
  M->vc.assign((size_t)M->n_layer * M->ctx * (M->vw ? M->vw : 1), 0.f);
  M->x.resize(H); M->h.resize(H); M->y.resize(H);
  M->qkv.resize(mla ? (size_t)(q_lora > 0 ? q_lora : 1) : (size_t)(M->n_q + 2 * M->n_kv) * M->head);
  M->qfull.resize(mla ? (size_t)M->n_q * (nope + rope_dim) : 1);
  M->qlat.resize(mla ? (size_t)M->n_q * kv_lora : 1);
  M->olat.resize(mla ? (size_t)M->n_q * kv_lora : 1);
  M->att.resize(M->att_w);
  M->logits_r.resize(M->n_expert > 0 ? M->n_expert : 1);
  M->scores.resize((size_t)M->n_q * M->ctx);
  return 0;
}

void blh_model_destroy(void* h) { delete (HostModel*)h; }

void blh_model_set_io(void* h, const uint8_t* embd, int embd_type, const uint8_t* out, int out_type, const float* out_norm) {
  auto* M = (HostModel*)h;
  M->embd = Mat{embd, embd_type, M->vocab, M->hidden};
  M->out = Mat{out, out_type, M->vocab, M->hidden};
  M->out_norm = out_norm;
}

int blh_model_set_mat(void* h, int il, int slot, const uint8_t* w, int type, int rows, int K) {
  auto* M = (HostModel*)h;
  if (il < 0 || il >= M->n_layer || slot < 0 || slot >= M_COUNT || K % 64 || resident_row_bytes(type, K) <= 0) return -1;
  M->layers[il].m[slot] = Mat{w, type, rows, K};
  return 0;
}

int blh_model_set_vec(void* h, int il, int slot, const float* v) {
  auto* M = (HostModel*)h;
  if (il < 0 || il >= M->n_layer || slot < 0 || slot >= V_COUNT) return -1;
  M->layers[il].v[slot] = v;
  return 0;
}

void blh_model_set_experts(void* h, int il, const uint8_t* gate, const uint8_t* up, const uint8_t* down, int gtype, int dtype) {
  HostLayer& L = ((HostModel*)h)->layers[il];
  L.gate = gate; L.up = up; L.down = down; L.gtype = gtype; L.dtype = dtype;
}

// The first n positions of the sequence's cache, out to / in from [layer][n][k width] (and [layer][n][v width]) floats
// (snapshots, shared prefixes, slot files).  0 on success.
int blh_model_kv_get(void* h, int n, float* k, float* v) {
  auto* M = (HostModel*)h;
  if (n < 0 || n > M->ctx) return -1;
  for (int il = 0; il < M->n_layer; ++il) {
    std::memcpy(k + (size_t)il * n * M->kw, M->kc.data() + (size_t)il * M->ctx * M->kw, (size_t)n * M->kw * sizeof(float));
    if (M->vw) std::memcpy(v + (size_t)il * n * M->vw, M->vc.data() + (size_t)il * M->ctx * M->vw, (size_t)n * M->vw * sizeof(float));
  }
  return 0;
}

int blh_model_kv_set(void* h, int n, const float* k, const float* v) {
  auto* M = (HostModel*)h;
  if (n < 0 || n > M->ctx) return -1;
  for (int il = 0; il < M->n_layer; ++il) {
    std::memcpy(M->kc.data() + (size_t)il * M->ctx * M->kw, k + (size_t)il * n * M->kw, (size_t)n * M->kw * sizeof(float));
    if (M->vw) std::memcpy(M->vc.data() + (size_t)il * M->ctx * M->vw, v + (size_t)il * n * M->vw, (size_t)n * M->vw * sizeof(float));
  }
  return 0;
}

// One token at position pos (0 <= pos < ctx; the positions before it hold this sequence's earlier tokens).
// logits == null skips the head (prompt positions whose next token is known).  0 on success.
int blh_model_step(void* h, int token, int pos, float* logits) {
  auto* Mp = (HostModel*)h;
  HostModel& M = *Mp;
  if (token < 0 || token >= M.vocab || pos < 0 || pos >= M.ctx || M.kw == 0) return -1;
  const int H = M.hidden;
  if (blh_decode_rows(M.embd.type, M.embd.w + (long)token * resident_row_bytes(M.embd.type, H), 1, H, M.x.data())) return -2;
  for (int il = 0; il < M.n_layer; ++il) {
    const HostLayer& L = M.layers[il];
    rms_norm(M.x.data(), L.v[V_ATTN_NORM], M.eps, H, M.h.data());
    quantise(M, M.h.data(), H);
    if (M.mla) attention_mla(M, L, il, pos); else attention_gqa(M, L, il, pos);
    quantise(M, M.att.data(), M.att_w);
    gemv(L.m[M_O], M.q8.data(), M.ds.data(), M.y.data());
    for (int i = 0; i < H; ++i) M.x[i] += M.y[i];
    rms_norm(M.x.data(), L.v[V_FFN_NORM], M.eps, H, M.h.data());
    if (il < M.first_dense || M.n_expert == 0) {
      quantise(M, M.h.data(), H);
      swiglu_ffn(M, L.m[M_GATE], L.m[M_UP], L.m[M_DOWN], M.y.data());
      for (int i = 0; i < H; ++i) M.x[i] += M.y[i];
      continue;
    }
    // router on the normed row in fp32
    const int E = M.n_expert, kk = M.n_used;
    blh::Pool::instance().parallel_for(E, 8, [&](int e0, int e1) {
      for (int e = e0; e < e1; ++e) {
        const float* wr = L.v[V_ROUTER] + (long)e * H;
        float acc = 0.f;
        for (int i = 0; i < H; ++i) acc += M.h[i] * wr[i];
        M.logits_r[e] = acc;
      }
    });
    std::vector<int> ids(kk);
    std::vector<float> wts(kk);
    route(M, L, M.logits_r.data(), ids.data(), wts.data());
    quantise(M, M.h.data(), H);
    if (blh_moe_experts(1, H, M.inter, E, kk, ids.data(), wts.data(), M.q8.data(), M.ds.data(), L.gate, L.up, L.down, L.gtype,
                        L.dtype, M.y.data())) return -3;
    for (int i = 0; i < H; ++i) M.x[i] += M.y[i];
    if (M.shared_inter) {
      swiglu_ffn(M, L.m[M_SH_GATE], L.m[M_SH_UP], L.m[M_SH_DOWN], M.y.data());    // M.q8 still holds the normed row
      for (int i = 0; i < H; ++i) M.x[i] += M.y[i];
    }
  }
  if (!logits) return 0;
  rms_norm(M.x.data(), M.out_norm, M.eps, H, M.h.data());
  quantise(M, M.h.data(), H);
  gemv(M.out, M.q8.data(), M.ds.data(), logits);
  return 0;
}

}  // extern "C"
