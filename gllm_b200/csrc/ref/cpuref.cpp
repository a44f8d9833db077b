// Scalar fp32 CPU reference: the correctness oracle and the timed CPU baseline.
//
// Restates the reference's scalar math (src/compat/scalar_ops.rs:11-378: scalar_rms_norm, scalar_gemm,
// scalar_rope half-split, cached_gqa_attention, swiglu_ffn, scalar_moe_gate softmax over all experts,
// scalar_top_k_experts renormalised) and its CPU sampler order of operations (src/compat/sampling.rs:28-135:
// greedy if T <= 0; else sort-desc -> top-k -> /T -> softmax -> top-p cumulative cut -> renorm -> multinomial).
// A Llama-style decoder (RMSNorm, GQA, RoPE, SwiGLU, optional per-head q/k norm, tied or untied head) runs on a
// paged KV cache with 16-token pages: [layer][page][K|V][kv_head][token][D].
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

inline void rms_norm(const float* x, const float* w, float eps, int n, float* y) {
  double ss = 0;
  for (int i = 0; i < n; ++i) ss += double(x[i]) * x[i];
  const float inv = 1.0f / std::sqrt(float(ss / n) + eps);
  for (int i = 0; i < n; ++i) y[i] = x[i] * inv * w[i];
}

// y[M,N] = x[M,K] @ w[N,K]^T
void gemm_tn(const float* x, const float* w, int M, int N, int K, float* y) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const float* wr = w + size_t(n) * K;
    for (int m = 0; m < M; ++m) {
      const float* xr = x + size_t(m) * K;
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
      y[size_t(m) * N + n] = acc;
    }
  }
}

inline void rope_half(float* v, int d, int pos, float theta) {
  const int half = d / 2;
  for (int i = 0; i < half; ++i) {
    const float freq = std::pow(theta, -2.0f * i / d);
    const float a = pos * freq, c = std::cos(a), s = std::sin(a);
    const float x0 = v[i], x1 = v[i + half];
    v[i] = x0 * c - x1 * s;
    v[i + half] = x1 * c + x0 * s;
  }
}

struct Model {
  int layers, hidden, heads, kv_heads, head_dim, inter, vocab, qk_norm;
  float eps, theta;
  const float* embed;
  const float* lm_head;
  const float* final_norm;
  std::vector<const float*> in_norm, post_norm, wq, wk, wv, wo, q_norm, k_norm, w_gate, w_up, w_down;
  // paged KV
  int num_pages = 0;
  std::vector<float> kv;          // [layer][page][2][kv_heads][16][D]
  std::vector<int> block_table;   // logical page -> physical page
  int len = 0;
};

inline float* kv_ptr(Model& m, int layer, int page, int kv, int head, int tok) {
  const size_t per_page = size_t(2) * m.kv_heads * 16 * m.head_dim;
  return m.kv.data() + (size_t(layer) * m.num_pages + page) * per_page +
         ((size_t(kv) * m.kv_heads + head) * 16 + tok) * m.head_dim;
}

// one token at position pos; x in/out [hidden]
void forward_token(Model& m, int token, int pos, float* logits) {
  const int H = m.hidden, D = m.head_dim, nq = m.heads, nkv = m.kv_heads, group = nq / nkv;
  std::vector<float> x(m.embed + size_t(token) * H, m.embed + size_t(token + 1) * H);
  std::vector<float> h(H), q(nq * D), k(nkv * D), v(nkv * D), att(nq * D), o(H), g(m.inter), u(m.inter), d(H);
  std::vector<float> sc(pos + 1);
  const float scale = 1.0f / std::sqrt(float(D));
  const int page = m.block_table[pos / 16], off = pos % 16;
  for (int l = 0; l < m.layers; ++l) {
    rms_norm(x.data(), m.in_norm[l], m.eps, H, h.data());
    gemm_tn(h.data(), m.wq[l], 1, nq * D, H, q.data());
    gemm_tn(h.data(), m.wk[l], 1, nkv * D, H, k.data());
    gemm_tn(h.data(), m.wv[l], 1, nkv * D, H, v.data());
    for (int hd = 0; hd < nq; ++hd) {
      if (m.qk_norm) rms_norm(&q[hd * D], m.q_norm[l], m.eps, D, &q[hd * D]);
      rope_half(&q[hd * D], D, pos, m.theta);
    }
    for (int hd = 0; hd < nkv; ++hd) {
      if (m.qk_norm) rms_norm(&k[hd * D], m.k_norm[l], m.eps, D, &k[hd * D]);
      rope_half(&k[hd * D], D, pos, m.theta);
      std::memcpy(kv_ptr(m, l, page, 0, hd, off), &k[hd * D], sizeof(float) * D);
      std::memcpy(kv_ptr(m, l, page, 1, hd, off), &v[hd * D], sizeof(float) * D);
    }
#pragma omp parallel for schedule(static) firstprivate(sc)
    for (int hd = 0; hd < nq; ++hd) {
      const int kvh = hd / group;
      float mx = -INFINITY;
      for (int t = 0; t <= pos; ++t) {
        const float* kr = kv_ptr(m, l, m.block_table[t / 16], 0, kvh, t % 16);
        float s = 0.f;
        for (int i = 0; i < D; ++i) s += q[hd * D + i] * kr[i];
        sc[t] = s * scale;
        mx = std::max(mx, sc[t]);
      }
      float sum = 0.f;
      for (int t = 0; t <= pos; ++t) {
        sc[t] = std::exp(sc[t] - mx);
        sum += sc[t];
      }
      float* out = &att[hd * D];
      std::fill(out, out + D, 0.f);
      for (int t = 0; t <= pos; ++t) {
        const float* vr = kv_ptr(m, l, m.block_table[t / 16], 1, kvh, t % 16);
        const float p = sc[t] / sum;
        for (int i = 0; i < D; ++i) out[i] += p * vr[i];
      }
    }
    gemm_tn(att.data(), m.wo[l], 1, H, nq * D, o.data());
    for (int i = 0; i < H; ++i) x[i] += o[i];
    rms_norm(x.data(), m.post_norm[l], m.eps, H, h.data());
    gemm_tn(h.data(), m.w_gate[l], 1, m.inter, H, g.data());
    gemm_tn(h.data(), m.w_up[l], 1, m.inter, H, u.data());
    for (int i = 0; i < m.inter; ++i) g[i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
    gemm_tn(g.data(), m.w_down[l], 1, H, m.inter, d.data());
    for (int i = 0; i < H; ++i) x[i] += d[i];
  }
  if (logits) {
    rms_norm(x.data(), m.final_norm, m.eps, H, h.data());
    gemm_tn(h.data(), m.lm_head, 1, m.vocab, H, logits);
  }
}

}  // namespace

REF_API void* gllm_ref_create(int layers, int hidden, int heads, int kv_heads, int head_dim, int inter, int vocab,
                              int qk_norm, float eps, float theta, const float* embed, const float* lm_head,
                              const float* final_norm, int num_pages) {
  Model* m = new Model();
  m->layers = layers; m->hidden = hidden; m->heads = heads; m->kv_heads = kv_heads; m->head_dim = head_dim;
  m->inter = inter; m->vocab = vocab; m->qk_norm = qk_norm; m->eps = eps; m->theta = theta;
  m->embed = embed; m->lm_head = lm_head; m->final_norm = final_norm;
  m->num_pages = num_pages;
  m->kv.assign(size_t(layers) * num_pages * 2 * kv_heads * 16 * head_dim, 0.f);
  // a scrambled (but fixed) logical -> physical map: the paging is exercised, not the identity
  m->block_table.resize(num_pages);
  for (int i = 0; i < num_pages; ++i) m->block_table[i] = (i * 7 + 3) % num_pages;
  if (std::gcd(7, num_pages) != 1) std::iota(m->block_table.begin(), m->block_table.end(), 0);
  return m;
}

// per-layer pointers, in the order: in_norm, post_norm, wq, wk, wv, wo, q_norm, k_norm, gate, up, down
REF_API void gllm_ref_set_layer(void* h, int layer, const float* const* p) {
  Model* m = static_cast<Model*>(h);
  auto put = [&](std::vector<const float*>& v, const float* x) {
    if ((int)v.size() <= layer) v.resize(layer + 1);
    v[layer] = x;
  };
  put(m->in_norm, p[0]); put(m->post_norm, p[1]); put(m->wq, p[2]); put(m->wk, p[3]); put(m->wv, p[4]);
  put(m->wo, p[5]); put(m->q_norm, p[6]); put(m->k_norm, p[7]); put(m->w_gate, p[8]); put(m->w_up, p[9]);
  put(m->w_down, p[10]);
}

REF_API void gllm_ref_destroy(void* h) { delete static_cast<Model*>(h); }
REF_API void gllm_ref_reset(void* h) { static_cast<Model*>(h)->len = 0; }

// Feeds `n` tokens; writes the logits after the last one. Returns the new sequence length or -1.
REF_API int gllm_ref_forward(void* h, const int* tokens, int n, float* logits) {
  Model* m = static_cast<Model*>(h);
  if (m->len + n > m->num_pages * 16) return -1;
  for (int i = 0; i < n; ++i) {
    forward_token(*m, tokens[i], m->len, i == n - 1 ? logits : nullptr);
    ++m->len;
  }
  return m->len;
}

// Greedy generation: prompt then max_new tokens; stops at eos (if >= 0). Returns the number generated.
REF_API int gllm_ref_generate_greedy(void* h, const int* prompt, int n_prompt, int max_new, int eos, int* out) {
  Model* m = static_cast<Model*>(h);
  m->len = 0;
  std::vector<float> logits(m->vocab);
  if (gllm_ref_forward(h, prompt, n_prompt, logits.data()) < 0) return -1;
  int produced = 0;
  while (produced < max_new) {
    const int tok = int(std::max_element(logits.begin(), logits.end()) - logits.begin());
    out[produced++] = tok;
    if (tok == eos || produced == max_new) break;
    if (gllm_ref_forward(h, &tok, 1, logits.data()) < 0) break;
  }
  return produced;
}

// The reference sampler's order of operations. `u` in [0,1) is the uniform draw (the caller owns the RNG).
REF_API int gllm_ref_sample(const float* logits, int vocab, float temperature, int top_k, float top_p, float u) {
  if (temperature <= 0.f) return int(std::max_element(logits, logits + vocab) - logits);
  std::vector<int> idx(vocab);
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return logits[a] > logits[b]; });
  int n = (top_k > 0 && top_k < vocab) ? top_k : vocab;
  std::vector<float> p(n);
  const float mx = logits[idx[0]] / temperature;
  float sum = 0.f;
  for (int i = 0; i < n; ++i) {
    p[i] = std::exp(logits[idx[i]] / temperature - mx);
    sum += p[i];
  }
  for (int i = 0; i < n; ++i) p[i] /= sum;
  if (top_p < 1.0f) {
    float cum = 0.f;
    int keep = n;
    for (int i = 0; i < n; ++i) {
      cum += p[i];
      if (cum >= top_p) {
        keep = i + 1;
        break;
      }
    }
    n = keep;
    float s2 = 0.f;
    for (int i = 0; i < n; ++i) s2 += p[i];
    for (int i = 0; i < n; ++i) p[i] /= s2;
  }
  float cum = 0.f;
  for (int i = 0; i < n; ++i) {
    cum += p[i];
    if (u < cum) return idx[i];
  }
  return idx[n - 1];
}

// MoE pieces of the scalar reference: gate = softmax over ALL experts, top-k renormalised.
REF_API void gllm_ref_moe_gate_topk(const float* logits, int experts, int k, int* ids, float* weights) {
  std::vector<float> p(experts);
  const float mx = *std::max_element(logits, logits + experts);
  float sum = 0.f;
  for (int e = 0; e < experts; ++e) sum += (p[e] = std::exp(logits[e] - mx));
  for (int e = 0; e < experts; ++e) p[e] /= sum;
  std::vector<int> idx(experts);
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return p[a] > p[b]; });
  float s = 0.f;
  for (int i = 0; i < k; ++i) s += p[idx[i]];
  for (int i = 0; i < k; ++i) {
    ids[i] = idx[i];
    weights[i] = p[idx[i]] / s;
  }
}
