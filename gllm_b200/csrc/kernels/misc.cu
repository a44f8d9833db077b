// Bandwidth-bound helper kernels: embedding gather, RMSNorm / LayerNorm, standalone RoPE + paged KV
// write (any head_dim), GLU activation, generic paged attention for head dims other than 128,
// pooling, and the sampling pipeline.
//
// Reference semantics: src/compat/scalar_ops.rs:11-63 (rms norm, half-split RoPE),
// src/compat/sampling.rs:28-135 (greedy if T<=0, else top-k -> 1/T -> softmax -> top-p -> multinomial),
// src/arch/auto_graph_fragments/build_graph.inc.rs:213 (Gather), :2424 (MeanPool).
#include <cuda_fp8.h>

#include "common.cuh"

namespace gllm {

// ---------------------------------------------------------------------------------------------
// block reductions
// ---------------------------------------------------------------------------------------------
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}

// ---------------------------------------------------------------------------------------------
// embedding gather: out[m,:] = table[ids[m],:] * scale ; ss_out[m] = sum(out^2)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) embed_gather_kernel(const int* ids, const __nv_bfloat16* table, int vocab,
                                                           int hidden, float scale, __nv_bfloat16* out,
                                                           float* ss_out, int* err) {
  __shared__ float red[32];
  const int m = blockIdx.x;
  int id = ids[m];
  if (id < 0 || id >= vocab) {
    if (err && threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_ARG);
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<long long>(id) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(m) * hidden);
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    uint4 u = src[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __bfloat1622float2(h[e]);
      if (scale != 1.0f) {
        f.x = bf16_round(f.x * scale);
        f.y = bf16_round(f.y * scale);
        h[e] = __floats2bfloat162_rn(f.x, f.y);
      }
      ss += f.x * f.x + f.y * f.y;
    }
    dst[i] = u;
  }
  if (ss_out) {
    ss = block_sum<128>(ss, red);
    if (threadIdx.x == 0) ss_out[m] = ss;
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm (optionally fused residual add): h = x (+ residual); y = h * rsqrt(mean h^2 + eps) * (w | 1+w)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* x, const __nv_bfloat16* residual,
                                                      const float* w, int hidden, float eps, int one_plus_w,
                                                      __nv_bfloat16* h_out, __nv_bfloat16* y, float* ss_out) {
  __shared__ float red[32];
  extern __shared__ float row[];
  const long long off = static_cast<long long>(blockIdx.x) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = __bfloat162float(x[off + i]);
    if (residual) v = bf16_round(v + __bfloat162float(residual[off + i]));
    row[i] = v;
    ss += v * v;
    if (h_out) h_out[off + i] = __float2bfloat16_rn(v);
  }
  ss = block_sum<256>(ss, red);
  if (ss_out && threadIdx.x == 0) ss_out[blockIdx.x] = ss;
  if (!y) return;
  const float r = rsqrtf(ss / hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float g = w ? (one_plus_w ? 1.f + w[i] : w[i]) : 1.f;
    y[off + i] = __float2bfloat16_rn(row[i] * r * g);
  }
}

// LayerNorm with optional residual add (encoder models).
__global__ void __launch_bounds__(256) layernorm_kernel(const __nv_bfloat16* x, const __nv_bfloat16* residual,
                                                        const float* w, const float* b, int hidden, float eps,
                                                        __nv_bfloat16* y) {
  __shared__ float red[32];
  extern __shared__ float row[];
  const long long off = static_cast<long long>(blockIdx.x) * hidden;
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = __bfloat162float(x[off + i]);
    if (residual) v += __bfloat162float(residual[off + i]);
    row[i] = v;
    s += v;
  }
  const float mean = block_sum<256>(s, red) / hidden;
  float var = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row[i] - mean;
    var += d * d;
  }
  var = block_sum<256>(var, red) / hidden;
  const float r = rsqrtf(var + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    y[off + i] = __float2bfloat16_rn((row[i] - mean) * r * (w ? w[i] : 1.f) + (b ? b[i] : 0.f));
  }
}

// ---------------------------------------------------------------------------------------------
// GLU activation on a fused [M, 2I] buffer (gate | up halves): out[M, I]
// ---------------------------------------------------------------------------------------------
__global__ void glu_kernel(const __nv_bfloat16* gu, long long ld, int inter, int act, __nv_bfloat16* out) {
  const long long m = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= inter) return;
  const float g = __bfloat162float(gu[m * ld + i]);
  const float u = __bfloat162float(gu[m * ld + inter + i]);
  const float a = act == 0 ? silu_f(g) : (act == 1 ? gelu_tanh_f(g) : 0.5f * g * (1.f + erff(g * 0.70710678f)));
  out[m * inter + i] = __float2bfloat16_rn(a * u);
}

// ---------------------------------------------------------------------------------------------
// Standalone per-head norm + RoPE + paged KV write for any even head_dim <= 256.
// qkv: [M, (Hq + 2 Hkv) * D] (q heads, k heads, v heads). One warp per (token, head).
// ---------------------------------------------------------------------------------------------
// KV8: the cache holds fp8 e4m3 (value / kv_scale, saturating) instead of bf16; q stays bf16.
template <bool KV8>
__global__ void rope_kv_write_kernel(const __nv_bfloat16* qkv, long long ld, int M, int n_q, int n_kv, int D,
                                     int rot_dim, const int* positions, const int* slot_mapping,
                                     const float* cos_t, const float* sin_t, int max_pos, const float* q_norm_w,
                                     const float* k_norm_w, float qk_eps, __nv_bfloat16* q_out,
                                     void* kv_cache_v, int num_pages, float kv_inv_scale, int* err) {
  __nv_bfloat16* kv_cache = static_cast<__nv_bfloat16*>(kv_cache_v);
  uint8_t* kv_cache8 = static_cast<uint8_t*>(kv_cache_v);
  uint8_t* dst8 = nullptr;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = n_q + 2 * n_kv;
  if (warp_global >= M * heads) return;
  const int m = warp_global / heads, head = warp_global % heads;
  const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
  const __nv_bfloat16* src = qkv + static_cast<long long>(m) * ld + static_cast<long long>(head) * D;
  float x[8];  // D <= 256 -> up to 8 elements per lane, element index = lane + 32*i
  const int per = (D + 31) / 32;
  float ss = 0.f;
  for (int i = 0; i < per; ++i) {
    const int d = lane + 32 * i;
    x[i] = d < D ? __bfloat162float(src[d]) : 0.f;
    ss += x[i] * x[i];
  }
  const float* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
  if (nw) {
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / D + qk_eps);
    for (int i = 0; i < per; ++i) {
      const int d = lane + 32 * i;
      if (d < D) x[i] = bf16_round(x[i] * r * nw[d]);
    }
  }
  __nv_bfloat16* dst = nullptr;
  if (is_q) {
    dst = q_out + (static_cast<long long>(m) * n_q + head) * D;
  } else {
    const int slot = slot_mapping ? slot_mapping[m] : -1;
    if (slot >= 0) {
      const int page = slot / 16, off = slot % 16;
      if (page >= num_pages) {
        if (err && lane == 0) atomicCAS(err, 0, ERR_BAD_PAGE);
      } else {
        const int kvh = is_k ? head - n_q : head - n_q - n_kv;
        const long long eoff = (((static_cast<long long>(page) * 2 + (is_k ? 0 : 1)) * n_kv + kvh) * 16 + off) * D;
        if (KV8) dst8 = kv_cache8 + eoff; else dst = kv_cache + eoff;
      }
    }
  }
  if (!dst && !dst8) return;
  auto put = [&](int d, float v) {
    if (KV8 && dst8)
      dst8[d] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v * kv_inv_scale, __NV_SATFINITE, __NV_E4M3));
    else
      dst[d] = __float2bfloat16_rn(v);
  };
  if ((is_q || is_k) && rot_dim > 0) {
    int pos = positions[m];
    if (pos < 0 || pos >= max_pos) pos = 0;
    const int half = rot_dim / 2;
    // Partner of element d is d +- half. Every lane takes part in every shuffle (no divergence
    // around the warp-synchronous exchange); lanes without a partner read lane 0 and ignore it.
    float y[8];
    for (int i = 0; i < per; ++i) {
      const int d = lane + 32 * i;
      const bool rot = d < rot_dim;
      const int pd = rot ? (d < half ? d + half : d - half) : 0;
      float partner = 0.f;
      for (int s = 0; s < per; ++s) {
        const float cand = __shfl_sync(0xffffffffu, x[s], pd & 31);
        if (s == (pd >> 5)) partner = cand;
      }
      float v = x[i];
      if (rot) {
        const int fi = d < half ? d : d - half;
        const float c = cos_t[static_cast<long long>(pos) * half + fi];
        const float sn = sin_t[static_cast<long long>(pos) * half + fi];
        v = d < half ? v * c - partner * sn : v * c + partner * sn;
      }
      y[i] = v;
    }
    for (int i = 0; i < per; ++i) {
      const int d = lane + 32 * i;
      if (d < D) put(d, y[i]);
    }
  } else {
    for (int i = 0; i < per; ++i) {
      const int d = lane + 32 * i;
      if (d < D) put(d, x[i]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Generic paged attention (CUDA cores) for head dims other than 128: one warp per (query token, head).
// Used by small / encoder models; the tensor-core kernels cover head_dim 128.
// ---------------------------------------------------------------------------------------------
template <bool KV8>
__global__ void paged_attention_generic_kernel(const __nv_bfloat16* q, __nv_bfloat16* out,
                                               const void* kv_cache_v, const int* block_tables,
                                               int max_blocks, const int* q_start, const int* q_len,
                                               const int* ctx_lens, int n_q, int n_kv, int D, float scale,
                                               int causal, int window, int num_pages, float kv_scale) {
  const __nv_bfloat16* kv_cache = static_cast<const __nv_bfloat16*>(kv_cache_v);
  const uint8_t* kv_cache8 = static_cast<const uint8_t*>(kv_cache_v);
  auto ld_kv = [&](long long eoff) -> float {
    if (KV8) {
      const __half_raw h = __nv_cvt_fp8_to_halfraw(kv_cache8[eoff], __NV_E4M3);
      return __half2float(*reinterpret_cast<const __half*>(&h)) * kv_scale;
    }
    return __bfloat162float(kv_cache[eoff]);
  };
  const int seq = blockIdx.z, head = blockIdx.y;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int qlen = q_len[seq];
  if (row >= qlen) return;
  const int ctx = ctx_lens[seq];
  const int tok = q_start[seq] + row;
  const int kvh = head / (n_q / n_kv);
  const int hi = causal ? (ctx - qlen + row + 1) : ctx;
  const int lo = window > 0 ? max(0, hi - window) : 0;
  const int per = (D + 31) / 32;
  float qv[8], acc[8];
  for (int i = 0; i < per; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < D ? __bfloat162float(q[(static_cast<long long>(tok) * n_q + head) * D + d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;
  const int* bt = block_tables + static_cast<long long>(seq) * max_blocks;
  for (int t = lo; t < hi; ++t) {
    int page = bt[t / 16];
    if (page < 0 || page >= num_pages) page = 0;
    const long long kp = (((static_cast<long long>(page) * 2) * n_kv + kvh) * 16 + (t % 16)) * D;
    const long long vp = (((static_cast<long long>(page) * 2 + 1) * n_kv + kvh) * 16 + (t % 16)) * D;
    float s = 0.f;
    for (int i = 0; i < per; ++i) {
      const int d = lane + 32 * i;
      if (d < D) s += qv[i] * ld_kv(kp + d);
    }
    s = warp_sum(s);
    const float mn = fmaxf(mx, s);
    const float c = __expf(mx - mn), pnew = __expf(s - mn);
    l = l * c + pnew;
    for (int i = 0; i < per; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc[i] = acc[i] * c + pnew * ld_kv(vp + d);
    }
    mx = mn;
  }
  for (int i = 0; i < per; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out[(static_cast<long long>(tok) * n_q + head) * D + d] = __float2bfloat16_rn(l > 0.f ? acc[i] / l : 0.f);
  }
}

// ---------------------------------------------------------------------------------------------
// pooling: mean over each sequence's tokens, or pick one token (CLS / last)
// ---------------------------------------------------------------------------------------------
__global__ void pool_kernel(const __nv_bfloat16* h, const int* seq_start, const int* seq_len, int hidden, int mode,
                            float* out) {
  const int s = blockIdx.x;
  const int st = seq_start[s], n = seq_len[s];
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float v;
    if (mode == 0) {
      v = 0.f;
      for (int t = 0; t < n; ++t) v += __bfloat162float(h[static_cast<long long>(st + t) * hidden + d]);
      v /= (n > 0 ? n : 1);
    } else if (mode == 1) {
      v = __bfloat162float(h[static_cast<long long>(st) * hidden + d]);
    } else {
      v = __bfloat162float(h[static_cast<long long>(st + n - 1) * hidden + d]);
    }
    out[static_cast<long long>(s) * hidden + d] = v;
  }
}

// ---------------------------------------------------------------------------------------------
// sampling
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Philox4x32-10 -> one uniform in [0,1)
__device__ __forceinline__ float philox_uniform(unsigned long long seed, unsigned long long subseq,
                                                unsigned long long offset) {
  uint32_t c0 = static_cast<uint32_t>(offset), c1 = static_cast<uint32_t>(offset >> 32);
  uint32_t c2 = static_cast<uint32_t>(subseq), c3 = static_cast<uint32_t>(subseq >> 32);
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (c0 >> 8) * (1.0f / 16777216.0f);
}

constexpr int kSampleThreads = 1024;

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, int i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, int i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, int i) {
  return __bfloat162float(p[i]);
}

// Row argmax; NaN never wins; the lowest index wins ties. Also returns the max value.
template <typename T>
__device__ void block_argmax(const T* row, int vocab, float& best_v, int& best_i, float* sv, int* si) {
  float bv = -INFINITY;
  int bi = vocab;  // sentinel: nothing seen
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = load_logit(row, i);
    if (v == v && (v > bv || bi == vocab)) {
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi < vocab && (bi == vocab || ov > bv || (ov == bv && oi < bi))) {
      bv = ov;
      bi = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    bv = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : vocab;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi < vocab && (bi == vocab || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (threadIdx.x == 0) {
      sv[0] = bv;
      si[0] = bi == vocab ? 0 : bi;
    }
  }
  __syncthreads();
  best_v = sv[0];
  best_i = si[0];
  __syncthreads();
}

// One CTA per row. params[b] = {temperature, top_k, top_p, unused}. Sort-free equivalent of
// "sort desc -> keep k -> 1/T -> softmax -> smallest prefix with mass >= p -> renormalise -> multinomial":
// radix-select the k-th largest key, then radix-select the key where the descending cumulative
// probability mass reaches p, then draw by prefix sums over the surviving set.
template <typename T>
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const T* logits, long long ld, int vocab,
                                                                const float* params, unsigned long long seed,
                                                                const long long* step_offsets, int* out_tokens,
                                                                float* out_logprob) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float hist_f[256];
  __shared__ int hist_i[256];
  __shared__ uint32_t sh_prefix;
  __shared__ float sh_f[2];
  __shared__ int sh_i[2];
  __shared__ float scan[kSampleThreads / 32];

  const int b = blockIdx.x;
  const T* row = logits + static_cast<long long>(b) * ld;
  const float temp = params[b * 4 + 0];
  int top_k = static_cast<int>(params[b * 4 + 1]);
  const float top_p = params[b * 4 + 2];

  float mx;
  int amax;
  block_argmax(row, vocab, mx, amax, sv, si);
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) {
      out_tokens[b] = amax;
      if (out_logprob) out_logprob[b] = 0.f;
    }
    return;
  }
  const float inv_t = 1.0f / temp;

  // ---- top-k threshold key (k-th largest) ----
  uint32_t key_k = 0;
  if (top_k > 0 && top_k < vocab) {
    uint32_t prefix = 0;
    int remaining = top_k;
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = threadIdx.x; i < 256; i += blockDim.x) hist_i[i] = 0;
      __syncthreads();
      const uint32_t hmask = pass == 3 ? 0u : (0xFFFFFFFFu << ((pass + 1) * 8));
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = load_logit(row, i);
        if (v != v) continue;
        const uint32_t k = float_key(v);
        if ((k & hmask) == (prefix & hmask)) atomicAdd(&hist_i[(k >> (pass * 8)) & 255], 1);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int cum = 0, bin = 0;
        for (int j = 255; j >= 0; --j) {
          if (cum + hist_i[j] >= remaining) {
            bin = j;
            break;
          }
          cum += hist_i[j];
        }
        sh_prefix = prefix | (static_cast<uint32_t>(bin) << (pass * 8));
        sh_i[0] = remaining - cum;
      }
      __syncthreads();
      prefix = sh_prefix;
      remaining = sh_i[0];
      __syncthreads();
    }
    key_k = prefix;
  }

  // ---- total mass of the top-k set ----
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = load_logit(row, i);
    if (v == v && float_key(v) >= key_k) z += __expf((v - mx) * inv_t);
  }
  z = block_sum<kSampleThreads>(z, sv);

  // ---- top-p threshold key ----
  uint32_t key_p = key_k;
  if (top_p > 0.f && top_p < 1.f) {
    uint32_t prefix = 0;
    float remaining = top_p * z;
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = threadIdx.x; i < 256; i += blockDim.x) hist_f[i] = 0.f;
      __syncthreads();
      const uint32_t hmask = pass == 3 ? 0u : (0xFFFFFFFFu << ((pass + 1) * 8));
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = load_logit(row, i);
        if (v != v) continue;
        const uint32_t k = float_key(v);
        if (k >= key_k && (k & hmask) == (prefix & hmask))
          atomicAdd(&hist_f[(k >> (pass * 8)) & 255], __expf((v - mx) * inv_t));
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        float cum = 0.f;
        int bin = 0;
        for (int j = 255; j >= 0; --j) {
          if (cum + hist_f[j] >= remaining || j == 0) {
            bin = j;
            break;
          }
          cum += hist_f[j];
        }
        sh_prefix = prefix | (static_cast<uint32_t>(bin) << (pass * 8));
        sh_f[0] = remaining - cum;
      }
      __syncthreads();
      prefix = sh_prefix;
      remaining = sh_f[0];
      __syncthreads();
    }
    key_p = prefix > key_k ? prefix : key_k;
  }

  // ---- multinomial over the surviving set (contiguous chunk per thread, block prefix sum) ----
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int i0 = threadIdx.x * chunk, i1 = min(i0 + chunk, vocab);
  float local = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float v = load_logit(row, i);
    if (v == v && float_key(v) >= key_p) local += __expf((v - mx) * inv_t);
  }
  // inclusive scan over threads
  float incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if ((threadIdx.x & 31) >= o) incl += n;
  }
  if ((threadIdx.x & 31) == 31) scan[threadIdx.x >> 5] = incl;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < (blockDim.x >> 5) ? scan[threadIdx.x] : 0.f;
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, wi, o);
      if (threadIdx.x >= o) wi += n;
    }
    scan[threadIdx.x] = wi - w;  // exclusive warp offsets
    if (threadIdx.x == 31) sh_f[1] = wi;
  }
  __syncthreads();
  incl += scan[threadIdx.x >> 5];
  const float total = sh_f[1];
  const float u = philox_uniform(seed, static_cast<unsigned long long>(b), step_offsets ? step_offsets[b] : 0);
  const float target = u * total;
  if (threadIdx.x == 0) sh_i[1] = -1;
  __syncthreads();
  const float excl = incl - local;
  if (local > 0.f && target >= excl && target < incl) {
    float cum = excl;
    int pick = -1;
    for (int i = i0; i < i1; ++i) {
      const float v = load_logit(row, i);
      if (v == v && float_key(v) >= key_p) {
        cum += __expf((v - mx) * inv_t);
        pick = i;
        if (cum > target) break;
      }
    }
    atomicMax(&sh_i[1], pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tok = sh_i[1];
    if (tok < 0) tok = amax;  // numerical corner: fall back to the mode
    out_tokens[b] = tok;
    if (out_logprob) out_logprob[b] = (load_logit(row, tok) - mx) * inv_t - __logf(total);
  }
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads) argmax_kernel(const T* logits, long long ld, int vocab,
                                                                int* out_tokens, float* out_vals) {
  __shared__ float sv[32];
  __shared__ int si[32];
  float mx;
  int amax;
  block_argmax(logits + static_cast<long long>(blockIdx.x) * ld, vocab, mx, amax, sv, si);
  if (threadIdx.x == 0) {
    out_tokens[blockIdx.x] = amax;
    if (out_vals) out_vals[blockIdx.x] = mx;
  }
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();

#define CHECK_LAUNCH(name)                                                   \
  do {                                                                       \
    cudaError_t e__ = cudaGetLastError();                                    \
    if (e__ != cudaSuccess) {                                                \
      set_last_error(name " launch failed: %s", cudaGetErrorString(e__));    \
      return -1;                                                             \
    }                                                                        \
    return 0;                                                                \
  } while (0)

GLLM_API int gllm_embed_gather(const int* ids, const void* table, int vocab, int hidden, float scale, void* out,
                               float* ss_out, int M, void* stream) {
  if (hidden % 8 != 0) { set_last_error("embed_gather: hidden %d must be a multiple of 8", hidden); return -1; }
  embed_gather_kernel<<<M, 128, 0, (cudaStream_t)stream>>>(ids, static_cast<const __nv_bfloat16*>(table), vocab,
                                                           hidden, scale, static_cast<__nv_bfloat16*>(out), ss_out,
                                                           gllm_error_word());
  CHECK_LAUNCH("embed_gather");
}

GLLM_API int gllm_rmsnorm(const void* x, const void* residual, const float* w, int M, int hidden, float eps,
                          int one_plus_w, void* h_out, void* y, float* ss_out, void* stream) {
  rmsnorm_kernel<<<M, 256, hidden * sizeof(float), (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), w, hidden, eps, one_plus_w,
      static_cast<__nv_bfloat16*>(h_out), static_cast<__nv_bfloat16*>(y), ss_out);
  CHECK_LAUNCH("rmsnorm");
}

GLLM_API int gllm_layernorm(const void* x, const void* residual, const float* w, const float* b, int M, int hidden,
                            float eps, void* y, void* stream) {
  layernorm_kernel<<<M, 256, hidden * sizeof(float), (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), w, b, hidden, eps,
      static_cast<__nv_bfloat16*>(y));
  CHECK_LAUNCH("layernorm");
}

GLLM_API int gllm_glu(const void* gu, long long ld, int M, int inter, int act, void* out, void* stream) {
  dim3 grid((inter + 255) / 256, M);
  glu_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(static_cast<const __nv_bfloat16*>(gu), ld, inter, act,
                                                     static_cast<__nv_bfloat16*>(out));
  CHECK_LAUNCH("glu");
}

GLLM_API int gllm_rope_kv_write(const void* qkv, long long ld, int M, int n_q, int n_kv, int D, int rot_dim,
                                const int* positions, const int* slot_mapping, const float* cos_t,
                                const float* sin_t, int max_pos, const float* q_norm_w, const float* k_norm_w,
                                float qk_eps, void* q_out, void* kv_cache, int num_pages, void* stream) {
  if (D > 256 || (D & 1) || rot_dim > D || (rot_dim & 1)) {
    set_last_error("rope_kv_write: head_dim %d / rot_dim %d unsupported", D, rot_dim);
    return -1;
  }
  const long long warps = static_cast<long long>(M) * (n_q + 2 * n_kv);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  rope_kv_write_kernel<false><<<static_cast<unsigned>(blocks), threads, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, M, n_q, n_kv, D, rot_dim, positions, slot_mapping, cos_t, sin_t,
      max_pos, q_norm_w, k_norm_w, qk_eps, static_cast<__nv_bfloat16*>(q_out), kv_cache, num_pages, 1.0f,
      gllm_error_word());
  CHECK_LAUNCH("rope_kv_write");
}

// Same with an fp8 e4m3 KV cache: stored value = x / kv_scale.
GLLM_API int gllm_rope_kv_write_fp8(const void* qkv, long long ld, int M, int n_q, int n_kv, int D, int rot_dim,
                                    const int* positions, const int* slot_mapping, const float* cos_t,
                                    const float* sin_t, int max_pos, const float* q_norm_w, const float* k_norm_w,
                                    float qk_eps, void* q_out, void* kv_cache, int num_pages, float kv_scale,
                                    void* stream) {
  if (D > 256 || kv_scale <= 0.f) { set_last_error("rope_kv_write_fp8: head_dim %d > 256 or bad scale", D); return -1; }
  if (M <= 0) return 0;
  const long long warps = static_cast<long long>(M) * (n_q + 2 * n_kv);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  rope_kv_write_kernel<true><<<static_cast<unsigned>(blocks), threads, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(qkv), ld, M, n_q, n_kv, D, rot_dim, positions, slot_mapping, cos_t, sin_t,
      max_pos, q_norm_w, k_norm_w, qk_eps, static_cast<__nv_bfloat16*>(q_out), kv_cache, num_pages, 1.0f / kv_scale,
      gllm_error_word());
  CHECK_LAUNCH("rope_kv_write_fp8");
}

GLLM_API int gllm_paged_attention_generic(const void* q, void* out, const void* kv_cache, int num_pages,
                                          const int* block_tables, int max_blocks, const int* q_start,
                                          const int* q_len, const int* ctx_lens, int num_seqs, int max_q_len,
                                          int n_q, int n_kv, int D, float scale, int causal, int window,
                                          void* stream) {
  if (D > 256) { set_last_error("paged_attention_generic: head_dim %d > 256", D); return -1; }
  dim3 grid((max_q_len + 3) / 4, n_q, num_seqs);
  paged_attention_generic_kernel<false><<<grid, 128, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), kv_cache, block_tables, max_blocks,
      q_start, q_len, ctx_lens, n_q, n_kv, D, scale, causal, window, num_pages, 1.0f);
  CHECK_LAUNCH("paged_attention_generic");
}

// fp8 e4m3 KV cache (value = stored * kv_scale); any head_dim <= 256. Halves the cache footprint and the bytes
// the attention streams; CUDA-core kernel.
GLLM_API int gllm_paged_attention_fp8kv(const void* q, void* out, const void* kv_cache, int num_pages,
                                        const int* block_tables, int max_blocks, const int* q_start,
                                        const int* q_len, const int* ctx_lens, int num_seqs, int max_q_len,
                                        int n_q, int n_kv, int D, float scale, int causal, int window,
                                        float kv_scale, void* stream) {
  if (D > 256) { set_last_error("paged_attention_fp8kv: head_dim %d > 256", D); return -1; }
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  dim3 grid((max_q_len + 3) / 4, n_q, num_seqs);
  paged_attention_generic_kernel<true><<<grid, 128, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), kv_cache, block_tables, max_blocks,
      q_start, q_len, ctx_lens, n_q, n_kv, D, scale, causal, window, num_pages, kv_scale);
  CHECK_LAUNCH("paged_attention_fp8kv");
}

GLLM_API int gllm_pool(const void* h, const int* seq_start, const int* seq_len, int num_seqs, int hidden, int mode,
                       float* out, void* stream) {
  pool_kernel<<<num_seqs, 256, 0, (cudaStream_t)stream>>>(static_cast<const __nv_bfloat16*>(h), seq_start, seq_len,
                                                          hidden, mode, out);
  CHECK_LAUNCH("pool");
}

// logits: fp32 (is_bf16 = 0) or bf16 rows of pitch ld; params [B,4] = {temperature, top_k, top_p, 0}.
GLLM_API int gllm_sample(const void* logits, long long ld, int is_bf16, int batch, int vocab, const float* params,
                         unsigned long long seed, const long long* step_offsets, int* out_tokens,
                         float* out_logprob, void* stream) {
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<batch, kSampleThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, vocab, params, seed, step_offsets, out_tokens, out_logprob);
  else
    sample_kernel<float><<<batch, kSampleThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const float*>(logits), ld, vocab, params, seed, step_offsets, out_tokens, out_logprob);
  CHECK_LAUNCH("sample");
}

GLLM_API int gllm_argmax(const void* logits, long long ld, int is_bf16, int batch, int vocab, int* out_tokens,
                         float* out_vals, void* stream) {
  if (is_bf16)
    argmax_kernel<__nv_bfloat16><<<batch, kSampleThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, vocab, out_tokens, out_vals);
  else
    argmax_kernel<float><<<batch, kSampleThreads, 0, (cudaStream_t)stream>>>(static_cast<const float*>(logits), ld,
                                                                              vocab, out_tokens, out_vals);
  CHECK_LAUNCH("argmax");
}
