// Multi-head latent attention (DeepSeek-style) over a paged latent cache.
//
// The cache keeps one row per token: [c_kv (d_c) | k_pe (d_r)] (page layout [page][16 tokens][d_c + d_r]). With
// the K up-projection absorbed into the query and the V up-projection applied after attention, every query
// head attends over the SAME latent rows: key = the whole row, value = its first d_c entries.
//
//   gllm_mla_latent_write : RMSNorm(c_kv) * w, RoPE(k_pe) at the token's position, write into the page slot
//   gllm_mla_attention    : scores = q_abs . c_kv + q_pe . k_pe (q row = [q_abs | q_pe]), online softmax,
//                           out = probs . c_kv   -> [tokens, heads, d_c]
//
// Reference parity: MlaKvCompress / MlaQAbsorb / MlaAttention graph ops
// (src/arch/auto_graph_fragments/build_graph.inc.rs:1486-1578); MLA page stride
// L * page_size * (d_c + d_rope) (src/compat/cpu_backend.rs:254-271).
#include "common.cuh"

namespace gllm {

constexpr int kMlaPage = 16;
constexpr int kMlaTile = 32;      // kv tokens per step
constexpr int kMlaHeads = 8;      // heads per CTA (one warp each)
constexpr int kMlaMaxDk = 576;
constexpr int kMlaMaxDv = 512;

__global__ void __launch_bounds__(128) mla_latent_write_kernel(
    const __nv_bfloat16* kv_a, long long ld, int d_c, int d_r, const float* norm_w, float eps, const int* positions,
    const int* slot_mapping, const float* cos_t, const float* sin_t, int max_pos, __nv_bfloat16* cache, int num_pages,
    int* err) {
  __shared__ float red[4];
  const int t = blockIdx.x;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int page = slot / kMlaPage, off = slot % kMlaPage;
  if (page >= num_pages) {
    if (threadIdx.x == 0 && err) atomicCAS(err, 0, ERR_BAD_PAGE);
    return;
  }
  const __nv_bfloat16* src = kv_a + static_cast<long long>(t) * ld;
  __nv_bfloat16* dst = cache + (static_cast<long long>(page) * kMlaPage + off) * (d_c + d_r);
  float ss = 0.f;
  for (int i = threadIdx.x; i < d_c; i += blockDim.x) {
    const float v = __bfloat162float(src[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float tot = red[0] + red[1] + red[2] + red[3];
  const float inv = rsqrtf(tot / d_c + eps);
  for (int i = threadIdx.x; i < d_c; i += blockDim.x)
    dst[i] = __float2bfloat16(__bfloat162float(src[i]) * inv * norm_w[i]);
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) pos = 0;
  const int half = d_r / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float x0 = __bfloat162float(src[d_c + i]), x1 = __bfloat162float(src[d_c + half + i]);
    const float cs = cos_t[static_cast<long long>(pos) * half + i], sn = sin_t[static_cast<long long>(pos) * half + i];
    dst[d_c + i] = __float2bfloat16(x0 * cs - x1 * sn);
    dst[d_c + half + i] = __float2bfloat16(x1 * cs + x0 * sn);
  }
}

// grid (query token, head block). Sequence s owns query rows [q_start[s], q_start[s]+q_len[s]) which sit at the
// END of its context (ctx_lens[s] tokens); row_seq[t] gives the sequence of row t.
__global__ void __launch_bounds__(256) mla_attention_kernel(
    const __nv_bfloat16* q, __nv_bfloat16* out, const __nv_bfloat16* cache, int num_pages, const int* block_tables,
    int max_blocks, const int* row_seq, const int* q_start, const int* q_len, const int* ctx_lens, int n_heads, int d_k,
    int d_v, float scale, int causal, int* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = d_k + 8;  // bf16 elements; (stride * 2 / 16) is odd -> 16-byte row reads spread over banks
  __nv_bfloat16* s_kv = reinterpret_cast<__nv_bfloat16*>(smem_raw);                       // [32][stride]
  float* s_q = reinterpret_cast<float*>(smem_raw + kMlaTile * stride * 2);                 // [8][d_k]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * kMlaHeads + warp;
  const int s = row_seq[t];
  const int ctx = ctx_lens[s];
  const int row_in_seq = t - q_start[s];
  const int ql = q_len[s];
  int kv_len = causal ? (ctx - ql + row_in_seq + 1) : ctx;
  if (kv_len > ctx) kv_len = ctx;
  if (head < n_heads) {
    const __nv_bfloat16* qrow = q + (static_cast<long long>(t) * n_heads + head) * d_k;
    for (int i = lane; i < d_k; i += 32) s_q[warp * d_k + i] = __bfloat162float(qrow[i]) * scale;
  }
  float acc[kMlaMaxDv / 32];
#pragma unroll
  for (int i = 0; i < kMlaMaxDv / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int vec_per_row = d_k / 8;
  for (int k0 = 0; k0 < kv_len; k0 += kMlaTile) {
    __syncthreads();
    const int nt = min(kMlaTile, kv_len - k0);
    for (int idx = threadIdx.x; idx < nt * vec_per_row; idx += blockDim.x) {
      const int r = idx / vec_per_row, v = idx - r * vec_per_row;
      const int tok = k0 + r;
      int page = block_tables[static_cast<long long>(s) * max_blocks + tok / kMlaPage];
      if (page < 0 || page >= num_pages) {
        if (err) atomicCAS(err, 0, ERR_BAD_PAGE);
        page = 0;
      }
      const uint4* src = reinterpret_cast<const uint4*>(cache + (static_cast<long long>(page) * kMlaPage + tok % kMlaPage) * d_k);
      *reinterpret_cast<uint4*>(s_kv + r * stride + v * 8) = src[v];
    }
    __syncthreads();
    if (head >= n_heads) continue;
    // lane = token of the tile
    float sc = -INFINITY;
    if (lane < nt) {
      const float* qv = s_q + warp * d_k;
      const __nv_bfloat16* kr = s_kv + lane * stride;
      float d = 0.f;
      for (int i = 0; i < d_k; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kr + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          d += f.x * qv[i + 2 * e] + f.y * qv[i + 2 * e + 1];
        }
      }
      sc = d;
    }
    float tile_max = sc;
    for (int o = 16; o > 0; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
    const float m_new = fmaxf(m, tile_max);
    const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
    const float p = (lane < nt) ? __expf(sc - m_new) : 0.f;
    float psum = p;
    for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * corr + psum;
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMlaMaxDv / 32; ++i) acc[i] *= corr;
    for (int tok = 0; tok < nt; ++tok) {
      const float pt = __shfl_sync(0xffffffffu, p, tok);
      const __nv_bfloat16* vr = s_kv + tok * stride;
#pragma unroll
      for (int i = 0; i < kMlaMaxDv / 32; ++i)
        if (i * 32 < d_v) acc[i] += pt * __bfloat162float(vr[i * 32 + lane]);
    }
  }
  if (head < n_heads) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* orow = out + (static_cast<long long>(t) * n_heads + head) * d_v;
#pragma unroll
    for (int i = 0; i < kMlaMaxDv / 32; ++i)
      if (i * 32 < d_v) orow[i * 32 + lane] = __float2bfloat16(acc[i] * inv);
  }
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();

GLLM_API int gllm_mla_latent_write(const void* kv_a, long long ld, int T, int d_c, int d_r, const float* norm_w,
                                   float eps, const int* positions, const int* slot_mapping, const float* cos_t,
                                   const float* sin_t, int max_pos, void* cache, int num_pages, void* stream) {
  if (T <= 0) return 0;
  if (d_r % 2 != 0) {
    set_last_error("mla_latent_write: rope dim %d must be even", d_r);
    return -1;
  }
  mla_latent_write_kernel<<<T, 128, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(kv_a), ld, d_c, d_r, norm_w, eps, positions, slot_mapping, cos_t, sin_t, max_pos,
      static_cast<__nv_bfloat16*>(cache), num_pages, gllm_error_word());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("mla_latent_write launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

GLLM_API int gllm_mla_attention(const void* q, void* out, const void* cache, int num_pages, const int* block_tables,
                                int max_blocks, const int* row_seq, const int* q_start, const int* q_len,
                                const int* ctx_lens, int T, int n_heads, int d_k, int d_v, float scale, int causal,
                                void* stream) {
  if (T <= 0) return 0;
  if (d_k > kMlaMaxDk || d_v > kMlaMaxDv || d_k % 8 != 0 || d_v % 32 != 0 || d_v > d_k) {
    set_last_error("mla_attention: d_k=%d (<=576, %%8) d_v=%d (<=512, %%32, <= d_k) unsupported", d_k, d_v);
    return -1;
  }
  const int smem = kMlaTile * (d_k + 8) * 2 + kMlaHeads * d_k * 4;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaFuncSetAttribute(mla_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr_set[dev & 63] = true;
  }
  dim3 grid(T, (n_heads + kMlaHeads - 1) / kMlaHeads);
  mla_attention_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(cache),
      num_pages, block_tables, max_blocks, row_seq, q_start, q_len, ctx_lens, n_heads, d_k, d_v, scale, causal,
      gllm_error_word());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("mla_attention launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
