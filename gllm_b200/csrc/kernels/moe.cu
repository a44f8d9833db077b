// Mixture-of-experts routing on the device: router scores -> top-k, token permutation into per-expert
// row blocks for the grouped tcgen05 GEMM, and the weighted combine on the way back.
//
// Reference semantics (src/compat/scalar_ops.rs:70-181, src/moe/routing.rs:100-307): router GEMM ->
// softmax over ALL experts -> top-k -> renormalise the k weights to sum 1 -> sum_k w_k * expert_k(x)
// (+ shared expert). DeepSeek-style scoring (sigmoid, selection bias, routed scaling) is the `scoring`
// / `sel_bias` / `scale` options. The reference loops over all experts with masks
// (build_graph.inc.rs:2076-2123); here only routed rows are computed: rows are bucketed per expert,
// each bucket padded to a multiple of 128 rows so one GEMM row block belongs to exactly one expert.
//
// Everything is sized for the worst case and driven by device-side counts, so the whole MoE layer can
// sit inside a CUDA graph: no host round trip for the routing decision.
#include "common.cuh"

namespace gllm {

constexpr int kMoeBlockRows = 128;

// One warp per token. E <= 512.
__global__ void moe_route_kernel(const float* logits, long long ld, int T, int E, int k, int norm_topk, int scoring,
                                 const float* sel_bias, float scale, int* out_ids, float* out_w, int* err) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* row = logits + static_cast<long long>(t) * ld;
  constexpr int kPer = 16;  // 512 / 32
  float score[kPer], sel[kPer];
  const int per = (E + 31) / 32;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = lane + 32 * i;
    const float v = e < E ? row[e] : -INFINITY;
    score[i] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (scoring == 0) {  // softmax over all experts
    float z = 0.f;
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < E ? __expf(score[i] - mx) : 0.f;
      z += score[i];
    }
    z = warp_sum(z);
    for (int i = 0; i < per; ++i) score[i] /= z;
  } else {  // sigmoid
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < E ? 1.f / (1.f + __expf(-score[i])) : 0.f;
    }
  }
  for (int i = 0; i < per; ++i) {
    const int e = lane + 32 * i;
    sel[i] = e < E ? score[i] + (sel_bias ? sel_bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;   // lane j keeps the j-th pick
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = 0; i < per; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (sel[i] > bv || (sel[i] == bv && e < bi))) {
        bv = sel[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    // weight = the (unbiased) score of the winner
    const int owner = bi & 31, slot = bi >> 5;
    float w = 0.f;
    for (int i = 0; i < per; ++i)
      if (i == slot) w = score[i];
    w = __shfl_sync(0xffffffffu, w, owner);
    if (lane == owner) {
      for (int i = 0; i < per; ++i)
        if (i == slot) sel[i] = -INFINITY;
    }
    wsum += w;
    if (lane == j) {
      my_w = w;
      my_id = bi;
    }
  }
  if (lane < k) {
    if (my_id < 0 || my_id >= E) {
      if (err) atomicCAS(err, 0, ERR_BAD_EXPERT);
      my_id = 0;
    }
    float w = my_w;
    if (norm_topk) w = w / fmaxf(wsum, 1e-20f);
    out_ids[t * k + lane] = my_id;
    out_w[t * k + lane] = w * scale;
  }
}

// counts[e] = number of (token, slot) pairs routed to local expert e (ids outside [e0, e0+E_local) ignored)
__global__ void moe_count_kernel(const int* ids, int n, int e0, int e_local, int* counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i] - e0;
  if (e >= 0 && e < e_local) atomicAdd(&counts[e], 1);
}

// Single block: padded bucket offsets, block -> expert map, cursors reset. blk_group holds 2 * max_blocks ints: the
// expert of every 128-row block (-1: inactive), then the number of routed rows in every block (the rest is padding),
// which lets the grouped GEMMs load and store only the rows that exist.
__global__ void moe_plan_kernel(const int* counts, int e_local, int* offsets, int* cursors, int* blk_group,
                                int max_blocks, int* total_rows) {
  __shared__ int s_off[513];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < e_local; ++e) {
      s_off[e] = acc;
      acc += (counts[e] + kMoeBlockRows - 1) / kMoeBlockRows * kMoeBlockRows;
    }
    s_off[e_local] = acc;
    *total_rows = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= e_local; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < e_local) cursors[e] = 0;
  }
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
    const int row = b * kMoeBlockRows;
    int g = -1;
    if (row < s_off[e_local]) {
      int lo = 0, hi = e_local;  // last e with s_off[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    blk_group[b] = g;
    blk_group[max_blocks + b] = g < 0 ? 0 : min(kMoeBlockRows, counts[g] - (row - s_off[g]));
  }
}

// One warp per (token, slot): claim a row in the expert's bucket and copy the hidden row there.
__global__ void moe_scatter_kernel(const __nv_bfloat16* x, const float* row_ss, int ss_parts, const int* ids, int T,
                                   int k, int hidden, int e0, int e_local, const int* offsets, int* cursors,
                                   __nv_bfloat16* a_perm, float* ss_perm, int* dest_rows, int max_rows) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * k) return;
  const int t = w / k;
  const int e = ids[w] - e0;
  int dest = -1;
  if (e >= 0 && e < e_local) {
    if (lane == 0) dest = offsets[e] + atomicAdd(&cursors[e], 1);
    dest = __shfl_sync(0xffffffffu, dest, 0);
    if (dest >= max_rows) dest = -1;
  }
  if (lane == 0) dest_rows[w] = dest;
  if (dest < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(a_perm + static_cast<long long>(dest) * hidden);
  for (int i = lane; i < hidden / 8; i += 32) dst[i] = src[i];
  if (ss_perm && lane == 0) {
    float s = 0.f;
    for (int p = 0; p < ss_parts; ++p) s += row_ss[static_cast<long long>(t) * ss_parts + p];
    ss_perm[dest] = s;
  }
}

// x[t] += sum_k w[t,k] * y_perm[dest[t,k]] (+ shared[t]); writes bf16 x and the row sum of squares.
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* y_perm, const int* dest_rows,
                                                          const float* weights, int k, int hidden,
                                                          const __nv_bfloat16* shared, __nv_bfloat16* x,
                                                          float* ss_out) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int c = threadIdx.x * 2; c < hidden; c += blockDim.x * 2) {
    float2 acc = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<long long>(t) * hidden + c));
    if (shared) {
      const float2 s = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(shared + static_cast<long long>(t) * hidden + c));
      acc.x += s.x;
      acc.y += s.y;
    }
    for (int j = 0; j < k; ++j) {
      const int d = dest_rows[t * k + j];
      if (d < 0) continue;
      const float w = weights[t * k + j];
      const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(y_perm + static_cast<long long>(d) * hidden + c));
      acc.x += w * y.x;
      acc.y += w * y.y;
    }
    const __nv_bfloat162 o = __floats2bfloat162_rn(acc.x, acc.y);
    *reinterpret_cast<__nv_bfloat162*>(x + static_cast<long long>(t) * hidden + c) = o;
    const float2 r = __bfloat1622float2(o);
    ss += r.x * r.x + r.y * r.y;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0 && ss_out) ss_out[t] = v;
  }
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();

#define MOE_CHECK(name)                                                      \
  do {                                                                       \
    cudaError_t e__ = cudaGetLastError();                                    \
    if (e__ != cudaSuccess) {                                                \
      set_last_error(name " launch failed: %s", cudaGetErrorString(e__));    \
      return -1;                                                             \
    }                                                                        \
  } while (0)

GLLM_API int gllm_moe_route(const float* logits, long long ld, int T, int E, int k, int norm_topk, int scoring,
                            const float* sel_bias, float scale, int* out_ids, float* out_w, void* stream) {
  if (E > 512 || k > 32 || k > E) {
    set_last_error("moe_route: E=%d (max 512) / k=%d (max 32) unsupported", E, k);
    return -1;
  }
  const int threads = 256;
  const int blocks = (T * 32 + threads - 1) / threads;
  moe_route_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(logits, ld, T, E, k, norm_topk, scoring, sel_bias,
                                                                 scale, out_ids, out_w, gllm_error_word());
  MOE_CHECK("moe_route");
  return 0;
}

// Buckets the T*k routed (token, slot) pairs of local experts [e0, e0+e_local) into 128-row blocks.
// counts / offsets (e_local+1) / cursors / blk_group (2 * max_blocks: experts, then row counts) / total_rows (1) are int32 device
// buffers; counts must be zero on entry (the call re-zeroes nothing: the caller owns them).
GLLM_API int gllm_moe_permute(const void* x, const float* row_ss, int ss_parts, const int* ids, int T, int k,
                              int hidden, int e0, int e_local, int* counts, int* offsets, int* cursors,
                              int* blk_group, int max_blocks, int* total_rows, void* a_perm, float* ss_perm,
                              int* dest_rows, void* stream) {
  if (e_local > 512 || hidden % 8 != 0) {
    set_last_error("moe_permute: e_local=%d (max 512), hidden %d must be a multiple of 8", e_local, hidden);
    return -1;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int n = T * k;
  cudaMemsetAsync(counts, 0, sizeof(int) * e_local, s);
  if (n > 0) moe_count_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, n, e0, e_local, counts);
  MOE_CHECK("moe_count");
  moe_plan_kernel<<<1, 256, 0, s>>>(counts, e_local, offsets, cursors, blk_group, max_blocks, total_rows);
  MOE_CHECK("moe_plan");
  const int threads = 256;
  const long long blocks = (static_cast<long long>(n) * 32 + threads - 1) / threads;
  if (n > 0) moe_scatter_kernel<<<static_cast<unsigned>(blocks), threads, 0, s>>>(
      static_cast<const __nv_bfloat16*>(x), row_ss, ss_parts, ids, T, k, hidden, e0, e_local, offsets, cursors,
      static_cast<__nv_bfloat16*>(a_perm), ss_perm, dest_rows, max_blocks * kMoeBlockRows);
  MOE_CHECK("moe_scatter");
  return 0;
}

GLLM_API int gllm_moe_combine(const void* y_perm, const int* dest_rows, const float* weights, int T, int k,
                              int hidden, const void* shared, void* x, float* ss_out, void* stream) {
  if (hidden % 2 != 0) {
    set_last_error("moe_combine: hidden %d must be even", hidden);
    return -1;
  }
  if (T <= 0) return 0;
  moe_combine_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(static_cast<const __nv_bfloat16*>(y_perm), dest_rows, weights,
                                                          k, hidden, static_cast<const __nv_bfloat16*>(shared),
                                                          static_cast<__nv_bfloat16*>(x), ss_out);
  MOE_CHECK("moe_combine");
  return 0;
}
