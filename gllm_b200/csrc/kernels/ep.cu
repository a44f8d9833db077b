// Expert-parallel dispatch / combine over NVLink peer memory (sm_100a).
//
// Every rank owns E / world consecutive experts and a symmetric buffer that its peers can address. One MoE
// layer runs as:
//   1. ep_count_publish : count this rank's (token, slot) pairs per expert, store the counts in every peer's
//                         count table, arrive on their "counts" flag.
//   2. ep_dispatch      : wait for all count rows; every rank derives the same row plan (expert blocks padded to
//                         128 rows, sources in rank order inside a block); copy each routed hidden row STRAIGHT
//                         into the owning rank's grouped-GEMM input buffer with peer stores, together with its
//                         row statistic and a return address (source rank, slot); arrive on the "data" flag.
//   3. ep_recv_plan     : wait for all data; build the block -> expert table for the grouped GEMMs.
//   4. grouped GEMMs    : the second one scatters its output rows into the token owners' memory as tiles retire
//                         (gllm_gemm_bf16_grouped_scatter).
//   5. ep_combine       : arrive on the "done" flag, wait for all peers, weighted top-k sum from LOCAL memory.
// Flags are monotonically increasing arrival counters (expected value = epoch * world), so nothing is reset
// and the sequence can be replayed from a CUDA graph. Every wait is bounded and reports ERR_TIMEOUT_PEER.
//
// Buffer reuse is safe without extra barriers: a rank only starts layer l+1's dispatch after its layer-l combine
// saw every peer's "done", and a rank only runs layer l+1's GEMMs after every peer's layer-l+1 dispatch arrived.
//
// Reference parity: src/moe/distributed_dispatch.rs:250-284 exchanges per-rank counts with an all-gather and
// stops there (the token exchange was never implemented); this file is the exchange.
#include "common.cuh"

namespace gllm {

constexpr int kEpBlockRows = 128;
constexpr int kEpMaxExperts = 512;

struct EpComm {
  int world, rank, num_experts, e_local, hidden, max_rows;
  int* counts[8];                 // [world][E] on each rank; row s is written by rank s
  unsigned long long* flags[8];   // [0] counts arrived, [1] data arrived, [2] outputs done
  __nv_bfloat16* x[8];            // [max_rows][hidden] grouped-GEMM input
  float* ss[8];                   // [max_rows] row sum of squares (fused RMSNorm) or unused
  int* meta[8];                   // [max_rows] (source rank << 24) | slot, or -1 for padding rows
  unsigned long long* state;      // local: [0] epoch
  unsigned int* cta_done;         // local: dispatch CTA completion counter
  int* err;
};

__device__ __forceinline__ unsigned long long ep_ld_acquire(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ep_signal(unsigned long long* p) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(1ull) : "memory");
}
// thread 0 waits (bounded) until *flag >= target; result broadcast to the CTA
__device__ __forceinline__ bool ep_wait(const unsigned long long* flag, unsigned long long target, int* err) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    int ok = 1;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    while (ep_ld_acquire(flag) < target) {
      if (((++spins) & 0x3F) == 0 && globaltimer_ns() - t0 > kPeerWaitLimitNs) {
        if (err) atomicCAS(err, 0, ERR_TIMEOUT_PEER);
        ok = 0;
        break;
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  return ok_flag != 0;
}

__global__ void __launch_bounds__(1024) ep_count_publish_kernel(EpComm c, const int* ids, int n, int* cursors) {
  __shared__ int s_cnt[kEpMaxExperts];
  const int E = c.num_experts;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&s_cnt[e], 1);
    else if (c.err) atomicCAS(c.err, 0, ERR_BAD_EXPERT);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < E * c.world; idx += blockDim.x) {
    const int r = idx / E, e = idx - r * E;
    c.counts[r][c.rank * E + e] = s_cnt[e];
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) cursors[e] = 0;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.world) ep_signal(c.flags[threadIdx.x] + 0);
  if (threadIdx.x == 0) c.state[0] = c.state[0] + 1ull;
}

__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpComm c, const __nv_bfloat16* x, const float* row_ss,
                                                          int ss_parts, const int* ids, int n, int k, int* cursors) {
  __shared__ int s_tot[kEpMaxExperts];
  __shared__ int s_base[kEpMaxExperts];
  const int E = c.num_experts;
  const unsigned long long epoch = c.state[0];
  if (!ep_wait(c.flags[c.rank] + 0, epoch * c.world, c.err)) return;
  const int* my_counts = c.counts[c.rank];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, pre = 0;
    for (int s = 0; s < c.world; ++s) {
      const int v = __ldcg(my_counts + s * E + e);
      tot += v;
      if (s < c.rank) pre += v;
    }
    s_tot[e] = tot;
    s_base[e] = pre;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int first = (e / c.e_local) * c.e_local;
    int off = 0;
    for (int e2 = first; e2 < e; ++e2) off += (s_tot[e2] + kEpBlockRows - 1) / kEpBlockRows * kEpBlockRows;
    s_base[e] += off;  // s_base held the prefix over lower source ranks; only this thread touches entry e
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < n; w += warps) {
    const int t = w / k;
    const int e = ids[w];
    if (e < 0 || e >= E) continue;
    const int owner = e / c.e_local;
    int row = 0;
    if (lane == 0) row = s_base[e] + atomicAdd(&cursors[e], 1);
    row = __shfl_sync(0xffffffffu, row, 0);
    if (row >= c.max_rows) {
      if (lane == 0 && c.err) atomicCAS(c.err, 0, ERR_BAD_ARG);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * c.hidden);
    uint4* dst = reinterpret_cast<uint4*>(c.x[owner] + static_cast<long long>(row) * c.hidden);
    for (int i = lane; i < c.hidden / 8; i += 32) dst[i] = src[i];
    if (lane == 0) {
      c.meta[owner][row] = (c.rank << 24) | w;
      if (row_ss) {
        float s = 0.f;
        for (int p = 0; p < ss_parts; ++p) s += row_ss[static_cast<long long>(t) * ss_parts + p];
        c.ss[owner][row] = s;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(c.cta_done, 1u) == gridDim.x - 1) {
      *c.cta_done = 0u;
      __threadfence_system();
      for (int r = 0; r < c.world; ++r) ep_signal(c.flags[r] + 1);
    }
  }
}

__global__ void __launch_bounds__(256) ep_recv_plan_kernel(EpComm c, int* blk_group, int max_blocks, int* total_rows) {
  __shared__ int s_tot[kEpMaxExperts];
  __shared__ int s_off[kEpMaxExperts + 1];
  const int E = c.num_experts, EL = c.e_local;
  const unsigned long long epoch = c.state[0];
  const bool ok = ep_wait(c.flags[c.rank] + 1, epoch * c.world, c.err);
  if (!ok) {  // nothing trustworthy arrived: make the GEMMs skip every block
    for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
      blk_group[b] = -1;
      blk_group[max_blocks + b] = 0;
    }
    if (threadIdx.x == 0) *total_rows = 0;
    return;
  }
  const int* my_counts = c.counts[c.rank];
  for (int el = threadIdx.x; el < EL; el += blockDim.x) {
    int tot = 0;
    for (int s = 0; s < c.world; ++s) tot += __ldcg(my_counts + s * E + c.rank * EL + el);
    s_tot[el] = tot;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int el = 0; el < EL; ++el) {
      s_off[el] = acc;
      acc += (s_tot[el] + kEpBlockRows - 1) / kEpBlockRows * kEpBlockRows;
    }
    if (acc > c.max_rows) {
      if (c.err) atomicCAS(c.err, 0, ERR_BAD_ARG);
      acc = 0;
    }
    s_off[EL] = acc;
    *total_rows = acc;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x) {
    const int row = b * kEpBlockRows;
    int g = -1;
    if (row < s_off[EL]) {
      int lo = 0, hi = EL;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid;
      }
      g = lo;
    }
    blk_group[b] = g;
    // second half of the table: received rows in this block (the rest is padding), for the grouped GEMMs
    blk_group[max_blocks + b] = g < 0 ? 0 : min(kEpBlockRows, s_tot[g] - (row - s_off[g]));
  }
  // padding rows of every block: no return address, benign statistic
  int* meta = c.meta[c.rank];
  float* ss = c.ss[c.rank];
  if (s_off[EL] > 0) {
    for (int el = threadIdx.x >> 5; el < EL; el += blockDim.x >> 5)
      for (int r = s_off[el] + s_tot[el] + (threadIdx.x & 31); r < s_off[el + 1]; r += 32) {
        meta[r] = -1;
        ss[r] = 1.0f;
      }
  }
}

// x[t] += sum_j w[t,j] * y[t*k+j] (+ shared[t]); y is this rank's own buffer, filled by the peers' GEMMs.
__global__ void __launch_bounds__(256) ep_combine_kernel(EpComm c, const __nv_bfloat16* y, const float* weights, int T,
                                                         int k, const __nv_bfloat16* shared, __nv_bfloat16* x,
                                                         float* ss_out) {
  __shared__ float red[32];
  const int hidden = c.hidden;
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    __threadfence_system();
    ep_signal(c.flags[threadIdx.x] + 2);
  }
  const unsigned long long epoch = c.state[0];
  if (!ep_wait(c.flags[c.rank] + 2, epoch * c.world, c.err)) return;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    float ss = 0.f;
    for (int col = threadIdx.x * 2; col < hidden; col += blockDim.x * 2) {
      float2 acc = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + static_cast<long long>(t) * hidden + col));
      if (shared) {
        const float2 s = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(shared + static_cast<long long>(t) * hidden + col));
        acc.x += s.x;
        acc.y += s.y;
      }
      for (int j = 0; j < k; ++j) {
        const float w = weights[t * k + j];
        const unsigned int raw = __ldcg(reinterpret_cast<const unsigned int*>(y + (static_cast<long long>(t) * k + j) * hidden + col));
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
        acc.x += w * v.x;
        acc.y += w * v.y;
      }
      const __nv_bfloat162 o = __floats2bfloat162_rn(acc.x, acc.y);
      *reinterpret_cast<__nv_bfloat162*>(x + static_cast<long long>(t) * hidden + col) = o;
      const float2 r = __bfloat1622float2(o);
      ss += r.x * r.x + r.y * r.y;
    }
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (threadIdx.x == 0 && ss_out) ss_out[t] = v;
    }
  }
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();
extern "C" int gllm_sm_count();

// Host mirror of the pointer tables (filled from Python with ctypes).
struct GllmEpDesc {
  int world, rank, num_experts, e_local, hidden, max_rows;
  void* counts[8];
  void* flags[8];
  void* x[8];
  void* ss[8];
  void* meta[8];
  void* state;
  void* cta_done;
};

static int ep_make(const GllmEpDesc* d, EpComm& c) {
  if (!d || d->world < 1 || d->world > 8 || d->rank < 0 || d->rank >= d->world || d->num_experts > kEpMaxExperts ||
      d->num_experts != d->e_local * d->world || d->hidden % 8 != 0) {
    set_last_error("ep: bad descriptor (world 1..8, experts <= 512 and divisible by world, hidden %% 8 == 0)");
    return -1;
  }
  c.world = d->world; c.rank = d->rank; c.num_experts = d->num_experts; c.e_local = d->e_local;
  c.hidden = d->hidden; c.max_rows = d->max_rows;
  for (int r = 0; r < d->world; ++r) {
    c.counts[r] = static_cast<int*>(d->counts[r]);
    c.flags[r] = static_cast<unsigned long long*>(d->flags[r]);
    c.x[r] = static_cast<__nv_bfloat16*>(d->x[r]);
    c.ss[r] = static_cast<float*>(d->ss[r]);
    c.meta[r] = static_cast<int*>(d->meta[r]);
  }
  c.state = static_cast<unsigned long long*>(d->state);
  c.cta_done = static_cast<unsigned int*>(d->cta_done);
  c.err = gllm_error_word();
  return 0;
}

#define EP_CHECK(name)                                                       \
  do {                                                                       \
    cudaError_t e__ = cudaGetLastError();                                    \
    if (e__ != cudaSuccess) {                                                \
      set_last_error(name " launch failed: %s", cudaGetErrorString(e__));    \
      return -1;                                                             \
    }                                                                        \
  } while (0)

// Steps 1-3 for T tokens with k routed experts each. x [T, hidden] bf16, row_ss [T, ss_parts] or null,
// ids [T, k]. cursors: local int[num_experts] scratch. After it returns (stream order) this rank's x / ss / meta
// buffers hold the rows routed to its experts and blk_group (2 * max_blocks ints: the expert of every 128-row block, then
// the received rows in every block) / total_rows describe them.
GLLM_API int gllm_ep_dispatch(const GllmEpDesc* desc, const void* x, const float* row_ss, int ss_parts, const int* ids,
                              int T, int k, int* cursors, int* blk_group, int max_blocks, int* total_rows,
                              void* stream) {
  EpComm c;
  if (ep_make(desc, c) != 0) return -1;
  if (static_cast<long long>(T) * k >= (1 << 24)) {
    set_last_error("ep: T * k must stay below 2^24");
    return -1;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int n = T * k;
  ep_count_publish_kernel<<<1, 1024, 0, s>>>(c, ids, n, cursors);
  EP_CHECK("ep_count_publish");
  int ctas = (n + 7) / 8;  // one warp per row, 8 warps per CTA
  const int cap = 4 * gllm_sm_count();
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  ep_dispatch_kernel<<<ctas, 256, 0, s>>>(c, static_cast<const __nv_bfloat16*>(x), row_ss, ss_parts, ids, n, k, cursors);
  EP_CHECK("ep_dispatch");
  ep_recv_plan_kernel<<<1, 256, 0, s>>>(c, blk_group, max_blocks, total_rows);
  EP_CHECK("ep_recv_plan");
  return 0;
}

// Step 5. y: this rank's return buffer [T*k, hidden] (peers wrote it); x updated in place.
GLLM_API int gllm_ep_combine(const GllmEpDesc* desc, const void* y, const float* weights, int T, int k,
                             const void* shared, void* x, float* ss_out, void* stream) {
  EpComm c;
  if (ep_make(desc, c) != 0) return -1;
  int ctas = T < 1 ? 1 : T;
  const int cap = 8 * gllm_sm_count();
  if (ctas > cap) ctas = cap;
  ep_combine_kernel<<<ctas, 256, 0, (cudaStream_t)stream>>>(c, static_cast<const __nv_bfloat16*>(y), weights, T, k,
                                                            static_cast<const __nv_bfloat16*>(shared),
                                                            static_cast<__nv_bfloat16*>(x), ss_out);
  EP_CHECK("ep_combine");
  return 0;
}
