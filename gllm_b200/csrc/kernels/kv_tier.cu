// Device-side 4-bit KV tier (KIVI layout): whole KV pages packed into a byte pool on the same GPU, unpacked back, and
// read in place by an attention kernel.
//
// A bf16 cache page is [2 (K, V)][n_kv][16 tokens][D]. Its packed form takes n_kv * (20 D + 64) bytes (2624 per head
// for D = 128 against 8192 in bf16), per head:
//   K part, 12 D bytes: codes [16 tokens][D / 2] (channel 2j in the low nibble of byte j, 2j + 1 in the high one),
//                       then scale[D], zero[D] as fp16: one asymmetric range PER CHANNEL over the page's 16 tokens
//                       (key outliers live in fixed channels, so each channel keeps its own range)
//   V part, 8 D + 64:   codes [16][D / 2], then scale[16], zero[16] as fp16: one range PER TOKEN
// value = code * scale + zero, code in 0..15, scale = (max - min) / 15 and zero = min, both rounded to fp16 BEFORE the
// codes are chosen, so that packing then unpacking is the nearest point of the grid the reader will see.
//
//   gllm_kivi4_pack_pages     cache pages -> pool slots        (a sequence leaves the hot tier, 3.1x smaller)
//   gllm_kivi4_unpack_pages   pool slots -> cache pages        (it comes back; the tensor-core kernels read bf16)
//   gllm_paged_attention_tiered   attention over a block table that mixes both: entry p >= 0 is a bf16 page,
//                             entry p < 0 is pool slot -p - 1, dequantised as it is read (CUDA cores, any even D <= 256)
//
// Reference parity: KIVI key-per-channel / value-per-token quantisation of cold pages and the precision tiers chosen
// per page (src/kv_cache/quant.rs:35-700, src/scheduler/kv_optimizer.rs:131-192,446-830).
#include <cuda_fp16.h>

#include "common.cuh"

extern "C" int* gllm_error_word();

namespace gllm {

__host__ __device__ inline long long kivi4_head_bytes(int D) { return 20LL * D + 64; }

__device__ __forceinline__ void kivi4_range(float lo, float hi, float& s, float& z, __half& sh, __half& zh) {
  sh = __float2half_rn(__fdiv_rn(hi - lo, 15.f));
  zh = __float2half_rn(lo);
  s = __half2float(sh);
  z = __half2float(zh);
  if (!(s > 0.f)) s = 1.f;      // a constant group: every code is 0 and the value is `zero`
}
__device__ __forceinline__ unsigned int kivi4_code(float x, float s, float z) {
  const float c = rintf(__fdiv_rn(x - z, s));
  return static_cast<unsigned int>(fminf(fmaxf(c, 0.f), 15.f));
}

// grid (n pages, n_kv, 2), 128 threads
__global__ void __launch_bounds__(128) kivi4_pack_kernel(const __nv_bfloat16* cache, uint8_t* pool, const int* src_pages,
                                                         const int* dst_slots, int n_kv, int D, int num_pages,
                                                         int pool_pages, int* err) {
  const int i = blockIdx.x, h = blockIdx.y, kv = blockIdx.z;
  const int page = src_pages[i], slot = dst_slots[i];
  if (page < 0 || page >= num_pages || slot < 0 || slot >= pool_pages) {
    if (err && threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_PAGE);
    return;
  }
  const int half_d = D / 2;
  const __nv_bfloat16* src = cache + ((static_cast<long long>(page) * 2 + kv) * n_kv + h) * 16 * D;
  uint8_t* dst = pool + static_cast<long long>(slot) * n_kv * kivi4_head_bytes(D) + h * kivi4_head_bytes(D) + (kv ? 12LL * D : 0);
  __half* meta = reinterpret_cast<__half*>(dst + 8LL * D);
  if (kv == 0) {
    // keys: a thread owns channels 2j and 2j + 1 of all 16 tokens
    for (int j = threadIdx.x; j < half_d; j += blockDim.x) {
      float s[2], z[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int d = 2 * j + c;
        float lo = INFINITY, hi = -INFINITY;
        for (int t = 0; t < 16; ++t) {
          const float x = __bfloat162float(src[t * D + d]);
          lo = fminf(lo, x);
          hi = fmaxf(hi, x);
        }
        __half sh, zh;
        kivi4_range(lo, hi, s[c], z[c], sh, zh);
        meta[d] = sh;
        meta[D + d] = zh;
      }
      for (int t = 0; t < 16; ++t) {
        const unsigned int c0 = kivi4_code(__bfloat162float(src[t * D + 2 * j]), s[0], z[0]);
        const unsigned int c1 = kivi4_code(__bfloat162float(src[t * D + 2 * j + 1]), s[1], z[1]);
        dst[t * half_d + j] = static_cast<uint8_t>(c0 | (c1 << 4));
      }
    }
  } else {
    // values: a warp owns a token
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int t = warp; t < 16; t += nwarps) {
      float lo = INFINITY, hi = -INFINITY;
      for (int d = lane; d < D; d += 32) {
        const float x = __bfloat162float(src[t * D + d]);
        lo = fminf(lo, x);
        hi = fmaxf(hi, x);
      }
      lo = -warp_max(-lo);
      hi = warp_max(hi);
      float s, z;
      __half sh, zh;
      kivi4_range(lo, hi, s, z, sh, zh);
      if (lane == 0) {
        meta[t] = sh;
        meta[16 + t] = zh;
      }
      for (int j = lane; j < half_d; j += 32) {
        const unsigned int c0 = kivi4_code(__bfloat162float(src[t * D + 2 * j]), s, z);
        const unsigned int c1 = kivi4_code(__bfloat162float(src[t * D + 2 * j + 1]), s, z);
        dst[t * half_d + j] = static_cast<uint8_t>(c0 | (c1 << 4));
      }
    }
  }
}

__device__ __forceinline__ float kivi4_scale(const __half* p) {
  const float s = __half2float(*p);
  return s > 0.f ? s : 1.f;
}

// grid (n pages, n_kv, 2), 128 threads
__global__ void __launch_bounds__(128) kivi4_unpack_kernel(__nv_bfloat16* cache, const uint8_t* pool, const int* src_slots,
                                                           const int* dst_pages, int n_kv, int D, int num_pages,
                                                           int pool_pages, int* err) {
  const int i = blockIdx.x, h = blockIdx.y, kv = blockIdx.z;
  const int slot = src_slots[i], page = dst_pages[i];
  if (page < 0 || page >= num_pages || slot < 0 || slot >= pool_pages) {
    if (err && threadIdx.x == 0) atomicCAS(err, 0, ERR_BAD_PAGE);
    return;
  }
  const int half_d = D / 2;
  __nv_bfloat16* dst = cache + ((static_cast<long long>(page) * 2 + kv) * n_kv + h) * 16 * D;
  const uint8_t* src = pool + static_cast<long long>(slot) * n_kv * kivi4_head_bytes(D) + h * kivi4_head_bytes(D) + (kv ? 12LL * D : 0);
  const __half* meta = reinterpret_cast<const __half*>(src + 8LL * D);
  for (int idx = threadIdx.x; idx < 16 * half_d; idx += blockDim.x) {
    const int t = idx / half_d, j = idx % half_d;
    const unsigned int b = src[idx];
    const float c0 = static_cast<float>(b & 15u), c1 = static_cast<float>(b >> 4);
    float v0, v1;
    if (kv == 0) {
      v0 = c0 * kivi4_scale(meta + 2 * j) + __half2float(meta[D + 2 * j]);
      v1 = c1 * kivi4_scale(meta + 2 * j + 1) + __half2float(meta[D + 2 * j + 1]);
    } else {
      const float s = kivi4_scale(meta + t), z = __half2float(meta[16 + t]);
      v0 = c0 * s + z;
      v1 = c1 * s + z;
    }
    dst[t * D + 2 * j] = __float2bfloat16_rn(v0);
    dst[t * D + 2 * j + 1] = __float2bfloat16_rn(v1);
  }
}

// One warp per (query token, head), like the generic kernel; a block-table entry p < 0 names pool slot -p - 1.
__global__ void paged_attention_tiered_kernel(const __nv_bfloat16* q, __nv_bfloat16* out, const __nv_bfloat16* cache,
                                              const uint8_t* pool, const int* block_tables, int max_blocks,
                                              const int* q_start, const int* q_len, const int* ctx_lens, int n_q,
                                              int n_kv, int D, float scale, int causal, int window, int num_pages,
                                              int pool_pages, int* err) {
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
  const int half_d = D / 2;
  float qv[8], acc[8];
  for (int i = 0; i < per; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < D ? __bfloat162float(q[(static_cast<long long>(tok) * n_q + head) * D + d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float mx = -INFINITY, l = 0.f;
  const int* bt = block_tables + static_cast<long long>(seq) * max_blocks;
  for (int t = lo; t < hi; ++t) {
    int page = (t / 16 < max_blocks) ? bt[t / 16] : 0;
    const int off = t % 16;
    float kx[8], vx[8];
    if (page >= 0) {
      if (page >= num_pages) {
        if (err && lane == 0) atomicCAS(err, 0, ERR_BAD_PAGE);
        page = 0;
      }
      const __nv_bfloat16* kp = cache + (((static_cast<long long>(page) * 2) * n_kv + kvh) * 16 + off) * D;
      const __nv_bfloat16* vp = cache + (((static_cast<long long>(page) * 2 + 1) * n_kv + kvh) * 16 + off) * D;
      for (int i = 0; i < per; ++i) {
        const int d = lane + 32 * i;
        kx[i] = d < D ? __bfloat162float(kp[d]) : 0.f;
        vx[i] = d < D ? __bfloat162float(vp[d]) : 0.f;
      }
    } else {
      int slot = -page - 1;
      if (slot >= pool_pages) {
        if (err && lane == 0) atomicCAS(err, 0, ERR_BAD_PAGE);
        slot = 0;
      }
      const uint8_t* kb = pool + static_cast<long long>(slot) * n_kv * kivi4_head_bytes(D) + kvh * kivi4_head_bytes(D);
      const uint8_t* vb = kb + 12LL * D;
      const __half* km = reinterpret_cast<const __half*>(kb + 8LL * D);
      const __half* vm = reinterpret_cast<const __half*>(vb + 8LL * D);
      const float vs = kivi4_scale(vm + off), vz = __half2float(vm[16 + off]);
      for (int i = 0; i < per; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
          const unsigned int kbyte = kb[off * half_d + (d >> 1)], vbyte = vb[off * half_d + (d >> 1)];
          const float kc = static_cast<float>((d & 1) ? (kbyte >> 4) : (kbyte & 15u));
          const float vc = static_cast<float>((d & 1) ? (vbyte >> 4) : (vbyte & 15u));
          kx[i] = kc * kivi4_scale(km + d) + __half2float(km[D + d]);
          vx[i] = vc * vs + vz;
        } else {
          kx[i] = 0.f;
          vx[i] = 0.f;
        }
      }
    }
    float s = 0.f;
    for (int i = 0; i < per; ++i) s += qv[i] * kx[i];
    s = warp_sum(s);
    const float mn = fmaxf(mx, s);
    const float c = __expf(mx - mn), pnew = __expf(s - mn);
    l = l * c + pnew;
    for (int i = 0; i < per; ++i) acc[i] = acc[i] * c + pnew * vx[i];
    mx = mn;
  }
  for (int i = 0; i < per; ++i) {
    const int d = lane + 32 * i;
    if (d < D) out[(static_cast<long long>(tok) * n_q + head) * D + d] = __float2bfloat16_rn(l > 0.f ? acc[i] / l : 0.f);
  }
}

}  // namespace gllm

using namespace gllm;

GLLM_API long long gllm_kivi4_page_bytes(int n_kv, int D) { return static_cast<long long>(n_kv) * kivi4_head_bytes(D); }

static int kivi4_check(const char* what, int n_kv, int D) {
  if (n_kv <= 0 || D <= 0 || D > 256 || (D & 1)) {
    set_last_error("%s: n_kv %d, head_dim %d (even, <= 256)", what, n_kv, D);
    return -1;
  }
  return 0;
}

// cache: bf16 [num_pages, 2, n_kv, 16, D]; pool: bytes [pool_pages, gllm_kivi4_page_bytes]; ids: device int32 [n].
GLLM_API int gllm_kivi4_pack_pages(const void* cache, int num_pages, void* pool, int pool_pages, const int* src_pages,
                                   const int* dst_slots, int n, int n_kv, int D, void* stream) {
  if (n <= 0) return 0;
  if (kivi4_check("kivi4_pack_pages", n_kv, D)) return -1;
  kivi4_pack_kernel<<<dim3(n, n_kv, 2), 128, 0, (cudaStream_t)stream>>>(static_cast<const __nv_bfloat16*>(cache),
                                                                       static_cast<uint8_t*>(pool), src_pages, dst_slots,
                                                                       n_kv, D, num_pages, pool_pages, gllm_error_word());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("kivi4_pack_pages launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

GLLM_API int gllm_kivi4_unpack_pages(void* cache, int num_pages, const void* pool, int pool_pages, const int* src_slots,
                                     const int* dst_pages, int n, int n_kv, int D, void* stream) {
  if (n <= 0) return 0;
  if (kivi4_check("kivi4_unpack_pages", n_kv, D)) return -1;
  kivi4_unpack_kernel<<<dim3(n, n_kv, 2), 128, 0, (cudaStream_t)stream>>>(static_cast<__nv_bfloat16*>(cache),
                                                                         static_cast<const uint8_t*>(pool), src_slots,
                                                                         dst_pages, n_kv, D, num_pages, pool_pages,
                                                                         gllm_error_word());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("kivi4_unpack_pages launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

GLLM_API int gllm_paged_attention_tiered(const void* q, void* out, const void* cache, int num_pages, const void* pool,
                                         int pool_pages, const int* block_tables, int max_blocks, const int* q_start,
                                         const int* q_len, const int* ctx_lens, int num_seqs, int max_q_len, int n_q,
                                         int n_kv, int D, float scale, int causal, int window, void* stream) {
  if (num_seqs <= 0 || max_q_len <= 0) return 0;
  if (kivi4_check("paged_attention_tiered", n_kv, D)) return -1;
  if (n_q <= 0 || n_q % n_kv != 0) {
    set_last_error("paged_attention_tiered: %d query heads over %d KV heads", n_q, n_kv);
    return -1;
  }
  const dim3 grid((max_q_len + 3) / 4, n_q, num_seqs);
  paged_attention_tiered_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(cache),
      static_cast<const uint8_t*>(pool), block_tables, max_blocks, q_start, q_len, ctx_lens, n_q, n_kv, D, scale, causal,
      window, num_pages, pool_pages, gllm_error_word());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("paged_attention_tiered launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
