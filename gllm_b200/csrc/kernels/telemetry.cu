// Layer telemetry and in-place KV page requantisation.
//
//   gllm_layer_telemetry   one pass over a layer's input / output residual stream and its FFN activation:
//                          ||x_out - x_in||^2, ||x_in||^2, count of near-zero activations -> residual delta and
//                          activation sparsity without a host round trip per tensor.
//   gllm_kv_requant_pages  rounds whole KV pages (bf16 container) through a lower precision tier in place:
//                          fp8 e4m3 with one scale per page, or asymmetric 4 / 2 bit per token row (KIVI style V
//                          quantisation). The page keeps its bf16 layout, so every attention kernel still reads it;
//                          what changes is the information it holds (and what a compressed swap-out would store).
//
// Reference parity: epilogue telemetry signals (src/jit/epilogue.rs; 64-byte page header fields
// src/kv_cache/mod.rs:119-135) and host-side page requantisation (src/scheduler/kv_optimizer.rs:446-830).
#include <cuda_fp8.h>

#include "common.cuh"

namespace gllm {

__global__ void __launch_bounds__(256) layer_telemetry_kernel(const __nv_bfloat16* x_in, const __nv_bfloat16* x_out,
                                                              long long n_x, const __nv_bfloat16* act, long long n_act,
                                                              float eps, float* out) {
  float d2 = 0.f, n2 = 0.f, zeros = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_x; i += stride) {
    const float a = __bfloat162float(x_in[i]), b = __bfloat162float(x_out[i]);
    d2 += (b - a) * (b - a);
    n2 += a * a;
  }
  if (act)
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_act; i += stride)
      zeros += fabsf(__bfloat162float(act[i])) < eps ? 1.f : 0.f;
  d2 = warp_sum(d2);
  n2 = warp_sum(n2);
  zeros = warp_sum(zeros);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(out + 0, d2);
    atomicAdd(out + 1, n2);
    atomicAdd(out + 2, zeros);
  }
}

// mode 1: fp8 e4m3, one scale per page; mode 2 / 3: asymmetric 4 / 2 bit per row of `row_len` elements.
__global__ void __launch_bounds__(256) kv_requant_kernel(__nv_bfloat16* cache, const int* page_ids, long long page_elems,
                                                         int row_len, int mode, int num_pages, int* err) {
  __shared__ float red[8], red2[8];
  const int page = page_ids[blockIdx.x];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0 && err) atomicCAS(err, 0, ERR_BAD_PAGE);
    return;
  }
  __nv_bfloat16* p = cache + static_cast<long long>(page) * page_elems;
  if (mode == 1) {
    float amax = 0.f;
    for (long long i = threadIdx.x; i < page_elems; i += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(p[i])));
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.f;
    for (int w = 0; w < 8; ++w) amax = fmaxf(amax, red[w]);
    const float scale = fmaxf(amax, 1e-12f) / 448.0f, inv = 1.0f / scale;
    for (long long i = threadIdx.x; i < page_elems; i += blockDim.x) {
      const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(__bfloat162float(p[i]) * inv, __NV_SATFINITE, __NV_E4M3);
      const __half_raw h = __nv_cvt_fp8_to_halfraw(q, __NV_E4M3);
      p[i] = __float2bfloat16_rn(__half2float(*reinterpret_cast<const __half*>(&h)) * scale);
    }
    return;
  }
  const int levels = mode == 2 ? 15 : 3;
  const int rows = static_cast<int>(page_elems / row_len);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < rows; r += blockDim.x >> 5) {   // one warp per row
    __nv_bfloat16* row = p + static_cast<long long>(r) * row_len;
    float lo = INFINITY, hi = -INFINITY;
    for (int i = lane; i < row_len; i += 32) {
      const float v = __bfloat162float(row[i]);
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
    lo = -warp_max(-lo);
    hi = warp_max(hi);
    const float scale = fmaxf(hi - lo, 1e-8f) / levels;
    for (int i = lane; i < row_len; i += 32) {
      const float q = fminf(fmaxf(rintf((__bfloat162float(row[i]) - lo) / scale), 0.f), static_cast<float>(levels));
      row[i] = __float2bfloat16_rn(q * scale + lo);
    }
  }
  (void)red2;
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();
extern "C" int gllm_sm_count();

// out: 3 floats {sum (x_out - x_in)^2, sum x_in^2, count |act| < eps}; zeroed here.
GLLM_API int gllm_layer_telemetry(const void* x_in, const void* x_out, long long n_x, const void* act, long long n_act,
                                  float eps, float* out, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  cudaMemsetAsync(out, 0, 3 * sizeof(float), s);
  if (n_x <= 0) return 0;
  int blocks = static_cast<int>((n_x + 256 * 8 - 1) / (256 * 8));
  const int cap = 4 * gllm_sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  layer_telemetry_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x_in), static_cast<const __nv_bfloat16*>(x_out),
                                                n_x, static_cast<const __nv_bfloat16*>(act), n_act, eps, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("layer_telemetry launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

// cache: bf16 [num_pages, page_elems]; page_ids: device int32 [n]; mode 1 fp8, 2 four-bit rows, 3 two-bit rows.
GLLM_API int gllm_kv_requant_pages(void* cache, int num_pages, long long page_elems, const int* page_ids, int n, int row_len,
                                   int mode, void* stream) {
  if (n <= 0) return 0;
  if (mode < 1 || mode > 3 || row_len <= 0 || page_elems % row_len != 0) {
    set_last_error("kv_requant_pages: mode %d row_len %d page_elems %lld", mode, row_len, page_elems);
    return -1;
  }
  kv_requant_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(static_cast<__nv_bfloat16*>(cache), page_ids, page_elems, row_len, mode,
                                                        num_pages, gllm_error_word());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("kv_requant_pages launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
