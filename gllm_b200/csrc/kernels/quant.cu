// Activation quantisation for the block-scaled tensor-core GEMMs (sm_100a): bf16 rows -> MXFP8 (e4m3 codes + one
// ue8m0 scale per 32 elements) or NVFP4 (e2m1 codes, two per byte, + one ue4m3 scale per 16 elements; a static
// per-tensor scale is divided out first). The scale bytes are written in the 512-byte chunk layout the GEMM's bulk
// copies and tcgen05.cp consume: chunk (row / 128, scale column / 4), byte (r % 32) * 16 + ((r % 128) / 32) * 4 + j.
//
// The reference quantises nothing at run time (its QuantGemm dequantises weights, activations stay f32:
// src/arch/auto_graph_fragments/build_graph.inc.rs:116); block-scaled tensor cores need both operands narrow.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace gllm {

__device__ __forceinline__ long long sf_byte_offset(int r, int col, int cols) {
  const long long chunk = static_cast<long long>(r >> 7) * (cols >> 2) + (col >> 2);
  return chunk * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (col & 3);
}

// Source row / destination row of work unit `u` (one unit per row): plain form u -> (u, u), bounded by *rows_limit
// when given (a device-side row count, e.g. the routed rows of an MoE step); scatter form: unit u is routed pair
// (token u / k, slot u % k) whose destination row is dest[u] (< 0: not for this rank).
struct RowMap {
  const int* rows_limit;
  const int* dest;
  int k;
};
__device__ __forceinline__ bool map_row(const RowMap& m, int u, int& src, int& dst) {
  if (m.dest) {
    dst = __ldg(m.dest + u);
    src = u / m.k;
    return dst >= 0;
  }
  src = dst = u;
  return m.rows_limit == nullptr || u < __ldg(m.rows_limit);
}

// one thread per (row, 32-element block)
__global__ void __launch_bounds__(256) quantize_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M,
                                                             int K, uint8_t* __restrict__ codes, long long ldc,
                                                             uint8_t* __restrict__ sf, RowMap map) {
  const int nblk = K >> 5;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int u = static_cast<int>(idx / nblk), b = static_cast<int>(idx % nblk);
  if (u >= M) return;
  int rs, r;
  if (!map_row(map, u, rs, r)) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(rs) * ldx + b * 32);
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 u = __ldg(src + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      v[i * 8 + e * 2] = f.x;
      v[i * 8 + e * 2 + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  // smallest power of two s with amax / s <= 448
  int e = -127;
  if (amax > 0.f) {
    int ex;
    const float m = frexpf(amax * (1.0f / 448.0f), &ex);   // value = m * 2^ex, m in [0.5, 1)
    e = (m == 0.5f) ? ex - 1 : ex;
    e = max(-127, min(127, e));
  }
  const float inv = exp2f(static_cast<float>(-e));
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[i] = lo | (hi << 16);
  }
  uint4* dst = reinterpret_cast<uint4*>(codes + static_cast<long long>(r) * ldc + b * 32);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  sf[sf_byte_offset(r, b, nblk)] = static_cast<uint8_t>(e + 127);
}

// one thread per (row, 16-element block)
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M,
                                                             int K, uint8_t* __restrict__ codes, long long ldc,
                                                             uint8_t* __restrict__ sf, float inv_tensor_scale,
                                                             RowMap map) {
  const int nblk = K >> 4;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int u = static_cast<int>(idx / nblk), b = static_cast<int>(idx % nblk);
  if (u >= M) return;
  int rs, r;
  if (!map_row(map, u, rs, r)) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(rs) * ldx + b * 16);
  float v[16];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 u = __ldg(src + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      v[i * 8 + e * 2] = f.x * inv_tensor_scale;
      v[i * 8 + e * 2 + 1] = f.y * inv_tensor_scale;
      amax = fmaxf(amax, fmaxf(fabsf(v[i * 8 + e * 2]), fabsf(v[i * 8 + e * 2 + 1])));
    }
  }
  // block scale: amax / 6 rounded to ue4m3 (the positive half of e4m3), then the codes against the ROUNDED scale
  const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(amax * (1.0f / 6.0f), __NV_SATFINITE, __NV_E4M3);
  const float s = __half2float(__half(__nv_cvt_fp8_to_halfraw(sb, __NV_E4M3)));
  const float inv = s > 0.f ? 1.0f / s : 0.f;
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t byte = __nv_cvt_float2_to_fp4x2(make_float2(v[2 * i] * inv, v[2 * i + 1] * inv), __NV_E2M1, cudaRoundNearest);
    w[i >> 2] |= (byte & 0xFFu) << (8 * (i & 3));
  }
  *reinterpret_cast<uint2*>(codes + static_cast<long long>(r) * ldc + b * 8) = make_uint2(w[0], w[1]);
  sf[sf_byte_offset(r, b, nblk)] = static_cast<uint8_t>(sb);
}

}  // namespace gllm

using namespace gllm;

// x [M, K] bf16 (row pitch ldx elements) -> codes (row pitch ldc BYTES) + scale chunks. fmt 2: MXFP8 (K % 128 == 0),
// fmt 3: NVFP4 (K % 256 == 0; tensor_scale is the static second-level scale). The scale buffer must cover the rows
// padded to 128 (ops/blockscale.py: sf_bytes).
// rows_limit (device int, nullable): only rows below *rows_limit are quantised (M then is the upper bound the launch is
// sized for). dest / k (nullable / 0): scatter form for routed MoE rows: work unit u = (token u / k, slot u % k) reads
// row u / k of x and writes destination row dest[u] (a negative entry is skipped); M is then the number of units.
static int quantize_launch(const void* x, long long ldx, int M, int K, int fmt, void* codes, long long ldc, void* sf,
                           float tensor_scale, const int* rows_limit, const int* dest, int k, void* stream) {
  if (!x || !codes || !sf || M <= 0 || K <= 0 || (fmt != 2 && fmt != 3) || K % (fmt == 2 ? 128 : 256) != 0 ||
      (ldx % 8) != 0 || (ldc % 16) != 0 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(codes)) & 15) ||
      (dest && k <= 0)) {
    set_last_error("quantize_act: bad arguments (M %d K %d fmt %d; 16-byte aligned rows required)", M, K, fmt);
    return -1;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long units = static_cast<long long>(M) * (K / (fmt == 2 ? 32 : 16));
  const unsigned grid = static_cast<unsigned>((units + 255) / 256);
  RowMap map{rows_limit, dest, k};
  if (fmt == 2)
    quantize_mxfp8_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, M, K,
                                               static_cast<uint8_t*>(codes), ldc, static_cast<uint8_t*>(sf), map);
  else
    quantize_nvfp4_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), ldx, M, K,
                                               static_cast<uint8_t*>(codes), ldc, static_cast<uint8_t*>(sf),
                                               tensor_scale > 0.f ? 1.0f / tensor_scale : 1.0f, map);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("quantize_act launch: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

GLLM_API int gllm_quantize_act(const void* x, long long ldx, int M, int K, int fmt, void* codes, long long ldc,
                               void* sf, float tensor_scale, void* stream) {
  return quantize_launch(x, ldx, M, K, fmt, codes, ldc, sf, tensor_scale, nullptr, nullptr, 0, stream);
}
GLLM_API int gllm_quantize_act_rows(const void* x, long long ldx, int max_rows, int K, int fmt, void* codes,
                                    long long ldc, void* sf, float tensor_scale, const int* rows_limit, void* stream) {
  return quantize_launch(x, ldx, max_rows, K, fmt, codes, ldc, sf, tensor_scale, rows_limit, nullptr, 0, stream);
}
GLLM_API int gllm_quantize_act_scatter(const void* x, long long ldx, int units, int k, int K, int fmt, void* codes,
                                       long long ldc, void* sf, float tensor_scale, const int* dest, void* stream) {
  return quantize_launch(x, ldx, units, K, fmt, codes, ldc, sf, tensor_scale, nullptr, dest, k, stream);
}
