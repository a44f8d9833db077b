// Persistent warp-specialised tcgen05 GEMM family for sm_100a:  D[M,N] = A[M,K] · B[N,K]ᵀ.
//
// Both operands are K-major (activations row-major, weights in checkpoint [out,in] order), so the
// kernel consumes weights exactly as they sit in the file — the same "trans_b = true" contract
// the reference's graph uses for every linear (src/arch/auto_graph_fragments/build_graph.inc.rs:1618).
//
// One CTA per SM, 256 threads:
//   warp 0      TMA producer: 128xBK A tile + BNxBK B tile per stage, 128-byte swizzle
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16|32) into TMEM
//   warp 2      TMEM allocator
//   warps 4..7  epilogue: tcgen05.ld -> registers -> fused epilogue -> global
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of tile i overlaps
// the main loop of tile i+1.
//
// Fused epilogues (the reference lowers these as separate graph ops; see build_graph.inc.rs
// RmsNorm :275, Add :1865, SwiGlu :1983, HeadRmsNorm :1708, RoPE :1754, attention kv_write :1777):
//   EPI_STORE     out = rowscale * acc (+bias)                 (bf16 or fp32)
//   EPI_RESIDUAL  out = acc (+bias) + residual ; per-row partial sum of squares of `out`
//   EPI_GLU       out = act(rowscale*gate) * (rowscale*up)     (SwiGLU / GeGLU, weights interleaved per tile)
//   EPI_QKV       per head: rowscale -> optional per-head RMSNorm -> RoPE -> q buffer / paged KV write
// `rowscale` is the RMSNorm-as-prologue trick: the norm weight is folded into B at load time and
// the per-row rsqrt(mean(x²)+eps) is applied to the accumulator, using the partial sums of squares
// that the producing kernel's epilogue left behind.
#include "common.cuh"

namespace gllm {

enum : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GLU = 2, EPI_QKV = 3 };

constexpr int kBM = 128;
constexpr int kTileKBytes = 128;  // one swizzle row
constexpr int kGemmThreads = 256;
constexpr int kPageTokens = 16;

struct GemmParams {
  int M, N, K;
  int num_m, num_n, num_kb;
  // output
  void* out;
  long long ldo;
  int out_f32;
  const float* bias;  // [N] or null
  // residual epilogue
  const __nv_bfloat16* residual;
  long long ldr;
  float* row_ss_out;  // [M, num_n] or null
  // rmsnorm-as-row-scale prologue
  const float* row_ss_in;  // [M, ss_in_parts] or null
  int ss_in_parts;
  float norm_inv_dim, norm_eps;
  // per-row / per-column dequant scales (fp8 path), nullable
  const float* a_scale;
  const float* b_scale;
  // GLU
  int glu_act;  // 0 = silu, 1 = gelu_tanh
  // grouped GEMM: m-block -> group id; B rows of group g start at g * group_rows
  const int* mblk_group;
  int group_rows;
  // QKV epilogue
  int n_q_heads, n_kv_heads;
  __nv_bfloat16* q_out;  // [M, n_q_heads*128]
  __nv_bfloat16* kv_cache;  // [pages][2][n_kv_heads][16][128]
  int num_pages;
  const int* slot_mapping;  // [M] slot = page*16 + offset, or -1
  const int* positions;     // [M]
  const float* cos_table;   // [max_pos][64]
  const float* sin_table;   // [max_pos][64]
  int max_pos;
  const float* q_norm_w;  // [128] or null
  const float* k_norm_w;  // [128] or null
  float qk_eps;
  int* err;
};

template <int BN>
struct GemmCfg {
  static constexpr int kStageBytes = kBM * kTileKBytes + BN * kTileKBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*align slack*/;
};

__device__ __forceinline__ float row_scale_of(const GemmParams& p, int m) {
  if (p.row_ss_in == nullptr) return 1.0f;
  float ss = 0.f;
  const float* src = p.row_ss_in + static_cast<long long>(m) * p.ss_in_parts;
  for (int i = 0; i < p.ss_in_parts; ++i) ss += src[i];
  return rsqrtf(ss * p.norm_inv_dim + p.norm_eps);
}

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&v)[32]) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 u;
    u.x = pack_bf16x2(v[i * 8 + 0], v[i * 8 + 1]);
    u.y = pack_bf16x2(v[i * 8 + 2], v[i * 8 + 3]);
    u.z = pack_bf16x2(v[i * 8 + 4], v[i * 8 + 5]);
    u.w = pack_bf16x2(v[i * 8 + 6], v[i * 8 + 7]);
    d4[i] = u;
  }
}

template <int BN, int EPI, bool FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kABytes = kBM * kTileKBytes;
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr int kElemsPerKB = FP8 ? 128 : 64;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tiles = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_ptr + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m * p.num_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 2) {
    tmem_alloc(tmem_base_ptr, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % p.num_m;
        const int n_blk = t / p.num_m;
        int b_row = n_blk * BN;
        if (p.mblk_group) b_row += p.mblk_group[m_blk] * p.group_rows;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, ERR_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = tiles + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kElemsPerKB, m_blk * kBM);
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kElemsPerKB, b_row);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kBM, BN, FP8 ? 0 : 1, FP8 ? 0 : 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.err, ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * kStageBytes);
          const uint64_t a_desc = umma_desc_sw128(sa);
          const uint64_t b_desc = umma_desc_sw128(sa + kABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 4 x 32-byte K slices per 128-byte swizzle row
            if (FP8)
              umma_f8f6f4(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
            else
              umma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------- epilogue -----------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const int m_blk = t % p.num_m;
      const int n_blk = t / p.num_m;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      // warp-uniform decision: tcgen05.ld below is warp-collective
      const bool got = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.err, ERR_TIMEOUT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int m = m_blk * kBM + q * 32 + lane;
      const bool row_ok = m < p.M;
      const int mm = row_ok ? m : (p.M - 1);
      float rs = row_scale_of(p, mm);
      if (p.a_scale) rs *= p.a_scale[mm];

      if constexpr (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
        float ss = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int n0 = n_blk * BN + c * 32;
          if (n0 >= p.N) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * rs;
          if (p.b_scale) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.b_scale[n0 + j];
          }
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += p.bias[n0 + j];
          }
          if constexpr (EPI == EPI_RESIDUAL) {
            if (row_ok) {
              const uint4* r4 = reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(m) * p.ldr + n0);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 u = r4[i];
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 f = __bfloat1622float2(h[e]);
                  v[i * 8 + e * 2] += f.x;
                  v[i * 8 + e * 2 + 1] += f.y;
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = bf16_round(v[j]);
              ss += v[j] * v[j];
            }
          }
          if (row_ok) {
            if (p.out_f32) {
              float4* o4 = reinterpret_cast<float4*>(static_cast<float*>(p.out) + static_cast<long long>(m) * p.ldo + n0);
#pragma unroll
              for (int i = 0; i < 8; ++i) o4[i] = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
            } else {
              store_bf16x32(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0, v);
            }
          }
        }
        if constexpr (EPI == EPI_RESIDUAL) {
          if (p.row_ss_out && row_ok) p.row_ss_out[static_cast<long long>(m) * p.num_n + n_blk] = ss;
        }
      } else if constexpr (EPI == EPI_GLU) {
        // tile columns [0, BN/2) hold gate rows, [BN/2, BN) the matching up rows
        constexpr int kHalf = BN / 2;
#pragma unroll 1
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c * 32, g);
          tmem_ld_32x32(taddr + kHalf + c * 32, u);
          tmem_ld_wait();
          const int n0 = n_blk * kHalf + c * 32;  // output column
          if (n0 >= p.N / 2) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float gv = __uint_as_float(g[j]) * rs;
            float uv = __uint_as_float(u[j]) * rs;
            if (p.b_scale) {
              gv *= p.b_scale[n_blk * BN + c * 32 + j];
              uv *= p.b_scale[n_blk * BN + kHalf + c * 32 + j];
            }
            v[j] = (p.glu_act == 0 ? silu_f(gv) : gelu_tanh_f(gv)) * uv;
          }
          if (row_ok) store_bf16x32(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0, v);
        }
      } else {  // EPI_QKV, BN == 128 == head_dim: this tile is exactly one head
        static_assert(EPI != EPI_QKV || BN == 128, "QKV epilogue needs BN == head_dim == 128");
        const int head = n_blk;
        const bool is_q = head < p.n_q_heads;
        const bool is_k = !is_q && head < p.n_q_heads + p.n_kv_heads;
        const float* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
        float inv_rms = 1.f;
        if (nw) {  // per-head RMSNorm over the 128 features of this row
          float ss = 0.f;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float x = __uint_as_float(r[j]) * rs;
              if (p.bias) x += p.bias[head * 128 + c * 32 + j];
              ss += x * x;
            }
          }
          inv_rms = rsqrtf(ss * (1.0f / 128.0f) + p.qk_eps);
        }
        int pos = 0, slot = -1;
        if (row_ok) {
          pos = p.positions[m];
          slot = p.slot_mapping ? p.slot_mapping[m] : -1;
          if (pos < 0 || pos >= p.max_pos) pos = 0;
        }
        __nv_bfloat16* dst = nullptr;
        if (row_ok) {
          if (is_q) {
            dst = p.q_out + (static_cast<long long>(m) * p.n_q_heads + head) * 128;
          } else if (slot >= 0) {
            const int page = slot / kPageTokens, off = slot % kPageTokens;
            if (page >= p.num_pages) {
              if (p.err) atomicCAS(p.err, 0, ERR_BAD_PAGE);
            } else {
              const int kvh = is_k ? head - p.n_q_heads : head - p.n_q_heads - p.n_kv_heads;
              const long long base = ((static_cast<long long>(page) * 2 + (is_k ? 0 : 1)) * p.n_kv_heads + kvh);
              dst = p.kv_cache + (base * kPageTokens + off) * 128;
            }
          }
        }
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {  // columns [32c, 32c+32) pair with [64+32c, 64+32c+32)
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(taddr + c * 32, lo);
          tmem_ld_32x32(taddr + 64 + c * 32, hi);
          tmem_ld_wait();
          float a[32], b[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float x0 = __uint_as_float(lo[j]) * rs;
            float x1 = __uint_as_float(hi[j]) * rs;
            if (p.bias) {
              x0 += p.bias[head * 128 + c * 32 + j];
              x1 += p.bias[head * 128 + 64 + c * 32 + j];
            }
            if (nw) {
              x0 *= inv_rms * nw[c * 32 + j];
              x1 *= inv_rms * nw[64 + c * 32 + j];
            }
            if (is_q || is_k) {
              const float cs = p.cos_table[static_cast<long long>(pos) * 64 + c * 32 + j];
              const float sn = p.sin_table[static_cast<long long>(pos) * 64 + c * 32 + j];
              a[j] = x0 * cs - x1 * sn;
              b[j] = x1 * cs + x0 * sn;
            } else {
              a[j] = x0;
              b[j] = x1;
            }
          }
          if (dst) {
            store_bf16x32(dst + c * 32, a);
            store_bf16x32(dst + 64 + c * 32, b);
          }
        }
      }
      // hand the accumulator slot back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

template <int BN, int EPI, bool FP8>
static int launch_gemm(const void* A, long long lda, const void* B, long long ldb, long long b_rows, GemmParams p,
                       cudaStream_t stream, int max_ctas) {
  using Cfg = GemmCfg<BN>;
  constexpr int kElemsPerKB = FP8 ? 128 : 64;
  const int esz = FP8 ? 1 : 2;
  const CUtensorMapDataType dt = FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  p.num_m = (p.M + kBM - 1) / kBM;
  p.num_n = (p.N + BN - 1) / BN;
  p.num_kb = (p.K + kElemsPerKB - 1) / kElemsPerKB;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) {
    set_last_error("gemm: empty problem M=%d N=%d K=%d", p.M, p.N, p.K);
    return -1;
  }
  if (p.N % 32 != 0) {
    set_last_error("gemm: N=%d must be a multiple of 32 (pad the weight at load time)", p.N);
    return -1;
  }
  CUtensorMap ta, tb;
  if (make_tmap_2d(&ta, A, dt, esz, uint64_t(p.M), uint64_t(p.K), uint64_t(lda), kBM, kElemsPerKB)) return -1;
  if (make_tmap_2d(&tb, B, dt, esz, uint64_t(b_rows), uint64_t(p.K), uint64_t(ldb), BN, kElemsPerKB)) return -1;
  static bool attr_set = false;
  auto kern = gemm_tn_kernel<BN, EPI, FP8>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      set_last_error("gemm: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
      return -1;
    }
    attr_set = true;
  }
  int sms = max_ctas;
  if (sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = p.num_m * p.num_n;
  const int grid = tiles < sms ? tiles : sms;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("gemm launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // namespace gllm

using namespace gllm;

extern "C" int* gllm_error_word();

// ---------------------------------------------------------------------------------------------
// C entry points. All pointers are device pointers; `stream` is a cudaStream_t.
// ---------------------------------------------------------------------------------------------

// out[M,N] = rowscale(A) · Bᵀ (+bias).  bn: 128 or 256.  row_ss_in may be null.
GLLM_API int gllm_gemm_bf16(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                            int M, int N, int K, int out_f32, const float* bias, const float* row_ss_in,
                            int ss_in_parts, float norm_inv_dim, float norm_eps, int bn, void* stream, int max_ctas) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32; p.bias = bias;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.err = gllm_error_word();
  if (bn == 256) return launch_gemm<256, EPI_STORE, false>(A, lda, B, ldb, N, p, (cudaStream_t)stream, max_ctas);
  return launch_gemm<128, EPI_STORE, false>(A, lda, B, ldb, N, p, (cudaStream_t)stream, max_ctas);
}

// out[M,N] = A · Bᵀ (+bias) + residual ; row_ss_out[M, ceil(N/bn)] receives per-tile sums of squares.
GLLM_API int gllm_gemm_bf16_residual(const void* A, long long lda, const void* B, long long ldb, void* out,
                                     long long ldo, const void* residual, long long ldr, float* row_ss_out, int M,
                                     int N, int K, const float* bias, int bn, void* stream, int max_ctas) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.row_ss_out = row_ss_out;
  p.err = gllm_error_word();
  if (bn == 256) return launch_gemm<256, EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, (cudaStream_t)stream, max_ctas);
  return launch_gemm<128, EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, (cudaStream_t)stream, max_ctas);
}

// out[M,N/2] = act(rowscale*gate) * rowscale*up ; B is the tile-interleaved gate/up weight [N,K]:
// rows [t*bn, t*bn+bn/2) = gate rows of output block t, rows [t*bn+bn/2, (t+1)*bn) = its up rows.
GLLM_API int gllm_gemm_bf16_glu(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                                int M, int N, int K, int act, const float* row_ss_in, int ss_in_parts,
                                float norm_inv_dim, float norm_eps, int bn, const int* mblk_group, int num_groups,
                                void* stream, int max_ctas) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.glu_act = act;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.mblk_group = mblk_group; p.group_rows = N;
  p.err = gllm_error_word();
  const long long b_rows = mblk_group ? static_cast<long long>(num_groups) * N : N;  // groups are stacked
  if (bn == 256) return launch_gemm<256, EPI_GLU, false>(A, lda, B, ldb, b_rows, p, (cudaStream_t)stream, max_ctas);
  return launch_gemm<128, EPI_GLU, false>(A, lda, B, ldb, b_rows, p, (cudaStream_t)stream, max_ctas);
}

// Grouped plain GEMM (MoE down projection): m-block i multiplies group mblk_group[i]'s [N,K] weight.
GLLM_API int gllm_gemm_bf16_grouped(const void* A, long long lda, const void* B, long long ldb, void* out,
                                    long long ldo, int M, int N, int K, const int* mblk_group, int num_groups,
                                    int bn, void* stream, int max_ctas) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo;
  p.mblk_group = mblk_group; p.group_rows = N;
  p.err = gllm_error_word();
  const long long b_rows = static_cast<long long>(num_groups) * N;
  if (bn == 256) return launch_gemm<256, EPI_STORE, false>(A, lda, B, ldb, b_rows, p, (cudaStream_t)stream, max_ctas);
  return launch_gemm<128, EPI_STORE, false>(A, lda, B, ldb, b_rows, p, (cudaStream_t)stream, max_ctas);
}

// Fused QKV projection for head_dim 128: rowscale -> per-head RMSNorm (optional) -> RoPE -> q buffer and
// paged KV write.  B is [(Hq+2Hkv)*128, K] with q heads first, then k heads, then v heads.
GLLM_API int gllm_gemm_bf16_qkv(const void* A, long long lda, const void* B, long long ldb, int M, int K,
                                int n_q_heads, int n_kv_heads, void* q_out, void* kv_cache, int num_pages,
                                const int* slot_mapping, const int* positions, const float* cos_table,
                                const float* sin_table, int max_pos, const float* q_norm_w, const float* k_norm_w,
                                float qk_eps, const float* row_ss_in, int ss_in_parts, float norm_inv_dim,
                                float norm_eps, const float* bias, void* stream, int max_ctas) {
  GemmParams p = {};
  p.M = M; p.N = (n_q_heads + 2 * n_kv_heads) * 128; p.K = K;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.q_out = static_cast<__nv_bfloat16*>(q_out); p.kv_cache = static_cast<__nv_bfloat16*>(kv_cache);
  p.num_pages = num_pages; p.slot_mapping = slot_mapping; p.positions = positions;
  p.cos_table = cos_table; p.sin_table = sin_table; p.max_pos = max_pos;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.qk_eps = qk_eps;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.bias = bias;
  p.err = gllm_error_word();
  return launch_gemm<128, EPI_QKV, false>(A, lda, B, ldb, p.N, p, (cudaStream_t)stream, max_ctas);
}

// FP8 (e4m3) GEMM with per-row activation scale and per-column weight scale applied in the epilogue.
GLLM_API int gllm_gemm_fp8(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                           int M, int N, int K, int out_f32, const float* a_scale, const float* b_scale, int bn,
                           void* stream, int max_ctas) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32;
  p.a_scale = a_scale; p.b_scale = b_scale;
  p.err = gllm_error_word();
  if (bn == 256) return launch_gemm<256, EPI_STORE, true>(A, lda, B, ldb, N, p, (cudaStream_t)stream, max_ctas);
  return launch_gemm<128, EPI_STORE, true>(A, lda, B, ldb, N, p, (cudaStream_t)stream, max_ctas);
}
