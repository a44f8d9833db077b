// Weight-quantised GEMM for sm_100a: out[M,N] = A[M,K] (bf16) @ dequant(W)[N,K]^T, with the dequantisation fused
// into the main loop.
//
// The quantised weight tile (fp8 e4m3, fp4 e2m1, int4 or int8 codes) is what crosses HBM: TMA brings the raw
// bytes of a [128 rows x 64 k] tile into shared memory, four "transform" warps expand them to bf16 (code ->
// value * group scale + group offset), writing the 128-byte-swizzled K-major layout that tcgen05.mma reads, and
// signal the MMA warp. A is loaded by TMA already swizzled. Accumulators live in TMEM; the epilogue reads them
// with tcgen05.ld and stores bf16 (or fp32 partials when K is split across CTAs, reduced by a second tiny kernel).
//
// Warp roles (512 threads): 0 TMA producer, 1 MMA issuer, 2 TMEM allocator, 3 idle, 4-7 epilogue, 8-15 transform
// (two groups of four warps taking alternate stages, so one group's scale-load latency hides behind the other's
// conversion).
//
// Canonical weight form (built by the Python packer from MXFP8 / FP8-block / NVFP4 / MXFP4 / AWQ / GPTQ / GGUF
// blocks): codes uint8 [N, K*bits/8] row-major (4-bit: low nibble = even k), scales bf16 [N, K/group],
// optional offsets bf16 [N, K/group]; value = decode(code) * scale + offset, or (decode(code) + offset) * scale when
// the offset is an integer zero point (exact in bf16).
//
// Reference parity: the QuantGemm graph op (src/arch/auto_graph_fragments/build_graph.inc.rs:116) dequantises in
// the JIT's GEMM main loop for 22 block formats; here every format is first repacked to the canonical form.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace gllm {

constexpr int kQBM = 128;       // rows of A per tile (UMMA M)
constexpr int kQBN = 128;       // rows of W per tile (UMMA N)
constexpr int kQBK = 64;        // k elements per stage (128 bytes of bf16)
constexpr int kQThreads = 512;

enum QMode { Q_FP8 = 0, Q_FP4 = 1, Q_INT4 = 2, Q_INT8 = 3 };

struct QGemmParams {
  int M, N, K;
  int num_m, num_n, num_kb, splits;
  int mode, group, group_shift;    // group: k elements per scale (a power of two); group_shift = log2(group)
  const __nv_bfloat16* scales;     // [N, K/group]
  const __nv_bfloat16* offsets;    // [N, K/group] or null
  int offset_in_codes;             // 1: value = (code + offset) * scale; 0: value = code * scale + offset
  long long ld_scale;
  __nv_bfloat16* out;              // [M, N] (splits == 1)
  float* partial;                  // [splits, M, N] (splits > 1)
  long long ldo;
  const float* row_ss_in;          // optional RMSNorm row statistics of A (sum of squares), [M, ss_parts]
  int ss_parts;
  float norm_inv_dim, norm_eps;
  int* err;
};

// MT = 128-row A tiles sharing one W tile: with MT = 2 every weight tile is fetched and expanded once for 256 rows.
template <int BYTES_PER_ROW, int MT>
struct QStage {
  static constexpr int kA1 = kQBM * 128;              // one swizzled bf16 A tile
  static constexpr int kA = MT * kA1;
  static constexpr int kB = kQBN * 128;               // swizzled bf16 W tile (written by the transform warps)
  static constexpr int kRaw = kQBN * BYTES_PER_ROW;   // raw codes
  static constexpr int kBytes = kA + kB + ((kRaw + 1023) / 1024) * 1024;
  static constexpr int kStages = MT == 1 ? 4 : 3;
  static constexpr int kTmemCols = 2 * MT * kQBN;     // double-buffered accumulators
};

__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint32_t bf16x2_from(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Expand `n` codes starting at byte pointer `src` into floats.
template <int MODE>
__device__ __forceinline__ void decode16(const uint8_t* bytes, float (&v)[16]) {
  if constexpr (MODE == Q_FP8) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_fp8x2_storage_t pr = static_cast<__nv_fp8x2_storage_t>(bytes[2 * i] | (bytes[2 * i + 1] << 8));
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  } else if constexpr (MODE == Q_INT8) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = static_cast<float>(static_cast<int8_t>(bytes[i]));
  } else if constexpr (MODE == Q_FP4) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(bytes[i]), __NV_E2M1);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
      v[2 * i] = f.x;       // low nibble = even k
      v[2 * i + 1] = f.y;
    }
  } else {  // Q_INT4 unsigned codes
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = static_cast<float>(bytes[i] & 0xF);
      v[2 * i + 1] = static_cast<float>(bytes[i] >> 4);
    }
  }
}

template <int MODE, int MT>
__global__ void __launch_bounds__(kQThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const QGemmParams p) {
  constexpr int kBits = (MODE == Q_FP8 || MODE == Q_INT8) ? 8 : 4;
  constexpr int kRowBytes = kQBK * kBits / 8;         // raw bytes of one W row per stage: 64 or 32
  using St = QStage<kRowBytes, MT>;
  constexpr int kQStages = St::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + kQStages * St::kBytes);
  uint64_t* full_bar = raw_full + kQStages;
  uint64_t* empty_bar = full_bar + kQStages;
  uint64_t* tmem_full = empty_bar + kQStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_ptr + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int splits = p.splits;
  const int num_items = p.num_m * p.num_n * splits;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&full_bar[s], 4);    // one arrival per transform warp
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
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 2) {
    tmem_alloc(tmem_base_ptr, St::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;

  auto decode_item = [&](int t, int& ks, int& m_blk, int& n_blk, int& kb0, int& kb1) {
    ks = t % splits;
    const int r = t / splits;
    m_blk = r % p.num_m;
    n_blk = r / p.num_m;
    kb0 = static_cast<int>(static_cast<long long>(ks) * p.num_kb / splits);
    kb1 = static_cast<int>(static_cast<long long>(ks + 1) * p.num_kb / splits);
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
        int ks, m_blk, n_blk, kb0, kb1;
        decode_item(t, ks, m_blk, n_blk, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, ERR_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * St::kBytes;
          uint8_t* sraw = sa + St::kA + St::kB;
          mbar_expect_tx(&raw_full[stage], St::kA + St::kRaw);
#pragma unroll
          for (int i = 0; i < MT; ++i)
            tma_load_2d(sa + i * St::kA1, &tmap_a, &raw_full[stage], kb * kQBK, (m_blk * MT + i) * kQBM);
          tma_load_2d(sraw, &tmap_w, &raw_full[stage], kb * kRowBytes, n_blk * kQBN);
          if (++stage == kQStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(kQBM, kQBN, 1, 1);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
        int ks, m_blk, n_blk, kb0, kb1;
        decode_item(t, ks, m_blk, n_blk, kb0, kb1);
        const int it_cur = it++;
        const int acc = it_cur & 1;
        const uint32_t acc_phase = (it_cur >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.err, ERR_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (MT * kQBN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * St::kBytes);
          const uint64_t b_desc = umma_desc_sw128(sa + St::kA);
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            const uint64_t a_desc = umma_desc_sw128(sa + i * St::kA1);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16(d_tmem + i * kQBN, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == kQStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else if (warp >= 8) {
    // ------------------------------- transform: codes -> swizzled bf16 -------------------------------
    const int grp = (warp - 8) >> 2;                  // transform group 0 / 1
    const int tt = threadIdx.x - 256 - grp * 128;     // 0..127 inside the group
    constexpr int kChunksPerRow = kRowBytes / 16;     // 16-byte raw chunks per row: 4 (8-bit) or 2 (4-bit)
    constexpr int kElemsPerChunk = 16 * 8 / kBits;    // 16 or 32
    constexpr int kChunks = kQBN * kChunksPerRow;
    int seq = 0;                                      // running stage counter over all (tile, k block) pairs
    bool ok = true;
    for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
      int ks, m_blk, n_blk, kb0, kb1;
      decode_item(t, ks, m_blk, n_blk, kb0, kb1);
      for (int kb = kb0; kb < kb1; ++kb, ++seq) {
        if ((seq & 1) != grp) continue;               // the other group's stage
        const int stage = seq % kQStages;
        const uint32_t phase = (seq / kQStages) & 1;
        const bool got = mbar_wait(&raw_full[stage], phase, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL);
        if (!__all_sync(0xffffffffu, got)) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + stage * St::kBytes + St::kA;
        const uint8_t* sraw = sb + St::kB;
        // issue every load of this stage first (raw codes from shared memory, scales / offsets from L2), then
        // convert: one memory latency per stage instead of one per chunk
        constexpr int kPer = kChunks / 128;                 // chunks per thread: 4 (8-bit) or 2 (4-bit)
        constexpr int kHalves = kElemsPerChunk / 16;        // 16-element pieces per chunk: 1 or 2
        uint4 raw[kPer];
        float sc[kPer][kHalves], of[kPer][kHalves];
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
          const int c = tt + i * 128;
          const int r = c / kChunksPerRow, cc = c % kChunksPerRow;
          raw[i] = *reinterpret_cast<const uint4*>(sraw + r * kRowBytes + cc * 16);
          const int n = n_blk * kQBN + r;
          const int nn = n < p.N ? n : p.N - 1;
#pragma unroll
          for (int half = 0; half < kHalves; ++half) {
            // 16 consecutive k share a scale when group >= 16 (every supported format)
            const int kk = kb * kQBK + cc * kElemsPerChunk + half * 16;
            const long long si = static_cast<long long>(nn) * p.ld_scale + (kk >> p.group_shift);
            sc[i][half] = __bfloat162float(p.scales[si]);
            of[i][half] = p.offsets ? __bfloat162float(p.offsets[si]) : 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
          const int c = tt + i * 128;
          const int r = c / kChunksPerRow, cc = c % kChunksPerRow;
          const uint8_t* bytes = reinterpret_cast<const uint8_t*>(&raw[i]);
#pragma unroll
          for (int half = 0; half < kHalves; ++half) {
            float v[16];
            decode16<MODE>(bytes + half * (16 * kBits / 8), v);
            const float s = sc[i][half];
            const float o = p.offset_in_codes ? of[i][half] * s : of[i][half];
            uint4 w0, w1;
            w0.x = bf16x2_from(v[0] * s + o, v[1] * s + o);
            w0.y = bf16x2_from(v[2] * s + o, v[3] * s + o);
            w0.z = bf16x2_from(v[4] * s + o, v[5] * s + o);
            w0.w = bf16x2_from(v[6] * s + o, v[7] * s + o);
            w1.x = bf16x2_from(v[8] * s + o, v[9] * s + o);
            w1.y = bf16x2_from(v[10] * s + o, v[11] * s + o);
            w1.z = bf16x2_from(v[12] * s + o, v[13] * s + o);
            w1.w = bf16x2_from(v[14] * s + o, v[15] * s + o);
            // 128-byte swizzle: 16-byte chunk j of row r lives at chunk (j ^ (r & 7)) of that row
            const int j = (cc * kElemsPerChunk + half * 16) / 8;   // first of two 16-byte chunks (8 bf16 each)
            uint8_t* row = sb + r * 128;
            *reinterpret_cast<uint4*>(row + ((j ^ (r & 7)) << 4)) = w0;
            *reinterpret_cast<uint4*>(row + (((j + 1) ^ (r & 7)) << 4)) = w1;
          }
        }
        fence_async_proxy();   // generic-proxy writes above must be visible to the tensor core's async-proxy reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------- epilogue -------------------------------
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
      int ks, m_blk, n_blk, kb0, kb1;
      decode_item(t, ks, m_blk, n_blk, kb0, kb1);
      const int it_cur = it++;
      const int acc = it_cur & 1;
      const uint32_t acc_phase = (it_cur >> 1) & 1;
      const bool got = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.err, ERR_TIMEOUT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int mi = 0; mi < MT; ++mi) {
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * (MT * kQBN) + mi * kQBN;
      const int m = (m_blk * MT + mi) * kQBM + q * 32 + lane;
      const bool row_ok = m < p.M;
      float rs = 1.f;
      if (p.row_ss_in && row_ok) {
        float ss = 0.f;
        for (int i = 0; i < p.ss_parts; ++i) ss += p.row_ss_in[static_cast<long long>(m) * p.ss_parts + i];
        rs = rsqrtf(ss * p.norm_inv_dim + p.norm_eps);
      }
#pragma unroll 1
      for (int c = 0; c < kQBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int n0 = n_blk * kQBN + c * 32;
        if (!row_ok || n0 >= p.N) continue;
        if (splits > 1) {
          float4* d4 = reinterpret_cast<float4*>(p.partial + (static_cast<long long>(ks) * p.M + m) * p.ldo + n0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (n0 + 4 * j < p.N)
              d4[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                  __uint_as_float(r[4 * j + 3]));
        } else {
          uint4* d4 = reinterpret_cast<uint4*>(p.out + static_cast<long long>(m) * p.ldo + n0);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (n0 + 8 * j >= p.N) continue;
            uint4 w;
            w.x = bf16x2_from(__uint_as_float(r[8 * j]) * rs, __uint_as_float(r[8 * j + 1]) * rs);
            w.y = bf16x2_from(__uint_as_float(r[8 * j + 2]) * rs, __uint_as_float(r[8 * j + 3]) * rs);
            w.z = bf16x2_from(__uint_as_float(r[8 * j + 4]) * rs, __uint_as_float(r[8 * j + 5]) * rs);
            w.w = bf16x2_from(__uint_as_float(r[8 * j + 6]) * rs, __uint_as_float(r[8 * j + 7]) * rs);
            d4[j] = w;
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 2) tmem_dealloc(tmem_base, St::kTmemCols);
}

// out[m][n] = bf16(rowscale(m) * sum_s partial[s][m][n])
__global__ void qgemm_reduce_kernel(const float* partial, int splits, int M, int N, long long ldo, __nv_bfloat16* out,
                                    const float* row_ss_in, int ss_parts, float inv_dim, float eps) {
  const long long idx = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (idx >= static_cast<long long>(M) * N) return;
  const int m = static_cast<int>(idx / N), n = static_cast<int>(idx % N);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(partial + (static_cast<long long>(s) * M + m) * ldo + n);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  float rs = 1.f;
  if (row_ss_in) {
    float ss = 0.f;
    for (int i = 0; i < ss_parts; ++i) ss += row_ss_in[static_cast<long long>(m) * ss_parts + i];
    rs = rsqrtf(ss * inv_dim + eps);
  }
  uint2 w;
  w.x = bf16x2_from(acc.x * rs, acc.y * rs);
  w.y = bf16x2_from(acc.z * rs, acc.w * rs);
  *reinterpret_cast<uint2*>(out + static_cast<long long>(m) * ldo + n) = w;
}

static int make_raw_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch_bytes,
                         uint32_t box_rows, uint32_t box_bytes) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || pitch_bytes % 16 != 0 || box_bytes % 16 != 0) {
    set_last_error("quantised weight: base / row pitch / box must be 16-byte aligned (pitch %llu)", (unsigned long long)pitch_bytes);
    return -1;
  }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return -1;
  }
  cuuint64_t gdim[2] = {row_bytes, rows};
  cuuint64_t gstride[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled (raw codes) failed with CUresult %d", int(r));
    return -1;
  }
  return 0;
}

template <int MODE, int MT>
static int launch_qgemm_mt(const CUtensorMap& ta, const CUtensorMap& tw, const QGemmParams& p, int ctas, cudaStream_t s) {
  constexpr int kBits = (MODE == Q_FP8 || MODE == Q_INT8) ? 8 : 4;
  using St = QStage<kQBK * kBits / 8, MT>;
  const int smem = St::kStages * St::kBytes + 1024 + 1024;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaFuncSetAttribute(qgemm_kernel<MODE, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done[dev & 63] = true;
  }
  qgemm_kernel<MODE, MT><<<ctas, kQThreads, smem, s>>>(ta, tw, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("qgemm launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

template <int MODE>
static int launch_qgemm(const CUtensorMap& ta, const CUtensorMap& tw, const QGemmParams& p, int mt, int ctas, cudaStream_t s) {
  return mt == 2 ? launch_qgemm_mt<MODE, 2>(ta, tw, p, ctas, s) : launch_qgemm_mt<MODE, 1>(ta, tw, p, ctas, s);
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();
extern "C" int gllm_sm_count();

// A [M, K] bf16 (lda elements); codes [N, K*bits/8] uint8 (pitch bytes); scales / offsets bf16 [N, K/group].
// partial: fp32 scratch of at least splits*M*N floats when the call may split K (pass null to forbid splitting).
GLLM_API int gllm_qgemm(const void* A, long long lda, const void* codes, long long pitch_bytes, int mode, int group,
                        const void* scales, const void* offsets, int offset_in_codes, long long ld_scale, void* out, long long ldo, int M,
                        int N, int K, const float* row_ss_in, int ss_parts, float norm_inv_dim, float norm_eps,
                        float* partial, long long partial_floats, int force_splits, void* stream) {
  if (mode < 0 || mode > 3 || K % kQBK != 0 || N % 8 != 0 || group < 16 || (group & (group - 1)) != 0 || K % group != 0) {
    set_last_error("qgemm: mode %d group %d K %d N %d unsupported (K %% 64 == 0, N %% 8 == 0, group a power of two >= 16 dividing K)",
                   mode, group, K, N);
    return -1;
  }
  if (M <= 0) return 0;
  const int bits = (mode == Q_FP8 || mode == Q_INT8) ? 8 : 4;
  QGemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  const int mt = M > kQBM ? 2 : 1;
  p.num_m = (M + mt * kQBM - 1) / (mt * kQBM); p.num_n = (N + kQBN - 1) / kQBN; p.num_kb = K / kQBK;
  p.mode = mode; p.group = group;
  p.group_shift = 0;
  while ((1 << p.group_shift) < group) ++p.group_shift;
  p.scales = static_cast<const __nv_bfloat16*>(scales);
  p.offsets = static_cast<const __nv_bfloat16*>(offsets);
  p.offset_in_codes = offset_in_codes;
  p.ld_scale = ld_scale;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.row_ss_in = row_ss_in; p.ss_parts = ss_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.err = gllm_error_word();
  const int sms = gllm_sm_count();
  const int tiles = p.num_m * p.num_n;
  int splits = 1;
  if (force_splits > 0) {
    splits = force_splits;
  } else if (partial && tiles < 2 * sms) {
    // fewest waves of work per unit of K, with a small charge per split for the partial dump and the reduce
    double best = 1e30;
    for (int sp = 1; sp <= 16 && sp * 4 <= p.num_kb; ++sp) {
      const int waves = (tiles * sp + sms - 1) / sms;
      const double cost = static_cast<double>(waves) / sp + 0.03 * (sp - 1);
      if (cost < best - 1e-9) {
        best = cost;
        splits = sp;
      }
    }
  }
  if (splits < 1) splits = 1;
  if (splits > p.num_kb) splits = p.num_kb;
  if (splits > 1 && (!partial || static_cast<long long>(splits) * M * ldo > partial_floats || N % 4 != 0)) splits = 1;
  p.splits = splits;
  p.partial = partial;
  CUtensorMap ta, tw;
  if (make_tmap_2d(&ta, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(M), uint64_t(K), uint64_t(lda), kQBM, kQBK)) return -1;
  const uint32_t row_bytes = kQBK * bits / 8;
  if (make_raw_tmap(&tw, codes, uint64_t(N), uint64_t(K) * bits / 8, uint64_t(pitch_bytes), kQBN, row_bytes)) return -1;
  int ctas = tiles * splits;
  if (ctas > sms) ctas = sms;
  cudaStream_t s = (cudaStream_t)stream;
  int rc = 0;
  switch (mode) {
    case Q_FP8: rc = launch_qgemm<Q_FP8>(ta, tw, p, mt, ctas, s); break;
    case Q_FP4: rc = launch_qgemm<Q_FP4>(ta, tw, p, mt, ctas, s); break;
    case Q_INT4: rc = launch_qgemm<Q_INT4>(ta, tw, p, mt, ctas, s); break;
    default: rc = launch_qgemm<Q_INT8>(ta, tw, p, mt, ctas, s); break;
  }
  if (rc) return rc;
  if (splits > 1) {
    const long long quads = (static_cast<long long>(M) * N + 3) / 4;
    qgemm_reduce_kernel<<<static_cast<unsigned>((quads + 255) / 256), 256, 0, s>>>(
        partial, splits, M, N, ldo, p.out, row_ss_in, ss_parts, norm_inv_dim, norm_eps);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_error("qgemm reduce launch failed: %s", cudaGetErrorString(e));
      return -1;
    }
  }
  return 0;
}
