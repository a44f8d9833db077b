// MLA absorbed decode attention on tensor cores (mma.sync m16n8k16, bf16, fp32 accumulate).
//
// One CTA (4 warps) serves one (sequence, tile of 16 query heads, KV split). Every head attends over the SAME
// latent rows [c_kv (d_c = 512) | k_pe (d_r = 64)], so the 16 heads are the 16 rows of the MMA tile and each
// latent byte is read from HBM once per head tile. Per 32-token tile:
//   phase 1  warp w: S_w[16 heads x 8 tokens] = Q[16 x 576] . K_w^T   (36 k-steps, A and B through ldmatrix)
//            block-wide online softmax (row maxima / sums exchanged through shared memory), P written as bf16
//   phase 2  warp w: O_w[16 x 128 columns] += P[16 x 32] . V[32 x (its 128 of the 512 latent columns)]
// The latent tile is fetched by TMA (boxes of 16 tokens x 64 columns, 128-byte swizzle) into a two-stage ring;
// two CTAs share an SM so that one computes while the other waits for its tile.
// With more than one KV split the unnormalised partial outputs and their (max, sum) go to scratch and a second
// small kernel merges them.
//
// Reference parity: MlaAttention over the latent cache with the absorbed query
// (src/arch/auto_graph_fragments/build_graph.inc.rs:1513-1578).
#include "common.cuh"

namespace gllm {

constexpr int kMdDc = 512, kMdDr = 64, kMdDk = kMdDc + kMdDr;   // 576
constexpr int kMdPage = 16;
constexpr int kMdTile = 32;                 // tokens per stage (two CTAs per SM hide each other's load latency)
constexpr int kMdChunks = kMdDk / 64;       // 9 column chunks of 64 bf16 (128 bytes)
constexpr int kMdStageBytes = kMdChunks * kMdTile * 128;   // 36864
constexpr int kMdPStride = kMdTile + 8;     // bf16 elements per row of the probability tile (16-byte rows, odd multiple)
constexpr int kMdQBytes = kMdChunks * 16 * 128;            // 18432
constexpr int kMdThreads = 128;

__device__ __forceinline__ void md_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void md_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void md_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t md_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

struct MlaDecodeParams {
  const __nv_bfloat16* q;     // [B, n_heads, 576]
  __nv_bfloat16* out;         // [B, n_heads, 512]
  const int* block_tables;    // [B, max_blocks]
  const int* ctx_lens;        // [B]
  int max_blocks, n_heads, num_pages, splits;
  float scale_log2;           // softmax scale * log2(e)
  float* part_o;              // [B, head_tiles, splits, 16, 512] unnormalised partial outputs (splits > 1)
  float* part_ml;             // [B, head_tiles, splits, 16, 2] (max in log2 domain, sum)
  int* err;
};

// shared-memory address of the 16-byte chunk holding columns [8j, 8j+8) of row `row` inside a [rows x 64 col] box
// group laid out as TMA writes it with the 128-byte swizzle: box c (64 columns) at c * rows * 128.
__device__ __forceinline__ uint32_t md_addr(uint32_t base, int rows, int row, int col8) {
  const int c = col8 >> 3, j = col8 & 7;
  return base + c * rows * 128 + row * 128 + ((j ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(kMdThreads, 2)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmap, const MlaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_kv = smem;                                   // 2 stages
  uint8_t* s_q = smem + 2 * kMdStageBytes;                // Q tile, same swizzled layout with 16 rows
  __nv_bfloat16* s_p = reinterpret_cast<__nv_bfloat16*>(s_q + kMdQBytes);        // P [16][kMdPStride] bf16
  float* s_red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(s_p) + 16 * kMdPStride * 2);   // [4 warps][16 rows][2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_red + 4 * 16 * 2);              // full[2]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2);

  const int b = blockIdx.x, ht = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctx = p.ctx_lens[b];
  const int n_tiles_total = (ctx + kMdTile - 1) / kMdTile;
  const int t_begin = static_cast<int>(static_cast<long long>(split) * n_tiles_total / p.splits);
  const int t_end = static_cast<int>(static_cast<long long>(split + 1) * n_tiles_total / p.splits);
  const int head0 = ht * 16;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  // Q tile -> shared memory (rows beyond n_heads are zero), swizzled like the KV boxes
  for (int idx = threadIdx.x; idx < 16 * (kMdDk / 8); idx += kMdThreads) {
    const int row = idx / (kMdDk / 8), col8 = idx % (kMdDk / 8);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (head0 + row < p.n_heads)
      v = *reinterpret_cast<const uint4*>(p.q + (static_cast<long long>(b) * p.n_heads + head0 + row) * kMdDk + col8 * 8);
    const uint32_t a = md_addr(0, 16, row, col8);
    *reinterpret_cast<uint4*>(s_q + a) = v;
  }
  __syncthreads();

  auto issue_tile = [&](int t, int stage) {   // one thread: 2 pages x 9 boxes
    uint8_t* dst = s_kv + stage * kMdStageBytes;
    const int tok0 = t * kMdTile;
    int n_pages = (min(ctx, tok0 + kMdTile) - tok0 + kMdPage - 1) / kMdPage;
    mbar_expect_tx(&bars[stage], n_pages * kMdChunks * kMdPage * 128);
    for (int pg = 0; pg < n_pages; ++pg) {
      int page = p.block_tables[static_cast<long long>(b) * p.max_blocks + tok0 / kMdPage + pg];
      if (page < 0 || page >= p.num_pages) {
        if (p.err) atomicCAS(p.err, 0, ERR_BAD_PAGE);
        page = 0;
      }
      for (int c = 0; c < kMdChunks; ++c)
        tma_load_2d(dst + c * kMdTile * 128 + pg * kMdPage * 128, &tmap, &bars[stage], c * 64, page * kMdPage);
    }
  };

  float o[16][4];     // this warp's 128 output columns: 16 n-tiles of 8
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows lane/4 and lane/4 + 8
  const uint32_t q_base = smem_u32(s_q);

  if (threadIdx.x == 0 && t_begin < t_end) issue_tile(t_begin, 0);
  for (int t = t_begin, it = 0; t < t_end; ++t, ++it) {
    const int stage = it & 1;
    if (threadIdx.x == 0 && t + 1 < t_end) issue_tile(t + 1, stage ^ 1);   // the other stage was released by the sync below
    mbar_wait(&bars[stage], (it >> 1) & 1, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL);   // on a timeout the status word is set
    const uint32_t kv_base = smem_u32(s_kv + stage * kMdStageBytes);
    const int tok0 = t * kMdTile;
    {
      // the last tile of a sequence may bring fewer than four pages: rows nothing was copied into must not hold
      // NaN bit patterns (their probabilities are zero, but 0 * NaN is NaN in the P.V product)
      const int rows_valid = ((min(ctx, tok0 + kMdTile) - tok0 + kMdPage - 1) / kMdPage) * kMdPage;
      if (rows_valid < kMdTile) {
        uint8_t* st = s_kv + stage * kMdStageBytes;
        const int per_chunk = (kMdTile - rows_valid) * 8;     // 16-byte pieces per column chunk
        for (int idx = threadIdx.x; idx < kMdChunks * per_chunk; idx += kMdThreads) {
          const int c = idx / per_chunk, r = idx % per_chunk;
          *reinterpret_cast<uint4*>(st + c * kMdTile * 128 + rows_valid * 128 + r * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    // ---------------- phase 1: S_w = Q . K_w^T for tokens [8w, 8w+8) of the tile ----------------
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int a_row = (lane & 7) + (((lane >> 3) & 1) << 3);      // A: rows 0-15, two k halves per k-step
      const int a_csel = lane >> 4;
      const int b_tok = warp * 8 + (lane & 7);                      // B: 8 token rows, four k chunks = two k-steps
      const int b_csel = lane >> 3;
#pragma unroll 3
      for (int ks2 = 0; ks2 < kMdDk / 32; ++ks2) {
        uint32_t a0[4], a1[4], b0, b1, b2, b3;
        md_ldsm_x4(md_addr(q_base, 16, a_row, ks2 * 4 + a_csel), a0[0], a0[1], a0[2], a0[3]);
        md_ldsm_x4(md_addr(q_base, 16, a_row, ks2 * 4 + 2 + a_csel), a1[0], a1[1], a1[2], a1[3]);
        md_ldsm_x4(md_addr(kv_base, kMdTile, b_tok, ks2 * 4 + b_csel), b0, b1, b2, b3);
        md_mma(s, a0, b0, b1);
        md_mma(s, a1, b2, b3);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int tok = tok0 + warp * 8 + (lane & 3) * 2 + e;
      float v0 = s[e] * p.scale_log2, v1 = s[2 + e] * p.scale_log2;
      if (tok >= ctx) v0 = v1 = -INFINITY;
      s[e] = v0;
      s[2 + e] = v1;
      mx0 = fmaxf(mx0, v0);
      mx1 = fmaxf(mx1, v1);
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const int r0 = lane >> 2, r1 = r0 + 8;
    if ((lane & 3) == 0) {
      s_red[(warp * 16 + r0) * 2] = mx0;
      s_red[(warp * 16 + r1) * 2] = mx1;
    }
    __syncthreads();
    float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      tm0 = fmaxf(tm0, s_red[(w * 16 + r0) * 2]);
      tm1 = fmaxf(tm1, s_red[(w * 16 + r1) * 2]);
    }
    const float mn0 = fmaxf(m0, tm0), mn1 = fmaxf(m1, tm1);
    const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float corr0 = exp2f(m0 - ms0), corr1 = exp2f(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
    {
      const float p00 = exp2f(s[0] - ms0), p01 = exp2f(s[1] - ms0);
      const float p10 = exp2f(s[2] - ms1), p11 = exp2f(s[3] - ms1);
      rs0 = p00 + p01;
      rs1 = p10 + p11;
      const int col = warp * 8 + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(s_p + r0 * kMdPStride + col) = md_pack(p00, p01);
      *reinterpret_cast<uint32_t*>(s_p + r1 * kMdPStride + col) = md_pack(p10, p11);
    }
    rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
    rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
    rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
    rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
    if ((lane & 3) == 0) {
      s_red[(warp * 16 + r0) * 2 + 1] = rs0;
      s_red[(warp * 16 + r1) * 2 + 1] = rs1;
    }
    __syncthreads();
    float ts0 = 0.f, ts1 = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      ts0 += s_red[(w * 16 + r0) * 2 + 1];
      ts1 += s_red[(w * 16 + r1) * 2 + 1];
    }
    l0 = l0 * corr0 + ts0;
    l1 = l1 * corr1 + ts1;
    // ---------------- phase 2: O_w += P . V[:, 128w .. 128w+128) ----------------
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= corr0;
      o[i][1] *= corr0;
      o[i][2] *= corr1;
      o[i][3] *= corr1;
    }
    {
      const uint32_t p_base = smem_u32(s_p);
      const int a_row = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int a_csel = lane >> 4;
      const int v_tok = (lane & 7) + (((lane >> 3) & 1) << 3);
      const int v_csel = lane >> 4;
#pragma unroll
      for (int kt = 0; kt < kMdTile / 16; ++kt) {
        uint32_t a[4];
        md_ldsm_x4(p_base + (a_row * kMdPStride + kt * 16 + a_csel * 8) * 2, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {     // 16 output columns per ldmatrix.x4.trans
          uint32_t b0, b1, b2, b3;
          md_ldsm_x4_t(md_addr(kv_base, kMdTile, kt * 16 + v_tok, (warp * 128 + nb * 16) / 8 + v_csel), b0, b1, b2, b3);
          md_mma(o[nb * 2], a, b0, b1);
          md_mma(o[nb * 2 + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();   // P, the reduction scratch and this stage's tile are free again
  }

  // ---------------- write-out ----------------
  const int r0 = lane >> 2, r1 = r0 + 8;
  if (p.splits == 1) {
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int col = warp * 128 + i * 8 + (lane & 3) * 2;
      if (head0 + r0 < p.n_heads)
        *reinterpret_cast<uint32_t*>(p.out + (static_cast<long long>(b) * p.n_heads + head0 + r0) * kMdDc + col) =
            md_pack(o[i][0] * inv0, o[i][1] * inv0);
      if (head0 + r1 < p.n_heads)
        *reinterpret_cast<uint32_t*>(p.out + (static_cast<long long>(b) * p.n_heads + head0 + r1) * kMdDc + col) =
            md_pack(o[i][2] * inv1, o[i][3] * inv1);
    }
  } else {
    const long long unit = (static_cast<long long>(b) * gridDim.y + ht) * p.splits + split;
    float* po = p.part_o + unit * 16 * kMdDc;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int col = warp * 128 + i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(po + r0 * kMdDc + col) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(po + r1 * kMdDc + col) = make_float2(o[i][2], o[i][3]);
    }
    if (warp == 0 && (lane & 3) == 0) {
      float* ml = p.part_ml + unit * 16 * 2;
      ml[r0 * 2] = m0; ml[r0 * 2 + 1] = l0;
      ml[r1 * 2] = m1; ml[r1 * 2 + 1] = l1;
    }
  }
}

// out[b, h, :] = sum_s exp2(m_s - M) * o_s / sum_s exp2(m_s - M) * l_s
__global__ void mla_decode_merge_kernel(const float* part_o, const float* part_ml, __nv_bfloat16* out, int n_heads,
                                        int head_tiles, int splits) {
  const int b = blockIdx.x, ht = blockIdx.y, row = blockIdx.z;
  const int head = ht * 16 + row;
  if (head >= n_heads) return;
  const long long unit0 = (static_cast<long long>(b) * head_tiles + ht) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[((unit0 + s) * 16 + row) * 2]);
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* ml = part_ml + ((unit0 + s) * 16 + row) * 2;
    L += exp2f(ml[0] - Ms) * ml[1];
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int c = threadIdx.x; c < kMdDc; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float w = exp2f(part_ml[((unit0 + s) * 16 + row) * 2] - Ms);
      acc += w * part_o[((unit0 + s) * 16 + row) * kMdDc + c];
    }
    out[(static_cast<long long>(b) * n_heads + head) * kMdDc + c] = __float2bfloat16(acc * inv);
  }
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();
extern "C" int gllm_sm_count();

// Floats of scratch the call needs for `splits` KV splits (0 when splits == 1).
GLLM_API long long gllm_mla_decode_scratch_floats(int batch, int n_heads, int splits) {
  if (splits <= 1) return 0;
  const long long units = static_cast<long long>(batch) * ((n_heads + 15) / 16) * splits;
  return units * 16 * (kMdDc + 2);
}

// q [B, n_heads, 576] bf16 ([q_abs | q_pe] per head); cache [num_pages, 16, 576] bf16; out [B, n_heads, 512] bf16.
// One query token per sequence (decode). splits <= 0 picks a split count that fills the GPU.
GLLM_API int gllm_mla_decode(const void* q, void* out, const void* cache, int num_pages, const int* block_tables,
                             int max_blocks, const int* ctx_lens, int batch, int n_heads, int max_ctx, float scale,
                             int splits, float* scratch, long long scratch_floats, void* stream) {
  if (batch <= 0) return 0;
  const int head_tiles = (n_heads + 15) / 16;
  if (splits <= 0) {
    const int ctas = batch * head_tiles;
    const int tiles = (max_ctx + kMdTile - 1) / kMdTile;
    splits = 1;
    const int sms = gllm_sm_count();
    while (ctas * splits < 2 * sms && splits * 2 <= tiles && splits < 16) splits *= 2;   // two CTAs fit on an SM
  }
  if (splits > 1 && (!scratch || gllm_mla_decode_scratch_floats(batch, n_heads, splits) > scratch_floats)) splits = 1;
  CUtensorMap tmap;
  if (make_tmap_2d(&tmap, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(num_pages) * kMdPage, uint64_t(kMdDk),
                   uint64_t(kMdDk), kMdPage, 64))
    return -1;
  MlaDecodeParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_tables = block_tables;
  p.ctx_lens = ctx_lens;
  p.max_blocks = max_blocks; p.n_heads = n_heads; p.num_pages = num_pages; p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + static_cast<long long>(batch) * head_tiles * splits * 16 * kMdDc : nullptr;
  p.err = gllm_error_word();
  const int smem = 2 * kMdStageBytes + kMdQBytes + 16 * kMdPStride * 2 + 4 * 16 * 2 * 4 + 64 + 1024;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_done[dev & 63] = true;
  }
  cudaStream_t s = (cudaStream_t)stream;
  mla_decode_kernel<<<dim3(batch, head_tiles, splits), kMdThreads, smem, s>>>(tmap, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("mla_decode launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  if (splits > 1) {
    mla_decode_merge_kernel<<<dim3(batch, head_tiles, 16), 128, 0, s>>>(p.part_o, p.part_ml, p.out, n_heads, head_tiles, splits);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_last_error("mla_decode merge launch failed: %s", cudaGetErrorString(e));
      return -1;
    }
  }
  return 0;
}
