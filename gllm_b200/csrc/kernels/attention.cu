// Paged attention for head_dim 128 over 16-token KV pages (bf16 KV cache).
//
//   * paged_decode_kernel   flash-decode: one CTA per (sequence, kv head, KV split); the G = Hq/Hkv
//                           query heads that share a KV head are packed as the rows of one MMA tile, so
//                           each KV byte is read from HBM exactly once per step. Splits are merged by the
//                           last CTA to finish (ticket counter), no second launch.
//   * paged_prefill_kernel  causal flash attention for (chunked) prefill: 64 query rows per CTA, KV
//                           streamed page by page from the same paged cache (prefix pages included).
//
// KV pages are fetched with tiled TMA copies (128-byte swizzle) into a per-warp / per-CTA ring and read
// back with ldmatrix; the math is mma.sync m16n8k16 bf16 with fp32 online softmax. Decode attention is
// bandwidth bound (4 FLOP per KV byte at G = 4), so the roofline here is HBM, not the tensor pipe.
//
// Semantics follow the reference's CPU attention (src/compat/scalar_ops.rs:196-278, 316-378):
// scale 1/sqrt(d), kv head = q head / (Hq/Hkv), causal mask, max-subtracted softmax; optional sliding
// window and learnable sinks (src/arch/auto_graph_fragments/build_graph.inc.rs:1775-1781).
//
// Cache layout per layer: [page][K|V][kv_head][16 tokens][128] bf16, or the same shape in fp8 (e4m3, one per-tensor
// scale). The fp8 variants of both kernels (template parameter KV8) fetch 2 KB page tiles, convert the ldmatrix
// fragments to f16 in registers (cvt.f16x2.e4m3x2) and run the same tiles on mma.sync f16: a 16-byte shared-memory
// chunk then holds 16 features instead of 8, so the K fragments pair features (4t..4t+3) with a matching permutation
// of the Q fragment's k index, and a transposed V fragment yields the even and the odd features of a 16-feature block
// as two n-tiles; the output columns are un-permuted when they are written.
#include <cuda_fp8.h>

#include "common.cuh"

namespace gllm {

constexpr int kHD = 128;
constexpr int kPage = 16;
constexpr int kPageBytes = kPage * kHD * 2;  // 4 KB per (page, K|V, head)
template <bool KV8>
struct KvFmt {
  static constexpr int kBytes = KV8 ? kPage * kHD : kPage * kHD * 2;   // one K or V tile of a page
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two e4m3 bytes (low 16 bits of x) -> f16x2, low byte in the low half
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t x) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(x & 0xFFFFu), __NV_E4M3);
  return static_cast<uint32_t>(h.x) | (static_cast<uint32_t>(h.y) << 16);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t x) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
  return pack_f16x2(f.x, f.y);
}

// Q fragments of one 16-row tile. bf16 cache: the standard m16n8k16 A layout over feature blocks of 16. fp8 cache:
// f16 values, and within each block thread t holds features 4t, 4t+1 (k = 2t, 2t+1) and 4t+2, 4t+3 (k = 2t+8, 2t+9),
// the order in which a 16-byte ldmatrix chunk of fp8 K delivers them.
template <bool KV8>
__device__ __forceinline__ void load_q_frags(const __nv_bfloat16* q0, const __nv_bfloat16* q1, bool ok0, bool ok1,
                                             uint32_t (&qf)[8][4]) {
  const int t = threadIdx.x & 3;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    if constexpr (KV8) {
      const int c = ks * 16 + t * 4;
      const uint2 v0 = ok0 ? *reinterpret_cast<const uint2*>(q0 + c) : make_uint2(0u, 0u);
      const uint2 v1 = ok1 ? *reinterpret_cast<const uint2*>(q1 + c) : make_uint2(0u, 0u);
      qf[ks][0] = bf16x2_to_f16x2(v0.x);
      qf[ks][1] = bf16x2_to_f16x2(v1.x);
      qf[ks][2] = bf16x2_to_f16x2(v0.y);
      qf[ks][3] = bf16x2_to_f16x2(v1.y);
    } else {
      const int c = ks * 16 + t * 2;
      qf[ks][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
      qf[ks][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
      qf[ks][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
      qf[ks][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
    }
  }
}
// Feature index of accumulator element e (0/1: the two columns of the row) of n-tile dt.
template <bool KV8>
__device__ __forceinline__ int out_feature(int dt, int e) {
  const int t = threadIdx.x & 3;
  if constexpr (KV8) return 16 * (dt >> 1) + 4 * t + 2 * e + (dt & 1);
  return dt * 8 + t * 2 + e;
}

// Online-softmax state of one warp: rows r0 = lane/4 and r1 = r0 + 8 of a 16-row tile.
struct SoftmaxState {
  float m0, m1, l0, l1;
};

// One 16-token page: S = Q·Kᵀ (16x16), mask, online softmax, O += P·V.
// k_smem / v_smem: shared addresses of the page's K and V tiles, each two 2 KB boxes
// ([d half][token][64 bf16], 128-byte swizzle). Row r may attend tokens in [lo_r, hi_r).
template <bool KV8>
__device__ __forceinline__ void attend_page(const uint32_t (&qf)[8][4], uint32_t k_smem, uint32_t v_smem,
                                            int tok_base, int lo0, int hi0, int lo1, int hi1, float scale_log2,
                                            float (&o)[16][4], SoftmaxState& st) {
  const int lane = threadIdx.x & 31;
  float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  if constexpr (KV8) {
    // K tile: [16 tokens][128 bytes]; one x4 load = tokens 0-7 / 8-15 x feature blocks 2i, 2i+1
    const int tok = (lane & 7) + ((lane >> 4) << 3);
    const int csel = (lane >> 3) & 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int chunk = 2 * i + csel;
      const uint32_t addr = k_smem + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(addr, b0, b1, b2, b3);
      mma_f16_16816(s[0], qf[2 * i], e4m3x2_to_f16x2(b0), e4m3x2_to_f16x2(b0 >> 16));
      mma_f16_16816(s[0], qf[2 * i + 1], e4m3x2_to_f16x2(b1), e4m3x2_to_f16x2(b1 >> 16));
      mma_f16_16816(s[1], qf[2 * i], e4m3x2_to_f16x2(b2), e4m3x2_to_f16x2(b2 >> 16));
      mma_f16_16816(s[1], qf[2 * i + 1], e4m3x2_to_f16x2(b3), e4m3x2_to_f16x2(b3 >> 16));
    }
  } else {
    const int tok = (lane & 7) + ((lane >> 4) << 3);
    const int csel = (lane >> 3) & 1;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int chunk = (ks & 3) * 2 + csel;
      const uint32_t addr = k_smem + (ks >> 2) * 2048 + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(addr, b0, b1, b2, b3);
      mma_bf16_16816(s[0], qf[ks], b0, b1);
      mma_bf16_16816(s[1], qf[ks], b2, b3);
    }
  }
  // mask + scale (log2 domain); pages that every row of the warp may attend in full skip the mask tests
  float mx0 = -INFINITY, mx1 = -INFINITY;
  const bool whole = __all_sync(0xffffffffu, tok_base >= lo0 && tok_base >= lo1 && tok_base + kPage <= hi0 &&
                                                 tok_base + kPage <= hi1);
  if (whole) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s[nt][e] *= scale_log2;
        s[nt][2 + e] *= scale_log2;
        mx0 = fmaxf(mx0, s[nt][e]);
        mx1 = fmaxf(mx1, s[nt][2 + e]);
      }
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = tok_base + nt * 8 + (lane & 3) * 2 + e;
        float v0 = s[nt][e] * scale_log2, v1 = s[nt][2 + e] * scale_log2;
        if (t < lo0 || t >= hi0) v0 = -INFINITY;
        if (t < lo1 || t >= hi1) v1 = -INFINITY;
        s[nt][e] = v0;
        s[nt][2 + e] = v1;
        mx0 = fmaxf(mx0, v0);
        mx1 = fmaxf(mx1, v1);
      }
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m0, mx0), mn1 = fmaxf(st.m1, mx1);
  const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
  const float corr0 = exp2f(st.m0 - ms0), corr1 = exp2f(st.m1 - ms1);  // exp2(-inf) = 0 on first use
  // in steady state the running maxima rarely move: then every correction factor is exactly 1 and the 64
  // multiplies on the output accumulators can be skipped (warp-uniform decision)
  const bool rescale = __any_sync(0xffffffffu, corr0 != 1.f || corr1 != 1.f);
  st.m0 = mn0;
  st.m1 = mn1;
  float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      s[nt][e] = exp2f(s[nt][e] - ms0);
      s[nt][2 + e] = exp2f(s[nt][2 + e] - ms1);
      rs0 += s[nt][e];
      rs1 += s[nt][2 + e];
    }
  }
  rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
  rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
  rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
  rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
  st.l0 = st.l0 * corr0 + rs0;
  st.l1 = st.l1 * corr1 + rs1;
  uint32_t pf[4];
  if constexpr (KV8) {
    pf[0] = pack_f16x2(s[0][0], s[0][1]);
    pf[1] = pack_f16x2(s[0][2], s[0][3]);
    pf[2] = pack_f16x2(s[1][0], s[1][1]);
    pf[3] = pack_f16x2(s[1][2], s[1][3]);
  } else {
    pf[0] = pack_bf16x2(s[0][0], s[0][1]);
    pf[1] = pack_bf16x2(s[0][2], s[0][3]);
    pf[2] = pack_bf16x2(s[1][0], s[1][1]);
    pf[3] = pack_bf16x2(s[1][2], s[1][3]);
  }
  if constexpr (KV8) {
    // V tile: [16 tokens][128 bytes]; a transposed 8x8 b16 matrix hands thread (g, t) the bytes
    // {tok 2t: features 2g, 2g+1 | tok 2t+1: features 2g, 2g+1} of a 16-feature block: bytes 0,2 are the even-feature
    // B fragment, bytes 1,3 the odd one. One x4 load = tokens 0-7 / 8-15 x blocks 2i, 2i+1.
    const int tok = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int csel = lane >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int chunk = 2 * i + csel;
      const uint32_t addr = v_smem + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t r0, r1, r2, r3;   // (tok 0-7, blk 2i), (tok 8-15, blk 2i), (tok 0-7, blk 2i+1), (tok 8-15, blk 2i+1)
      ldsm_x4_t(addr, r0, r1, r2, r3);
      if (rescale) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) o[4 * i + q4][e] *= (e < 2) ? corr0 : corr1;
        }
      }
      mma_f16_16816(o[4 * i + 0], pf, e4m3x2_to_f16x2(__byte_perm(r0, 0u, 0x4420)), e4m3x2_to_f16x2(__byte_perm(r1, 0u, 0x4420)));
      mma_f16_16816(o[4 * i + 1], pf, e4m3x2_to_f16x2(__byte_perm(r0, 0u, 0x4431)), e4m3x2_to_f16x2(__byte_perm(r1, 0u, 0x4431)));
      mma_f16_16816(o[4 * i + 2], pf, e4m3x2_to_f16x2(__byte_perm(r2, 0u, 0x4420)), e4m3x2_to_f16x2(__byte_perm(r3, 0u, 0x4420)));
      mma_f16_16816(o[4 * i + 3], pf, e4m3x2_to_f16x2(__byte_perm(r2, 0u, 0x4431)), e4m3x2_to_f16x2(__byte_perm(r3, 0u, 0x4431)));
    }
  } else {
    const int tok = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int csel = lane >> 4;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int chunk = (j * 2 + csel) & 7;
      const int box = (j * 2) >> 3;
      const uint32_t addr = v_smem + box * 2048 + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(addr, b0, b1, b2, b3);
      if (rescale) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[2 * j][e] *= (e < 2) ? corr0 : corr1;
          o[2 * j + 1][e] *= (e < 2) ? corr0 : corr1;
        }
      }
      mma_bf16_16816(o[2 * j], pf, b0, b1);
      mma_bf16_16816(o[2 * j + 1], pf, b2, b3);
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Decode with the roles of the operands swapped (bf16 pages): S^T = K Q^T and O^T = V^T P^T. The 16 tokens of a page
// are the M rows of the MMA tile and the query heads of the group (at most 8) are its 8 columns, so a page costs 8 + 8
// MMAs instead of 16 + 16, four exponentials per thread instead of eight, and the output accumulators are 32 registers
// instead of 64. (With the queries as rows, a group of 4 heads fills 4 of 16 rows and the kernel is bound by its own
// instruction stream, not by HBM, whenever few warps share an SM: one KV head per rank under tensor parallelism.)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// B fragments of Q^T: thread (g = lane / 4, t = lane % 4) holds Q[head g][16 ks + 2t, +1] and [.. + 8 + 2t, +1].
__device__ __forceinline__ void load_qT_frags(const __nv_bfloat16* qb, int group, uint32_t (&qt)[8][2]) {
  const int g = (threadIdx.x & 31) >> 2, t = threadIdx.x & 3;
  const __nv_bfloat16* row = qb + g * kHD;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int c = ks * 16 + t * 2;
    qt[ks][0] = g < group ? *reinterpret_cast<const uint32_t*>(row + c) : 0u;
    qt[ks][1] = g < group ? *reinterpret_cast<const uint32_t*>(row + c + 8) : 0u;
  }
}
// Softmax state per thread: the two query heads 2t and 2t + 1. The maxima are the same in the eight threads that share
// t; the sums are partial (this thread's tokens) until `softmax_t_finish`.
struct SoftmaxStateT {
  float mA, mB, lA, lB;
};
__device__ __forceinline__ void softmax_t_finish(SoftmaxStateT& st) {
#pragma unroll
  for (int d = 4; d <= 16; d <<= 1) {
    st.lA += __shfl_xor_sync(0xffffffffu, st.lA, d);
    st.lB += __shfl_xor_sync(0xffffffffu, st.lB, d);
  }
}
// One page: tokens [tok_base, tok_base + 16) of which [lo, hi) may be attended (the same range for every head).
__device__ __forceinline__ void attend_page_t(const uint32_t (&qt)[8][2], uint32_t k_smem, uint32_t v_smem, int tok_base,
                                              int lo, int hi, float scale_log2, float (&o)[8][4], SoftmaxStateT& st) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};   // two accumulation chains over the 8 k-steps
  {
    // A = K: matrices (tokens 0-7 | 8-15) x (chunk 2 ks | 2 ks + 1)
    const int tok = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int csel = lane >> 4;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int chunk = (ks & 3) * 2 + csel;
      const uint32_t addr = k_smem + (ks >> 2) * 2048 + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t a[4];
      ldsm_x4(addr, a[0], a[1], a[2], a[3]);
      if (ks & 1) mma_bf16_16816(sb, a, qt[ks][0], qt[ks][1]);
      else mma_bf16_16816(sa, a, qt[ks][0], qt[ks][1]);
    }
  }
  // c0: (token g, head 2t)  c1: (token g, head 2t + 1)  c2, c3: token g + 8
  float s0 = (sa[0] + sb[0]) * scale_log2, s1 = (sa[1] + sb[1]) * scale_log2;
  float s2 = (sa[2] + sb[2]) * scale_log2, s3 = (sa[3] + sb[3]) * scale_log2;
  const int t0 = tok_base + g, t1 = t0 + 8;
  if (t0 < lo || t0 >= hi) s0 = s1 = -INFINITY;
  if (t1 < lo || t1 >= hi) s2 = s3 = -INFINITY;
  float mxA = fmaxf(s0, s2), mxB = fmaxf(s1, s3);
#pragma unroll
  for (int d = 4; d <= 16; d <<= 1) {
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, d));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, d));
  }
  const float mnA = fmaxf(st.mA, mxA), mnB = fmaxf(st.mB, mxB);
  const float msA = (mnA == -INFINITY) ? 0.f : mnA, msB = (mnB == -INFINITY) ? 0.f : mnB;
  const float corrA = exp2f(st.mA - msA), corrB = exp2f(st.mB - msB);
  const bool rescale = __any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f);
  st.mA = mnA;
  st.mB = mnB;
  s0 = exp2f(s0 - msA);
  s1 = exp2f(s1 - msB);
  s2 = exp2f(s2 - msA);
  s3 = exp2f(s3 - msB);
  // the row sums stay per thread (its own two tokens of every page): the correction factors are the same in the eight
  // threads of a head pair, so the sum over those threads can wait until the last page
  st.lA = st.lA * corrA + (s0 + s2);
  st.lB = st.lB * corrB + (s1 + s3);
  // P^T as the B operand (k = token, n = head): the accumulator layout transposed 8 x 8 at a time
  const uint32_t pb0 = movmatrix_trans(pack_bf16x2(s0, s1));
  const uint32_t pb1 = movmatrix_trans(pack_bf16x2(s2, s3));
  {
    // A = V^T: transposed loads of (tokens 0-7 | 8-15) x (chunk 2 mt | 2 mt + 1)
    const int tok = (lane & 7) + ((lane >> 4) << 3);
    const int csel = (lane >> 3) & 1;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int chunk = (mt & 3) * 2 + csel;
      const uint32_t addr = v_smem + (mt >> 2) * 2048 + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t a[4];
      ldsm_x4_t(addr, a[0], a[1], a[2], a[3]);
      if (rescale) {
        o[mt][0] *= corrA;
        o[mt][1] *= corrB;
        o[mt][2] *= corrA;
        o[mt][3] *= corrB;
      }
      mma_bf16_16816(o[mt], a, pb0, pb1);
    }
  }
}

// The same for fp8 (e4m3) pages, on f16 MMAs. A 16-byte shared-memory chunk holds 16 features, so ldmatrix hands a thread
// four consecutive features (4t .. 4t + 3) of a token: the contraction index of the S^T product is permuted inside each
// 16-feature block (MMA k = 2t, 2t + 1 <-> features 4t, 4t + 1; k = 2t + 8, 2t + 9 <-> features 4t + 2, 4t + 3) and the
// Q^T fragments are loaded in the same order. A transposed 8 x 8 b16 matrix of V hands a thread the bytes {token 2t:
// features 2g, 2g + 1 | token 2t + 1: features 2g, 2g + 1}: bytes 0, 2 are an A fragment of the even features, bytes
// 1, 3 of the odd ones, so a 32-feature span gives two MMA row tiles: rows g / g + 8 of tile 2i + e are the features
// 32 i + 2g + e and 32 i + 16 + 2g + e.
__device__ __forceinline__ void load_qT_frags8(const __nv_bfloat16* qb, int group, uint32_t (&qt)[8][2]) {
  const int g = (threadIdx.x & 31) >> 2, t = threadIdx.x & 3;
  const __nv_bfloat16* row = qb + g * kHD;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint2 v = g < group ? *reinterpret_cast<const uint2*>(row + ks * 16 + t * 4) : make_uint2(0u, 0u);
    qt[ks][0] = bf16x2_to_f16x2(v.x);
    qt[ks][1] = bf16x2_to_f16x2(v.y);
  }
}
// Feature of accumulator register pair (c0, c1 | c2, c3) of row tile `mt` in the fp8 form.
__device__ __forceinline__ int out_feature_t8(int mt, int half) {
  const int g = (threadIdx.x & 31) >> 2;
  return 32 * (mt >> 1) + 16 * half + 2 * g + (mt & 1);
}
__device__ __forceinline__ void attend_page_t8(const uint32_t (&qt)[8][2], uint32_t k_smem, uint32_t v_smem, int tok_base,
                                               int lo, int hi, float scale_log2, float (&o)[8][4], SoftmaxStateT& st) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
  {
    const int tok = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int csel = lane >> 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {      // chunks 2i and 2i + 1 = k-steps 2i and 2i + 1
      const int chunk = 2 * i + csel;
      const uint32_t addr = k_smem + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t r0, r1, r2, r3;        // (tokens 0-7, chunk 2i) (tokens 8-15, chunk 2i) (0-7, 2i + 1) (8-15, 2i + 1)
      ldsm_x4(addr, r0, r1, r2, r3);
      const uint32_t a0[4] = {e4m3x2_to_f16x2(r0), e4m3x2_to_f16x2(r1), e4m3x2_to_f16x2(r0 >> 16), e4m3x2_to_f16x2(r1 >> 16)};
      const uint32_t a1[4] = {e4m3x2_to_f16x2(r2), e4m3x2_to_f16x2(r3), e4m3x2_to_f16x2(r2 >> 16), e4m3x2_to_f16x2(r3 >> 16)};
      mma_f16_16816(sa, a0, qt[2 * i][0], qt[2 * i][1]);
      mma_f16_16816(sb, a1, qt[2 * i + 1][0], qt[2 * i + 1][1]);
    }
  }
  float s0 = (sa[0] + sb[0]) * scale_log2, s1 = (sa[1] + sb[1]) * scale_log2;
  float s2 = (sa[2] + sb[2]) * scale_log2, s3 = (sa[3] + sb[3]) * scale_log2;
  const int t0 = tok_base + g, t1 = t0 + 8;
  if (t0 < lo || t0 >= hi) s0 = s1 = -INFINITY;
  if (t1 < lo || t1 >= hi) s2 = s3 = -INFINITY;
  float mxA = fmaxf(s0, s2), mxB = fmaxf(s1, s3);
#pragma unroll
  for (int d = 4; d <= 16; d <<= 1) {
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, d));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, d));
  }
  const float mnA = fmaxf(st.mA, mxA), mnB = fmaxf(st.mB, mxB);
  const float msA = (mnA == -INFINITY) ? 0.f : mnA, msB = (mnB == -INFINITY) ? 0.f : mnB;
  const float corrA = exp2f(st.mA - msA), corrB = exp2f(st.mB - msB);
  const bool rescale = __any_sync(0xffffffffu, corrA != 1.f || corrB != 1.f);
  st.mA = mnA;
  st.mB = mnB;
  s0 = exp2f(s0 - msA);
  s1 = exp2f(s1 - msB);
  s2 = exp2f(s2 - msA);
  s3 = exp2f(s3 - msB);
  st.lA = st.lA * corrA + (s0 + s2);
  st.lB = st.lB * corrB + (s1 + s3);
  const uint32_t pb0 = movmatrix_trans(pack_f16x2(s0, s1));
  const uint32_t pb1 = movmatrix_trans(pack_f16x2(s2, s3));
  {
    const int tok = (lane & 7) + ((lane >> 4) << 3);
    const int csel = (lane >> 3) & 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int chunk = 2 * i + csel;
      const uint32_t addr = v_smem + tok * 128 + ((chunk ^ (tok & 7)) << 4);
      uint32_t r0, r1, r2, r3;        // (tokens 0-7, chunk 2i) (0-7, 2i + 1) (8-15, 2i) (8-15, 2i + 1)
      ldsm_x4_t(addr, r0, r1, r2, r3);
      if (rescale) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          o[2 * i + e][0] *= corrA;
          o[2 * i + e][1] *= corrB;
          o[2 * i + e][2] *= corrA;
          o[2 * i + e][3] *= corrB;
        }
      }
      const uint32_t ae[4] = {e4m3x2_to_f16x2(__byte_perm(r0, 0u, 0x4420)), e4m3x2_to_f16x2(__byte_perm(r1, 0u, 0x4420)),
                              e4m3x2_to_f16x2(__byte_perm(r2, 0u, 0x4420)), e4m3x2_to_f16x2(__byte_perm(r3, 0u, 0x4420))};
      const uint32_t ao[4] = {e4m3x2_to_f16x2(__byte_perm(r0, 0u, 0x4431)), e4m3x2_to_f16x2(__byte_perm(r1, 0u, 0x4431)),
                              e4m3x2_to_f16x2(__byte_perm(r2, 0u, 0x4431)), e4m3x2_to_f16x2(__byte_perm(r3, 0u, 0x4431))};
      mma_f16_16816(o[2 * i], ae, pb0, pb1);
      mma_f16_16816(o[2 * i + 1], ao, pb0, pb1);
    }
  }
}

template <bool KV8>
__device__ __forceinline__ void load_page_kv(const CUtensorMap* tmap, uint8_t* dst, uint64_t* bar, int page,
                                             int n_kv_heads, int kvh) {
  const int krow = ((page * 2 + 0) * n_kv_heads + kvh) * kPage;
  const int vrow = ((page * 2 + 1) * n_kv_heads + kvh) * kPage;
  mbar_expect_tx(bar, 2 * KvFmt<KV8>::kBytes);
  if constexpr (KV8) {   // one 16 x 128-byte box per tile
    tma_load_2d(dst, tmap, bar, 0, krow);
    tma_load_2d(dst + 2048, tmap, bar, 0, vrow);
  } else {
    tma_load_2d(dst, tmap, bar, 0, krow);
    tma_load_2d(dst + 2048, tmap, bar, 64, krow);
    tma_load_2d(dst + 4096, tmap, bar, 0, vrow);
    tma_load_2d(dst + 6144, tmap, bar, 64, vrow);
  }
}

// ---------------------------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------------------------
struct DecodeParams {
  const __nv_bfloat16* q;  // [B, Hq, 128]
  __nv_bfloat16* out;      // [B, Hq, 128]
  const int* block_tables;  // [B, max_blocks]
  const int* ctx_lens;      // [B] tokens in the cache including the one just written; <= 0 = empty slot
  int max_blocks;
  int n_q_heads, n_kv_heads, group;
  float scale_log2;
  int pages_per_split, max_splits;
  float* part_o;    // [B, Hq, max_splits, 128]
  float* part_lse;  // [B, Hq, max_splits]
  int* counters;    // [B, Hkv], zero before the first launch; the kernel leaves them zero
  int num_pages;
  int window;          // 0 = full attention
  const float* sinks;  // [Hq] learnable sink logits or null
  float v_scale;       // fp8 cache: value = stored * scale (the K scale is folded into scale_log2)
  int* err;
};

constexpr int kDecWarps = 4;
constexpr int kDecStages = 3;
constexpr int kDecSmem = kDecWarps * kDecStages * 2 * kPageBytes + 1024 + 1024;
// fp8 pages: half the ring (still larger than the 33 KB the cross-warp merge needs), so three CTAs fit per SM; the
// extra warps hide the latency of the per-fragment conversions
constexpr int kDecSmem8 = kDecWarps * kDecStages * 2 * (kPageBytes / 2) + 1024 + 1024;

template <bool KV8>
__global__ void __launch_bounds__(kDecWarps * 32, KV8 ? 3 : 2)
paged_decode_kernel(const __grid_constant__ CUtensorMap tmap_kv, const DecodeParams p) {
  constexpr int kTile = KvFmt<KV8>::kBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDecWarps * kDecStages * 2 * kTile);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kDecWarps * kDecStages);
  int* is_last = const_cast<int*>(abort_flag) + 1;

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();                // q and the KV rows of this step come from the kernel before this one
  pdl_launch_dependents();
  int ctx = p.ctx_lens[b];
  if (ctx <= 0) return;
  if (ctx > p.max_blocks * kPage) {   // a context longer than the block table: report it and attend what the table covers
    if (p.err && threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_ARG);
    ctx = p.max_blocks * kPage;
  }
  const int n_pages = (ctx + kPage - 1) / kPage;
  const int first_tok = (p.window > 0 && ctx > p.window) ? ctx - p.window : 0;
  const int first_page = first_tok / kPage;
  // never more splits than the scratch was sized for: widen the split when the context is long
  const int span = n_pages - first_page;
  const int pps = max(p.pages_per_split, (span + p.max_splits - 1) / p.max_splits);
  const int n_splits = (span + pps - 1) / pps;
  if (split >= n_splits) return;
  const int p0 = first_page + split * pps;
  const int p1 = min(p0 + pps, n_pages);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kDecWarps * kDecStages; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_kv);
  }
  __syncthreads();

  // bf16 pages with at most 8 heads per group take the swapped form (tokens as MMA rows, heads as columns); fp8
  // pages and larger groups keep the heads as rows
  constexpr bool kSwapOk = true;
  const bool swapped = kSwapOk && p.group <= 8;
  // Q fragments: rows = the `group` q heads of this kv head (rows >= group are zero)
  uint32_t qf[8][4];
  [[maybe_unused]] uint32_t qt[8][2];
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    const __nv_bfloat16* qb = p.q + (static_cast<long long>(b) * p.n_q_heads + kvh * p.group) * kHD;
    if (swapped) {
      if constexpr (KV8) load_qT_frags8(qb, p.group, qt);
      else load_qT_frags(qb, p.group, qt);
    } else {
      load_q_frags<KV8>(qb + r0 * kHD, qb + r1 * kHD, r0 < p.group, r1 < p.group, qf);
    }
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  SoftmaxState st{-INFINITY, -INFINITY, 0.f, 0.f};
  [[maybe_unused]] SoftmaxStateT stt{-INFINITY, -INFINITY, 0.f, 0.f};

  uint8_t* my_ring = smem + warp * kDecStages * 2 * kTile;
  uint64_t* my_bars = bars + warp * kDecStages;
  const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
  const int n_my = (p1 - p0 - warp + kDecWarps - 1) / kDecWarps;  // pages p0+warp, p0+warp+4, ...

  // The page ids of this warp's pages are fetched 32 at a time, one per lane, ahead of their use: a load of the block
  // table in front of every TMA issue would put an L2 round trip into each page's critical path (at one KV head per
  // rank, with few warps per SM to hide it, that round trip was most of the kernel's time).
  auto fetch_ids = [&](int base) {
    const int i = base + lane;
    int page = 0;
    if (i < n_my) {
      page = bt[p0 + warp + i * kDecWarps];
      if (page < 0 || page >= p.num_pages) {
        if (p.err) atomicCAS(p.err, 0, ERR_BAD_PAGE);
        page = 0;
      }
    }
    return page;
  };
  int ids = fetch_ids(0);        // pages [0, 32) of this warp
  int ids_next = 0;              // pages [32 * c + 32, 32 * c + 64): fetched one chunk ahead
  if (n_my > 32) ids_next = fetch_ids(32);
  auto issue = [&](int i, int page) {   // lane 0 only
    const int stg = i % kDecStages;
    load_page_kv<KV8>(&tmap_kv, my_ring + stg * 2 * kTile, &my_bars[stg], page, p.n_kv_heads, kvh);
  };
  for (int i = 0; i < n_my && i < kDecStages; ++i) {
    const int page = __shfl_sync(0xffffffffu, ids, i);
    if (lane == 0) issue(i, page);
  }
  __syncwarp();
  for (int i = 0; i < n_my; ++i) {
    const int stg = i % kDecStages;
    // warp-uniform decision: the page body uses warp-synchronous instructions
    const bool got = mbar_wait(&my_bars[stg], (i / kDecStages) & 1, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL);
    if (!__all_sync(0xffffffffu, got)) break;
    const uint32_t kaddr = smem_u32(my_ring + stg * 2 * kTile);
    const int tok_base = (p0 + warp + i * kDecWarps) * kPage;
    if (swapped) {
      if constexpr (KV8)
        attend_page_t8(qt, kaddr, kaddr + kTile, tok_base, first_tok, ctx, p.scale_log2,
                       *reinterpret_cast<float(*)[8][4]>(&o[0][0]), stt);
      else
        attend_page_t(qt, kaddr, kaddr + kTile, tok_base, first_tok, ctx, p.scale_log2,
                      *reinterpret_cast<float(*)[8][4]>(&o[0][0]), stt);
    } else {
      attend_page<KV8>(qf, kaddr, kaddr + kTile, tok_base, first_tok, ctx, first_tok, ctx, p.scale_log2, o, st);
    }
    __syncwarp();
    const int nxt = i + kDecStages;
    if ((nxt & 31) == 0 && nxt < n_my) {   // the next issue opens a new chunk of 32 page ids
      ids = ids_next;
      if (nxt + 32 < n_my) ids_next = fetch_ids(nxt + 32);
    }
    if (nxt < n_my) {
      const int page = __shfl_sync(0xffffffffu, ids, nxt & 31);
      if (lane == 0) {
        fence_proxy_async_smem();
        issue(nxt, page);
      }
    }
  }
  // every issued copy has been waited for above (or the wait was abandoned after the limit)
  __syncthreads();

  // cross-warp merge through shared memory (the rings are idle now)
  float* mo = reinterpret_cast<float*>(smem);            // [warp][16][128]
  float* mml = mo + kDecWarps * 16 * kHD;                // [warp][16][2]
  if (swapped) {
    // swapped form: o[mt] = (feature 16 mt + g | + 8, head 2t | 2t + 1)
    const int g = lane >> 2, t = lane & 3;
    if constexpr (kSwapOk) softmax_t_finish(stt);
    float* wA = mo + (warp * 16 + 2 * t) * kHD;
    float* wB = wA + kHD;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int d0 = KV8 ? out_feature_t8(mt, 0) : mt * 16 + g;
      const int d1 = KV8 ? out_feature_t8(mt, 1) : mt * 16 + g + 8;
      wA[d0] = o[mt][0];
      wB[d0] = o[mt][1];
      wA[d1] = o[mt][2];
      wB[d1] = o[mt][3];
    }
    if (g == 0) {
      mml[(warp * 16 + 2 * t) * 2 + 0] = stt.mA;
      mml[(warp * 16 + 2 * t) * 2 + 1] = stt.lA;
      mml[(warp * 16 + 2 * t + 1) * 2 + 0] = stt.mB;
      mml[(warp * 16 + 2 * t + 1) * 2 + 1] = stt.lB;
    }
  } else {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int dt = 0; dt < 16; ++dt) {
      const int c0 = out_feature<KV8>(dt, 0), c1 = out_feature<KV8>(dt, 1);
      float* w0 = mo + (warp * 16 + r0) * kHD;
      float* w1 = mo + (warp * 16 + r1) * kHD;
      w0[c0] = o[dt][0];
      w0[c1] = o[dt][1];
      w1[c0] = o[dt][2];
      w1[c1] = o[dt][3];
    }
    if ((lane & 3) == 0) {
      mml[(warp * 16 + r0) * 2 + 0] = st.m0;
      mml[(warp * 16 + r0) * 2 + 1] = st.l0;
      mml[(warp * 16 + r1) * 2 + 0] = st.m1;
      mml[(warp * 16 + r1) * 2 + 1] = st.l1;
    }
  }
  __syncthreads();
  const int d = threadIdx.x;  // 128 threads <-> 128 features
  const bool single = (n_splits == 1);
  for (int r = 0; r < p.group; ++r) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, mml[(w * 16 + r) * 2]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = mml[(w * 16 + r) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += mml[(w * 16 + r) * 2 + 1] * f;
      acc += mo[(w * 16 + r) * kHD + d] * f;
    }
    const int qh = kvh * p.group + r;
    if (single) {
      if (p.sinks) L += exp2f(p.sinks[qh] * 1.4426950408889634f - M);
      p.out[(static_cast<long long>(b) * p.n_q_heads + qh) * kHD + d] = __float2bfloat16_rn(acc / L * (KV8 ? p.v_scale : 1.f));
    } else {
      const long long pi = (static_cast<long long>(b) * p.n_q_heads + qh) * p.max_splits + split;
      p.part_o[pi * kHD + d] = acc / L * (KV8 ? p.v_scale : 1.f);
      if (d == 0) p.part_lse[pi] = M + log2f(L);
    }
  }
  if (single) return;

  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&p.counters[b * p.n_kv_heads + kvh], 1);
    *is_last = (ticket == n_splits - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!*is_last) return;
  __threadfence();
  for (int r = 0; r < p.group; ++r) {
    const int qh = kvh * p.group + r;
    const long long pb = (static_cast<long long>(b) * p.n_q_heads + qh) * p.max_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, __ldcg(&p.part_lse[pb + s]));
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float f = exp2f(__ldcg(&p.part_lse[pb + s]) - M);
      L += f;
      acc += __ldcg(&p.part_o[(pb + s) * kHD + d]) * f;
    }
    if (p.sinks) L += exp2f(p.sinks[qh] * 1.4426950408889634f - M);
    p.out[(static_cast<long long>(b) * p.n_q_heads + qh) * kHD + d] = __float2bfloat16_rn(acc / L);
  }
  if (threadIdx.x == 0) p.counters[b * p.n_kv_heads + kvh] = 0;
}

// ---------------------------------------------------------------------------------------------
// prefill (varlen, causal, chunk-aware)
// ---------------------------------------------------------------------------------------------
struct PrefillParams {
  const __nv_bfloat16* q;  // [T, Hq, 128] flat tokens of every sequence in the batch
  __nv_bfloat16* out;      // [T, Hq, 128]
  const int* q_start;      // [S] first flat token of sequence i
  const int* q_len;        // [S] query tokens of sequence i in this step
  const int* ctx_lens;     // [S] KV tokens after this step (queries are the last q_len of them)
  const int* block_tables;  // [S, max_blocks]
  int max_blocks;
  int n_q_heads, n_kv_heads, group;
  float scale_log2;
  int num_pages;
  int window;
  int causal;  // 0 = bidirectional over [0, ctx)
  const float* sinks;
  float v_scale;   // fp8 cache: value = stored * scale (the K scale is folded into scale_log2)
  int* err;
};

constexpr int kPfWarps = 4;
constexpr int kPfRows = kPfWarps * 16;  // 64 query rows per CTA
constexpr int kPfBlockPages = 4;        // 64 KV tokens per stage
constexpr int kPfStages = 2;
constexpr int kPfStageBytes = kPfBlockPages * 2 * kPageBytes;  // 32 KB (the fp8 variant fills half of it)
constexpr int kPfSmem = kPfStages * kPfStageBytes + 1024 + 1024;

template <bool KV8>
__global__ void __launch_bounds__(kPfWarps * 32)
paged_prefill_kernel(const __grid_constant__ CUtensorMap tmap_kv, const PrefillParams p) {
  constexpr int kTile = KvFmt<KV8>::kBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPfStages * kPfStageBytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + kPfStages);

  const int qblk = blockIdx.x, qh = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_wait();
  pdl_launch_dependents();
  const int qlen = p.q_len[seq];
  if (qblk * kPfRows >= qlen) return;
  int ctx = p.ctx_lens[seq];
  if (ctx > p.max_blocks * kPage) {   // longer than the block table: report, never index past the table
    if (p.err && threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_ARG);
    ctx = p.max_blocks * kPage;
  }
  const int qstart = p.q_start[seq];
  const int kvh = qh / p.group;
  const int pos0 = ctx - qlen;  // position of query row 0 of this sequence

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kPfStages; ++i) mbar_init(&bars[i], 1);
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_kv);
  }
  __syncthreads();

  const int row0 = qblk * kPfRows + warp * 16 + (lane >> 2), row1 = row0 + 8;
  uint32_t qf[8][4];
  {
    const __nv_bfloat16* q0 = p.q + (static_cast<long long>(qstart + row0) * p.n_q_heads + qh) * kHD;
    const __nv_bfloat16* q1 = p.q + (static_cast<long long>(qstart + row1) * p.n_q_heads + qh) * kHD;
    load_q_frags<KV8>(q0, q1, row0 < qlen, row1 < qlen, qf);
  }
  // allowed token ranges per row
  int hi0, hi1, lo0 = 0, lo1 = 0;
  if (p.causal) {
    hi0 = pos0 + row0 + 1;
    hi1 = pos0 + row1 + 1;
  } else {
    hi0 = hi1 = ctx;
  }
  if (p.window > 0) {
    lo0 = max(0, hi0 - p.window);
    lo1 = max(0, hi1 - p.window);
  }
  if (row0 >= qlen) hi0 = lo0 = 0;
  if (row1 >= qlen) hi1 = lo1 = 0;
  // KV range needed by this CTA
  const int last_row = min(qblk * kPfRows + kPfRows, qlen) - 1;
  const int kv_hi = p.causal ? (pos0 + last_row + 1) : ctx;
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, (p.causal ? pos0 + qblk * kPfRows + 1 : ctx) - p.window);
  const int page_lo = kv_lo / kPage;
  const int page_hi = (kv_hi + kPage - 1) / kPage;
  const int n_blocks = (page_hi - page_lo + kPfBlockPages - 1) / kPfBlockPages;
  const int* bt = p.block_tables + static_cast<long long>(seq) * p.max_blocks;

  auto issue = [&](int blk) {
    const int stg = blk % kPfStages;
    uint8_t* dst = smem + stg * kPfStageBytes;
    const int pg0 = page_lo + blk * kPfBlockPages;
    const int npg = min(kPfBlockPages, page_hi - pg0);
    mbar_expect_tx(&bars[stg], npg * 2 * kTile);
    for (int j = 0; j < npg; ++j) {
      int page = bt[pg0 + j];
      if (page < 0 || page >= p.num_pages) {
        if (p.err) atomicCAS(p.err, 0, ERR_BAD_PAGE);
        page = 0;
      }
      const int krow = ((page * 2 + 0) * p.n_kv_heads + kvh) * kPage;
      const int vrow = ((page * 2 + 1) * p.n_kv_heads + kvh) * kPage;
      uint8_t* d = dst + j * 2 * kTile;
      if constexpr (KV8) {
        tma_load_2d(d, &tmap_kv, &bars[stg], 0, krow);
        tma_load_2d(d + 2048, &tmap_kv, &bars[stg], 0, vrow);
      } else {
        tma_load_2d(d, &tmap_kv, &bars[stg], 0, krow);
        tma_load_2d(d + 2048, &tmap_kv, &bars[stg], 64, krow);
        tma_load_2d(d + 4096, &tmap_kv, &bars[stg], 0, vrow);
        tma_load_2d(d + 6144, &tmap_kv, &bars[stg], 64, vrow);
      }
    }
  };

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  SoftmaxState st{-INFINITY, -INFINITY, 0.f, 0.f};

  if (threadIdx.x == 0) {
    for (int blk = 0; blk < n_blocks && blk < kPfStages; ++blk) issue(blk);
  }
  // rows of this warp need tokens below warp_hi only
  const int warp_last_row = min(qblk * kPfRows + warp * 16 + 15, qlen - 1);
  const int warp_hi = p.causal ? (pos0 + warp_last_row + 1) : ctx;
  for (int blk = 0; blk < n_blocks; ++blk) {
    const int stg = blk % kPfStages;
    // the decision to stop must be CTA-uniform because the loop body contains a block barrier
    const int got = mbar_wait(&bars[stg], (blk / kPfStages) & 1, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL) ? 1 : 0;
    if (!__syncthreads_and(got)) break;
    const int pg0 = page_lo + blk * kPfBlockPages;
    const int npg = min(kPfBlockPages, page_hi - pg0);
    const uint32_t base = smem_u32(smem + stg * kPfStageBytes);
    for (int j = 0; j < npg; ++j) {
      const int tok_base = (pg0 + j) * kPage;
      if (tok_base >= warp_hi) break;  // fully masked for every row of this warp
      attend_page<KV8>(qf, base + j * 2 * kTile, base + j * 2 * kTile + kTile, tok_base, lo0, hi0, lo1, hi1,
                       p.scale_log2, o, st);
    }
    __syncthreads();
    if (threadIdx.x == 0 && blk + kPfStages < n_blocks) {
      fence_proxy_async_smem();
      issue(blk + kPfStages);
    }
  }

  float L0 = st.l0, L1 = st.l1;
  if (p.sinks) {
    const float sk = p.sinks[qh] * 1.4426950408889634f;
    L0 += exp2f(sk - (st.m0 == -INFINITY ? 0.f : st.m0));
    L1 += exp2f(sk - (st.m1 == -INFINITY ? 0.f : st.m1));
  }
  const float vs = KV8 ? p.v_scale : 1.f;
  const float inv0 = L0 > 0.f ? vs / L0 : 0.f, inv1 = L1 > 0.f ? vs / L1 : 0.f;
  __nv_bfloat16* o0 = p.out + (static_cast<long long>(qstart + row0) * p.n_q_heads + qh) * kHD;
  __nv_bfloat16* o1 = p.out + (static_cast<long long>(qstart + row1) * p.n_q_heads + qh) * kHD;
  if constexpr (KV8) {
    // n-tiles 2j / 2j+1 hold the even / odd features of block j: features 16j + 4t .. 4t+3 are
    // (even[0], odd[0], even[1], odd[1])
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = 16 * j + 4 * (lane & 3);
      if (row0 < qlen) {
        uint2 w;
        w.x = pack_bf16x2(o[2 * j][0] * inv0, o[2 * j + 1][0] * inv0);
        w.y = pack_bf16x2(o[2 * j][1] * inv0, o[2 * j + 1][1] * inv0);
        *reinterpret_cast<uint2*>(o0 + c) = w;
      }
      if (row1 < qlen) {
        uint2 w;
        w.x = pack_bf16x2(o[2 * j][2] * inv1, o[2 * j + 1][2] * inv1);
        w.y = pack_bf16x2(o[2 * j][3] * inv1, o[2 * j + 1][3] * inv1);
        *reinterpret_cast<uint2*>(o1 + c) = w;
      }
    }
  } else {
#pragma unroll
    for (int dt = 0; dt < 16; ++dt) {
      const int c = dt * 8 + (lane & 3) * 2;
      if (row0 < qlen) *reinterpret_cast<uint32_t*>(o0 + c) = pack_bf16x2(o[dt][0] * inv0, o[dt][1] * inv0);
      if (row1 < qlen) *reinterpret_cast<uint32_t*>(o1 + c) = pack_bf16x2(o[dt][2] * inv1, o[dt][3] * inv1);
    }
  }
}

static int kv_tmap(CUtensorMap* t, const void* kv_cache, int num_pages, int n_kv_heads, bool fp8 = false) {
  const uint64_t rows = uint64_t(num_pages) * 2 * n_kv_heads * kPage;
  if (fp8) return make_tmap_2d(t, kv_cache, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows, kHD, kHD, kPage, 128);
  return make_tmap_2d(t, kv_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, kHD, kHD, kPage, 64);
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();

// Scratch sizes for the split-KV decode path (floats / ints).
GLLM_API long long gllm_decode_scratch_floats(int batch, int n_q_heads, int max_splits) {
  return static_cast<long long>(batch) * n_q_heads * max_splits * (kHD + 1);
}

template <bool KV8>
static int paged_decode_impl(const void* q, void* out, const void* kv_cache, int num_pages,
                             const int* block_tables, int max_blocks, const int* ctx_lens, int batch,
                             int n_q_heads, int n_kv_heads, float scale, int pages_per_split, int max_splits,
                             float* scratch, int* counters, int window, const float* sinks, float kv_scale,
                             void* stream) {
  if (n_q_heads % n_kv_heads != 0 || n_q_heads / n_kv_heads > 16) {
    set_last_error("paged_decode: group size %d/%d unsupported (must divide, <= 16)", n_q_heads, n_kv_heads);
    return -1;
  }
  if (max_splits > 1 && (!scratch || !counters)) {
    set_last_error("paged_decode: split-KV needs scratch and counters");
    return -1;
  }
  CUtensorMap t;
  if (kv_tmap(&t, kv_cache, num_pages, n_kv_heads, KV8)) return -1;
  DecodeParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.max_blocks = max_blocks;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = n_q_heads / n_kv_heads;
  p.scale_log2 = scale * 1.4426950408889634f * (KV8 ? kv_scale : 1.f);
  p.v_scale = KV8 ? kv_scale : 1.f;
  p.pages_per_split = pages_per_split > 0 ? pages_per_split : (1 << 30);
  p.max_splits = max_splits > 0 ? max_splits : 1;
  p.part_o = scratch;
  p.part_lse = scratch ? scratch + static_cast<long long>(batch) * n_q_heads * p.max_splits * kHD : nullptr;
  p.counters = counters; p.num_pages = num_pages; p.window = window; p.sinks = sinks;
  p.err = gllm_error_word();
  static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the kernel
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(paged_decode_kernel<KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         KV8 ? kDecSmem8 : kDecSmem);
    if (e != cudaSuccess) { set_last_error("paged_decode: %s", cudaGetErrorString(e)); return -1; }
    attr_set[dev & 63] = true;
  }
  dim3 grid(p.max_splits, n_kv_heads, batch);
  cudaError_t e = launch_kernel(paged_decode_kernel<KV8>, grid, dim3(kDecWarps * 32), KV8 ? kDecSmem8 : kDecSmem,
                                (cudaStream_t)stream, true, 0, t, p);
  if (e != cudaSuccess) { (void)cudaGetLastError(); set_last_error("paged_decode launch: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

GLLM_API int gllm_paged_decode(const void* q, void* out, const void* kv_cache, int num_pages,
                               const int* block_tables, int max_blocks, const int* ctx_lens, int batch,
                               int n_q_heads, int n_kv_heads, float scale, int pages_per_split, int max_splits,
                               float* scratch, int* counters, int window, const float* sinks, void* stream) {
  return paged_decode_impl<false>(q, out, kv_cache, num_pages, block_tables, max_blocks, ctx_lens, batch, n_q_heads,
                                  n_kv_heads, scale, pages_per_split, max_splits, scratch, counters, window, sinks,
                                  1.f, stream);
}
// Same kernel over an fp8 (e4m3) cache of the same shape; cached value = stored byte * kv_scale.
GLLM_API int gllm_paged_decode_fp8(const void* q, void* out, const void* kv_cache, int num_pages,
                                   const int* block_tables, int max_blocks, const int* ctx_lens, int batch,
                                   int n_q_heads, int n_kv_heads, float scale, int pages_per_split, int max_splits,
                                   float* scratch, int* counters, int window, const float* sinks, float kv_scale,
                                   void* stream) {
  return paged_decode_impl<true>(q, out, kv_cache, num_pages, block_tables, max_blocks, ctx_lens, batch, n_q_heads,
                                 n_kv_heads, scale, pages_per_split, max_splits, scratch, counters, window, sinks,
                                 kv_scale, stream);
}

template <bool KV8>
static int paged_prefill_impl(const void* q, void* out, const void* kv_cache, int num_pages,
                              const int* block_tables, int max_blocks, const int* q_start, const int* q_len,
                              const int* ctx_lens, int num_seqs, int max_q_len, int n_q_heads, int n_kv_heads,
                              float scale, int causal, int window, const float* sinks, float kv_scale, void* stream) {
  if (n_q_heads % n_kv_heads != 0) {
    set_last_error("paged_prefill: heads %d not divisible by kv heads %d", n_q_heads, n_kv_heads);
    return -1;
  }
  CUtensorMap t;
  if (kv_tmap(&t, kv_cache, num_pages, n_kv_heads, KV8)) return -1;
  PrefillParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_start = q_start; p.q_len = q_len; p.ctx_lens = ctx_lens;
  p.block_tables = block_tables; p.max_blocks = max_blocks;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = n_q_heads / n_kv_heads;
  p.scale_log2 = scale * 1.4426950408889634f * (KV8 ? kv_scale : 1.f);
  p.v_scale = KV8 ? kv_scale : 1.f;
  p.num_pages = num_pages; p.window = window; p.causal = causal; p.sinks = sinks;
  p.err = gllm_error_word();
  static bool attr_set[64] = {};   // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(paged_prefill_kernel<KV8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem);
    if (e != cudaSuccess) { set_last_error("paged_prefill: %s", cudaGetErrorString(e)); return -1; }
    attr_set[dev & 63] = true;
  }
  dim3 grid((max_q_len + kPfRows - 1) / kPfRows, n_q_heads, num_seqs);
  cudaError_t e = launch_kernel(paged_prefill_kernel<KV8>, grid, dim3(kPfWarps * 32), kPfSmem, (cudaStream_t)stream,
                                true, 0, t, p);
  if (e != cudaSuccess) { (void)cudaGetLastError(); set_last_error("paged_prefill launch: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

GLLM_API int gllm_paged_prefill(const void* q, void* out, const void* kv_cache, int num_pages,
                                const int* block_tables, int max_blocks, const int* q_start, const int* q_len,
                                const int* ctx_lens, int num_seqs, int max_q_len, int n_q_heads, int n_kv_heads,
                                float scale, int causal, int window, const float* sinks, void* stream) {
  return paged_prefill_impl<false>(q, out, kv_cache, num_pages, block_tables, max_blocks, q_start, q_len, ctx_lens,
                                   num_seqs, max_q_len, n_q_heads, n_kv_heads, scale, causal, window, sinks, 1.f, stream);
}
GLLM_API int gllm_paged_prefill_fp8(const void* q, void* out, const void* kv_cache, int num_pages,
                                    const int* block_tables, int max_blocks, const int* q_start, const int* q_len,
                                    const int* ctx_lens, int num_seqs, int max_q_len, int n_q_heads, int n_kv_heads,
                                    float scale, int causal, int window, const float* sinks, float kv_scale,
                                    void* stream) {
  return paged_prefill_impl<true>(q, out, kv_cache, num_pages, block_tables, max_blocks, q_start, q_len, ctx_lens,
                                  num_seqs, max_q_len, n_q_heads, n_kv_heads, scale, causal, window, sinks, kv_scale,
                                  stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of gllm_paged_decode (declared and documented in gllm_noalloc.h).
//
// Who needs it: callers that cannot allocate device memory when they need attention — under a fixed
// start-up memory plan, on a thread where the owning framework forbids allocator calls, or in a
// latency-critical loop. The split-KV scratch is the
// static array below; the caller still owns q, out, the KV cache and the index tensors.
// ---------------------------------------------------------------------------------------------
#include <mutex>

#include "gllm_noalloc.h"

namespace gllm {
// partial outputs [units][128] followed by their log-sum-exps [units]; units = batch * n_q * max_splits
static __device__ __align__(256) float g_noalloc_scratch[GLLM_NOALLOC_MAX_UNITS * (kHD + 1)];
static __device__ __align__(256) int g_noalloc_counters[GLLM_NOALLOC_MAX_COUNTERS];
static __device__ __align__(256) int g_noalloc_err[4];

struct NoAllocDeviceState {
  bool ready = false;
  float* scratch = nullptr;   // device addresses obtained with cudaGetSymbolAddress: in host code the
  int* counters = nullptr;    // array names above are only host-side stand-ins, never device pointers
  int* err = nullptr;
};
static NoAllocDeviceState g_noalloc_state[64];
static std::mutex g_noalloc_mutex;   // the per-device set-up may be reached by several host threads at once

// Resolves (once per device, under the mutex) the device addresses of the static arrays. Returns null on failure.
static NoAllocDeviceState* noalloc_state_for_current_device(const char* who) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_last_error("%s: no current device", who);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDeviceState& st = g_noalloc_state[dev];
  if (!st.ready) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st.scratch), g_noalloc_scratch);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st.counters), g_noalloc_counters);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st.err), g_noalloc_err);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(paged_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmem);
    if (e != cudaSuccess) {
      set_last_error("%s: set-up failed: %s", who, cudaGetErrorString(e));
      return nullptr;
    }
    st.ready = true;
  }
  return &st;
}
}  // namespace gllm

// Status of the allocation-free path on the current device (see gllm_noalloc.h). Copies the 4-byte status word
// to the host on `stream`, waits for that stream, and clears the word when it was non-zero. Allocates nothing.
GLLM_API int gllm_paged_decode_noalloc_status(void* stream) {
  NoAllocDeviceState* st = noalloc_state_for_current_device("paged_decode_noalloc_status");
  if (!st) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int code = 0;
  cudaError_t e = cudaMemcpyAsync(&code, st->err, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && code != 0) e = cudaMemsetAsync(st->err, 0, sizeof(int), s);
  if (e != cudaSuccess) {
    set_last_error("paged_decode_noalloc_status: %s", cudaGetErrorString(e));
    return -1;
  }
  return code;
}

GLLM_API int gllm_paged_decode_noalloc(const void* q, void* out, const void* kv_cache, int num_pages,
                                       const int* block_tables, int max_blocks, const int* ctx_lens, int batch,
                                       int n_q_heads, int n_kv_heads, float scale, int pages_per_split,
                                       int max_splits, int window, const float* sinks, void* stream) {
  if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 ||
      n_q_heads / n_kv_heads > 16) {
    set_last_error("paged_decode_noalloc: bad shape batch %d heads %d/%d", batch, n_q_heads, n_kv_heads);
    return -1;
  }
  if (max_splits < 1) max_splits = 1;
  const long long units = static_cast<long long>(batch) * n_q_heads * max_splits;
  if (units > GLLM_NOALLOC_MAX_UNITS) {
    set_last_error("paged_decode_noalloc: batch*heads*splits = %lld exceeds the built-in scratch (%d); lower "
                   "max_splits or use gllm_paged_decode with caller scratch", units, GLLM_NOALLOC_MAX_UNITS);
    return -1;
  }
  if (static_cast<long long>(batch) * n_kv_heads > GLLM_NOALLOC_MAX_COUNTERS) {
    set_last_error("paged_decode_noalloc: batch*kv_heads = %lld exceeds the built-in counters (%d)",
                   static_cast<long long>(batch) * n_kv_heads, GLLM_NOALLOC_MAX_COUNTERS);
    return -1;
  }
  // one-time set-up for this device (do it before any stream capture): resolve the device addresses
  NoAllocDeviceState* stp = noalloc_state_for_current_device("paged_decode_noalloc");
  if (!stp) return -1;
  NoAllocDeviceState& st = *stp;
  // tensor map built on the stack (the cached encoder used elsewhere grows a host-side table)
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) {
    set_last_error("paged_decode_noalloc: cuTensorMapEncodeTiled is not available from this driver");
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(kv_cache) & 15) != 0) {
    set_last_error("paged_decode_noalloc: kv_cache must be 16-byte aligned");
    return -1;
  }
  CUtensorMap t;
  {
    cuuint64_t gdim[2] = {kHD, static_cast<cuuint64_t>(num_pages) * 2 * n_kv_heads * kPage};
    cuuint64_t gstride[1] = {kHD * 2};
    cuuint32_t box[2] = {64, kPage};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv_cache), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_last_error("paged_decode_noalloc: tensor map encode failed (CUresult %d)", int(r));
      return -1;
    }
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the scratch keeps the last call's contents; only the ticket counters must start at zero
  cudaError_t e = cudaMemsetAsync(st.counters, 0, sizeof(int) * static_cast<size_t>(batch) * n_kv_heads, s);
  if (e != cudaSuccess) {
    set_last_error("paged_decode_noalloc: counter clear failed: %s", cudaGetErrorString(e));
    return -1;
  }
  DecodeParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.block_tables = block_tables; p.ctx_lens = ctx_lens; p.max_blocks = max_blocks;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = n_q_heads / n_kv_heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.pages_per_split = pages_per_split > 0 ? pages_per_split : (1 << 30);
  p.max_splits = max_splits;
  p.part_o = st.scratch;
  p.part_lse = st.scratch + units * kHD;
  p.counters = st.counters; p.num_pages = num_pages; p.window = window; p.sinks = sinks;
  p.err = st.err;
  dim3 grid(max_splits, n_kv_heads, batch);
  paged_decode_kernel<false><<<grid, kDecWarps * 32, kDecSmem, s>>>(t, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("paged_decode_noalloc launch: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
