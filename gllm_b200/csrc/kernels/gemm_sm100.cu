// Persistent warp-specialised tcgen05 GEMM family for sm_100a:  D[M,N] = A[M,K] · B[N,K]ᵀ.
//
// Both operands are K-major (activations row-major, weights in checkpoint [out,in] order), so the
// kernel consumes weights exactly as they sit in the file — the same "trans_b = true" contract
// the reference's graph uses for every linear (src/arch/auto_graph_fragments/build_graph.inc.rs:1618).
//
// One CTA per SM, 256 threads:
//   warp 0      TMA producer: MT x (128 x BK) A tiles + one BN x BK B tile per stage, 128-byte swizzle
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16|32) into TMEM, MT
//               accumulators per B tile so a weight tile fetched once serves up to 256 rows
//   warp 2      TMEM allocator
//   warps 4..7  epilogue: tcgen05.ld -> registers -> fused epilogue -> global
// When two accumulator sets fit in TMEM (2*MT*BN <= 512 columns) they are double-buffered so the
// epilogue of work item i overlaps the main loop of item i+1.
//
// Small-M (decode) shapes have too few output tiles to occupy 148 SMs and are bound by how fast
// one SM can pull bytes into shared memory (about 100 GB/s), so the K dimension is split across
// CTAs. The kernel then has two phases separated by a grid barrier (all CTAs are resident: one per
// SM): phase 1 streams distinct weight slices and dumps fp32 partial tiles to scratch; phase 2 has
// every warp of every CTA sum the partials in split order (deterministic) with coalesced loads and
// apply the same fused epilogue.
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
#include <cuda_fp8.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

extern "C" int gllm_sm_count();

namespace gllm {

enum : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GLU = 2, EPI_QKV = 3 };

// Phase stamps of CTA 0 (SM clocks) exist only in builds with -DGLLM_TRACE (python -m gllm_b200.build --trace).
#ifdef GLLM_TRACE
#define GLLM_TRACE_DECL const bool tracing = p.trace != nullptr && blockIdx.x == 0
#define GLLM_STAMP(cond, slot)                           \
  do {                                                   \
    if (tracing && (cond)) p.trace[slot] = clock64();    \
  } while (0)
#else
#define GLLM_TRACE_DECL
#define GLLM_STAMP(cond, slot) \
  do {                         \
  } while (0)
#endif

constexpr int kBM = 128;
constexpr int kTileKBytes = 128;  // one swizzle row
constexpr int kGemmThreads = 256;
constexpr int kPageTokens = 16;
constexpr int kMaxSplits = 16;
constexpr int kClusterPartStride = 128 + 4;  // floats per row of a parked fp32 tile in shared memory (padded: no bank conflicts)

struct GemmParams {
  int M, N, K;
  int num_m, num_n, num_kb;  // num_m counts MT*128-row super tiles
  int splits;
  float* sk_scratch;        // [split][M][num_n*BN] fp32 partial sums
  unsigned int* sk_barrier;  // {arrival count, generation} of the grid barrier
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
  // block-scaled operands (OPM_MXFP8 / OPM_NVFP4): scale-factor chunks of A and B, and one factor for the whole
  // product (NVFP4's per-tensor scales); out_scale == 0 means 1
  const uint8_t* sfa;
  const uint8_t* sfb;
  float out_scale;
  // GLU
  int glu_act;  // 0 = silu, 1 = gelu_tanh
  // grouped GEMM: 128-row m-block -> group id; B rows of group g start at g * group_rows
  const int* mblk_group;
  int group_rows;
  // QKV epilogue
  int n_q_heads, n_kv_heads;
  __nv_bfloat16* q_out;     // [M, n_q_heads*128]
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
  int kv_fp8;             // 1: kv_cache holds fp8 e4m3 bytes of the same shape, stored = value * kv_inv_scale (saturating)
  float kv_inv_scale;
  // fused all-reduce (row-parallel GEMM across `ar_world` GPUs): every rank stores its bf16 partial
  // tiles in its own symmetric buffer as they retire; after the arrival barrier each rank pulls the
  // sum of all ranks' partials (multimem.ld_reduce through NVSwitch when a multicast mapping exists,
  // else plain peer loads over NVLink) and finishes locally. ar_world == 0 disables it.
  int ar_world;
  __nv_bfloat16* ar_mc_buf;               // multicast address of the partial buffers, or null
  __nv_bfloat16* ar_peer_buf[8];          // unicast addresses (index = rank); [ar_rank] is local
  unsigned long long* ar_mc_counter;      // multicast address of the arrival counter, or null
  unsigned long long* ar_peer_counter[8];
  unsigned long long* ar_state;           // local {expected rank arrivals, launch index, CTA arrivals, expected CTA
                                          // arrivals, expected rank arrivals of the second meeting}
  int ar_rank;
  int ar_two_shot;                        // 1: reduce-scatter + broadcast through the result region at 2 * ar_buf_elems
  long long ar_buf_elems;                 // elements of one partial buffer (two alternate per launch)
  // row scatter (expert-parallel return path): output row m goes to scatter_peer[meta >> 24] + (meta & 0xFFFFFF) * ldo
  // where meta = scatter_meta[m]; a negative meta drops the row. The stores go straight into the token owner's
  // memory over NVLink as each tile retires.
  const int* scatter_meta;
  __nv_bfloat16* scatter_peer[8];
  int park;           // 1: one work item per CTA: the fp32 accumulator tile is parked in shared memory and written out
                      //    by all warps with row-contiguous stores (split-K scratch or the all-reduce buffer)
  int cluster_sk;     // 1: the splits of a tile form a thread-block cluster and reduce through distributed shared memory
  // Push form of the fused all-reduce (ar_push == 1). Rank r owns output rows [r * rows_per, (r + 1) * rows_per),
  // rows_per = ceil(M / world). As a tile retires its bf16 rows are stored straight into the row owner's receive
  // slots [source][local row][column] (peer stores over NVLink, no atomics) and one flag per (source, m tile, n tile)
  // is released with the launch epoch; the owner's warps wait on those flags tile by tile, add the sources in a fixed
  // order, add the residual, and store the finished rows and their row statistics into `out` / `row_ss_out` of EVERY
  // rank (one multimem.st per 16 bytes, or a store per peer): both must lie inside the symmetric region. A last
  // meeting on per-rank "done" words ends the kernel. All regions are offsets from the symmetric base of each rank.
  int ar_push;
  long long ar_recv_off;      // bf16 elements from the base: receive slots
  long long ar_out_off;       // bf16 elements from the base: `out` (== residual) rows
  long long ar_ss_off;        // BYTES from the base: row statistics [M, n_pad / 256] fp32
  long long ar_flag_off;      // BYTES from the base: tile flags (u32)
  long long ar_done_off;      // BYTES from the base: done words (u64 per rank)
  long long ar_flag_cap;      // number of u32 flags at ar_flag_off
  // Low-latency form (ar_ll == 1, decode-sized M): no flags, no fences, no meeting. Every 32-bit word of the receive
  // and result slots holds either the sentinel 0x80008000 (two bf16 negative zeros, which the writers never store:
  // they write +0 instead) or data; a reader polls the data words themselves until none is the sentinel and puts the
  // sentinel back after reading, so the slots clean themselves. Two parity sets of slots alternate between launches.
  // Producers store bf16 partial rows into the owner's receive slots, the owner adds them and stores the finished rows
  // into the result slots of EVERY rank, and every rank copies all rows from its own result slots into `out` (plain
  // local memory) with their row statistics.
  int ar_ll;
  long long ar_ll_recv_off, ar_ll_recv_bytes;   // BYTES from the base / bytes of one parity set of receive slots
  long long ar_ll_res_off, ar_ll_res_bytes;     // same for the result slots ([M][n_pad] bf16)
  int ar_drop_flags;          // test hook: leave the tile flags unset (push) / the tiles unsent (ll): the waits run out
  float softcap;              // EPI_STORE, unsplit launches only: out = softcap * tanh(out / softcap) (0 = off)
  // Grouped GEMMs: rows that exist in every 128-row block (the rest of a block is padding: a block of an expert with
  // 16 routed rows has 112 of them). When given, the producer loads only ceil(rows / 32) * 32 rows of the A tile
  // (32-row boxes through the third tensor map) and the epilogue neither reads nor stores the padding rows.
  const int* mblk_rows;
  // Reduce-scatter output of the low-latency form (ar_rs_only == 1): rank r keeps the finished rows [r * ceil(M / W), ...)
  // in `out` / `residual` / `row_ss_out`, which then are SHARDS indexed by the local row; nothing is broadcast.
  int ar_rs_only;
  // All-gather of the A operand before the main loop (ag_world > 0): every rank holds rows [r * ceil(M / W), ...) of A in
  // `ag_src`; the kernel stores them into every rank's slots (self-validating words as in the low-latency all-reduce:
  // sentinel 0x80008000, two parity sets), copies all rows from its own slots into `ag_dst` (the tensor the A tensor
  // map describes, local memory), meets the other CTAs of the grid and only then starts the A loads. The weight tiles
  // of the first stages are requested before that, so they travel while the rows are exchanged.
  int ag_world, ag_rank;
  const __nv_bfloat16* ag_src; long long ag_src_ld;
  __nv_bfloat16* ag_dst; long long ag_dst_ld;
  char* ag_peer[8]; char* ag_mc;            // symmetric region bases (and the multicast mapping or null)
  long long ag_slot_off, ag_slot_bytes;     // bytes: offset of the slots in the region, size of one parity set
  unsigned long long* ag_state;             // local: [0] launch index (parity)
  float* ag_ss_out;                         // optional [M, K / 256]: sums of squares of the gathered rows per 256 columns
                                            // (the row statistics a fused-norm epilogue of the same GEMM reads)
  unsigned long long wait_ns, peer_wait_ns;   // limits of the bounded waits
  long long* trace;   // debugging aid (GLLM_TRACE builds): CTA 0 writes SM clock stamps of its phases here (9 slots)
  int* err;
};

// Operand modes of the kernel (template parameter OPM; the two first values are what `false` / `true` of the former
// boolean meant):
//   0  bf16 x bf16                      tcgen05.mma.kind::f16
//   1  e4m3 x e4m3, scales in the epilogue (per row / per column)   kind::f8f6f4
//   2  MXFP8: e4m3 x e4m3, one ue8m0 scale per 32 elements along K of both operands   kind::mxf8f6f4.block_scale
//   3  NVFP4: e2m1 x e2m1 (two per byte), one ue4m3 scale per 16 elements             kind::mxf4nvf4.block_scale.scale_vec::4X
// In modes 2 and 3 the scale factors of a (128 rows x one 128-byte K block) piece of an operand are one contiguous
// chunk of global memory in the layout the tensor core wants (see sf_chunk_offset in the host code): the producer
// brings the chunks into the stage with bulk copies, the MMA thread moves them to tensor memory with tcgen05.cp and
// issues the block-scaled MMAs, which multiply every 32- (16-) element slice by its two scales in hardware.
enum : int { OPM_BF16 = 0, OPM_FP8 = 1, OPM_MXFP8 = 2, OPM_NVFP4 = 3 };
constexpr int kSfChunkBytes = 512;   // scale factors of 128 rows x 4 consecutive scale columns

template <int BN, int MT, bool PAIR = false, int OPM = 0>
struct GemmCfg {
  static constexpr bool kBlockScaled = OPM >= OPM_MXFP8;
  static constexpr int kSfChunks = OPM == OPM_MXFP8 ? 1 : (OPM == OPM_NVFP4 ? 4 : 0);   // chunks per 128 rows and stage
  static constexpr int kSfABytes = MT * kSfChunks * kSfChunkBytes;
  static constexpr int kSfBBytes = (BN / 128) * kSfChunks * kSfChunkBytes;
  // PAIR: each CTA of a pair stages its own 128 rows of A and half of the B tile's rows
  static constexpr int kTileBytes = MT * kBM * kTileKBytes + (PAIR ? BN / 2 : BN) * kTileKBytes;
  static constexpr int kTxBytes = kTileBytes + kSfABytes + kSfBBytes;        // bytes that arrive per stage
  static constexpr int kStageBytes = (kTxBytes + 1023) / 1024 * 1024;         // stages stay 1024-byte aligned (swizzle atoms)
  static constexpr int kStages = (196608 / kStageBytes) > 8 ? 8 : (196608 / kStageBytes);
  // tensor-memory columns of the scale factors: two buffers (stage parity) of [A: MT x chunks x 4 | B: BN/128 x chunks x 4]
  static constexpr int kSfColsA = MT * kSfChunks * 4;
  static constexpr int kSfColsB = (BN / 128) * kSfChunks * 4;
  static constexpr int kSfCols = 2 * (kSfColsA + kSfColsB);
  static constexpr int kAccStages = (2 * MT * BN + kSfCols <= 512) ? 2 : 1;
  static_assert(!kBlockScaled || (MT * BN + kSfCols <= 512 && BN % 128 == 0 && !PAIR), "block-scaled tile does not fit tensor memory");
  static constexpr int kCols = kAccStages * MT * BN + kSfCols;
  static constexpr int kTmemCols = kCols <= 32 ? 32 : (kCols <= 64 ? 64 : (kCols <= 128 ? 128 : (kCols <= 256 ? 256 : 512)));
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*barriers*/ + 1024 /*align slack*/;
};

__device__ __forceinline__ float row_scale_of(const GemmParams& p, int m) {
  if (p.row_ss_in == nullptr) return p.out_scale != 0.f ? p.out_scale : 1.0f;
  float ss = 0.f;
  const float* src = p.row_ss_in + static_cast<long long>(m) * p.ss_in_parts;
  if (p.ag_ss_out != nullptr) {
    // the statistics were written by this very launch (all-gather phase, other SMs): read them from L2
    for (int i = 0; i < p.ss_in_parts; ++i) ss += __ldcg(src + i);
  } else if ((p.ss_in_parts & 3) == 0 && (reinterpret_cast<uintptr_t>(p.row_ss_in) & 15) == 0) {
    for (int i = 0; i < p.ss_in_parts; i += 4) {   // 16-byte loads: a row has up to hidden/128 partial sums
      const float4 f = *reinterpret_cast<const float4*>(src + i);
      ss += (f.x + f.y) + (f.z + f.w);
    }
  } else {
    for (int i = 0; i < p.ss_in_parts; ++i) ss += src[i];
  }
  return rsqrtf(ss * p.norm_inv_dim + p.norm_eps) * (p.out_scale != 0.f ? p.out_scale : 1.0f);
}
// The same for a whole warp working on one row: the partial sums are spread over the lanes (one load + a warp
// reduction instead of up to 32 dependent loads per unit; measured: the QKV reduce phase of the serving step went
// from 45.6 k clocks with 32 partials per row).
__device__ __forceinline__ float row_scale_warp(const GemmParams& p, int m, int lane) {
  if (p.row_ss_in == nullptr) return p.out_scale != 0.f ? p.out_scale : 1.0f;
  const float* src = p.row_ss_in + static_cast<long long>(m) * p.ss_in_parts;
  float ss = 0.f;
  if (p.ag_ss_out != nullptr) {
    for (int i = lane; i < p.ss_in_parts; i += 32) ss += __ldcg(src + i);
  } else {
    for (int i = lane; i < p.ss_in_parts; i += 32) ss += __ldg(src + i);
  }
  ss = warp_sum(ss);
  return rsqrtf(ss * p.norm_inv_dim + p.norm_eps) * (p.out_scale != 0.f ? p.out_scale : 1.0f);
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

// 32 floats -> 32 fp8 e4m3 bytes (saturating) at a 16-byte aligned address
__device__ __forceinline__ void store_fp8x32(uint8_t* dst, const float (&v)[32], float inv_scale) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i] * inv_scale, v[4 * i + 1] * inv_scale),
                                                 __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2] * inv_scale, v[4 * i + 3] * inv_scale),
                                                 __NV_SATFINITE, __NV_E4M3);
    w[i] = lo | (hi << 16);
  }
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
  d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Accumulator access for the epilogue: 32 consecutive fp32 columns of this thread's TMEM lane.
struct AccReader {
  uint32_t taddr;  // TMEM address of (lane quadrant, accumulator, column 0)
  __device__ __forceinline__ void load(int col, float (&v)[32]) const {
    uint32_t r[32];
    tmem_ld_32x32(taddr + col, r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  }
};

// Sum over all GPUs of a multicast group of 8 bf16 values (fp32 accumulation inside the switch).
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const __nv_bfloat16* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Cross-GPU arrival barrier of the fused all-reduce, in two levels so that a rank's counter takes one remote atomic
// per rank and launch instead of one per CTA: every CTA adds one to a LOCAL counter after a device-scope fence; the CTA
// that completes the local count (`local_target`) issues a system-scope fence and adds one to the arrival counter of
// every rank (one multimem.red, or one red per peer); everybody then waits until the own rank's counter has reached
// `target`. Bounded; returns false on timeout.
__device__ __forceinline__ bool ar_barrier(const GemmParams& p, unsigned long long target,
                                           unsigned long long local_target, int word = 0) {
  // `word` selects one of two adjacent arrival counters: the two-shot form meets twice per launch and keeps the
  // rounds on separate words, so an early second-round arrival can never stand in for a late first-round one.
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    if (word)
      __threadfence_system();   // second meeting: this CTA's stores went to the other GPUs' memory
    else
      __threadfence();
    const unsigned long long prev = atomicAdd(p.ar_state + 2, 1ull);
    if (prev + 1ull == local_target) {
      __threadfence_system();
      if (p.ar_mc_counter) {
        asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(p.ar_mc_counter + word), "l"(1ull) : "memory");
      } else {
        for (int r = 0; r < p.ar_world; ++r)
          asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p.ar_peer_counter[r] + word), "l"(1ull) : "memory");
      }
    }
    const unsigned long long* mine = p.ar_peer_counter[p.ar_rank] + word;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    while (ld_acquire_sys_u64(mine) < target) {
      if (((++spins) & 0x3F) == 0 && globaltimer_ns() - t0 > p.peer_wait_ns) {
        if (p.err) atomicCAS(p.err, 0, ERR_TIMEOUT_PEER);
        ok = 0;
        break;
      }
    }
    ok_flag = ok;
  }
  __syncthreads();
  return ok_flag != 0;
}

// Sense-reversing grid barrier over {count, generation}; bounded. Returns false on timeout.
__device__ __forceinline__ bool grid_barrier(unsigned int* bar, unsigned int num_ctas, int* err,
                                             unsigned long long limit_ns) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    __threadfence();
    const unsigned int gen = *reinterpret_cast<volatile unsigned int*>(bar + 1);
    if (atomicAdd(bar, 1u) == num_ctas - 1) {
      *reinterpret_cast<volatile unsigned int*>(bar) = 0u;
      __threadfence();
      atomicAdd(bar + 1, 1u);
    } else {
      const unsigned long long t0 = globaltimer_ns();
      unsigned int spins = 0;
      while (*reinterpret_cast<volatile unsigned int*>(bar + 1) == gen) {
        if (((++spins) & 0x3F) == 0 && globaltimer_ns() - t0 > limit_ns) {
          if (err) atomicCAS(err, 0, ERR_TIMEOUT_GRID);
          ok = 0;
          break;
        }
      }
    }
    __threadfence();
    ok_flag = ok;
  }
  __syncthreads();
  return ok_flag != 0;
}

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float2 ldcg2(const float* p) { return __ldcg(reinterpret_cast<const float2*>(p)); }

// The fused epilogue of EPI for one (row m, n tile) unit whose summed accumulator values a lane holds in v
// (lane -> column mapping as in splitk_reduce_phase). Shared by the global-memory and the cluster reduce phases.
// Inputs of the QKV epilogue of one unit that the reduce phases fetch ahead of time for all the units they keep in
// flight: position and cache slot of the row, and this lane's two cos / sin pairs. Without it every unit pays two
// dependent L2 round trips (row -> position -> rope table) after its partial sums arrived, one unit after the other
// (measured: 43 k clocks for the QKV reduce phase of the serving step against 9.6 k for the residual one).
struct QkvPre {
  int pos, slot;
  float2 cs, sn;
};
__device__ __forceinline__ void qkv_pre_row(const GemmParams& p, int m, QkvPre& q) {
  int pos = __ldg(p.positions + m);
  if (pos < 0 || pos >= p.max_pos) pos = 0;
  q.pos = pos;
  q.slot = p.slot_mapping ? __ldg(p.slot_mapping + m) : -1;
}
__device__ __forceinline__ void qkv_pre_rope(const GemmParams& p, int lane, QkvPre& q) {
  q.cs = __ldg(reinterpret_cast<const float2*>(p.cos_table + static_cast<long long>(q.pos) * 64 + lane * 2));
  q.sn = __ldg(reinterpret_cast<const float2*>(p.sin_table + static_cast<long long>(q.pos) * 64 + lane * 2));
}

template <int BN, int EPI, int NV, int SEGW>
__device__ __forceinline__ void apply_unit_epilogue(const GemmParams& p, int m, int n_blk, int lane, float (&v)[NV],
                                                    const uint2* pre_residual = nullptr,
                                                    const QkvPre* qpre = nullptr) {
      float rs = row_scale_warp(p, m, lane);   // every lane of the warp is here with the same row
      if (p.a_scale) rs *= p.a_scale[m];
      if constexpr (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
        const int n0 = n_blk * BN + lane * NV;
        float ss = 0.f;
        if (n0 < p.N) {
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            v[j] *= rs;
            if (p.b_scale) v[j] *= p.b_scale[n0 + j];
            if (p.bias) v[j] += p.bias[n0 + j];
          }
          if constexpr (EPI == EPI_RESIDUAL) {
            // pre_residual: the 4 residual values of this lane, loaded by the caller ahead of a long-latency phase
            const __nv_bfloat16* r = (NV == 4 && pre_residual) ? reinterpret_cast<const __nv_bfloat16*>(pre_residual)
                                                               : p.residual + static_cast<long long>(m) * p.ldr + n0;
#pragma unroll
            for (int j = 0; j < NV; j += 2) {
              const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(r + j));
              v[j] = bf16_round(v[j] + f.x);
              v[j + 1] = bf16_round(v[j + 1] + f.y);
              ss += v[j] * v[j] + v[j + 1] * v[j + 1];
            }
          }
          if (p.out_f32) {
            float* o = static_cast<float*>(p.out) + static_cast<long long>(m) * p.ldo + n0;
#pragma unroll
            for (int j = 0; j < NV; j += 4)
              *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0;
#pragma unroll
            for (int j = 0; j < NV; j += 4) {
              uint2 w;
              w.x = pack_bf16x2(v[j], v[j + 1]);
              w.y = pack_bf16x2(v[j + 2], v[j + 3]);
              *reinterpret_cast<uint2*>(o + j) = w;
            }
          }
        }
        if constexpr (EPI == EPI_RESIDUAL) {
          ss = warp_sum(ss);
          if (p.row_ss_out && lane == 0) p.row_ss_out[static_cast<long long>(m) * p.num_n + n_blk] = ss;
        }
      } else if constexpr (EPI == EPI_GLU) {
        constexpr int kHalf = BN / 2;
        const int n0 = n_blk * kHalf + lane * SEGW;
        if (n0 < p.N / 2) {
          float o4[SEGW];
#pragma unroll
          for (int j = 0; j < SEGW; ++j) {
            float gv = v[j] * rs, uv = v[SEGW + j] * rs;
            if (p.b_scale) {   // gate column of output o sits at 64 * (o / 32) + o % 32 of the tile, its up column 32 further
              const int o_in = lane * SEGW + j;
              const int gcol = n_blk * BN + (o_in >> 5) * 64 + (o_in & 31);
              gv *= p.b_scale[gcol];
              uv *= p.b_scale[gcol + 32];
            }
            o4[j] = (p.glu_act == 0 ? silu_f(gv) : gelu_tanh_f(gv)) * uv;
          }
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0;
          if constexpr (SEGW == 4) {
            uint2 w;
            w.x = pack_bf16x2(o4[0], o4[1]);
            w.y = pack_bf16x2(o4[2], o4[3]);
            *reinterpret_cast<uint2*>(o) = w;
          } else {
            *reinterpret_cast<uint32_t*>(o) = pack_bf16x2(o4[0], o4[1]);
          }
        }
      } else {  // EPI_QKV: the tile is one head; lane covers features {2l, 2l+1} and their RoPE partners
        const int head = n_blk;
        const bool is_q = head < p.n_q_heads;
        const bool is_k = !is_q && head < p.n_q_heads + p.n_kv_heads;
        float x0[2] = {v[0] * rs, v[1] * rs}, x1[2] = {v[2] * rs, v[3] * rs};
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            x0[j] += __ldg(p.bias + head * 128 + lane * 2 + j);
            x1[j] += __ldg(p.bias + head * 128 + 64 + lane * 2 + j);
          }
        }
        const float* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
        if (nw) {
          float ss = x0[0] * x0[0] + x0[1] * x0[1] + x1[0] * x1[0] + x1[1] * x1[1];
          ss = warp_sum(ss);
          const float inv_rms = rsqrtf(ss * (1.0f / 128.0f) + p.qk_eps);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            x0[j] *= inv_rms * __ldg(nw + lane * 2 + j);
            x1[j] *= inv_rms * __ldg(nw + 64 + lane * 2 + j);
          }
        }
        QkvPre qp;
        if (qpre) {
          qp = *qpre;
        } else {
          qkv_pre_row(p, m, qp);
          qkv_pre_rope(p, lane, qp);
        }
        const int slot = qp.slot;
        __nv_bfloat16* dst = nullptr;
        uint8_t* dst8 = nullptr;     // fp8 cache row
        if (is_q) {
          dst = p.q_out + (static_cast<long long>(m) * p.n_q_heads + head) * 128;
        } else if (slot >= 0) {
          const int page = slot / kPageTokens, off = slot % kPageTokens;
          if (page >= p.num_pages) {
            if (p.err && lane == 0) atomicCAS(p.err, 0, ERR_BAD_PAGE);
          } else {
            const int kvh = is_k ? head - p.n_q_heads : head - p.n_q_heads - p.n_kv_heads;
            const long long b2 = ((static_cast<long long>(page) * 2 + (is_k ? 0 : 1)) * p.n_kv_heads + kvh);
            if (p.kv_fp8)
              dst8 = reinterpret_cast<uint8_t*>(p.kv_cache) + (b2 * kPageTokens + off) * 128;
            else
              dst = p.kv_cache + (b2 * kPageTokens + off) * 128;
          }
        }
        if (dst || dst8) {
          float a[2], b[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (is_q || is_k) {
              const float cs = j == 0 ? qp.cs.x : qp.cs.y;
              const float sn = j == 0 ? qp.sn.x : qp.sn.y;
              a[j] = x0[j] * cs - x1[j] * sn;
              b[j] = x1[j] * cs + x0[j] * sn;
            } else {
              a[j] = x0[j];
              b[j] = x1[j];
            }
          }
          if (dst8) {
            const float is = p.kv_inv_scale;
            *reinterpret_cast<uint16_t*>(dst8 + lane * 2) = static_cast<uint16_t>(
                __nv_cvt_float2_to_fp8x2(make_float2(a[0] * is, a[1] * is), __NV_SATFINITE, __NV_E4M3));
            *reinterpret_cast<uint16_t*>(dst8 + 64 + lane * 2) = static_cast<uint16_t>(
                __nv_cvt_float2_to_fp8x2(make_float2(b[0] * is, b[1] * is), __NV_SATFINITE, __NV_E4M3));
          } else {
            *reinterpret_cast<uint32_t*>(dst + lane * 2) = pack_bf16x2(a[0], a[1]);
            *reinterpret_cast<uint32_t*>(dst + 64 + lane * 2) = pack_bf16x2(b[0], b[1]);
          }
        }
      }
}

// Phase 2 of a split-K GEMM: a warp owns (row, n tile) units, four at a time; lanes cover a unit's
// columns with vector loads. Loads of several units and several splits are issued together (the phase
// is latency bound: few threads, L2 round trips), the adds happen in split order so the result does
// not depend on timing, then the fused epilogue of EPI is applied.
template <int BN, int EPI>
__device__ void splitk_reduce_phase(const GemmParams& p, float* src_base, int nsplits, bool zero_after) {
  constexpr bool kGlu = (EPI == EPI_GLU), kQkv = (EPI == EPI_QKV);
  constexpr int NSEG = (kGlu || kQkv) ? 2 : BN / 128;            // vector segments per lane and unit
  constexpr int SEGW = (kQkv || (kGlu && BN == 128)) ? 2 : 4;    // floats per segment
  constexpr int NV = NSEG * SEGW;
  constexpr int U = 4;                                           // units in flight per warp
  constexpr int SU = (NV == 8) ? 2 : 4;                          // splits in flight
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const long long split_stride = static_cast<long long>(p.M) * n_pad;
  const int units = p.M * p.num_n;
  int seg_off[NSEG];
  if constexpr (kGlu) {
    // gate / up are interleaved in 64-column groups (32 gate, 32 up): output o of the tile pairs columns
    // 64 * (o / 32) + o % 32 and that + 32, whatever the tile width
    const int o_in = lane * SEGW;
    seg_off[0] = (o_in >> 5) * 64 + (o_in & 31);
    seg_off[1] = seg_off[0] + 32;
  } else if constexpr (kQkv) {
    seg_off[0] = lane * SEGW;
    seg_off[1] = BN / 2 + lane * SEGW;
  } else {
#pragma unroll
    for (int g = 0; g < NSEG; ++g) seg_off[g] = lane * NV + g * 4;
  }
  for (int u0 = (blockIdx.x * warps_per_cta + (threadIdx.x >> 5)) * U; u0 < units;
       u0 += gridDim.x * warps_per_cta * U) {
    float acc[U][NV];
    float* base[U];
    QkvPre qpre[kQkv ? U : 1];
    constexpr bool kPreRes = (EPI == EPI_RESIDUAL && NV == 4);
    uint2 pre_res[kPreRes ? U : 1];     // the residual values travel with the partial sums, not unit after unit
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = min(u0 + k, units - 1);
      base[k] = src_base + static_cast<long long>(u / p.num_n) * n_pad + static_cast<long long>(u % p.num_n) * BN;
      if constexpr (kQkv) qkv_pre_row(p, u / p.num_n, qpre[k]);   // in flight together with the partial sums
      if constexpr (kPreRes) {
        const int n0 = (u % p.num_n) * BN + lane * 4;
        pre_res[k] = make_uint2(0u, 0u);
        if (n0 < p.N)
          pre_res[k] = *reinterpret_cast<const uint2*>(p.residual + static_cast<long long>(u / p.num_n) * p.ldr + n0);
      }
#pragma unroll
      for (int j = 0; j < NV; ++j) acc[k][j] = 0.f;
    }
    for (int s0 = 0; s0 < nsplits; s0 += SU) {
      float tmp[SU][U][NV];
#pragma unroll
      for (int ds = 0; ds < SU; ++ds) {
        const int s = min(s0 + ds, nsplits - 1);
#pragma unroll
        for (int k = 0; k < U; ++k) {
          if constexpr (kQkv) {
            if (p.park) {   // parked tiles were published with the two 64-column halves interleaved per lane
              const float4 f = ldcg4(base[k] + s * split_stride + lane * 4);
              tmp[ds][k][0] = f.x; tmp[ds][k][1] = f.y; tmp[ds][k][2] = f.z; tmp[ds][k][3] = f.w;
              continue;
            }
          }
#pragma unroll
          for (int g = 0; g < NSEG; ++g) {
            const float* src = base[k] + s * split_stride + seg_off[g];
            if constexpr (SEGW == 4) {
              const float4 f = ldcg4(src);
              tmp[ds][k][g * 4 + 0] = f.x; tmp[ds][k][g * 4 + 1] = f.y;
              tmp[ds][k][g * 4 + 2] = f.z; tmp[ds][k][g * 4 + 3] = f.w;
            } else {
              const float2 f = ldcg2(src);
              tmp[ds][k][g * 2 + 0] = f.x; tmp[ds][k][g * 2 + 1] = f.y;
            }
          }
        }
      }
      if constexpr (kQkv) {
        if (s0 == 0) {   // the positions have arrived by now; the rope rows travel while the partial sums are added
#pragma unroll
          for (int k = 0; k < U; ++k) qkv_pre_rope(p, lane, qpre[k]);
        }
      }
#pragma unroll
      for (int ds = 0; ds < SU; ++ds) {
        if (s0 + ds < nsplits) {
#pragma unroll
          for (int k = 0; k < U; ++k)
#pragma unroll
            for (int j = 0; j < NV; ++j) acc[k][j] += tmp[ds][k][j];
        }
      }
    }
    if (zero_after) {  // the all-reduce accumulation buffer must be zero again before its next use
#pragma unroll
      for (int k = 0; k < U; ++k) {
        if (u0 + k < units) {
#pragma unroll
          for (int g = 0; g < NSEG; ++g) {
            if constexpr (SEGW == 4)
              __stcg(reinterpret_cast<float4*>(base[k] + seg_off[g]), make_float4(0.f, 0.f, 0.f, 0.f));
            else
              __stcg(reinterpret_cast<float2*>(base[k] + seg_off[g]), make_float2(0.f, 0.f));
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {  // fully unrolled: acc[k] must stay in registers
      const int u = u0 + k;
      if (u >= units) continue;
      const int n_blk = u % p.num_n;
      const int m = u / p.num_n;
      float v[NV];
#pragma unroll
      for (int j = 0; j < NV; ++j) v[j] = acc[k][j];
      apply_unit_epilogue<BN, EPI, NV, SEGW>(p, m, n_blk, lane, v, kPreRes ? &pre_res[k] : nullptr,
                                             kQkv ? &qpre[k] : nullptr);
    }
  }
}

// Phase 2 of the fused all-reduce: a warp owns (row, 256-column group) units, four at a time; a lane
// covers 8 columns = one 16-byte vector. The sum over ranks comes from one multimem.ld_reduce per
// vector (NVSwitch adds in fp32) or from one plain load per peer; then residual add, bf16 store and
// the row statistics for the next norm.
// When the rank split K locally (`nsplits` partial buffers, `split_elems` apart) every split is pulled and added in
// split order, identically on every rank.
// Two-shot form (bcast_off >= 0): the call covers only rows [row_lo, row_hi), this rank's share, and every finished
// 16-byte piece is also stored into the result region of every rank (one multimem.st, or one store per peer), from
// where ar_gather_phase copies the other ranks' rows after a second barrier. Each rank then pulls 1/W of the output
// instead of all of it (at eight ranks the one-shot pull reads 8 x 2 MB out of every GPU per GEMM).
__device__ __forceinline__ void multimem_st_b128(__nv_bfloat16* mc, const uint4& w) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(w.x), "r"(w.y),
               "r"(w.z), "r"(w.w)
               : "memory");
}
template <int BN, int U>
__device__ void ar_reduce_phase(const GemmParams& p, long long buf_off, int nsplits, long long split_elems, int row_lo,
                                int row_hi, long long bcast_off) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const int groups = static_cast<int>(n_pad / 256);
  const int units = (row_hi - row_lo) * groups;
  if (units <= 0) return;
  for (int u0 = (blockIdx.x * warps_per_cta + (threadIdx.x >> 5)) * U; u0 < units;
       u0 += gridDim.x * warps_per_cta * U) {
    float acc[U][8];
    long long off[U];
    uint4 res[U];     // residual rows: requested before the pull so that they do not cost a round trip per unit
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = min(u0 + k, units - 1);
      const int mrow = row_lo + u / groups;
      off[k] = buf_off + static_cast<long long>(mrow) * n_pad + static_cast<long long>(u % groups) * 256 + lane * 8;
      const int n0 = (u % groups) * 256 + lane * 8;
      res[k] = make_uint4(0u, 0u, 0u, 0u);
      if (n0 < p.N) res[k] = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(mrow) * p.ldr + n0);
    }
#pragma unroll
    for (int k = 0; k < U; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
    if (p.ar_mc_buf) {
      if (nsplits == 2) {   // both splits' round trips through the switch in flight together
        uint4 raw[2][U];
#pragma unroll
        for (int sp = 0; sp < 2; ++sp)
#pragma unroll
          for (int k = 0; k < U; ++k) raw[sp][k] = multimem_ld_reduce_bf16x8(p.ar_mc_buf + off[k] + sp * split_elems);
#pragma unroll
        for (int sp = 0; sp < 2; ++sp)
#pragma unroll
          for (int k = 0; k < U; ++k) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[sp][k]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h[e]);
              acc[k][2 * e] += f.x;
              acc[k][2 * e + 1] += f.y;
            }
          }
      } else {
        for (int sp = 0; sp < nsplits; ++sp) {
          uint4 raw[U];
#pragma unroll
          for (int k = 0; k < U; ++k) raw[k] = multimem_ld_reduce_bf16x8(p.ar_mc_buf + off[k] + sp * split_elems);
#pragma unroll
          for (int k = 0; k < U; ++k) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h[e]);
              acc[k][2 * e] += f.x;
              acc[k][2 * e + 1] += f.y;
            }
          }
        }
      }
    } else {
      for (int rs = 0; rs < p.ar_world * nsplits; ++rs) {  // (split, rank) order: every rank computes the identical sum
        const int r = rs % p.ar_world;
        const long long soff = static_cast<long long>(rs / p.ar_world) * split_elems;
        uint4 raw[U];
#pragma unroll
        for (int k = 0; k < U; ++k) raw[k] = __ldcg(reinterpret_cast<const uint4*>(p.ar_peer_buf[r] + off[k] + soff));
#pragma unroll
        for (int k = 0; k < U; ++k) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            acc[k][2 * e] += f.x;
            acc[k][2 * e + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = u0 + k;
      if (u >= units) continue;
      const int m = row_lo + u / groups, grp = u % groups;
      const int n0 = grp * 256 + lane * 8;
      float ss = 0.f;
      if (n0 < p.N) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] = acc[k][j];
          if (p.bias) v[j] += p.bias[n0 + j];
        }
        const uint4 rr = res[k];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[2 * e] = bf16_round(v[2 * e] + f.x);
          v[2 * e + 1] = bf16_round(v[2 * e + 1] + f.y);
          ss = fmaf(v[2 * e], v[2 * e], fmaf(v[2 * e + 1], v[2 * e + 1], ss));   // same order in ar_gather_phase
        }
        uint4 w;
        w.x = pack_bf16x2(v[0], v[1]);
        w.y = pack_bf16x2(v[2], v[3]);
        w.z = pack_bf16x2(v[4], v[5]);
        w.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0) = w;
        if (bcast_off >= 0) {
          const long long roff = bcast_off + static_cast<long long>(m) * n_pad + n0;
          if (p.ar_mc_buf) {
            multimem_st_b128(p.ar_mc_buf + roff, w);
          } else {
            for (int r = 0; r < p.ar_world; ++r)
              if (r != p.ar_rank) *reinterpret_cast<uint4*>(p.ar_peer_buf[r] + roff) = w;
          }
        }
      }
      ss = warp_sum(ss);
      if (p.row_ss_out && lane == 0) p.row_ss_out[static_cast<long long>(m) * groups + grp] = ss;
    }
  }
}

// Second half of the two-shot form: rows finished by the other ranks are copied from this GPU's result region into
// the output, with their row statistics (the same bf16 values, so every rank ends up with identical numbers).
template <int BN>
__device__ void ar_gather_phase(const GemmParams& p, long long bcast_off, int own_lo, int own_hi) {
  constexpr int U = 4;
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const int groups = static_cast<int>(n_pad / 256);
  const int other_rows = p.M - (own_hi - own_lo);
  const int units = other_rows * groups;
  const __nv_bfloat16* src = p.ar_peer_buf[p.ar_rank] + bcast_off;
  for (int u0 = (blockIdx.x * warps_per_cta + (threadIdx.x >> 5)) * U; u0 < units;
       u0 += gridDim.x * warps_per_cta * U) {
    uint4 w[U];
    int mr[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = min(u0 + k, units - 1);
      int m = u / groups;
      if (m >= own_lo) m += own_hi - own_lo;     // skip this rank's own rows
      mr[k] = m;
      const int n0 = (u % groups) * 256 + lane * 8;
      w[k] = make_uint4(0u, 0u, 0u, 0u);
      if (n0 < p.N) w[k] = __ldcg(reinterpret_cast<const uint4*>(src + static_cast<long long>(m) * n_pad + n0));
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = u0 + k;
      if (u >= units) continue;
      const int grp = u % groups;
      const int n0 = grp * 256 + lane * 8;
      float ss = 0.f;
      if (n0 < p.N) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
        }
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(mr[k]) * p.ldo + n0) = w[k];
      }
      ss = warp_sum(ss);
      if (p.row_ss_out && lane == 0) p.row_ss_out[static_cast<long long>(mr[k]) * groups + grp] = ss;
    }
  }
}


// ---------------------------------------------------------------------------------------------
// Push form of the fused all-reduce (GemmParams::ar_push): no meeting of all ranks before data moves. A producer
// stores the bf16 rows of a retired tile straight into the receive slots of the rank that owns those rows and then
// releases one flag per (source, m tile, n tile) with the launch epoch; the owner's warps wait for the flags of the
// tiles their units need, add the sources in (split, rank) order, finish the rows (bias, residual, rounding, row
// statistics) and store them into every rank's output. The flags carry values, not counts, so nothing is reset
// between launches; every rank issues the same launches in the same order, so the epochs agree.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys_u32(unsigned int* ptr, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_u64(unsigned long long* ptr, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(ptr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed_sys_u32(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void multimem_st_f32(float* mc, float v) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(v) : "memory");
}
__device__ __forceinline__ int ar_rows_per(const GemmParams& p) { return (p.M + p.ar_world - 1) / p.ar_world; }
__device__ __forceinline__ unsigned int* ar_flag_ptr(const GemmParams& p, int r) {
  return reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(p.ar_peer_buf[r]) + p.ar_flag_off);
}
__device__ __forceinline__ unsigned long long* ar_done_ptr(const GemmParams& p, int r) {
  return reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(p.ar_peer_buf[r]) + p.ar_done_off);
}
// Receive slot of (source, output row m, column n) in the memory of the rank that owns row m.
__device__ __forceinline__ __nv_bfloat16* ar_recv_slot(const GemmParams& p, int src, int m, long long n_pad, int n) {
  const int rows_per = ar_rows_per(p);
  const int owner = m / rows_per;
  const int lrow = m - owner * rows_per;
  return p.ar_peer_buf[owner] + p.ar_recv_off + (static_cast<long long>(src) * rows_per + lrow) * n_pad + n;
}
// After a barrier among all threads that stored tile (m_sup, n_blk) of source `src`: thread `tid` < world releases
// the tile's flag on rank `tid` when the tile holds rows of that rank.
__device__ __forceinline__ void ar_push_signal(const GemmParams& p, int tid, int src, int m_sup, int n_blk,
                                               int tile_rows, unsigned int epoch) {
  if (tid < p.ar_world && !p.ar_drop_flags) {
    const int rows_per = ar_rows_per(p);
    const int lo = tid * rows_per, hi = min(p.M, lo + rows_per);
    const int t_lo = m_sup * tile_rows, t_hi = min(p.M, t_lo + tile_rows);
    if (t_lo < hi && t_hi > lo) {
      __threadfence_system();
      st_release_sys_u32(ar_flag_ptr(p, tid) + (static_cast<long long>(src) * p.num_m + m_sup) * p.num_n + n_blk, epoch);
    }
  }
}
// The parked fp32 tile of this CTA (BN = 128) goes out row by row: a warp stores 256 contiguous bytes per row.
__device__ void ar_push_parked(const GemmParams& p, const float* part, int rows, int m_row0, int n_blk, int src) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * 128;
  for (int r = warp; r < rows; r += nwarps) {
    const int m = m_row0 + r;
    if (m >= p.M) continue;
    const float4 v = *reinterpret_cast<const float4*>(part + r * kClusterPartStride + lane * 4);
    uint2 w;
    w.x = pack_bf16x2(v.x, v.y);
    w.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(ar_recv_slot(p, src, m, n_pad, n_blk * 128 + lane * 4)) = w;
  }
}

// The owner's side: a warp takes (row, 256-column group) units of this rank's rows, four at a time; a lane covers 8
// columns. tile_rows: rows of one producer tile (the m index of the flags). abort: the CTA's shared abort word.
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
// U: units a warp keeps in flight. Decode-sized launches have fewer units than the grid has warps, so they run with
// U = 1 (every warp that has a unit works on it at once); large M uses 4 for memory-level parallelism.
template <int BN, int U>
__device__ void ar_push_reduce_u(const GemmParams& p, unsigned int epoch, int tile_rows, volatile int* abort) {
  constexpr int NB = 256 / BN;   // n tiles per 256-column group
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int W = p.ar_world, nsrc = W * p.splits;
  const int rows_per = ar_rows_per(p);
  const int own_lo = min(p.M, p.ar_rank * rows_per), own_hi = min(p.M, own_lo + rows_per);
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const int groups = static_cast<int>(n_pad / 256);
  const int units = (own_hi - own_lo) * groups;
  if (units <= 0) return;
  const __nv_bfloat16* recv = p.ar_peer_buf[p.ar_rank] + p.ar_recv_off;
  const unsigned int* flags = ar_flag_ptr(p, p.ar_rank);
  const long long src_stride = static_cast<long long>(rows_per) * n_pad;
  for (int u0 = (blockIdx.x * warps_per_cta + (threadIdx.x >> 5)) * U; u0 < units;
       u0 += gridDim.x * warps_per_cta * U) {
    // ---- wait (bounded) for the tiles these units are made of: one lane per (source, n tile) flag ----
    bool ok = true;
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = min(u0 + k, units - 1);
      const int m = own_lo + u / groups, grp = u % groups;
      if (lane < nsrc * NB) {
        const unsigned int* f = flags + (static_cast<long long>(lane / NB) * p.num_m + m / tile_rows) * p.num_n +
                                grp * NB + (lane % NB);
        // acquire loads: the tile's rows, stored before its flag was released, are visible to this lane afterwards and,
        // through the warp-level meeting below, to the whole warp
        if (ld_acquire_sys_u32(f) != epoch) {
          const unsigned long long t0 = globaltimer_ns();
          unsigned int spins = 0;
          while (ld_acquire_sys_u32(f) != epoch) {
            if (((++spins) & 0x3F) == 0) {
              if (*abort) { ok = false; break; }
              if (globaltimer_ns() - t0 > p.peer_wait_ns) {
                *abort = 1;
                if (p.err) atomicCAS(p.err, 0, ERR_TIMEOUT_PEER);
                ok = false;
                break;
              }
            }
          }
        }
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) continue;
    // ---- add the sources in (split, rank) order ----
    float acc[U][8];
    long long off[U];
    uint4 res[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = min(u0 + k, units - 1);
      const int lrow = u / groups, grp = u % groups;
      off[k] = static_cast<long long>(lrow) * n_pad + static_cast<long long>(grp) * 256 + lane * 8;
      const int n0 = grp * 256 + lane * 8;
      res[k] = make_uint4(0u, 0u, 0u, 0u);
      if (n0 < p.N) res[k] = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(own_lo + lrow) * p.ldr + n0);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
    }
    for (int s0 = 0; s0 < nsrc; s0 += 4) {
      uint4 raw[4][U];
#pragma unroll
      for (int ds = 0; ds < 4; ++ds) {
        const int sidx = min(s0 + ds, nsrc - 1);
#pragma unroll
        for (int k = 0; k < U; ++k) raw[ds][k] = __ldcg(reinterpret_cast<const uint4*>(recv + sidx * src_stride + off[k]));
      }
#pragma unroll
      for (int ds = 0; ds < 4; ++ds) {
        if (s0 + ds < nsrc) {
#pragma unroll
          for (int k = 0; k < U; ++k) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[ds][k]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(h[e]);
              acc[k][2 * e] += f.x;
              acc[k][2 * e + 1] += f.y;
            }
          }
        }
      }
    }
    // ---- finish the rows and hand them to every rank ----
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int u = u0 + k;
      if (u >= units) continue;
      const int m = own_lo + u / groups, grp = u % groups;
      const int n0 = grp * 256 + lane * 8;
      float ss = 0.f;
      if (n0 < p.N) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[j] = acc[k][j];
          if (p.bias) v[j] += p.bias[n0 + j];
        }
        const uint4 rr = res[k];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[2 * e] = bf16_round(v[2 * e] + f.x);
          v[2 * e + 1] = bf16_round(v[2 * e + 1] + f.y);
          ss = fmaf(v[2 * e], v[2 * e], fmaf(v[2 * e + 1], v[2 * e + 1], ss));
        }
        uint4 w;
        w.x = pack_bf16x2(v[0], v[1]);
        w.y = pack_bf16x2(v[2], v[3]);
        w.z = pack_bf16x2(v[4], v[5]);
        w.w = pack_bf16x2(v[6], v[7]);
        const long long o = p.ar_out_off + static_cast<long long>(m) * p.ldo + n0;
        if (p.ar_mc_buf) {
          multimem_st_b128(p.ar_mc_buf + o, w);
        } else {
          for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(p.ar_peer_buf[r] + o) = w;
        }
      }
      ss = warp_sum(ss);
      if (p.row_ss_out && lane == 0) {
        const long long so = p.ar_ss_off + (static_cast<long long>(m) * groups + grp) * 4;
        if (p.ar_mc_buf) {
          multimem_st_f32(reinterpret_cast<float*>(reinterpret_cast<char*>(p.ar_mc_buf) + so), ss);
        } else {
          for (int r = 0; r < W; ++r) *reinterpret_cast<float*>(reinterpret_cast<char*>(p.ar_peer_buf[r]) + so) = ss;
        }
      }
    }
  }
}

template <int BN>
__device__ __forceinline__ void ar_push_reduce(const GemmParams& p, unsigned int epoch, int tile_rows, volatile int* abort) {
  const int rows_per = ar_rows_per(p);
  const int own = max(0, min(p.M, (p.ar_rank + 1) * rows_per) - min(p.M, p.ar_rank * rows_per));
  const long long units = static_cast<long long>(own) * (static_cast<long long>(p.num_n) * BN / 256);
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  if (units <= warps) ar_push_reduce_u<BN, 1>(p, epoch, tile_rows, abort);
  else if (units <= 2 * warps) ar_push_reduce_u<BN, 2>(p, epoch, tile_rows, abort);
  else ar_push_reduce_u<BN, 4>(p, epoch, tile_rows, abort);
}

// End of a push launch: the last CTA of this rank to get here tells every rank that this rank's rows are out, then
// every CTA waits (bounded) until all ranks have said so. After that the outputs of all ranks are in local memory and
// nobody still reads this rank's receive slots, so the next launch may overwrite them.
__device__ __forceinline__ bool ar_push_finish(const GemmParams& p, unsigned long long epoch, unsigned long long launch) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();   // this CTA's stores went to the other GPUs' memory
    const unsigned long long prev = atomicAdd(p.ar_state + 5, 1ull);
    if (prev + 1ull == gridDim.x) {
      p.ar_state[5] = 0ull;             // every CTA has arrived, so every CTA has read the launch index
      p.ar_state[1] = launch + 1ull;
      __threadfence_system();
      for (int r = 0; r < p.ar_world; ++r) st_release_sys_u64(ar_done_ptr(p, r) + p.ar_rank, epoch);
    }
  }
  if (threadIdx.x < 32) {
    bool ok = true;
    if (threadIdx.x < p.ar_world) {
      const unsigned long long* d = ar_done_ptr(p, p.ar_rank) + threadIdx.x;
      const unsigned long long t0 = globaltimer_ns();
      unsigned int spins = 0;
      while (ld_acquire_sys_u64(d) != epoch) {
        if (((++spins) & 0x3F) == 0 && globaltimer_ns() - t0 > p.peer_wait_ns) {
          if (p.err) atomicCAS(p.err, 0, ERR_TIMEOUT_PEER);
          ok = false;
          break;
        }
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (threadIdx.x == 0) ok_flag = ok ? 1 : 0;
  }
  __syncthreads();
  return ok_flag != 0;
}

// ---------------------------------------------------------------------------------------------
// Low-latency (self-validating data) form of the fused all-reduce, see GemmParams::ar_ll.
// ---------------------------------------------------------------------------------------------
constexpr unsigned int kLlSentinel = 0x80008000u;   // bf16x2 (-0, -0): never stored as data
__device__ __forceinline__ unsigned int ll_word(unsigned int w) { return w == kLlSentinel ? 0u : w; }
__device__ __forceinline__ uint4 ld_volatile_u4(const void* ptr) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u4(void* ptr, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_volatile_u2(void* ptr, unsigned int a, unsigned int b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(ptr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ bool ll_valid(const uint4& v) {
  return v.x != kLlSentinel && v.y != kLlSentinel && v.z != kLlSentinel && v.w != kLlSentinel;
}
__device__ __forceinline__ __nv_bfloat16* ar_ll_recv(const GemmParams& p, int r, int parity) {
  return reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(p.ar_peer_buf[r]) + p.ar_ll_recv_off + parity * p.ar_ll_recv_bytes);
}
__device__ __forceinline__ __nv_bfloat16* ar_ll_res(const GemmParams& p, int r, int parity) {
  return reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(p.ar_peer_buf[r]) + p.ar_ll_res_off + parity * p.ar_ll_res_bytes);
}
// Bounded poll of one 16-byte slot piece; puts the sentinel back once the data has been taken.
__device__ __forceinline__ bool ll_take(__nv_bfloat16* slot, uint4& v, const GemmParams& p, volatile int* abort) {
  v = ld_volatile_u4(slot);
  if (!ll_valid(v)) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    do {
      if (((++spins) & 0x3F) == 0) {
        if (*abort) return false;
        if (globaltimer_ns() - t0 > p.peer_wait_ns) {
          *abort = 1;
          if (p.err) atomicCAS(p.err, 0, ERR_TIMEOUT_PEER);
          return false;
        }
      }
      v = ld_volatile_u4(slot);
    } while (!ll_valid(v));
  }
  st_volatile_u4(slot, make_uint4(kLlSentinel, kLlSentinel, kLlSentinel, kLlSentinel));
  return true;
}
// The parked fp32 tile (BN = 128) of this CTA -> bf16 rows in the receive slots of the rows' owners.
__device__ void ar_ll_push_parked(const GemmParams& p, const float* part, int rows, int m_row0, int n_blk, int src, int parity) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * 128;
  const int rows_per = ar_rows_per(p);
  for (int r = warp; r < rows; r += nwarps) {
    const int m = m_row0 + r;
    if (m >= p.M) continue;
    const int owner = m / rows_per, lrow = m - owner * rows_per;
    float4 v = *reinterpret_cast<const float4*>(part + r * kClusterPartStride + lane * 4);
    if (p.out_scale != 0.f) {      // block-scaled operands with per-tensor scales: the partial products carry them
      v.x *= p.out_scale; v.y *= p.out_scale; v.z *= p.out_scale; v.w *= p.out_scale;
    }
    __nv_bfloat16* dst = ar_ll_recv(p, owner, parity) + (static_cast<long long>(src) * rows_per + lrow) * n_pad + n_blk * 128 + lane * 4;
    st_volatile_u2(dst, ll_word(pack_bf16x2(v.x, v.y)), ll_word(pack_bf16x2(v.z, v.w)));
  }
}
// Owner: add the sources of this rank's rows, finish them, store them into every rank's result slots.
template <int BN>
__device__ void ar_ll_reduce(const GemmParams& p, int parity, volatile int* abort) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int W = p.ar_world, nsrc = W * p.splits;
  const int rows_per = ar_rows_per(p);
  const int own_lo = min(p.M, p.ar_rank * rows_per), own_hi = min(p.M, own_lo + rows_per);
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const int groups = static_cast<int>(n_pad / 256);
  const int units = (own_hi - own_lo) * groups;
  __nv_bfloat16* recv = ar_ll_recv(p, p.ar_rank, parity);
  const long long src_stride = static_cast<long long>(rows_per) * n_pad;
  for (int u = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); u < units; u += gridDim.x * warps_per_cta) {
    const int lrow = u / groups, grp = u % groups, m = own_lo + lrow;
    const int n0 = grp * 256 + lane * 8;
    const long long off = static_cast<long long>(lrow) * n_pad + n0;
    uint4 rr = make_uint4(0u, 0u, 0u, 0u);
    const long long rrow = p.ar_rs_only ? lrow : m;    // reduce-scatter output: residual / out / statistics are shards
    if (n0 < p.N) rr = *reinterpret_cast<const uint4*>(p.residual + rrow * p.ldr + n0);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    bool ok = true;
    for (int s0 = 0; s0 < nsrc && ok; ++s0) {   // (split, rank) order; the polls of later sources overlap the earlier adds
      uint4 raw;
      ok = ll_take(recv + s0 * src_stride + off, raw, p, abort);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    if (!__all_sync(0xffffffffu, ok)) continue;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (n0 < p.N) {
      float v[8];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        v[2 * e] = acc[2 * e] + (p.bias ? p.bias[n0 + 2 * e] : 0.f) + f.x;
        v[2 * e + 1] = acc[2 * e + 1] + (p.bias ? p.bias[n0 + 2 * e + 1] : 0.f) + f.y;
      }
      w.x = ll_word(pack_bf16x2(v[0], v[1]));
      w.y = ll_word(pack_bf16x2(v[2], v[3]));
      w.z = ll_word(pack_bf16x2(v[4], v[5]));
      w.w = ll_word(pack_bf16x2(v[6], v[7]));
    }
    if (p.ar_rs_only) {
      float ss = 0.f;
      if (n0 < p.N) {
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
        }
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + rrow * p.ldo + n0) = w;
      }
      ss = warp_sum(ss);
      if (p.row_ss_out && lane == 0) p.row_ss_out[rrow * groups + grp] = ss;
      continue;
    }
    const long long ro = static_cast<long long>(m) * n_pad + n0;
    if (p.ar_mc_buf) {   // one store, replicated to every rank's result slots by the switch
      multimem_st_b128(reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(p.ar_mc_buf) + p.ar_ll_res_off +
                                                        parity * p.ar_ll_res_bytes) + ro, w);
    } else {
      for (int r = 0; r < W; ++r) st_volatile_u4(ar_ll_res(p, r, parity) + ro, w);
    }
  }
}
// Every rank: all rows from the own result slots into `out`, with the row statistics of the next norm.
template <int BN>
__device__ void ar_ll_gather(const GemmParams& p, int parity, volatile int* abort) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const int groups = static_cast<int>(n_pad / 256);
  const int units = p.M * groups;
  __nv_bfloat16* res = ar_ll_res(p, p.ar_rank, parity);
  for (int u = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); u < units; u += gridDim.x * warps_per_cta) {
    const int m = u / groups, grp = u % groups;
    const int n0 = grp * 256 + lane * 8;
    uint4 w;
    const bool ok = ll_take(res + static_cast<long long>(m) * n_pad + n0, w, p, abort);
    if (!__all_sync(0xffffffffu, ok)) continue;
    float ss = 0.f;
    if (n0 < p.N) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
      }
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0) = w;
    }
    ss = warp_sum(ss);
    if (p.row_ss_out && lane == 0) p.row_ss_out[static_cast<long long>(m) * groups + grp] = ss;
  }
}
// The launch index advances once per launch: the last CTA to pass here does it (a local, relaxed counter).
__device__ __forceinline__ void ar_ll_advance(const GemmParams& p, unsigned long long launch) {
  if (threadIdx.x == 0) {
    const unsigned long long prev = atomicAdd(p.ar_state + 5, 1ull);
    if (prev + 1ull == gridDim.x) {
      p.ar_state[5] = 0ull;
      p.ar_state[1] = launch + 1ull;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// All-gather of the A rows in front of the main loop, see GemmParams::ag_world.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ bool ag_ll_phase(const GemmParams& p, int parity, volatile int* abort) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpc = blockDim.x >> 5;
  const int W = p.ag_world;
  const int rows_per = (p.M + W - 1) / W;
  const int own_lo = min(p.M, p.ag_rank * rows_per), own_hi = min(p.M, own_lo + rows_per);
  const int groups = p.K / 256;
  const long long set_off = p.ag_slot_off + parity * p.ag_slot_bytes;
  // this rank's rows -> every rank's slots
  for (int u = blockIdx.x * wpc + warp; u < (own_hi - own_lo) * groups; u += gridDim.x * wpc) {
    const int lrow = u / groups, grp = u % groups;
    const int c0 = grp * 256 + lane * 8;
    uint4 v = *reinterpret_cast<const uint4*>(p.ag_src + static_cast<long long>(lrow) * p.ag_src_ld + c0);
    v.x = ll_word(v.x); v.y = ll_word(v.y); v.z = ll_word(v.z); v.w = ll_word(v.w);
    const long long off = (static_cast<long long>(own_lo + lrow) * p.K + c0) * 2;
    if (p.ag_mc) {
      multimem_st_b128(reinterpret_cast<__nv_bfloat16*>(p.ag_mc + set_off + off), v);
    } else {
      for (int r = 0; r < W; ++r) st_volatile_u4(p.ag_peer[r] + set_off + off, v);
    }
  }
  // all rows: own slots -> the A tensor
  bool all_ok = true;
  for (int u = blockIdx.x * wpc + warp; u < p.M * groups; u += gridDim.x * wpc) {
    const int m = u / groups, grp = u % groups;
    const int c0 = grp * 256 + lane * 8;
    uint4 v;
    const bool ok = ll_take(reinterpret_cast<__nv_bfloat16*>(p.ag_peer[p.ag_rank] + set_off) + static_cast<long long>(m) * p.K + c0,
                            v, p, abort);
    if (!__all_sync(0xffffffffu, ok)) {
      all_ok = false;
      break;
    }
    *reinterpret_cast<uint4*>(p.ag_dst + static_cast<long long>(m) * p.ag_dst_ld + c0) = v;
    if (p.ag_ss_out) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        ss = fmaf(f.x, f.x, fmaf(f.y, f.y, ss));
      }
      ss = warp_sum(ss);
      if (lane == 0) p.ag_ss_out[static_cast<long long>(m) * groups + grp] = ss;
    }
  }
  fence_proxy_async_global();   // the rows were written by ordinary stores and are read by TMA
  return all_ok;
}

// ---------------------------------------------------------------------------------------------
// split-K inside a thread-block cluster: the S CTAs that share an output tile park their fp32 partial tiles in
// their own shared memory, write the rows that OTHER members will finish to the global scratch with coalesced
// stores, meet at one cluster barrier (instead of a grid-wide one) and each finishes 1/S of the rows: its own
// partial from shared memory, the others' from L2. Measured on B200: reading peers' tiles through distributed
// shared memory was 3-4x slower than through L2 (the SM-to-SM path moves far fewer bytes per clock than the
// 64 B/clk L2 port), so DSMEM is not used for the bulk data.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t cta) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(cta));
  return ra;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float2 ld_dsmem_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}


// Rows of the tile that cluster member `rank` finishes.
__device__ __forceinline__ void cluster_row_range(int rows, int S, int rank, int& b, int& e) {
  b = static_cast<int>(static_cast<long long>(rank) * rows / S);
  e = static_cast<int>(static_cast<long long>(rank + 1) * rows / S);
}

// part: this CTA's partial tile [rows][kClusterPartStride] fp32 in shared memory. Writes every row that another
// member finishes to scratch[ks][m][n_pad] (one warp per row: 512 contiguous bytes per store instruction).
// halves_interleaved: a lane's float4 holds columns (2l, 2l+1, 64+2l, 64+2l+1) instead of (4l .. 4l+3): the layout in
// which the QKV reduce phase wants its RoPE pairs, so that it reads one 16-byte piece per lane instead of two 8-byte ones.
__device__ void cluster_publish_partials(const GemmParams& p, const float* part, int rows, int m_row0, int n_blk, int S,
                                         int ks, bool skip_own = true, bool halves_interleaved = false) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const long long n_pad = static_cast<long long>(p.num_n) * 128;
  int own_b = 0, own_e = 0;
  if (skip_own) cluster_row_range(rows, S, ks, own_b, own_e);
  float* dst_base = p.sk_scratch + (static_cast<long long>(ks) * p.M) * n_pad + static_cast<long long>(n_blk) * 128 + lane * 4;
  for (int r = warp; r < rows; r += nwarps) {
    if (r >= own_b && r < own_e) continue;
    const int m = m_row0 + r;
    if (m >= p.M) continue;
    float4 v;
    if (halves_interleaved) {
      const float2 a = *reinterpret_cast<const float2*>(part + r * kClusterPartStride + lane * 2);
      const float2 b = *reinterpret_cast<const float2*>(part + r * kClusterPartStride + 64 + lane * 2);
      v = make_float4(a.x, a.y, b.x, b.y);
    } else {
      v = *reinterpret_cast<const float4*>(part + r * kClusterPartStride + lane * 4);
    }
    __stcg(reinterpret_cast<float4*>(dst_base + static_cast<long long>(m) * n_pad), v);
  }
}

// After the cluster barrier: this member (split index ks == cluster rank) finishes its rows of tile (m_sup, n_blk).
template <int EPI>
__device__ void cluster_reduce_phase(const GemmParams& p, const float* part, int rows, int m_row0, int n_blk, int S,
                                     int ks) {
  constexpr int BN = 128;
  constexpr bool kGlu = (EPI == EPI_GLU), kQkv = (EPI == EPI_QKV);
  constexpr int NSEG = (kGlu || kQkv) ? 2 : 1;
  constexpr int SEGW = (kGlu || kQkv) ? 2 : 4;
  constexpr int NV = NSEG * SEGW;
  constexpr int U = (SEGW == 4) ? 8 : 4;   // rows in flight per warp: with 8 warps that is the whole share of a 4-way split
  constexpr int SU = 4;   // splits in flight
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  int r_begin, r_end;
  cluster_row_range(rows, S, ks, r_begin, r_end);
  int seg_off[NSEG];
  if constexpr (kGlu) {
    const int o_in = lane * SEGW;
    seg_off[0] = (o_in >> 5) * 64 + (o_in & 31);
    seg_off[1] = seg_off[0] + 32;
  } else if constexpr (kQkv) {
    seg_off[0] = lane * SEGW;
    seg_off[1] = BN / 2 + lane * SEGW;
  } else {
    seg_off[0] = lane * 4;
  }
  const long long n_pad = static_cast<long long>(p.num_n) * BN;
  const long long split_stride = static_cast<long long>(p.M) * n_pad;
  for (int r0 = r_begin + warp; r0 < r_end; r0 += nwarps * U) {
    float acc[U][NV];
    uint2 pre[U];
    QkvPre qpre[kQkv ? U : 1];
    const float* gbase[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
#pragma unroll
      for (int j = 0; j < NV; ++j) acc[k][j] = 0.f;
      pre[k] = make_uint2(0u, 0u);
      const int r = min(r0 + k * nwarps, r_end - 1);
      const int m = min(m_row0 + r, p.M - 1);
      gbase[k] = p.sk_scratch + static_cast<long long>(m) * n_pad + static_cast<long long>(n_blk) * BN;
      if constexpr (kQkv) qkv_pre_row(p, m, qpre[k]);
      if constexpr (EPI == EPI_RESIDUAL) {   // ask for the residual together with the partials
        const int n0 = n_blk * BN + lane * 4;
        if (n0 < p.N) pre[k] = *reinterpret_cast<const uint2*>(p.residual + static_cast<long long>(m) * p.ldr + n0);
      }
    }
    for (int s0 = 0; s0 < S; s0 += SU) {   // split order: the sum does not depend on timing
      float tmp[SU][U][NV];
#pragma unroll
      for (int ds = 0; ds < SU; ++ds) {
        const int sidx = min(s0 + ds, S - 1);
#pragma unroll
        for (int k = 0; k < U; ++k) {
          const int r = min(r0 + k * nwarps, r_end - 1);
#pragma unroll
          for (int g = 0; g < NSEG; ++g) {
            if (sidx == ks) {   // own partial: shared memory
              const float* src = part + r * kClusterPartStride + seg_off[g];
              if constexpr (SEGW == 4) {
                const float4 f = *reinterpret_cast<const float4*>(src);
                tmp[ds][k][0] = f.x; tmp[ds][k][1] = f.y; tmp[ds][k][2] = f.z; tmp[ds][k][3] = f.w;
              } else {
                const float2 f = *reinterpret_cast<const float2*>(src);
                tmp[ds][k][g * 2] = f.x; tmp[ds][k][g * 2 + 1] = f.y;
              }
            } else {
              const float* src = gbase[k] + sidx * split_stride + seg_off[g];
              if constexpr (SEGW == 4) {
                const float4 f = ldcg4(src);
                tmp[ds][k][0] = f.x; tmp[ds][k][1] = f.y; tmp[ds][k][2] = f.z; tmp[ds][k][3] = f.w;
              } else {
                const float2 f = ldcg2(src);
                tmp[ds][k][g * 2] = f.x; tmp[ds][k][g * 2 + 1] = f.y;
              }
            }
          }
        }
      }
      if constexpr (kQkv) {
        if (s0 == 0) {
#pragma unroll
          for (int k = 0; k < U; ++k) qkv_pre_rope(p, lane, qpre[k]);
        }
      }
#pragma unroll
      for (int ds = 0; ds < SU; ++ds) {
        if (s0 + ds < S) {
#pragma unroll
          for (int k = 0; k < U; ++k)
#pragma unroll
            for (int j = 0; j < NV; ++j) acc[k][j] += tmp[ds][k][j];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int r = r0 + k * nwarps;
      if (r >= r_end) continue;
      const int m = m_row0 + r;
      if (m >= p.M) continue;
      float v[NV];
#pragma unroll
      for (int j = 0; j < NV; ++j) v[j] = acc[k][j];
      apply_unit_epilogue<BN, EPI, NV, SEGW>(p, m, n_blk, lane, v, EPI == EPI_RESIDUAL ? &pre[k] : nullptr,
                                             kQkv ? &qpre[k] : nullptr);
    }
  }
}

template <int BN, int MT, int EPI, int FP8 /* operand mode, OPM_* */, bool PAIR = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_a32, const GemmParams p) {
  static_assert(!PAIR || (MT == 1 && !FP8), "CTA pairs: one 128-row block per CTA, bf16");
  using Cfg = GemmCfg<BN, MT, PAIR, FP8>;
  constexpr bool kBS = Cfg::kBlockScaled;
  constexpr int kTxBytes = Cfg::kTxBytes;
  constexpr int kSfAOff = Cfg::kTileBytes;                       // scale chunks inside a stage: A's, then B's
  constexpr int kSfBOff = Cfg::kTileBytes + Cfg::kSfABytes;
  // CTA pair (launched as clusters of two): one work item is a 256-row x BN tile; the even CTA issues the MMAs for
  // both, each CTA loads its own operand halves and finishes its own 128 accumulator rows.
  constexpr int MTE = PAIR ? 2 : MT;          // 128-row blocks per work item
  const uint32_t crank = PAIR ? cluster_cta_rank() : 0u;
  const bool leader = crank == 0;
  const int work_id = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int work_stride = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int kStages = Cfg::kStages;
  constexpr int kABytes = kBM * kTileKBytes;
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr int kElemsPerKB = FP8 ? 128 : 64;
  constexpr int kAcc = Cfg::kAccStages;

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
  const int splits = p.splits;
  const bool fused_ar = p.ar_world > 0;
  GLLM_TRACE_DECL;
  GLLM_STAMP(threadIdx.x == 0, 0);
  __shared__ unsigned long long ar_expected_s;
  __shared__ unsigned long long ar_launch_s;
  __shared__ unsigned long long ar_local_base_s;
  __shared__ unsigned long long ar_expected2_s;
  const int num_items = p.num_m * p.num_n * splits;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], PAIR ? 8 : 4);   // the epilogue warps of both CTAs of a pair
    }
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  // work item -> (k split, m super tile, n tile); the splits of one output tile are adjacent so
  // they run at the same time and the reduction does not wait long
  auto decode_item = [&](int t, int& ks, int& m_sup, int& n_blk, int& kb0, int& kb1) {
    ks = t % splits;
    const int r = t / splits;
    m_sup = r % p.num_m;
    n_blk = r / p.num_m;
    kb0 = static_cast<int>(static_cast<long long>(ks) * p.num_kb / splits);
    kb1 = static_cast<int>(static_cast<long long>(ks + 1) * p.num_kb / splits);
  };
  // Weight tiles do not depend on the kernel before this one: the producer thread requests the B halves of its
  // first stages before it waits for that kernel (programmatic dependent launch), the A halves after.
  int b_prefetched = 0;
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if constexpr (!PAIR) {
      if (p.mblk_group == nullptr && work_id < num_items) {
        int ks, m_sup, n_blk, kb0, kb1;
        decode_item(work_id, ks, m_sup, n_blk, kb0, kb1);
        const int n_pre = min(kStages, kb1 - kb0);
        for (int i = 0; i < n_pre; ++i) {
          mbar_expect_tx(&full_bar[i], kTxBytes);
          tma_load_2d(tiles + i * kStageBytes + MT * kABytes, &tmap_b, &full_bar[i], (kb0 + i) * kElemsPerKB, n_blk * BN);
          if constexpr (kBS) {
#pragma unroll
            for (int blk = 0; blk < BN / 128; ++blk)
              bulk_load(tiles + i * kStageBytes + kSfBOff + blk * Cfg::kSfChunks * kSfChunkBytes,
                        p.sfb + (static_cast<long long>(n_blk * (BN / 128) + blk) * p.num_kb + (kb0 + i)) *
                                    (Cfg::kSfChunks * kSfChunkBytes),
                        Cfg::kSfChunks * kSfChunkBytes, &full_bar[i]);
          }
        }
        b_prefetched = n_pre;
      }
    }
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_base_ptr, Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_base_ptr, Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  // From here on the kernel reads and writes memory that the kernel before it in the stream may still be using.
  pdl_wait();
  if (fused_ar && threadIdx.x == 0) {
    ar_expected_s = p.ar_state[0];
    ar_launch_s = p.ar_state[1];
    ar_local_base_s = p.ar_state[3];
    ar_expected2_s = p.ar_state[4];
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (!PAIR && FP8 == 0) {
    if (p.ag_world > 0) {
      // the A rows of the other ranks arrive before any A tile is loaded; every CTA of the (co-resident) grid helps
      const unsigned long long ag_launch = p.ag_state[0];
      const bool ag_ok = ag_ll_phase(p, static_cast<int>(ag_launch & 1ull), abort_flag);
      const bool bar_ok = grid_barrier(p.sk_barrier, gridDim.x, p.err, p.wait_ns);
      if (blockIdx.x == 0 && threadIdx.x == 0) p.ag_state[0] = ag_launch + 1ull;   // every CTA read it before the barrier
      if (!ag_ok || !bar_ok) *abort_flag = 1;
      fence_proxy_async_global();
      __syncthreads();
    }
  }
  pdl_launch_dependents();   // the next kernel's CTAs may be scheduled (they wait for this grid in their own pdl_wait)
  if constexpr (PAIR) cluster_barrier();   // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  GLLM_STAMP(threadIdx.x == 0, 1);
  // push all-reduce: epoch of this launch (never 0, the value of untouched flags) and this rank's source index base
  const unsigned int ar_epoch = static_cast<unsigned int>(ar_launch_s & 0x7fffffffull) + 1u;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = work_id; t < num_items && ok; t += work_stride) {
        int ks, m_sup, n_blk, kb0, kb1;
        decode_item(t, ks, m_sup, n_blk, kb0, kb1);
        int b_row = n_blk * BN;
        if (p.mblk_group) {
          const int grp = p.mblk_group[m_sup * MTE];
          if (grp < 0) continue;  // inactive row block of a grouped GEMM (fewer routed rows than the launch was sized for)
          b_row += grp * p.group_rows;
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.err, ERR_TIMEOUT_SMEM_EMPTY, p.wait_ns)) {
            ok = false;
            break;
          }
          uint8_t* sa = tiles + stage * kStageBytes;
          uint8_t* sb = sa + MT * kABytes;
          if constexpr (PAIR) {
            // both CTAs' bytes are credited to the even CTA's barrier, which expects the sum
            if (leader) mbar_expect_tx(&full_bar[stage], 2 * kStageBytes);
            const uint32_t bar0 = cluster_map_addr(smem_u32(&full_bar[stage]), 0);
            tma_load_2d_pair(sa, &tmap_a, bar0, kb * kElemsPerKB, (m_sup * 2 + static_cast<int>(crank)) * kBM);
            tma_load_2d_pair(sb, &tmap_b, bar0, kb * kElemsPerKB, b_row + static_cast<int>(crank) * (BN / 2));
          } else {
            const bool b_done = b_prefetched > 0;   // the first stages' weight halves were requested before pdl_wait
            // grouped GEMM with row counts: only the 32-row pieces of the A tile that hold routed rows travel
            int a_pieces = 4;
            if constexpr (MT == 1) {
              if (p.mblk_rows) a_pieces = min(4, max(1, (p.mblk_rows[m_sup] + 31) >> 5));
            }
            if (b_done) --b_prefetched;
            else mbar_expect_tx(&full_bar[stage], kTxBytes - (4 - a_pieces) * (kABytes / 4));
            if (a_pieces < 4) {
              for (int pc = 0; pc < a_pieces; ++pc)
                tma_load_2d(sa + pc * (kABytes / 4), &tmap_a32, &full_bar[stage], kb * kElemsPerKB, m_sup * kBM + pc * 32);
            } else {
#pragma unroll
              for (int i = 0; i < MT; ++i)
                tma_load_2d(sa + i * kABytes, &tmap_a, &full_bar[stage], kb * kElemsPerKB, (m_sup * MT + i) * kBM);
            }
            if (!b_done) tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kElemsPerKB, b_row);
            if constexpr (kBS) {
              constexpr int kChunkBytes = Cfg::kSfChunks * kSfChunkBytes;   // scale factors of 128 rows for this K block
#pragma unroll
              for (int i = 0; i < MT; ++i)
                bulk_load(sa + kSfAOff + i * kChunkBytes,
                          p.sfa + (static_cast<long long>(m_sup * MT + i) * p.num_kb + kb) * kChunkBytes, kChunkBytes,
                          &full_bar[stage]);
              if (!b_done) {
#pragma unroll
                for (int blk = 0; blk < BN / 128; ++blk)
                  bulk_load(sa + kSfBOff + blk * kChunkBytes,
                            p.sfb + (static_cast<long long>(b_row / 128 + blk) * p.num_kb + kb) * kChunkBytes, kChunkBytes,
                            &full_bar[stage]);
              }
            }
          }
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
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = kBS ? umma_idesc_bs(kBM, BN, FP8 == OPM_NVFP4 ? 1 : 0, FP8 == OPM_MXFP8 ? 1 : 0)
                                     : umma_idesc(PAIR ? 2 * kBM : kBM, BN, FP8 ? 0 : 1, FP8 ? 0 : 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      [[maybe_unused]] uint32_t sf_flip = 0;   // block-scaled modes: which of the two scale-factor column buffers is next
      for (int t = work_id; t < num_items && ok; t += work_stride) {
        int ks, m_sup, n_blk, kb0, kb1;
        decode_item(t, ks, m_sup, n_blk, kb0, kb1);
        if (p.mblk_group && p.mblk_group[m_sup * MTE] < 0) continue;  // skipped by every role alike
        const int it_cur = it++;
        const int acc = it_cur % kAcc;
        const uint32_t acc_phase = (it_cur / kAcc) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.err, ERR_TIMEOUT_TMEM_EMPTY, p.wait_ns)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * (MT * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL, p.wait_ns)) {
            ok = false;
            break;
          }
          tc_fence_after();
          GLLM_STAMP(it_cur == 0 && kb == kb0, 2);
          const uint32_t sa = smem_u32(tiles + stage * kStageBytes);
          const uint64_t b_desc = umma_desc_sw128(sa + MT * kABytes);
          if constexpr (kBS) {
            // scale factors: shared memory -> tensor memory (one of two column buffers, by stage parity), then the
            // block-scaled MMAs; tcgen05.cp and tcgen05.mma of one thread run in issue order
            constexpr int kCh = Cfg::kSfChunks;
            const uint32_t sf_t = tmem_base + kAcc * (MT * BN) + (sf_flip & 1) * (Cfg::kSfColsA + Cfg::kSfColsB);
            ++sf_flip;
            const uint32_t sfb_t = sf_t + Cfg::kSfColsA;
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
              for (int j = 0; j < kCh; ++j)
                tmem_cp_sf(sf_t + (i * kCh + j) * 4, umma_desc_sf(sa + kSfAOff + (i * kCh + j) * kSfChunkBytes));
#pragma unroll
            for (int blk = 0; blk < BN / 128; ++blk)
#pragma unroll
              for (int j = 0; j < kCh; ++j)
                tmem_cp_sf(sfb_t + (j * (BN / 128) + blk) * 4, umma_desc_sf(sa + kSfBOff + (blk * kCh + j) * kSfChunkBytes));
#pragma unroll
            for (int i = 0; i < MT; ++i) {
              const uint64_t a_desc = umma_desc_sw128(sa + i * kABytes);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
                if constexpr (FP8 == OPM_MXFP8) {
                  // one scale per row and MMA (32 elements): byte k of the 32-bit scale columns of this K block
                  umma_mxf8_bs(d_tmem + i * BN, a_desc + 2 * k, b_desc + 2 * k,
                               idesc | (static_cast<uint32_t>(k) << 4) | (static_cast<uint32_t>(k) << 29), accum,
                               sf_t + i * 4, sfb_t);
                } else {
                  // four scales per row and MMA (64 elements in 16s): chunk k of this K block
                  umma_nvf4_bs(d_tmem + i * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, accum, sf_t + (i * kCh + k) * 4,
                               sfb_t + k * (BN / 128) * 4);
                }
              }
            }
          } else {
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            const uint64_t a_desc = umma_desc_sw128(sa + i * kABytes);
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // 4 x 32-byte K slices per 128-byte swizzle row
              const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
              if constexpr (PAIR)
                umma_f16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, accum);
              else if (FP8)
                umma_f8f6f4(d_tmem + i * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, accum);
              else
                umma_f16(d_tmem + i * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, accum);
            }
          }
          }
          if constexpr (PAIR) {   // the stage is free in both CTAs once these MMAs retire
            umma_commit_pair(smem_u32(&empty_bar[stage]));
            umma_commit_pair(cluster_map_addr(smem_u32(&empty_bar[stage]), 1));
          } else {
            umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) {
          if constexpr (PAIR) {
            umma_commit_pair(smem_u32(&tmem_full[acc]));
            umma_commit_pair(cluster_map_addr(smem_u32(&tmem_full[acc]), 1));
          } else {
            umma_commit(&tmem_full[acc]);
          }
        }
        GLLM_STAMP(it_cur == 0, 3);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------- epilogue -----------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int it = 0;
    bool ok = true;
    for (int t = work_id; t < num_items && ok; t += work_stride) {
      int ks, m_sup, n_blk, kb0, kb1;
      decode_item(t, ks, m_sup, n_blk, kb0, kb1);
      if (p.mblk_group && p.mblk_group[m_sup * MTE] < 0) continue;  // skipped by every role alike
      const int it_cur = it++;
      const int acc = it_cur % kAcc;
      const uint32_t acc_phase = (it_cur / kAcc) & 1;
      // warp-uniform decision: tcgen05.ld below is warp-collective
      const bool got = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.err, ERR_TIMEOUT_TMEM_FULL, p.wait_ns);
      if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
      GLLM_STAMP(it_cur == 0 && warp == 4 && lane == 0, 4);
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * (MT * BN);

      // ---- split-K phase 1: dump this CTA's fp32 partial tile; the fused epilogue runs in phase 2 ----
      bool finisher = true;
      if constexpr (BN == 128) {
        if (p.cluster_sk || p.park) {
          // park the fp32 partial tile in shared memory (the pipeline stages are idle: every load of
          // this CTA's only work item was consumed before the accumulator became ready)
          finisher = false;
          float* part = reinterpret_cast<float*>(tiles);
#pragma unroll 1
          for (int i = 0; i < MT; ++i) {
            float* prow = part + static_cast<long long>(i * kBM + q * 32 + lane) * kClusterPartStride;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(taddr0 + i * BN + c * 32, r);
              tmem_ld_wait();
              float4* d4 = reinterpret_cast<float4*>(prow + c * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                d4[j] = make_float4(__uint_as_float(r[j * 4]), __uint_as_float(r[j * 4 + 1]), __uint_as_float(r[j * 4 + 2]),
                                    __uint_as_float(r[j * 4 + 3]));
            }
          }
        }
      }
      bool staged_ll = false;
      if constexpr (EPI == EPI_RESIDUAL && MT == 1 && !PAIR && BN % 128 == 0) {
        if (!p.cluster_sk && !p.park && fused_ar && p.ar_ll) {
          // Low-latency form, several tiles per CTA: the tile's rows go to their owners' receive slots. A thread holds
          // one ROW of the accumulator, so storing from registers would put 16 bytes of 32 different rows into every
          // store instruction (16-byte NVLink writes: measured 80 GB/s). The warp transposes 32 rows x 128 columns
          // through its 8 KB staging area instead and stores 256 contiguous bytes of a row per half warp.
          finisher = false;
          staged_ll = true;
          const long long n_pad = static_cast<long long>(p.num_n) * BN;
          const int rows_per = ar_rows_per(p);
          const int parity = static_cast<int>(ar_launch_s & 1ull);
          uint8_t* stg = smem + kStages * kStageBytes + 1024 + q * 8192;     // [32 rows][16 chunks of 16 bytes], swizzled
          const int m_base = m_sup * kBM + q * 32;
          const float osc = p.out_scale != 0.f ? p.out_scale : 1.0f;
#pragma unroll 1
          for (int h = 0; h < BN / 128; ++h) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(taddr0 + h * 128 + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 w;
                w.x = ll_word(pack_bf16x2(osc * __uint_as_float(r[j * 8 + 0]), osc * __uint_as_float(r[j * 8 + 1])));
                w.y = ll_word(pack_bf16x2(osc * __uint_as_float(r[j * 8 + 2]), osc * __uint_as_float(r[j * 8 + 3])));
                w.z = ll_word(pack_bf16x2(osc * __uint_as_float(r[j * 8 + 4]), osc * __uint_as_float(r[j * 8 + 5])));
                w.w = ll_word(pack_bf16x2(osc * __uint_as_float(r[j * 8 + 6]), osc * __uint_as_float(r[j * 8 + 7])));
                *reinterpret_cast<uint4*>(stg + lane * 256 + (((c * 4 + j) ^ (lane & 15)) << 4)) = w;
              }
            }
            __syncwarp();
            if (!p.ar_drop_flags) {
              const int chunk = lane & 15;
#pragma unroll 1
              for (int rr = 0; rr < 16; ++rr) {
                const int row = 2 * rr + (lane >> 4);
                const int m = m_base + row;
                if (m >= p.M) continue;
                const uint4 w = *reinterpret_cast<const uint4*>(stg + row * 256 + ((chunk ^ (row & 15)) << 4));
                const int owner = m / rows_per, lrow = m - owner * rows_per;
                __nv_bfloat16* dst = ar_ll_recv(p, owner, parity) +
                                     (static_cast<long long>(p.ar_rank) * rows_per + lrow) * n_pad + n_blk * BN + h * 128 +
                                     chunk * 8;
                st_volatile_u4(dst, w);
              }
            }
            __syncwarp();
          }
        }
      }
      if (!staged_ll && !p.cluster_sk && !p.park && (splits > 1 || fused_ar)) {
        finisher = false;
        const long long n_pad = static_cast<long long>(p.num_n) * BN;
        const long long ar_off = fused_ar ? static_cast<long long>(ar_launch_s & 1u) * p.ar_buf_elems : 0;
#pragma unroll 1
        for (int i = 0; i < MT; ++i) {
          const int m = (m_sup * MTE + (PAIR ? static_cast<int>(crank) : i)) * kBM + q * 32 + lane;
          float* dst = p.sk_scratch + (static_cast<long long>(ks) * p.M + m) * n_pad + static_cast<long long>(n_blk) * BN;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr0 + i * BN + c * 32, r);
            tmem_ld_wait();
            if (m < p.M && fused_ar) {
              float v[32];
              const float osc = p.out_scale != 0.f ? p.out_scale : 1.0f;
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = osc * __uint_as_float(r[j]);
              if (p.ar_ll) {
                // low-latency form with several tiles per CTA (prefill sizes): the same self-validating words, stored
                // by the epilogue warps tile after tile; the reduce and gather phases follow the tile loop
                if (!p.ar_drop_flags) {
                  const int rows_per = ar_rows_per(p);
                  const int owner = m / rows_per, lrow = m - owner * rows_per;
                  __nv_bfloat16* dst = ar_ll_recv(p, owner, static_cast<int>(ar_launch_s & 1ull)) +
                                       (static_cast<long long>(ks * p.ar_world + p.ar_rank) * rows_per + lrow) * n_pad +
                                       n_blk * BN + c * 32;
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    uint4 w;
                    w.x = ll_word(pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]));
                    w.y = ll_word(pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]));
                    w.z = ll_word(pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]));
                    w.w = ll_word(pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]));
                    st_volatile_u4(dst + j * 8, w);
                  }
                }
              } else if (p.ar_push) {
                // straight into the receive slots of the rank that owns this row (a peer store over NVLink)
                store_bf16x32(ar_recv_slot(p, ks * p.ar_world + p.ar_rank, m, n_pad, n_blk * BN + c * 32), v);
              } else {
                // this rank's bf16 partial tile, in its own symmetric buffer (peers pull it after the barrier)
                const long long off = ar_off + static_cast<long long>(m) * n_pad + static_cast<long long>(n_blk) * BN + c * 32;
                store_bf16x32(p.ar_peer_buf[p.ar_rank] + off, v);
              }
            } else if (m < p.M) {
              float4* d4 = reinterpret_cast<float4*>(dst + c * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                __stcg(d4 + j, make_float4(__uint_as_float(r[j * 4]), __uint_as_float(r[j * 4 + 1]),
                                           __uint_as_float(r[j * 4 + 2]), __uint_as_float(r[j * 4 + 3])));
            }
          }
        }
        if (fused_ar && p.ar_push) {   // the four epilogue warps stored the tile: release its flags
          epi_bar_sync();
          ar_push_signal(p, static_cast<int>(threadIdx.x) - 128, ks * p.ar_world + p.ar_rank, m_sup, n_blk, MTE * kBM,
                         ar_epoch);
        }
      }

      if (finisher) {
#pragma unroll 1
        for (int i = 0; i < MT; ++i) {
          const int m = (m_sup * MTE + (PAIR ? static_cast<int>(crank) : i)) * kBM + q * 32 + lane;
          bool row_ok = m < p.M;
          if constexpr (MT == 1 && !PAIR) {
            if (p.mblk_rows) {   // padding rows of a grouped block: nothing to read or store
              const int blk_rows = p.mblk_rows[m_sup];
              if (q * 32 >= blk_rows) continue;     // warp-uniform: the whole quarter is padding
              row_ok = row_ok && (q * 32 + lane) < blk_rows;
            }
          }
          const int mm = row_ok ? m : (p.M - 1);
          float rs = row_scale_of(p, mm);
          if (p.a_scale) rs *= p.a_scale[mm];
          AccReader rd;
          rd.taddr = taddr0 + i * BN;

          if constexpr (EPI == EPI_STORE || EPI == EPI_RESIDUAL) {
            float ss = 0.f;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              float v[32];
              rd.load(c * 32, v);
              const int n0 = n_blk * BN + c * 32;
              if (n0 >= p.N) continue;
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= rs;
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
                  const uint4* r4 =
                      reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(m) * p.ldr + n0);
#pragma unroll
                  for (int ii = 0; ii < 4; ++ii) {
                    uint4 u = r4[ii];
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                      float2 f = __bfloat1622float2(h[e]);
                      v[ii * 8 + e * 2] += f.x;
                      v[ii * 8 + e * 2 + 1] += f.y;
                    }
                  }
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  v[j] = bf16_round(v[j]);
                  ss += v[j] * v[j];
                }
              }
              if constexpr (EPI == EPI_STORE) {
                if (p.softcap != 0.f) {   // final-logit soft cap: cap * tanh(x / cap)
                  const float inv_cap = 1.f / p.softcap;
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] = p.softcap * tanhf(v[j] * inv_cap);
                }
              }
              if (p.scatter_meta) {
                if (row_ok) {
                  const int meta = p.scatter_meta[m];
                  if (meta >= 0)
                    store_bf16x32(p.scatter_peer[meta >> 24] + static_cast<long long>(meta & 0xFFFFFF) * p.ldo + n0, v);
                }
              } else if (row_ok) {
                if (p.out_f32) {
                  float4* o4 =
                      reinterpret_cast<float4*>(static_cast<float*>(p.out) + static_cast<long long>(m) * p.ldo + n0);
#pragma unroll
                  for (int ii = 0; ii < 8; ++ii)
                    o4[ii] = make_float4(v[ii * 4], v[ii * 4 + 1], v[ii * 4 + 2], v[ii * 4 + 3]);
                } else {
                  store_bf16x32(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0, v);
                }
              }
            }
            if constexpr (EPI == EPI_RESIDUAL) {
              if (p.row_ss_out && row_ok) p.row_ss_out[static_cast<long long>(m) * p.num_n + n_blk] = ss;
            }
          } else if constexpr (EPI == EPI_GLU) {
            // every 64 tile columns hold 32 gate rows followed by the matching 32 up rows (independent of BN)
            constexpr int kHalf = BN / 2;
#pragma unroll 1
            for (int c = 0; c < kHalf / 32; ++c) {
              float g[32], u[32];
              rd.load(c * 64, g);
              rd.load(c * 64 + 32, u);
              const int n0 = n_blk * kHalf + c * 32;  // output column
              if (n0 >= p.N / 2) continue;
              float v[32];
              if (p.b_scale) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  g[j] *= p.b_scale[n_blk * BN + c * 64 + j];
                  u[j] *= p.b_scale[n_blk * BN + c * 64 + 32 + j];
                }
              }
              if (p.glu_act == 0) {   // the activation choice is hoisted out of the element loop
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = silu_f(g[j] * rs) * (u[j] * rs);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_f(g[j] * rs) * (u[j] * rs);
              }
              if (row_ok)
                store_bf16x32(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(m) * p.ldo + n0, v);
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
                float v[32];
                rd.load(c * 32, v);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  float x = v[j] * rs;
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
            uint8_t* dst8 = nullptr;     // fp8 cache row
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
                  if (p.kv_fp8)
                    dst8 = reinterpret_cast<uint8_t*>(p.kv_cache) + (base * kPageTokens + off) * 128;
                  else
                    dst = p.kv_cache + (base * kPageTokens + off) * 128;
                }
              }
            }
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {  // columns [32c, 32c+32) pair with [64+32c, 64+32c+32)
              float lo[32], hi[32];
              rd.load(c * 32, lo);
              rd.load(64 + c * 32, hi);
              float a[32], b[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x0 = lo[j] * rs;
                float x1 = hi[j] * rs;
                if (p.bias) {
                  x0 += p.bias[head * 128 + c * 32 + j];
                  x1 += p.bias[head * 128 + 64 + c * 32 + j];
                }
                a[j] = x0;
                b[j] = x1;
              }
              if (nw) {   // per-head norm weights as 16-byte loads (the same 128 floats for every row)
                const float4* w0 = reinterpret_cast<const float4*>(nw + c * 32);
                const float4* w1 = reinterpret_cast<const float4*>(nw + 64 + c * 32);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                  const float4 wa = __ldg(w0 + jj), wb = __ldg(w1 + jj);
                  a[jj * 4 + 0] *= inv_rms * wa.x; a[jj * 4 + 1] *= inv_rms * wa.y;
                  a[jj * 4 + 2] *= inv_rms * wa.z; a[jj * 4 + 3] *= inv_rms * wa.w;
                  b[jj * 4 + 0] *= inv_rms * wb.x; b[jj * 4 + 1] *= inv_rms * wb.y;
                  b[jj * 4 + 2] *= inv_rms * wb.z; b[jj * 4 + 3] *= inv_rms * wb.w;
                }
              }
              if (is_q || is_k) {
                // this row's 32 cos / sin values as 16-byte loads (table rows are 256 bytes, 128-byte aligned here)
                const float4* c4 = reinterpret_cast<const float4*>(p.cos_table + static_cast<long long>(pos) * 64 + c * 32);
                const float4* s4 = reinterpret_cast<const float4*>(p.sin_table + static_cast<long long>(pos) * 64 + c * 32);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                  const float4 cs = __ldg(c4 + jj), sn = __ldg(s4 + jj);
                  const float cv[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float x0 = a[jj * 4 + e], x1 = b[jj * 4 + e];
                    a[jj * 4 + e] = x0 * cv[e] - x1 * sv[e];
                    b[jj * 4 + e] = x1 * cv[e] + x0 * sv[e];
                  }
                }
              }
              if (dst) {
                store_bf16x32(dst + c * 32, a);
                store_bf16x32(dst + 64 + c * 32, b);
              } else if (dst8) {
                store_fp8x32(dst8 + c * 32, a, p.kv_inv_scale);
                store_fp8x32(dst8 + 64 + c * 32, b, p.kv_inv_scale);
              }
            }
          }
        }
      }
      // hand the accumulator slot back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && !leader)
          mbar_arrive_cluster(cluster_map_addr(smem_u32(&tmem_empty[acc]), 0));
        else
          mbar_arrive(&tmem_empty[acc]);
      }
      GLLM_STAMP(it_cur == 0 && warp == 4 && lane == 0, 5);
    }
  }

  tc_fence_before();
  __syncthreads();
  // a pair leaves together: the even CTA's MMAs read the partner's shared memory and signal its barriers
  if constexpr (PAIR) cluster_barrier();
  tc_fence_after();
  if (warp == 2) {
    if constexpr (PAIR)
      tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else
      tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  GLLM_STAMP(threadIdx.x == 0, 6);

  if constexpr (BN == 128) {
    if (p.cluster_sk) {
      // one work item per CTA: blockIdx.x is the item; its splits are the CTAs of this cluster
      int ks, m_sup, n_blk, kb0, kb1;
      decode_item(blockIdx.x, ks, m_sup, n_blk, kb0, kb1);
      const float* part = reinterpret_cast<const float*>(tiles);
      cluster_publish_partials(p, part, MT * kBM, m_sup * MT * kBM, n_blk, splits, ks);
      cluster_barrier();   // release / acquire at cluster scope: the members' scratch rows are visible
      GLLM_STAMP(threadIdx.x == 0, 7);
      cluster_reduce_phase<EPI>(p, part, MT * kBM, m_sup * MT * kBM, n_blk, splits, ks);
      GLLM_STAMP(threadIdx.x == 0, 8);
      return;
    }
  }
  if constexpr (BN == 128) {
    if (p.park) {
      // every warp writes whole rows of the parked tile: 512 (fp32 scratch) or 256 (bf16 all-reduce buffer)
      // contiguous bytes per store instruction instead of 64-byte pieces of 32 different rows
      int ks = 0, m_sup = 0, n_blk = 0, kb0, kb1;
      const bool has_item = static_cast<int>(blockIdx.x) < num_items;   // the fused all-reduce launches every SM
      if (has_item) decode_item(blockIdx.x, ks, m_sup, n_blk, kb0, kb1);
      const float* part = reinterpret_cast<const float*>(tiles);
      if (fused_ar && p.ar_ll) {
        if (has_item && !p.ar_drop_flags)
          ar_ll_push_parked(p, part, MT * kBM, m_sup * MT * kBM, n_blk, ks * p.ar_world + p.ar_rank,
                            static_cast<int>(ar_launch_s & 1ull));
      } else if (fused_ar && p.ar_push) {
        if (has_item) ar_push_parked(p, part, MT * kBM, m_sup * MT * kBM, n_blk, ks * p.ar_world + p.ar_rank);
        __syncthreads();
        if (has_item) ar_push_signal(p, threadIdx.x, ks * p.ar_world + p.ar_rank, m_sup, n_blk, MT * kBM, ar_epoch);
      } else if (fused_ar) {
        const long long n_pad = static_cast<long long>(p.num_n) * BN;
        __nv_bfloat16* dst = p.ar_peer_buf[p.ar_rank] + static_cast<long long>(ar_launch_s & 1u) * p.ar_buf_elems +
                             static_cast<long long>(ks) * p.M * n_pad + static_cast<long long>(n_blk) * BN + lane * 4;
        for (int r = warp; has_item && r < MT * kBM; r += kGemmThreads / 32) {
          const int m = m_sup * MT * kBM + r;
          if (m >= p.M) continue;
          const float4 v = *reinterpret_cast<const float4*>(part + r * kClusterPartStride + lane * 4);
          uint2 w;
          w.x = pack_bf16x2(v.x, v.y);
          w.y = pack_bf16x2(v.z, v.w);
          *reinterpret_cast<uint2*>(dst + static_cast<long long>(m) * n_pad) = w;
        }
      } else {
        if (has_item)
          cluster_publish_partials(p, part, MT * kBM, m_sup * MT * kBM, n_blk, /*S=*/1, /*ks=*/ks, /*skip_own=*/false,
                                   /*halves_interleaved=*/EPI == EPI_QKV);
      }
    }
  }
  if constexpr (BN % 128 == 0) {  // 192-wide tiles never split (their lanes would need 12-byte vectors)
    if (fused_ar && p.ar_ll) {
      if constexpr (EPI == EPI_RESIDUAL) {
        GLLM_STAMP(threadIdx.x == 0, 7);     // tile sent
        const int parity = static_cast<int>(ar_launch_s & 1ull);
        ar_ll_reduce<BN>(p, parity, abort_flag);
        GLLM_STAMP(threadIdx.x == 0, 9);     // this CTA's share of the owned rows reduced and sent to every rank
        if (!p.ar_rs_only) ar_ll_gather<BN>(p, parity, abort_flag);
        ar_ll_advance(p, ar_launch_s);
      }
    } else if (fused_ar && p.ar_push) {
      if constexpr (EPI == EPI_RESIDUAL) {
        GLLM_STAMP(threadIdx.x == 0, 7);     // tiles pushed, flags released
        ar_push_reduce<BN>(p, ar_epoch, MTE * kBM, abort_flag);
        GLLM_STAMP(threadIdx.x == 0, 9);     // this CTA's share of the rows reduced and stored to every rank
        ar_push_finish(p, static_cast<unsigned long long>(ar_epoch), ar_launch_s);
      }
    } else if (fused_ar) {
      // one arrival per rank once all of that rank's CTAs have published their tiles
      const unsigned long long target = ar_expected_s + static_cast<unsigned long long>(p.ar_world);
      const unsigned long long local_target = ar_local_base_s + gridDim.x;
      const bool ar_ok = ar_barrier(p, target, local_target);
      GLLM_STAMP(threadIdx.x == 0, 7);
      unsigned long long local_done = local_target;
      if constexpr (EPI == EPI_RESIDUAL) {
        const long long part_off = static_cast<long long>(ar_launch_s & 1u) * p.ar_buf_elems;
        const long long split_elems = static_cast<long long>(p.M) * p.num_n * BN;
        if (p.ar_two_shot) {
          // reduce-scatter by pull, broadcast by store, second meeting on the other counter word, local gather
          const int rows_per = (p.M + p.ar_world - 1) / p.ar_world;
          const int own_lo = min(p.M, p.ar_rank * rows_per), own_hi = min(p.M, own_lo + rows_per);
          const long long bcast_off = 2 * p.ar_buf_elems;
          if (ar_ok) ar_reduce_phase<BN, 1>(p, part_off, splits, split_elems, own_lo, own_hi, bcast_off);
          local_done = local_target + gridDim.x;
          const unsigned long long target2 = ar_expected2_s + static_cast<unsigned long long>(p.ar_world);
          const bool ok2 = ar_barrier(p, target2, local_done, 1);
          if (ar_ok && ok2) ar_gather_phase<BN>(p, bcast_off, own_lo, own_hi);
          if (blockIdx.x == 0 && threadIdx.x == 0) p.ar_state[4] = target2;
        } else if (ar_ok) {
          ar_reduce_phase<BN, 4>(p, part_off, splits, split_elems, 0, p.M, -1);
        }
      }
      // Safe to advance the launch state: every CTA of this rank read it before arriving at the barrier.
      if (blockIdx.x == 0 && threadIdx.x == 0) {
        p.ar_state[0] = target;
        p.ar_state[1] = static_cast<unsigned long long>(ar_launch_s) + 1ull;
        p.ar_state[3] = local_done;
      }
    } else if (splits > 1) {
      // every partial of every CTA must be visible before anyone reduces
      const bool bar_ok = grid_barrier(p.sk_barrier, gridDim.x, p.err, p.wait_ns);
      GLLM_STAMP(threadIdx.x == 0, 7);
      if (bar_ok) splitk_reduce_phase<BN, EPI>(p, p.sk_scratch, splits, false);
    }
  }
  GLLM_STAMP(threadIdx.x == 0, 8);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static long long* g_trace_ptr = nullptr;
static int g_trace_k = 0;   // when non-zero only launches with this K are traced
static int g_trace_n = 0;   // likewise for N

struct SplitKWorkspace {
  float* scratch = nullptr;
  long long scratch_floats = 0;
  unsigned int* barrier = nullptr;
};
static SplitKWorkspace g_splitk[64];          // per device: used by every stream without a workspace of its own
// Streams with their own split-K scratch and barrier words (gllm_gemm_set_splitk_workspace_stream): GEMMs launched on
// two such streams, or on one of them and on the default workspace, do not share a partial-sum buffer or a barrier,
// so they may overlap. Append-only; readers take no lock.
struct StreamWorkspace {
  int dev;
  cudaStream_t stream;
  SplitKWorkspace ws;
};
constexpr int kMaxStreamWorkspaces = 16;
static StreamWorkspace g_stream_ws[kMaxStreamWorkspaces];
static std::atomic<int> g_stream_ws_n{0};
static std::mutex g_stream_ws_mu;
static const SplitKWorkspace& workspace_for(int dev, cudaStream_t stream) {
  const int n = g_stream_ws_n.load(std::memory_order_acquire);
  for (int i = 0; i < n; ++i)
    if (g_stream_ws[i].dev == dev && g_stream_ws[i].stream == stream) return g_stream_ws[i].ws;
  return g_splitk[dev & 63];
}

// Pick the number of K splits with a small cost model (microseconds): one SM pulls about 100 GB/s into
// shared memory, work items run in waves of `sms`, a split costs the dump of its partial tile, and the
// reduce phase re-reads all partials at a few TB/s after one grid barrier.
static int choose_splits(int tiles, int num_kb, int stage_bytes, long long tile_floats, long long out_floats, int sms,
                         long long scratch_floats, bool cluster_ok) {
  if (tiles >= 2 * sms || num_kb < 4) return 1;
  double best = 1e30;
  int best_s = 1;
  for (int s = 1; s <= kMaxSplits && s * 2 <= num_kb; ++s) {
    if (s > 1 && s * out_floats > scratch_floats) break;
    const int items = tiles * s;
    const int waves = (items + sms - 1) / sms;
    const double kb = (num_kb + s - 1) / s;
    double t_item = kb * stage_bytes / 100e3 + 2.0;
    double total;
    if (s == 1) {
      total = waves * (t_item + tile_floats * 4 / 200e3);
    } else if (cluster_ok && s <= 8 && items <= sms) {
      // cluster split-K: partials stay in shared memory, one cluster barrier, rows reduced through DSMEM
      total = t_item + 2.5;
    } else {
      t_item += tile_floats * 4 / 100e3;
      total = waves * t_item + 2.0 + (double)s * out_floats * 4 / 3.5e6 + 1.5;
    }
    if (total < best * 0.95) {  // prefer fewer splits unless clearly better
      best = total;
      best_s = s;
    }
  }
  return best_s;
}

// The all-gather descriptor of the NEXT single-CTA bf16 GEMM launched by this thread (gllm_gemm_set_allgather_input).
struct PendingAllGather {
  bool active = false;
  int world = 0, rank = 0;
  const void* src = nullptr; long long src_ld = 0;
  void* dst = nullptr; long long dst_ld = 0;
  void* peer[8] = {}; void* mc = nullptr;
  long long slot_off = 0, slot_bytes = 0;
  unsigned long long* state = nullptr;
  float* ss_out = nullptr;
};
static thread_local PendingAllGather g_pending_ag;
static thread_local const int* g_pending_block_rows = nullptr;

template <int BN, int MT, int EPI, int FP8>
static int launch_gemm(const void* A, long long lda, const void* B, long long ldb, long long b_rows, GemmParams p,
                       cudaStream_t stream, int max_ctas, int force_splits) {
  using Cfg = GemmCfg<BN, MT, false, FP8>;
  if (g_pending_ag.active) {
    PendingAllGather ag = g_pending_ag;
    g_pending_ag.active = false;
    if (FP8 != 0 || p.mblk_group != nullptr || p.K % 256 != 0 || A != ag.dst || lda != ag.dst_ld || p.ar_world > 0 ||
        static_cast<long long>(p.M) * p.K * 2 > ag.slot_bytes) {
      set_last_error("gemm with all-gathered A: needs a bf16, ungrouped GEMM whose A is the gather destination, K %% 256 "
                     "== 0 and %lld slot bytes (have %lld)", static_cast<long long>(p.M) * p.K * 2, ag.slot_bytes);
      return -1;
    }
    p.ag_world = ag.world; p.ag_rank = ag.rank;
    p.ag_src = static_cast<const __nv_bfloat16*>(ag.src); p.ag_src_ld = ag.src_ld;
    p.ag_dst = static_cast<__nv_bfloat16*>(ag.dst); p.ag_dst_ld = ag.dst_ld;
    for (int r = 0; r < ag.world; ++r) p.ag_peer[r] = static_cast<char*>(ag.peer[r]);
    p.ag_mc = static_cast<char*>(ag.mc);
    p.ag_slot_off = ag.slot_off; p.ag_slot_bytes = ag.slot_bytes; p.ag_state = ag.state;
    p.ag_ss_out = ag.ss_out;
    p.peer_wait_ns = static_cast<unsigned long long>(settings().peer_wait_ns);
  }
  constexpr int kElemsPerKB = FP8 ? 128 : 64;
  const int esz = FP8 ? 1 : 2;
  const CUtensorMapDataType dt = FP8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) {
    set_last_error("gemm: empty problem M=%d N=%d K=%d", p.M, p.N, p.K);
    return -1;
  }
  if (p.N % 32 != 0) {
    set_last_error("gemm: N=%d must be a multiple of 32 (pad the weight at load time)", p.N);
    return -1;
  }
  p.trace = ((g_trace_k == 0 || g_trace_k == p.K) && (g_trace_n == 0 || g_trace_n == p.N)) ? g_trace_ptr : nullptr;
  const RuntimeSettings& rt = settings();
  p.wait_ns = rt.wait_ns;
  p.peer_wait_ns = rt.peer_wait_ns;
  p.num_m = (p.M + MT * kBM - 1) / (MT * kBM);
  p.num_n = (p.N + BN - 1) / BN;
  // tensor-map columns: elements for bf16 / fp8, BYTES for the packed 4-bit operands (two elements per byte)
  const int kcols = (FP8 == OPM_NVFP4) ? p.K / 2 : p.K;
  p.num_kb = (kcols + kElemsPerKB - 1) / kElemsPerKB;
  if (Cfg::kBlockScaled) {
    if (!p.sfa || !p.sfb || kcols % 128 != 0 || ((reinterpret_cast<uintptr_t>(p.sfa) | reinterpret_cast<uintptr_t>(p.sfb)) & 15) ||
        (p.mblk_group && p.group_rows % 128 != 0)) {
      set_last_error("block-scaled gemm: needs 16-byte aligned scale chunks, K a multiple of %d, expert rows %% 128",
                     FP8 == OPM_NVFP4 ? 256 : 128);
      return -1;
    }
  }
  CUtensorMap ta, tb, ta32;
  if (make_tmap_2d(&ta, A, dt, esz, uint64_t(p.M), uint64_t(kcols), uint64_t(lda), kBM, kElemsPerKB)) return -1;
  if (make_tmap_2d(&tb, B, dt, esz, uint64_t(b_rows), uint64_t(kcols), uint64_t(ldb), BN, kElemsPerKB)) return -1;
  if (make_tmap_2d(&ta32, A, dt, esz, uint64_t(p.M), uint64_t(kcols), uint64_t(lda), 32, kElemsPerKB)) return -1;
  if (g_pending_block_rows) {      // set for the next grouped launch of this thread (gllm_gemm_set_block_rows)
    if (p.mblk_group && MT == 1) p.mblk_rows = g_pending_block_rows;
    g_pending_block_rows = nullptr;
  }
  static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the kernel
  auto kern = gemm_tn_kernel<BN, MT, EPI, FP8>;
  // the residual kernels carry 32 KB of staging behind the barriers (four epilogue warps x 8 KB): the multi-tile
  // low-latency all-reduce transposes its rows there
  constexpr int kSmemLaunch = Cfg::kSmemBytes + ((EPI == EPI_RESIDUAL && MT == 1 && BN % 128 == 0) ? 32768 : 0);
  static_assert(kSmemLaunch <= 232448 - 512, "dynamic shared memory beyond 227 KB");
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLaunch);
    if (e != cudaSuccess) {
      set_last_error("gemm: cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
      return -1;
    }
    attr_set[dev & 63] = true;
  }
  int sms = max_ctas;
  if (sms <= 0) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = p.num_m * p.num_n;
  const SplitKWorkspace& ws = workspace_for(dev, stream);
  const long long tile_floats = static_cast<long long>(MT) * kBM * BN;
  const long long out_floats = static_cast<long long>(p.M) * p.num_n * BN;
  int splits = 1;
  if (p.mblk_group || BN % 128 != 0) force_splits = 1;  // grouped GEMMs have plenty of tiles
  const bool park_allowed = rt.park != 0;
  const bool part_fits = static_cast<long long>(MT) * kBM * kClusterPartStride * 4 <= static_cast<long long>(Cfg::kStages) * Cfg::kStageBytes;
  if (p.ar_world > 0) {
    // Fused all-reduce: a rank may split K locally when every work item gets its own CTA (the parked-tile path):
    // split s publishes its bf16 partial in buffer slice s and the pull adds the slices of every rank. Halves the
    // main loop of the decode-sized row-parallel GEMMs (64 tiles on 148 SMs).
    splits = 1;
    const bool ar_split_allowed = rt.ar_split != 0;
    // Pull forms, only with two ranks: the pull moves (ranks x splits) partial buffers per output element, and from
    // four ranks on that traffic (every rank reads every rank's buffer) costs more than the shorter main loop saves.
    // Push form, any rank count: the extra partials travel while the main loops run and are added from local memory.
    if (BN == 128 && park_allowed && part_fits && ar_split_allowed && force_splits <= 0 && p.mblk_group == nullptr &&
        (p.ar_world <= 2 || p.ar_push || p.ar_ll)) {
      int sp = sms / (tiles > 0 ? tiles : 1);
      if (sp > 4) sp = 4;
      if (sp > p.num_kb / 8) sp = p.num_kb / 8;
      if (p.ar_ll) {
        // every split is one more source the owner polls and adds and one more partial on the wire: from eight ranks
        // on the shorter main loop no longer pays (measured at eight ranks: 5.04 ms per step without, 5.08 ms with)
        if (p.ar_world >= 8) sp = 1;
        const long long rows_per = (p.M + p.ar_world - 1) / p.ar_world;
        while (sp > 1 && static_cast<long long>(p.ar_world) * sp * rows_per * p.num_n * BN * 2 > p.ar_ll_recv_bytes) --sp;
      } else if (p.ar_push) {
        // a warp waits with one lane per (source, n tile) flag; the receive slots hold (world x splits) sources
        while (sp > 1 && p.ar_world * sp * (256 / BN) > 32) --sp;
        const long long rows_per = (p.M + p.ar_world - 1) / p.ar_world;
        while (sp > 1 && static_cast<long long>(p.ar_world) * sp * rows_per * p.num_n * BN > p.ar_buf_elems) --sp;
      } else {
        while (sp > 1 && sp * out_floats > p.ar_buf_elems) --sp;
      }
      if (sp >= 2) splits = sp;
    }
  } else if (force_splits > 0)
    splits = force_splits;
  else if (ws.scratch)
    splits = choose_splits(tiles, p.num_kb, Cfg::kStageBytes, tile_floats, out_floats, sms, ws.scratch_floats,
                           BN == 128 && max_ctas <= 0 && rt.cluster_sk != 0);
  if (p.ar_world > 0 && p.ar_ll) {
    const long long rows_per = (p.M + p.ar_world - 1) / p.ar_world;
    const long long n_pad = static_cast<long long>(p.num_n) * BN;
    const long long need = static_cast<long long>(p.ar_world) * splits * rows_per * n_pad * 2;
    const long long need_res = static_cast<long long>(p.M) * n_pad * 2;
    // one parked tile per CTA (decode sizes), or any number of tiles per CTA without a local K split (prefill sizes)
    const bool parks = BN == 128 && park_allowed && part_fits && tiles * splits <= sms && p.mblk_group == nullptr;
    if ((!parks && splits != 1) || p.mblk_group != nullptr || need > p.ar_ll_recv_bytes ||
        (!p.ar_rs_only && need_res > p.ar_ll_res_bytes) || n_pad % 256 != 0) {
      set_last_error("fused all-reduce (low latency): %d tiles x %d splits on %d SMs, %lld receive bytes (have %lld), "
                     "%lld result bytes (have %lld), padded width %% 256",
                     tiles, splits, sms, need, p.ar_ll_recv_bytes, need_res, p.ar_ll_res_bytes);
      return -1;
    }
  } else if (p.ar_world > 0 && p.ar_push) {
    const long long rows_per = (p.M + p.ar_world - 1) / p.ar_world;
    const long long need = static_cast<long long>(p.ar_world) * splits * rows_per * p.num_n * BN;
    const long long nflags = static_cast<long long>(p.ar_world) * splits * p.num_m * p.num_n;
    if (need > p.ar_buf_elems || nflags > p.ar_flag_cap || (static_cast<long long>(p.num_n) * BN) % 256 != 0 ||
        p.ar_world * splits * (256 / BN) > 32) {
      set_last_error("fused all-reduce (push): needs %lld receive elements (have %lld) and %lld flags (have %lld), "
                     "padded width %% 256", need, p.ar_buf_elems, nflags, p.ar_flag_cap);
      return -1;
    }
  } else if (p.ar_world > 0) {
    if (splits * out_floats > p.ar_buf_elems || (static_cast<long long>(p.num_n) * BN) % 256 != 0) {
      set_last_error("fused all-reduce: output needs %lld elements per buffer (have %lld), padded width %% 256",
                     splits * out_floats, p.ar_buf_elems);
      return -1;
    }
  } else if (splits > 1) {
    if (!ws.scratch || splits * out_floats > ws.scratch_floats || splits > p.num_kb || splits > kMaxSplits) {
      set_last_error("gemm: split-K=%d needs %lld scratch floats (have %lld), K blocks %d", splits,
                     splits * out_floats, ws.scratch_floats, p.num_kb);
      return -1;
    }
  }
  p.splits = splits;
  p.sk_scratch = ws.scratch;
  p.sk_barrier = ws.barrier;
  const int items = tiles * splits;
  // the fused all-reduce launches every SM: CTAs without a tile still pull and finish their share of the rows
  const int grid = (p.ar_world > 0) ? sms : (items < sms ? items : sms);
  // Cluster split-K: the splits of a tile become one thread-block cluster (one work item per CTA) and reduce through
  // distributed shared memory instead of global scratch + grid barrier.
  const bool cluster_allowed = rt.cluster_sk != 0;
  if (BN == 128 && cluster_allowed && splits >= 2 && splits <= 8 && items <= sms && part_fits && p.ar_world == 0 &&
      p.ag_world == 0 &&
      p.mblk_group == nullptr && max_ctas <= 0) {
    p.cluster_sk = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(items, 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemLaunch;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // Clusters are placed inside one GPC; when the GPC sizes do not let every cluster of this launch run at once the
    // launch would take a second wave, which costs more than the reduce saves: use the global-scratch path then.
    static int max_clusters[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // per cluster size, 0 = not queried yet
    if (max_clusters[splits] == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        n = -1;
      }
      max_clusters[splits] = n > 0 ? n : -1;
    }
    if (max_clusters[splits] >= tiles) {
      cfg.numAttrs = rt.pdl ? 2 : 1;
      cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, ta, tb, ta32, p);
      if (ce == cudaSuccess) return 0;
      (void)cudaGetLastError();   // this cluster shape cannot be scheduled here: fall back
    }
    p.cluster_sk = 0;
  }
  p.park = (BN == 128 && park_allowed && (splits > 1 || p.ar_world > 0) && items <= grid && part_fits &&
            p.mblk_group == nullptr) ? 1 : 0;
  cudaError_t e = launch_kernel(kern, dim3(grid), dim3(kGemmThreads), kSmemLaunch, stream, true, 0, ta, tb, ta32, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_last_error("gemm launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

// Which GEMMs run on CTA pairs: 128 < M <= g_pair_max_m and the epilogue's bit set in g_pair_epi_mask. Measured at
// M = 256 (B200): the pair main loop issues one 256 x N x 16 MMA per ~150 clocks for N = 128 and N = 256 alike, so it
// only pays for wide tiles, and at decode sizes the single-CTA kernels end up ahead everywhere (gate/up with 192-wide
// tiles: 52.9 vs 57.0 us; o_proj 22 vs 28 us; QKV 33 vs 41 us), so no decode epilogue uses pairs by default.
// At prefill sizes (M = 8192) 256 x 256 pair tiles run 1.4-3.5 % faster than 256 x 256 single-CTA tiles (plain
// 1333 vs 1288 TFLOP/s, residual 1324 vs 1292, gate/up 1340 vs 1321), so 256-wide launches with M >= g_pair_big_m
// use them too; the one-head-per-tile QKV GEMM does not (729 vs 948 TFLOP/s).
// (settings pair_max_m / pair_epi_mask / pair_big_m of RuntimeSettings; the Python layer maps the GLLM_PAIR* environment
// variables onto them when it loads the library)
#define g_pair_max_m (settings().pair_max_m)
#define g_pair_epi_mask (settings().pair_epi_mask)
#define g_pair_big_m (settings().pair_big_m)
static int pair_max_m_setting() { return settings().pair_max_m; }

// CTA-pair launch (clusters of two, `tcgen05.mma.cta_group::2`): a work item is a 256-row x BN tile. Per 64-deep K
// block each SM ingests 16 KB of A and BN/2 rows of B instead of 32 KB + BN rows for a 256-row single-CTA tile, and the
// tensor core reads half as much B from shared memory per MMA; that is what decode-sized M (129..256 rows) is bound by.
template <int BN, int EPI>
static int launch_gemm_pair(const void* A, long long lda, const void* B, long long ldb, long long b_rows, GemmParams p,
                            cudaStream_t stream, int force_splits) {
  using Cfg = GemmCfg<BN, 1, true>;
  constexpr int kElemsPerKB = 64;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.N % 32 != 0) {
    set_last_error("gemm (pair): bad problem M=%d N=%d K=%d", p.M, p.N, p.K);
    return -1;
  }
  p.trace = ((g_trace_k == 0 || g_trace_k == p.K) && (g_trace_n == 0 || g_trace_n == p.N)) ? g_trace_ptr : nullptr;
  const RuntimeSettings& rt = settings();
  p.wait_ns = rt.wait_ns;
  p.peer_wait_ns = rt.peer_wait_ns;
  p.num_m = (p.M + 2 * kBM - 1) / (2 * kBM);
  p.num_n = (p.N + BN - 1) / BN;
  p.num_kb = (p.K + kElemsPerKB - 1) / kElemsPerKB;
  p.cluster_sk = 0;
  p.park = 0;
  CUtensorMap ta, tb;
  if (make_tmap_2d(&ta, A, dt, 2, uint64_t(p.M), uint64_t(p.K), uint64_t(lda), kBM, kElemsPerKB)) return -1;
  if (make_tmap_2d(&tb, B, dt, 2, uint64_t(b_rows), uint64_t(p.K), uint64_t(ldb), BN / 2, kElemsPerKB)) return -1;
  auto kern = gemm_tn_kernel<BN, 1, EPI, false, true>;
  static bool attr_set[64] = {};   // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) {
      set_last_error("gemm (pair): cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
      return -1;
    }
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // how many pairs can be resident at once (the split-K grid barrier needs every CTA of the launch running)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms & ~1, 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      n = -1;
    }
    max_pairs = n > 0 ? n : -1;
  }
  if (max_pairs <= 0) {
    set_last_error("gemm (pair): clusters of two cannot be scheduled on this device");
    return -1;
  }
  const int tiles = p.num_m * p.num_n;
  const SplitKWorkspace& ws = workspace_for(dev, stream);
  const long long tile_floats = 2ll * kBM * BN;
  const long long out_floats = static_cast<long long>(p.M) * p.num_n * BN;
  int splits = 1;
  if (BN % 128 != 0) force_splits = 1;
  if (force_splits > 0)
    splits = force_splits;
  else if (ws.scratch)
    splits = choose_splits(tiles, p.num_kb, Cfg::kStageBytes, tile_floats / 2, out_floats, max_pairs, ws.scratch_floats, false);
  if (splits > 1 && (!ws.scratch || splits * out_floats > ws.scratch_floats || splits > p.num_kb || splits > kMaxSplits)) {
    set_last_error("gemm (pair): split-K=%d needs %lld scratch floats (have %lld), K blocks %d", splits,
                   splits * out_floats, ws.scratch_floats, p.num_kb);
    return -1;
  }
  p.splits = splits;
  p.sk_scratch = ws.scratch;
  p.sk_barrier = ws.barrier;
  const int items = tiles * splits;
  const int pairs = items < max_pairs ? items : max_pairs;
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.numAttrs = rt.pdl ? 2 : 1;
  cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, ta, tb, ta, p);
  if (ce != cudaSuccess) {
    (void)cudaGetLastError();
    set_last_error("gemm (pair) launch failed: %s", cudaGetErrorString(ce));
    return -1;
  }
  return 0;
}

// Dispatch on (tile width, rows per CTA). Small M uses 256-row CTA tiles so a weight tile is pulled
// into shared memory once for the whole batch; large M keeps 128 x 256 tiles with a double-buffered
// accumulator so the epilogue overlaps the next main loop.
// Block-scaled operands: 128 x 128 and 256 x 128 (two accumulators share a weight tile) tiles, or 128 x 256 tiles at
// prefill sizes (tensor memory holds the accumulators and the scale-factor columns).
template <int EPI, int OPM>
static int dispatch_gemm_bs(const void* A, long long lda, const void* B, long long ldb, long long b_rows,
                            const GemmParams& p, int bn, cudaStream_t stream, int max_ctas, int force_splits) {
  // the fused all-reduce keeps 128-row tiles (one parked tile per CTA at decode sizes, staged rows at prefill sizes)
  const bool rows2 = p.M > 128 && p.M <= 1024 && p.mblk_group == nullptr && p.ar_world == 0;
  if constexpr (EPI != EPI_QKV) {
    if (bn == 256 && !rows2) return launch_gemm<256, 1, EPI, OPM>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
  }
  if (rows2 || (EPI == EPI_QKV && p.M > 128))
    return launch_gemm<128, 2, EPI, OPM>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
  return launch_gemm<128, 1, EPI, OPM>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
}

template <int EPI, int FP8>
static int dispatch_gemm(const void* A, long long lda, const void* B, long long ldb, long long b_rows,
                         const GemmParams& p, int bn, cudaStream_t stream, int max_ctas, int force_splits) {
  static_assert(FP8 < OPM_MXFP8, "block-scaled modes go through dispatch_gemm_bs");
  if constexpr (!FP8) {
    // decode-sized M: CTA pairs (gllm_gemm_set_pair / GLLM_PAIR / GLLM_PAIR_MAX_M choose where they are used)
    const int pair_max_m = pair_max_m_setting();
    bool use_pair = p.M > 128 && p.M <= pair_max_m && ((g_pair_epi_mask >> EPI) & 1) && p.mblk_group == nullptr &&
                    p.ar_world == 0 && p.scatter_meta == nullptr && max_ctas <= 0;
    const bool ag_pending = g_pending_ag.active;      // the CTA-pair kernels have no all-gather phase
    if (EPI == EPI_GLU && g_pair_epi_mask != 0xF && bn < 192) use_pair = false;   // narrow GLU tiles: single CTAs win
    if (EPI == EPI_GLU && !use_pair && g_pair_max_m > 0 && p.M > 128 && p.M <= g_pair_max_m && bn >= 192 &&
        p.mblk_group == nullptr && p.ar_world == 0 && max_ctas <= 0) {
      // gate/up shards of a tensor-parallel rank: when all tiles fit in one round of CTA pairs the pairs win (64 tiles
      // of 192 columns at two ranks: 51 vs 62 us per layer); with 128 tiles (one GPU) the single-CTA wave is ahead
      static int sms = 0;
      if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      }
      if ((p.N + bn - 1) / bn <= sms / 2) use_pair = true;
    }
    if (EPI != EPI_QKV && bn == 256 && g_pair_big_m > 0 && p.M >= g_pair_big_m && p.mblk_group == nullptr &&
        p.ar_world == 0 && p.scatter_meta == nullptr && max_ctas <= 0)
      use_pair = true;
    if (ag_pending) use_pair = false;
    if (use_pair) {
      if constexpr (EPI == EPI_GLU) {
        if (bn == 192) return launch_gemm_pair<192, EPI>(A, lda, B, ldb, b_rows, p, stream, 1);
      }
      if constexpr (EPI != EPI_QKV) {
        if (bn == 256) return launch_gemm_pair<256, EPI>(A, lda, B, ldb, b_rows, p, stream, force_splits);
      }
      return launch_gemm_pair<128, EPI>(A, lda, B, ldb, b_rows, p, stream, force_splits);
    }
  }
  // The fused all-reduce never splits K locally, so it keeps 128-row tiles: more tiles in flight.
  bool two_rows = p.M > 128 && p.M <= 1024 && p.mblk_group == nullptr && p.ar_world == 0;
  if constexpr (EPI == EPI_QKV) {
    // The QKV epilogue needs one head (128 columns) per tile, so its tiles cannot widen; 256 rows per CTA is what
    // lets a weight tile serve twice the MMAs at prefill sizes too.
    if (settings().qkv_two_rows && p.M > 128) two_rows = true;
  }
  // Decode-sized M without a K split (setting dec_tiles, one bit per epilogue): 128-row tiles, every tile streams its
  // whole K range. A CTA then pulls more bytes through its L2 port (all of A's rows for its tile), but nothing is
  // dumped, met at a barrier or reduced.
  // Measured in the serving step (M = 256, one GPU): QKV 49 -> 37 us per layer unsplit (its reduce phase was the slow
  // part); the residual GEMMs and gate/up get slower (down 43 -> 72 us), so only the QKV bit is on by default, and only
  // while the unsplit tiles fill at least half of the SMs (a tensor-parallel shard with few tiles keeps the split).
  if (p.M > 128 && p.M <= 256 && p.mblk_group == nullptr && p.ar_world == 0 && max_ctas <= 0 && force_splits <= 0 &&
      ((settings().dec_tiles >> EPI) & 1) && 2 * 2 * ((p.N + 127) / 128) >= gllm_sm_count()) {
    two_rows = false;
    force_splits = 1;
  }
  if constexpr (!FP8 && (EPI == EPI_STORE || EPI == EPI_RESIDUAL)) {
    // 64-wide tiles: twice the tiles of a narrow output (N = 4096 gives 128 tiles of 128 rows), never split
    if (bn == 64) return launch_gemm<64, 1, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, 1);
  }
  if constexpr (EPI == EPI_GLU) {
    // 192-wide tiles: 128 tiles for a 24576-row gate/up weight fill one wave of 148 SMs without splitting
    if (bn == 192) {
      if (two_rows) return launch_gemm<192, 2, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, 1);
      return launch_gemm<192, 1, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, 1);
    }
  }
  if constexpr (EPI != EPI_QKV) {
    if (bn == 256) {
      if (two_rows) return launch_gemm<256, 2, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
      return launch_gemm<256, 1, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
    }
  }
  if (two_rows) return launch_gemm<128, 2, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
  return launch_gemm<128, 1, EPI, FP8>(A, lda, B, ldb, b_rows, p, stream, max_ctas, force_splits);
}

}  // namespace gllm

using namespace gllm;

extern "C" int* gllm_error_word();
// Largest M that runs on CTA pairs (0 = never) and the set of epilogues (bit = EPI id; 0xF = all) that use them.
// Returns the previous setting as (mask << 16) | max_m.
GLLM_API int gllm_gemm_set_pair_big_m(int big_m) {   // 256-wide GEMMs with M >= big_m run on CTA pairs; 0 = never
  pair_max_m_setting();
  const int old = g_pair_big_m;
  g_pair_big_m = big_m < 0 ? 0 : big_m;
  return old;
}
GLLM_API int gllm_gemm_set_pair(int max_m, int epi_mask) {
  const int old = (g_pair_epi_mask << 16) | pair_max_m_setting();
  g_pair_max_m = max_m < 0 ? 0 : max_m;
  g_pair_epi_mask = epi_mask & 0xF;
  return old;
}


// ---------------------------------------------------------------------------------------------
// C entry points. All pointers are device pointers; `stream` is a cudaStream_t.
// ---------------------------------------------------------------------------------------------

// Registers the split-K scratch of the current device (caller-owned memory: `scratch_floats` fp32 for
// the partial sums and at least two zeroed int32 for the grid barrier). All GEMMs of a device share it,
// so GEMMs that may use split-K must not overlap on different streams, and a split-K launch needs every
// CTA of its grid resident at once (the grid never exceeds the SM count and uses one CTA per SM).
// Passing null pointers disables split-K.
GLLM_API int gllm_gemm_set_splitk_workspace(float* scratch, long long scratch_floats, int* counters,
                                            int num_counters) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  SplitKWorkspace& ws = g_splitk[dev & 63];
  if (scratch && (!counters || num_counters < 2)) {
    set_last_error("split-K workspace needs at least two zeroed counters for the grid barrier");
    return -1;
  }
  ws.scratch = scratch;
  ws.scratch_floats = scratch ? scratch_floats : 0;
  ws.barrier = reinterpret_cast<unsigned int*>(counters);
  return 0;
}

// The same for ONE stream of the current device: split-K GEMMs launched on `stream` (also while it captures a graph)
// reduce through this scratch and meet at these barrier words instead of the device-wide ones. At most 16 streams;
// registering a stream again replaces its workspace.
GLLM_API int gllm_gemm_set_splitk_workspace_stream(void* stream, float* scratch, long long scratch_floats, int* counters,
                                                   int num_counters) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (!scratch || !counters || num_counters < 2) {
    set_last_error("split-K stream workspace needs scratch and at least two zeroed counters");
    return -1;
  }
  std::lock_guard<std::mutex> lock(g_stream_ws_mu);
  const int n = g_stream_ws_n.load(std::memory_order_relaxed);
  int slot = -1;
  for (int i = 0; i < n; ++i)
    if (g_stream_ws[i].dev == dev && g_stream_ws[i].stream == static_cast<cudaStream_t>(stream)) slot = i;
  if (slot < 0) {
    if (n >= kMaxStreamWorkspaces) {
      set_last_error("split-K stream workspaces: table full (%d)", kMaxStreamWorkspaces);
      return -1;
    }
    slot = n;
  }
  g_stream_ws[slot].dev = dev;
  g_stream_ws[slot].stream = static_cast<cudaStream_t>(stream);
  g_stream_ws[slot].ws.scratch = scratch;
  g_stream_ws[slot].ws.scratch_floats = scratch_floats;
  g_stream_ws[slot].ws.barrier = reinterpret_cast<unsigned int*>(counters);
  if (slot == n) g_stream_ws_n.store(n + 1, std::memory_order_release);
  return 0;
}

// out[M,N] = rowscale(A) · Bᵀ (+bias).  bn: 128 or 256.  row_ss_in may be null.
GLLM_API int gllm_gemm_bf16(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                            int M, int N, int K, int out_f32, const float* bias, const float* row_ss_in,
                            int ss_in_parts, float norm_inv_dim, float norm_eps, int bn, void* stream, int max_ctas,
                            int force_splits) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32; p.bias = bias;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_STORE, false>(A, lda, B, ldb, N, p, bn, (cudaStream_t)stream, max_ctas, force_splits);
}

// gllm_gemm_bf16 with the final-logit soft cap in the epilogue (never split along K: the cap is not linear).
GLLM_API int gllm_gemm_bf16_softcap(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                                    int M, int N, int K, int out_f32, const float* bias, const float* row_ss_in,
                                    int ss_in_parts, float norm_inv_dim, float norm_eps, int bn, void* stream,
                                    float softcap) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32; p.bias = bias;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.softcap = softcap;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_STORE, false>(A, lda, B, ldb, N, p, bn, (cudaStream_t)stream, 0, 1);
}

// out[M,N] = A · Bᵀ (+bias) + residual ; row_ss_out[M, ceil(N/bn)] receives per-tile sums of squares.
GLLM_API int gllm_gemm_bf16_residual(const void* A, long long lda, const void* B, long long ldb, void* out,
                                     long long ldo, const void* residual, long long ldr, float* row_ss_out, int M,
                                     int N, int K, const float* bias, int bn, void* stream, int max_ctas,
                                     int force_splits) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.row_ss_out = row_ss_out;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, bn, (cudaStream_t)stream, max_ctas, force_splits);
}

// Form of the fused all-reduce: -1 = by rank count (two-shot from `kTwoShotMinWorld` ranks on), 0 = one-shot (every rank
// pulls every row), 1 = two-shot (each rank pulls its 1/W of the rows and broadcasts them). Every rank must use the same
// setting; the symmetric buffer must hold three regions of `buf_elems` (two partial buffers and the result region).
constexpr int kTwoShotMinWorld = 8;
static bool ar_two_shot_setting(int world) {
  const int v = settings().ar_two_shot;
  return v < 0 ? world >= kTwoShotMinWorld : v != 0;
}
GLLM_API int gllm_gemm_set_ar_two_shot(int mode) {
  const int old = settings().ar_two_shot;
  settings().ar_two_shot = mode;
  return old;
}

// Row-parallel GEMM fused with the tensor-parallel all-reduce: out = sum over ranks(A_r · B_rᵀ) (+bias)
// + residual, with the next norm's row statistics [M, ceil(N/256)]. Each rank stores its bf16 partial tiles
// in its own symmetric buffer as they retire; all CTAs of all ranks meet at an arrival counter (one
// multimem.red per CTA, or one red per peer); then every rank pulls the sum of all partials — one
// multimem.ld_reduce per 16 bytes through NVSwitch when `mc_buf` is given, else plain peer loads over
// NVLink — and finishes locally. Two buffers of `buf_elems` bf16 alternate between launches.
// Every rank must issue the same sequence of these calls. peer_buf / peer_counter: arrays of `world`
// pointers, index = rank. state: two local u64, zero at start.
GLLM_API int gllm_gemm_bf16_residual_allreduce(const void* A, long long lda, const void* B, long long ldb, void* out,
                                               long long ldo, const void* residual, long long ldr, float* row_ss_out,
                                               int M, int N, int K, const float* bias, int bn, void* stream,
                                               int max_ctas, int force_splits, int world, int rank, void* mc_buf,
                                               void* const* peer_buf, unsigned long long* mc_counter,
                                               unsigned long long* const* peer_counter, unsigned long long* state,
                                               long long buf_elems) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_buf || !peer_counter || !state) {
    set_last_error("gemm_allreduce: bad world/rank/pointers (world %d rank %d)", world, rank);
    return -1;
  }
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.row_ss_out = row_ss_out;
  p.ar_world = world; p.ar_rank = rank; p.ar_mc_buf = static_cast<__nv_bfloat16*>(mc_buf);
  p.ar_mc_counter = mc_counter;
  for (int r = 0; r < world; ++r) {
    p.ar_peer_buf[r] = static_cast<__nv_bfloat16*>(peer_buf[r]);
    p.ar_peer_counter[r] = peer_counter[r];
  }
  p.ar_state = state; p.ar_buf_elems = buf_elems;
  p.ar_two_shot = (world >= 2 && ar_two_shot_setting(world)) ? 1 : 0;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, bn, (cudaStream_t)stream, max_ctas, force_splits);
}

// Push form of the same fused op (see GemmParams::ar_push): no meeting before data moves. Each rank's symmetric
// region (`peer_base[r]`, all mapped by every rank; `mc_base` its multicast alias or null) holds, at the given
// offsets from its base: the receive slots (`recv_elems` bf16 at `recv_off` BYTES), the tile flags (`flag_count`
// u32, zero at start, at `flag_off` bytes) and the done words (8 u64, zero at start, at `done_off` bytes). `out`
// (which is also the residual: the op is x <- x + sum) and `row_ss_out` [M, ceil(N/256)] must themselves lie inside
// this rank's region, at the same offset on every rank: the owner of a row stores the finished row and its
// statistics into every rank's copy. `state`: 8 local u64, zero at start. Every rank issues the same calls in the
// same order. Waits are bounded by the `peer_wait_ns` setting and report ERR_TIMEOUT_PEER in the status word.
GLLM_API int gllm_gemm_bf16_residual_allreduce_push(const void* A, long long lda, const void* B, long long ldb,
                                                    void* out, long long ldo, float* row_ss_out, int M, int N, int K,
                                                    const float* bias, int bn, void* stream, int world, int rank,
                                                    void* mc_base, void* const* peer_base, long long region_bytes,
                                                    long long recv_off, long long recv_elems, long long flag_off,
                                                    long long flag_count, long long done_off,
                                                    unsigned long long* state) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_base || !state || !out) {
    set_last_error("gemm_allreduce_push: bad world/rank/pointers (world %d rank %d)", world, rank);
    return -1;
  }
  const char* base = static_cast<const char*>(peer_base[rank]);
  const long long out_off = static_cast<const char*>(out) - base;
  const long long ss_off = row_ss_out ? reinterpret_cast<const char*>(row_ss_out) - base : 0;
  const long long groups = (N + 255) / 256;
  if (out_off < 0 || out_off + (static_cast<long long>(M - 1) * ldo + N) * 2 > region_bytes || (out_off & 15) ||
      (row_ss_out && (ss_off < 0 || ss_off + static_cast<long long>(M) * groups * 4 > region_bytes || (ss_off & 3)))) {
    set_last_error("gemm_allreduce_push: out / row_ss_out must lie inside the symmetric region (16-byte aligned)");
    return -1;
  }
  if ((recv_off & 15) || (flag_off & 3) || (done_off & 7) || recv_off + recv_elems * 2 > region_bytes ||
      flag_off + flag_count * 4 > region_bytes || done_off + 64 > region_bytes) {
    set_last_error("gemm_allreduce_push: bad region layout");
    return -1;
  }
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(out); p.ldr = ldo; p.row_ss_out = row_ss_out;
  p.ar_world = world; p.ar_rank = rank; p.ar_mc_buf = static_cast<__nv_bfloat16*>(mc_base);
  for (int r = 0; r < world; ++r) p.ar_peer_buf[r] = static_cast<__nv_bfloat16*>(peer_base[r]);
  p.ar_state = state;
  p.ar_push = 1;
  p.ar_recv_off = recv_off / 2; p.ar_buf_elems = recv_elems;
  p.ar_out_off = out_off / 2; p.ar_ss_off = ss_off;
  p.ar_flag_off = flag_off; p.ar_flag_cap = flag_count; p.ar_done_off = done_off;
  p.ar_drop_flags = settings().ar_drop_flags;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, bn, (cudaStream_t)stream, 0, 0);
}

// Low-latency form of the fused all-reduce (GemmParams::ar_ll): `out` is plain local memory and holds the residual
// on entry; the receive and result slots ([2 parities] each) live in the symmetric region and hold the sentinel
// 0x80008000 in every word between launches (the caller fills them once, and again after a launch that timed out).
GLLM_API int gllm_gemm_bf16_residual_allreduce_ll(const void* A, long long lda, const void* B, long long ldb, void* out,
                                                  long long ldo, float* row_ss_out, int M, int N, int K,
                                                  const float* bias, int bn, void* stream, int world, int rank,
                                                  void* mc_base, void* const* peer_base, long long region_bytes, long long recv_off,
                                                  long long recv_bytes, long long res_off, long long res_bytes,
                                                  unsigned long long* state) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_base || !state || !out) {
    set_last_error("gemm_allreduce_ll: bad world/rank/pointers (world %d rank %d)", world, rank);
    return -1;
  }
  if ((recv_off & 15) || (res_off & 15) || (recv_bytes & 15) || (res_bytes & 15) || recv_off < 0 || res_off < 0 ||
      recv_off + 2 * recv_bytes > region_bytes || res_off + 2 * res_bytes > region_bytes) {
    set_last_error("gemm_allreduce_ll: bad region layout");
    return -1;
  }
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(out); p.ldr = ldo; p.row_ss_out = row_ss_out;
  p.ar_world = world; p.ar_rank = rank; p.ar_mc_buf = static_cast<__nv_bfloat16*>(mc_base);
  for (int r = 0; r < world; ++r) p.ar_peer_buf[r] = static_cast<__nv_bfloat16*>(peer_base[r]);
  p.ar_state = state;
  p.ar_ll = 1;
  p.ar_ll_recv_off = recv_off; p.ar_ll_recv_bytes = recv_bytes;
  p.ar_ll_res_off = res_off; p.ar_ll_res_bytes = res_bytes;
  p.ar_drop_flags = settings().ar_drop_flags;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, bn == 256 ? 256 : 128, (cudaStream_t)stream, 0, 0);
}

// Reduce-scatter form of the low-latency fused kernel: out_shard[lrow] = sum_ranks(A @ B^T)[rank * ceil(M / W) + lrow]
// + out_shard[lrow] for the rows this rank owns (`out_shard` holds the residual shard on entry, `row_ss_out` the
// statistics of the shard's rows per 256 columns); no rank receives the other rows. The sequence-parallel counterpart
// of gllm_gemm_bf16_residual_allreduce_ll: same receive slots, no result slots.
GLLM_API int gllm_gemm_bf16_residual_reduce_scatter(const void* A, long long lda, const void* B, long long ldb,
                                                    void* out_shard, long long ldo, float* row_ss_out, int M, int N,
                                                    int K, const float* bias, void* stream, int world, int rank,
                                                    void* const* peer_base, long long region_bytes, long long recv_off,
                                                    long long recv_bytes, unsigned long long* state) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_base || !state || !out_shard) {
    set_last_error("gemm_reduce_scatter: bad world/rank/pointers (world %d rank %d)", world, rank);
    return -1;
  }
  if ((recv_off & 15) || (recv_bytes & 15) || recv_off < 0 || recv_off + 2 * recv_bytes > region_bytes) {
    set_last_error("gemm_reduce_scatter: bad region layout");
    return -1;
  }
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out_shard; p.ldo = ldo; p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(out_shard); p.ldr = ldo; p.row_ss_out = row_ss_out;
  p.ar_world = world; p.ar_rank = rank;
  for (int r = 0; r < world; ++r) p.ar_peer_buf[r] = static_cast<__nv_bfloat16*>(peer_base[r]);
  p.ar_state = state;
  p.ar_ll = 1; p.ar_rs_only = 1;
  p.ar_ll_recv_off = recv_off; p.ar_ll_recv_bytes = recv_bytes;
  p.ar_ll_res_off = recv_off; p.ar_ll_res_bytes = 1ll << 40;   // result slots are not used by this form
  p.ar_drop_flags = settings().ar_drop_flags;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_RESIDUAL, false>(A, lda, B, ldb, N, p, 128, (cudaStream_t)stream, 0, 0);
}

// Row counts of the 128-row blocks of the NEXT grouped GEMM this thread launches (GemmParams::mblk_rows): one int per
// block, on the device. Consumed by that launch; launches that are not grouped ignore and clear it.
GLLM_API int gllm_gemm_set_block_rows(const int* rows) {
  g_pending_block_rows = rows;
  return 0;
}

// The NEXT bf16 GEMM this thread launches (plain, residual, GLU or QKV epilogue; not grouped, not a CTA-pair launch)
// first all-gathers its A operand: `src` holds this rank's rows [rank * ceil(M / W), ...) of A, `dst` is the [M, K]
// tensor passed as A to that GEMM (local memory, filled by the kernel), the slots ([2 parities][M][K] bf16, every word
// the sentinel 0x80008000 between launches) live at `slot_off` of the symmetric region. `state`: one local 64-bit
// launch counter owned by this all-gather site. The descriptor is consumed by the next launch, whatever its outcome.
GLLM_API int gllm_gemm_set_allgather_input(const void* src, long long src_ld, void* dst, long long dst_ld, int world,
                                           int rank, void* mc_base, void* const* peer_base, long long region_bytes,
                                           long long slot_off, long long slot_bytes, unsigned long long* state,
                                           float* ss_out) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !peer_base || !state || !src || !dst ||
      (slot_off & 15) || (slot_bytes & 15) || slot_off < 0 || slot_off + 2 * slot_bytes > region_bytes ||
      (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) || (src_ld & 7) || (dst_ld & 7)) {
    set_last_error("gemm_set_allgather_input: bad arguments (world %d rank %d)", world, rank);
    return -1;
  }
  PendingAllGather& ag = g_pending_ag;
  ag.active = true;
  ag.world = world; ag.rank = rank;
  ag.src = src; ag.src_ld = src_ld; ag.dst = dst; ag.dst_ld = dst_ld;
  for (int r = 0; r < world; ++r) ag.peer[r] = peer_base[r];
  ag.mc = mc_base;
  ag.slot_off = slot_off; ag.slot_bytes = slot_bytes; ag.state = state;
  ag.ss_out = ss_out;     // optional [M, K / 256] floats: row statistics of the gathered rows, written before the main loop
  return 0;
}

// out[M,N/2] = act(rowscale*gate) * rowscale*up ; B is the tile-interleaved gate/up weight [N,K]:
// rows [t*bn, t*bn+bn/2) = gate rows of output block t, rows [t*bn+bn/2, (t+1)*bn) = its up rows.
GLLM_API int gllm_gemm_bf16_glu(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                                int M, int N, int K, int act, const float* row_ss_in, int ss_in_parts,
                                float norm_inv_dim, float norm_eps, int bn, const int* mblk_group, int num_groups,
                                void* stream, int max_ctas, int force_splits) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.glu_act = act;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.mblk_group = mblk_group; p.group_rows = N;
  p.err = gllm_error_word();
  const long long b_rows = mblk_group ? static_cast<long long>(num_groups) * N : N;  // groups are stacked
  return dispatch_gemm<EPI_GLU, false>(A, lda, B, ldb, b_rows, p, bn, (cudaStream_t)stream, max_ctas, force_splits);
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
  return dispatch_gemm<EPI_STORE, false>(A, lda, B, ldb, b_rows, p, bn, (cudaStream_t)stream, max_ctas, 1);
}

// Grouped GEMM whose output rows are scattered by `scatter_meta` into up to 8 peers' buffers (see GemmParams).
GLLM_API int gllm_gemm_bf16_grouped_scatter(const void* A, long long lda, const void* B, long long ldb, long long ldo,
                                            int M, int N, int K, const int* mblk_group, int num_groups, int bn,
                                            const int* scatter_meta, void* const* scatter_peer, int world,
                                            void* stream, int max_ctas) {
  if (world < 1 || world > 8 || scatter_meta == nullptr) {
    set_last_error("gemm_grouped_scatter: world must be 1..8 and scatter_meta non-null");
    return -1;
  }
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = scatter_peer[0]; p.ldo = ldo;
  p.mblk_group = mblk_group; p.group_rows = N;
  p.scatter_meta = scatter_meta;
  for (int r = 0; r < world; ++r) p.scatter_peer[r] = static_cast<__nv_bfloat16*>(scatter_peer[r]);
  p.err = gllm_error_word();
  const long long b_rows = static_cast<long long>(num_groups) * N;
  return dispatch_gemm<EPI_STORE, false>(A, lda, B, ldb, b_rows, p, bn, (cudaStream_t)stream, max_ctas, 1);
}

// ---------------------------------------------------------------------------------------------
// Block-scaled GEMMs (MXFP8 / NVFP4 operands on kind::mxf8f6f4 / kind::mxf4nvf4 with hardware scale factors).
// One entry point with an argument block (the Python side fills a ctypes.Structure of the same layout); `epi`
// selects the epilogue, and the fields of the other epilogues are ignored. Operands:
//   a  [M, K] codes: e4m3 bytes (fmt 2) or packed e2m1, two per byte, low nibble first (fmt 3); lda / ldb in BYTES
//   b  [N, K] (grouped: num_groups stacked) in the same format
//   sfa / sfb  scale factors in 512-byte chunks: chunk (row block rb = row / 128, scale-column block cb) sits at
//              (rb * chunks_per_row_block + cb) * 512 and holds scale (row r, column 4 * cb + j) at byte
//              (r % 32) * 16 + ((r % 128) / 32) * 4 + j; rows padded to 128, K to 128 (fmt 2) / 256 (fmt 3) elements;
//              fmt 2: ue8m0, one per 32 elements; fmt 3: ue4m3, one per 16 elements
//   out_scale  factor for the whole product (NVFP4's per-tensor scales), 0 = 1
// ---------------------------------------------------------------------------------------------
struct GllmBsGemmArgs {
  const void* a; long long lda; const void* sfa;
  const void* b; long long ldb; const void* sfb;
  void* out; long long ldo;
  int M, N, K, fmt, epi, out_f32, bn, max_ctas, force_splits;
  float out_scale;
  const float* bias;
  const float* row_ss_in; int ss_in_parts; float norm_inv_dim, norm_eps;
  const void* residual; long long ldr; float* row_ss_out;          // EPI_RESIDUAL
  int glu_act;                                                     // EPI_GLU
  const int* mblk_group; int num_groups;                           // grouped (EPI_STORE / EPI_GLU)
  int n_q_heads, n_kv_heads; void* q_out; void* kv_cache; int num_pages;   // EPI_QKV
  const int* slot_mapping; const int* positions; const float* cos_table; const float* sin_table; int max_pos;
  const float* q_norm_w; const float* k_norm_w; float qk_eps; float kv_inv_scale;
  void* stream;
  const int* scatter_meta; void* const* scatter_peer; int scatter_world;   // EPI_STORE: rows scattered into peers
  // EPI_RESIDUAL fused with the tensor-parallel all-reduce (low-latency form, GemmParams::ar_ll): `out` holds the
  // residual on entry; ar_world == 0 = no all-reduce
  int ar_world, ar_rank; void* ar_mc_base; void* const* ar_peer_base; long long ar_region_bytes;
  long long ar_recv_off, ar_recv_bytes, ar_res_off, ar_res_bytes; unsigned long long* ar_state;
};

template <int OPM>
static int bs_gemm_call(const GllmBsGemmArgs& a) {
  GemmParams p = {};
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.out = a.out; p.ldo = a.ldo; p.out_f32 = a.out_f32; p.bias = a.bias;
  p.sfa = static_cast<const uint8_t*>(a.sfa); p.sfb = static_cast<const uint8_t*>(a.sfb); p.out_scale = a.out_scale;
  p.row_ss_in = a.row_ss_in; p.ss_in_parts = a.ss_in_parts; p.norm_inv_dim = a.norm_inv_dim; p.norm_eps = a.norm_eps;
  p.mblk_group = a.mblk_group; p.group_rows = a.N;
  p.err = gllm_error_word();
  const long long b_rows = a.mblk_group ? static_cast<long long>(a.num_groups) * a.N : a.N;
  const int fs = a.mblk_group ? 1 : a.force_splits;
  cudaStream_t st = static_cast<cudaStream_t>(a.stream);
  switch (a.epi) {
    case EPI_STORE:
      if (a.scatter_meta) {
        if (a.scatter_world < 1 || a.scatter_world > 8 || !a.scatter_peer) {
          set_last_error("gemm_blockscaled: bad scatter world %d", a.scatter_world);
          return -1;
        }
        p.scatter_meta = a.scatter_meta;
        for (int r = 0; r < a.scatter_world; ++r) p.scatter_peer[r] = static_cast<__nv_bfloat16*>(a.scatter_peer[r]);
        p.out = a.scatter_peer[0];
      }
      return dispatch_gemm_bs<EPI_STORE, OPM>(a.a, a.lda, a.b, a.ldb, b_rows, p, a.bn, st, a.max_ctas, fs);
    case EPI_RESIDUAL:
      p.residual = static_cast<const __nv_bfloat16*>(a.residual); p.ldr = a.ldr; p.row_ss_out = a.row_ss_out;
      if (a.ar_world > 0) {
        if (a.ar_world > 8 || a.ar_rank < 0 || a.ar_rank >= a.ar_world || !a.ar_peer_base || !a.ar_state || !a.out ||
            a.mblk_group) {
          set_last_error("block-scaled gemm + all-reduce: bad world/rank/pointers (world %d rank %d)", a.ar_world, a.ar_rank);
          return -1;
        }
        if ((a.ar_recv_off & 15) || (a.ar_res_off & 15) || (a.ar_recv_bytes & 15) || (a.ar_res_bytes & 15) ||
            a.ar_recv_off < 0 || a.ar_res_off < 0 || a.ar_recv_off + 2 * a.ar_recv_bytes > a.ar_region_bytes ||
            a.ar_res_off + 2 * a.ar_res_bytes > a.ar_region_bytes) {
          set_last_error("block-scaled gemm + all-reduce: bad region layout");
          return -1;
        }
        p.residual = static_cast<const __nv_bfloat16*>(a.out); p.ldr = a.ldo;
        p.ar_world = a.ar_world; p.ar_rank = a.ar_rank; p.ar_mc_buf = static_cast<__nv_bfloat16*>(a.ar_mc_base);
        for (int r = 0; r < a.ar_world; ++r) p.ar_peer_buf[r] = static_cast<__nv_bfloat16*>(a.ar_peer_base[r]);
        p.ar_state = a.ar_state;
        p.ar_ll = 1;
        p.ar_ll_recv_off = a.ar_recv_off; p.ar_ll_recv_bytes = a.ar_recv_bytes;
        p.ar_ll_res_off = a.ar_res_off; p.ar_ll_res_bytes = a.ar_res_bytes;
        p.ar_drop_flags = settings().ar_drop_flags;
      }
      return dispatch_gemm_bs<EPI_RESIDUAL, OPM>(a.a, a.lda, a.b, a.ldb, b_rows, p, a.bn, st, a.max_ctas, fs);
    case EPI_GLU:
      p.glu_act = a.glu_act;
      return dispatch_gemm_bs<EPI_GLU, OPM>(a.a, a.lda, a.b, a.ldb, b_rows, p, a.bn, st, a.max_ctas, fs);
    case EPI_QKV: {
      if (((reinterpret_cast<uintptr_t>(a.cos_table) | reinterpret_cast<uintptr_t>(a.sin_table) |
            reinterpret_cast<uintptr_t>(a.q_norm_w) | reinterpret_cast<uintptr_t>(a.k_norm_w)) & 15) != 0) {
        set_last_error("block-scaled qkv gemm: rope tables and q/k norm weights must be 16-byte aligned");
        return -1;
      }
      p.N = (a.n_q_heads + 2 * a.n_kv_heads) * 128;
      p.n_q_heads = a.n_q_heads; p.n_kv_heads = a.n_kv_heads;
      p.q_out = static_cast<__nv_bfloat16*>(a.q_out); p.kv_cache = static_cast<__nv_bfloat16*>(a.kv_cache);
      p.num_pages = a.num_pages; p.slot_mapping = a.slot_mapping; p.positions = a.positions;
      p.cos_table = a.cos_table; p.sin_table = a.sin_table; p.max_pos = a.max_pos;
      p.q_norm_w = a.q_norm_w; p.k_norm_w = a.k_norm_w; p.qk_eps = a.qk_eps;
      p.kv_fp8 = a.kv_inv_scale > 0.f ? 1 : 0; p.kv_inv_scale = a.kv_inv_scale;
      return dispatch_gemm_bs<EPI_QKV, OPM>(a.a, a.lda, a.b, a.ldb, p.N, p, 128, st, a.max_ctas, fs);
    }
  }
  set_last_error("block-scaled gemm: unknown epilogue %d", a.epi);
  return -1;
}

GLLM_API int gllm_gemm_blockscaled(const GllmBsGemmArgs* args) {
  if (!args || !args->a || !args->b || !args->sfa || !args->sfb) {
    set_last_error("block-scaled gemm: null operand");
    return -1;
  }
  if (args->fmt == OPM_MXFP8) return bs_gemm_call<OPM_MXFP8>(*args);
  if (args->fmt == OPM_NVFP4) return bs_gemm_call<OPM_NVFP4>(*args);
  set_last_error("block-scaled gemm: fmt must be 2 (MXFP8) or 3 (NVFP4), got %d", args->fmt);
  return -1;
}

// Debugging aid (trace builds): CTA 0 of every following GEMM launch writes SM-clock stamps to `buf` (device memory,
// 12 x int64; slot 9 = push all-reduce: this CTA's rows reduced):
// entry, set-up done, first stage landed, MMAs of the first item issued, first accumulator ready, first epilogue
// done, main loop left, split-K barrier passed, exit. Pass null to switch it off.
GLLM_API int gllm_gemm_trace_enabled() {   // 1 when the library was built with -DGLLM_TRACE
#ifdef GLLM_TRACE
  return 1;
#else
  return 0;
#endif
}
GLLM_API void gllm_gemm_set_trace(long long* buf) { g_trace_ptr = buf; }
GLLM_API void gllm_gemm_set_trace_k(int k) { g_trace_k = k; }
GLLM_API void gllm_gemm_set_trace_n(int n) { g_trace_n = n; }

// Fused QKV projection for head_dim 128: rowscale -> per-head RMSNorm (optional) -> RoPE -> q buffer and
// paged KV write.  B is [(Hq+2Hkv)*128, K] with q heads first, then k heads, then v heads.
static int gemm_qkv_impl(const void* A, long long lda, const void* B, long long ldb, int M, int K,
                         int n_q_heads, int n_kv_heads, void* q_out, void* kv_cache, int num_pages,
                         const int* slot_mapping, const int* positions, const float* cos_table,
                         const float* sin_table, int max_pos, const float* q_norm_w, const float* k_norm_w,
                         float qk_eps, const float* row_ss_in, int ss_in_parts, float norm_inv_dim,
                         float norm_eps, const float* bias, float kv_inv_scale, void* stream, int max_ctas,
                         int force_splits) {
  // the epilogue reads the rope tables and the per-head norm weights with 16-byte loads
  if (((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table) |
        reinterpret_cast<uintptr_t>(q_norm_w) | reinterpret_cast<uintptr_t>(k_norm_w)) & 15) != 0) {
    set_last_error("gemm_qkv: rope tables and q/k norm weights must be 16-byte aligned");
    return -1;
  }
  GemmParams p = {};
  p.M = M; p.N = (n_q_heads + 2 * n_kv_heads) * 128; p.K = K;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.q_out = static_cast<__nv_bfloat16*>(q_out); p.kv_cache = static_cast<__nv_bfloat16*>(kv_cache);
  p.num_pages = num_pages; p.slot_mapping = slot_mapping; p.positions = positions;
  p.cos_table = cos_table; p.sin_table = sin_table; p.max_pos = max_pos;
  p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w; p.qk_eps = qk_eps;
  p.kv_fp8 = kv_inv_scale > 0.f ? 1 : 0;
  p.kv_inv_scale = kv_inv_scale;
  p.row_ss_in = row_ss_in; p.ss_in_parts = ss_in_parts; p.norm_inv_dim = norm_inv_dim; p.norm_eps = norm_eps;
  p.bias = bias;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_QKV, false>(A, lda, B, ldb, p.N, p, 128, (cudaStream_t)stream, max_ctas, force_splits);
}
GLLM_API int gllm_gemm_bf16_qkv(const void* A, long long lda, const void* B, long long ldb, int M, int K,
                                int n_q_heads, int n_kv_heads, void* q_out, void* kv_cache, int num_pages,
                                const int* slot_mapping, const int* positions, const float* cos_table,
                                const float* sin_table, int max_pos, const float* q_norm_w, const float* k_norm_w,
                                float qk_eps, const float* row_ss_in, int ss_in_parts, float norm_inv_dim,
                                float norm_eps, const float* bias, void* stream, int max_ctas, int force_splits) {
  return gemm_qkv_impl(A, lda, B, ldb, M, K, n_q_heads, n_kv_heads, q_out, kv_cache, num_pages, slot_mapping, positions,
                       cos_table, sin_table, max_pos, q_norm_w, k_norm_w, qk_eps, row_ss_in, ss_in_parts, norm_inv_dim,
                       norm_eps, bias, 0.f, stream, max_ctas, force_splits);
}
// Same with an fp8 (e4m3) KV cache of the same shape: K / V rows are stored as value / kv_scale (saturating).
GLLM_API int gllm_gemm_bf16_qkv_fp8kv(const void* A, long long lda, const void* B, long long ldb, int M, int K,
                                      int n_q_heads, int n_kv_heads, void* q_out, void* kv_cache, int num_pages,
                                      const int* slot_mapping, const int* positions, const float* cos_table,
                                      const float* sin_table, int max_pos, const float* q_norm_w, const float* k_norm_w,
                                      float qk_eps, const float* row_ss_in, int ss_in_parts, float norm_inv_dim,
                                      float norm_eps, const float* bias, float kv_scale, void* stream, int max_ctas,
                                      int force_splits) {
  if (!(kv_scale > 0.f)) {
    set_last_error("gemm_qkv_fp8kv: kv_scale must be positive");
    return -1;
  }
  return gemm_qkv_impl(A, lda, B, ldb, M, K, n_q_heads, n_kv_heads, q_out, kv_cache, num_pages, slot_mapping, positions,
                       cos_table, sin_table, max_pos, q_norm_w, k_norm_w, qk_eps, row_ss_in, ss_in_parts, norm_inv_dim,
                       norm_eps, bias, 1.0f / kv_scale, stream, max_ctas, force_splits);
}

// FP8 (e4m3) GEMM with per-row activation scale and per-column weight scale applied in the epilogue.
GLLM_API int gllm_gemm_fp8(const void* A, long long lda, const void* B, long long ldb, void* out, long long ldo,
                           int M, int N, int K, int out_f32, const float* a_scale, const float* b_scale, int bn,
                           void* stream, int max_ctas, int force_splits) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32;
  p.a_scale = a_scale; p.b_scale = b_scale;
  p.err = gllm_error_word();
  return dispatch_gemm<EPI_STORE, true>(A, lda, B, ldb, N, p, bn, (cudaStream_t)stream, max_ctas, force_splits);
}
