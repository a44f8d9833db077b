// Flash attention for (chunked) prefill on the 5th-generation tensor cores: head_dim 128, bf16 paged KV cache.
//
// One CTA works on TWO query tiles of 128 rows that share their K/V stream: two query heads of one KV head over the
// same 128 query tokens (grouped-query models: both tiles then have the same causal range), or, when the group size
// is odd, two consecutive row blocks of one head. Roles:
//
//   warp 0      TMA producer: the Q tiles once, then K and V tiles of 64 tokens (four 16-token pages, each page two
//               64-column boxes with the 128-byte swizzle) into two three-stage rings
//   warp 1      tcgen05.mma issuer (one thread) and TMEM owner: S_t = Q_t K^T (128 x 64, accumulator in TMEM),
//               O_t += P_t V (128 x 128, accumulator stays in TMEM for the whole KV range). V is the MN-major operand
//               of the second product: it is used exactly as the pages store it (tokens x head_dim).
//   warps 2-5   softmax of tile 0: each thread owns one query row = one TMEM lane. tcgen05.ld of the S row, online
//   warps 6-9   softmax of tile 1   softmax in the exp2 domain, P written as bf16 into shared memory in the K-major
//               128-byte-swizzled layout the second product reads; when a row maximum of the warp moved, the warp
//               rescales its 32 lanes of the O accumulator in TMEM (tcgen05.ld / tcgen05.st).
//
// The issuer interleaves the tiles (PV_0(j), S_0(j+1), PV_1(j), S_1(j+1), ...), so the tensor core works on one tile
// while the other tile's softmax runs. A commit after S_t(j+1) also covers PV_t(j): "S ready" tells the softmax
// warps that the P buffer and the O accumulator of their tile are theirs again.
//
// Semantics are those of paged_prefill_kernel (attention.cu): the queries of a sequence are the last q_len of its ctx
// tokens, causal (or bidirectional) mask, optional sliding window and learnable sinks; scale 1/sqrt(d) folded into
// the exp2 argument. Reference behaviour: src/compat/scalar_ops.rs:196-278, 316-378 and the MultiHeadAttention node
// of src/arch/auto_graph_fragments/build_graph.inc.rs:1775-1781.
//
// Every wait is bounded (settings().wait_ns); a wait that runs out raises the status word, all roles leave their
// loops, the producer waits (bounded) for its copies in flight and the TMEM columns are freed.
#include "common.cuh"

namespace gllm {

constexpr int kFaD = 128;
constexpr int kFaRows = 128;                   // query rows per tile
constexpr int kFaKv = 64;                      // KV tokens per stage
constexpr int kFaStages = 3;
constexpr int kFaQTile = kFaRows * kFaD * 2;   // 32 KB: two 64-column panels of 128 rows x 128 bytes
constexpr int kFaKvTile = kFaKv * kFaD * 2;    // 16 KB: two panels of 64 rows x 128 bytes
constexpr int kFaPTile = kFaRows * kFaKv * 2;  // 16 KB: 128 rows x 128 bytes
constexpr int kFaOffK = 2 * kFaQTile;
constexpr int kFaOffV = kFaOffK + kFaStages * kFaKvTile;
constexpr int kFaOffP = kFaOffV + kFaStages * kFaKvTile;
constexpr int kFaOffBar = kFaOffP + 2 * kFaPTile;
constexpr int kFaSmem = kFaOffBar + 256 + 1024;
constexpr int kFaThreads = 320;
constexpr int kFaTmemCols = 512;               // S_0, S_1: 64 columns each; O_0, O_1: 128 columns each (384 used)

struct FaParams {
  __nv_bfloat16* out;        // [T, Hq, 128]
  const int* q_start;        // [S]
  const int* q_len;          // [S]
  const int* ctx_lens;       // [S]
  const int* block_tables;   // [S, max_blocks]
  int max_blocks;
  int n_q_heads, n_kv_heads, group;
  int pair_heads;            // 1: the tiles are heads 2y, 2y+1 over the same rows; 0: row blocks 2x, 2x+1 of head y
  float scale_log2;
  int num_pages;
  int window, causal;
  const float* sinks;
  int* err;
  unsigned long long wait_ns;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// MN-major operand with the 128-byte swizzle: 64 contiguous elements of the M/N dimension per 128-byte row, eight
// K rows per 1024-byte atom; `lbo` = bytes from one 64-element M/N panel to the next, atoms along K 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128_mn(uint32_t smem_addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// KV token range of one query tile: tiles [j0, j1) of 64 tokens.
struct FaTile {
  int head, row0, rows;   // rows = valid query rows (0: the tile does not exist)
  int j0, j1;
};

__global__ void __launch_bounds__(kFaThreads, 1)
fa_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                  const FaParams p) {
  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kFaOffBar);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // 3
  uint64_t* k_empty = bars + 4;            // 3
  uint64_t* v_full = bars + 7;             // 3
  uint64_t* v_empty = bars + 10;           // 3
  uint64_t* s_full = bars + 13;            // 2 (per tile)
  uint64_t* p_full = bars + 15;            // 2
  uint64_t* o_full = bars + 17;            // 2
  uint32_t* tmem_base_ptr = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 20);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z;
  pdl_wait();
  pdl_launch_dependents();
  const int qlen = p.q_len[seq];
  int ctx = p.ctx_lens[seq];
  if (qlen <= 0 || ctx <= 0) return;
  if (ctx > p.max_blocks * 16) {
    if (p.err && threadIdx.x == 0) atomicCAS(p.err, 0, ERR_BAD_ARG);
    ctx = p.max_blocks * 16;
  }
  const int qstart = p.q_start[seq];
  const int n_pages = (ctx + 15) / 16;

  FaTile tile[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    FaTile& ti = tile[t];
    if (p.pair_heads) {
      ti.head = blockIdx.y * 2 + t;
      ti.row0 = blockIdx.x * kFaRows;
    } else {
      ti.head = blockIdx.y;
      ti.row0 = (blockIdx.x * 2 + t) * kFaRows;
    }
    ti.rows = min(kFaRows, qlen - ti.row0);
    if (ti.rows <= 0 || ti.head >= p.n_q_heads) {
      ti.rows = 0; ti.j0 = 0; ti.j1 = 0;
      continue;
    }
    const int pos_first = ctx - qlen + ti.row0;
    const int pos_last = pos_first + ti.rows - 1;
    const int hi = p.causal ? min(ctx - 1, pos_last) : ctx - 1;
    const int lo = (p.window > 0) ? max(0, pos_first - p.window + 1) : 0;
    ti.j0 = lo / kFaKv;
    ti.j1 = hi / kFaKv + 1;
  }
  if (tile[0].rows == 0) return;   // tile 1 never exists without tile 0
  const int kvh = tile[0].head / p.group;
  const int J0 = tile[1].rows ? min(tile[0].j0, tile[1].j0) : tile[0].j0;
  const int J1 = tile[1].rows ? max(tile[0].j1, tile[1].j1) : tile[0].j1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < kFaStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 128);
      mbar_init(&o_full[t], 1);
    }
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_kv);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_ptr, kFaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_ptr;
  const unsigned long long wait_ns = p.wait_ns;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      const int ntiles = tile[1].rows ? 2 : 1;
      mbar_expect_tx(q_full, ntiles * kFaQTile);
      for (int t = 0; t < ntiles; ++t)
        for (int pn = 0; pn < 2; ++pn)
          tma_load_2d(smem + t * kFaQTile + pn * (kFaQTile / 2), &tmap_q, q_full, tile[t].head * kFaD + pn * 64,
                      qstart + tile[t].row0);
    }
    const int* bt = p.block_tables + static_cast<long long>(seq) * p.max_blocks;
    bool ok = true;
    int issued = 0;
    for (int j = J0; j < J1 && ok; ++j, ++issued) {
      const int n = j - J0, stg = n % kFaStages;
      const uint32_t par = ((n / kFaStages) & 1) ^ 1;
      // lanes 0..3 fetch the page ids of this tile (clamped to the sequence's last page: masked tokens then read
      // finite values), lanes 0..7 issue one box each
      int page = 0;
      if (lane < 4) {
        const int pi = min(j * 4 + lane, n_pages - 1);
        page = bt[pi];
        if (page < 0 || page >= p.num_pages) {
          if (p.err) atomicCAS(p.err, 0, ERR_BAD_PAGE);
          page = 0;
        }
      }
      const int my_page = __shfl_sync(0xffffffffu, page, (lane >> 1) & 3);
      const int pn = lane & 1;
      for (int kv = 0; kv < 2 && ok; ++kv) {
        uint64_t* empty = kv ? &v_empty[stg] : &k_empty[stg];
        uint64_t* full = kv ? &v_full[stg] : &k_full[stg];
        bool got = true;
        if (lane == 0) got = mbar_wait(empty, par, abort_flag, p.err, ERR_TIMEOUT_SMEM_EMPTY, wait_ns);
        ok = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(full, kFaKvTile);
        __syncwarp();
        if (lane < 8) {
          const int row = ((my_page * 2 + kv) * p.n_kv_heads + kvh) * 16;
          uint8_t* dst = smem + (kv ? kFaOffV : kFaOffK) + stg * kFaKvTile + pn * (kFaKvTile / 2) + (lane >> 1) * 2048;
          tma_load_2d(dst, &tmap_kv, full, pn * 64, row);
        }
      }
    }
    // copies in flight when the loop was abandoned: wait (bounded) for the last stages issued
    if (!ok && lane == 0) {
      for (int n = max(0, issued - kFaStages); n < issued; ++n) {
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(&v_full[n % kFaStages], (n / kFaStages) & 1) && globaltimer_ns() - t0 < wait_ns) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(kFaRows, kFaKv, 1, 1);
      constexpr uint32_t idesc_o = umma_idesc(kFaRows, kFaD, 1, 1) | (1u << 16);   // B (V) is MN-major
      const uint32_t q_addr = smem_u32(smem);
      const uint32_t k_addr = smem_u32(smem + kFaOffK);
      const uint32_t v_addr = smem_u32(smem + kFaOffV);
      const uint32_t p_addr = smem_u32(smem + kFaOffP);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL, wait_ns);
      auto in_range = [&](int t, int j) { return tile[t].rows > 0 && j >= tile[t].j0 && j < tile[t].j1; };
      auto issue_s = [&](int t, int j) {
        const int stg = (j - J0) % kFaStages;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t a = umma_desc_sw128(q_addr + t * kFaQTile + (k >> 2) * (kFaQTile / 2) + (k & 3) * 32);
          const uint64_t b = umma_desc_sw128(k_addr + stg * kFaKvTile + (k >> 2) * (kFaKvTile / 2) + (k & 3) * 32);
          umma_f16(tmem_base + t * kFaKv, a, b, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int j) {
        const int stg = (j - J0) % kFaStages;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t a = umma_desc_sw128(p_addr + t * kFaPTile + k * 32);
          const uint64_t b = umma_desc_sw128_mn(v_addr + stg * kFaKvTile + k * 2048, kFaKvTile / 2);
          umma_f16(tmem_base + 128 + t * kFaD, a, b, idesc_o, (j > tile[t].j0 || k > 0) ? 1u : 0u);
        }
      };
      // prologue: the first S of every tile whose range starts at J0
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL, wait_ns);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (in_range(t, J0)) issue_s(t, J0);
        // the K stage of tile J0 is free once these products (and every earlier one) are done, unless a tile whose
        // range starts later still needs... it cannot: ranges are contiguous and J0 is the smallest start
        umma_commit(&k_empty[0]);
      }
      int np[2] = {0, 0};   // P buffers consumed so far, per tile
      for (int j = J0; j < J1 && ok; ++j) {
        const int n = j - J0, stg = n % kFaStages;
        const bool has_next = j + 1 < J1;
        const int stg1 = (n + 1) % kFaStages;
        bool k_ready = false;
        ok = mbar_wait(&v_full[stg], (n / kFaStages) & 1, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL, wait_ns);
        for (int t = 0; t < 2 && ok; ++t) {
          if (in_range(t, j)) {
            ok = mbar_wait(&p_full[t], np[t] & 1, abort_flag, p.err, ERR_TIMEOUT_TMEM_FULL, wait_ns);
            if (!ok) break;
            ++np[t];
            tc_fence_after();
            issue_pv(t, j);
            if (j + 1 == tile[t].j1) umma_commit(&o_full[t]);
          }
          if (has_next && in_range(t, j + 1)) {
            if (!k_ready) {
              ok = mbar_wait(&k_full[stg1], ((n + 1) / kFaStages) & 1, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL, wait_ns);
              if (!ok) break;
              k_ready = true;
              tc_fence_after();
            }
            issue_s(t, j + 1);
          }
        }
        if (!ok) break;
        umma_commit(&v_empty[stg]);
        if (has_next) {
          if (!k_ready) ok = mbar_wait(&k_full[stg1], ((n + 1) / kFaStages) & 1, abort_flag, p.err, ERR_TIMEOUT_TMA_FULL, wait_ns);
          umma_commit(&k_empty[stg1]);
        }
      }
    }
  } else {
    // ------------------------------- softmax -------------------------------
    const int t = (warp - 2) >> 2;
    const FaTile ti = tile[t];
    if (ti.rows > 0) {
      const int quarter = warp & 3;                    // the TMEM lanes this warp may touch: 32 * (warp % 4) ...
      const int row = quarter * 32 + lane;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t s_addr = lane_addr + t * kFaKv;
      const uint32_t o_addr = lane_addr + 128 + t * kFaD;
      const bool row_ok = row < ti.rows;
      const int pos = ctx - qlen + ti.row0 + (row_ok ? row : 0);
      const int hi = p.causal ? min(ctx - 1, pos) : ctx - 1;
      const int lo = (p.window > 0) ? max(0, pos - p.window + 1) : 0;
      uint8_t* p_row = smem + kFaOffP + t * kFaPTile + (row >> 3) * 1024 + (row & 7) * 128;
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = ti.j0; j < ti.j1; ++j) {
        const int c = j - ti.j0;
        ok = mbar_wait(&s_full[t], c & 1, abort_flag, p.err, ERR_TIMEOUT_TMEM_FULL, wait_ns);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        tc_fence_after();
        uint32_t sr[2][32];
        tmem_ld_32x32(s_addr, sr[0]);
        tmem_ld_32x32(s_addr + 32, sr[1]);
        tmem_ld_wait();
        const int t0 = j * kFaKv;
        const bool full_tile = t0 >= lo && t0 + kFaKv - 1 <= hi;
        float mx = -INFINITY;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = __uint_as_float(sr[h][i]) * p.scale_log2;
            if (!full_tile) {
              const int tk = t0 + h * 32 + i;
              if (tk < lo || tk > hi) x = -INFINITY;
            }
            sr[h][i] = __float_as_uint(x);
            mx = fmaxf(mx, x);
          }
        const float m_new = fmaxf(m, mx);
        const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = ex2_approx(m - m_ref);        // m = -inf: 0
        float sum = 0.f;
        uint32_t pk[32];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = ex2_approx(__uint_as_float(sr[h][i]) - m_ref);
            const float e1 = ex2_approx(__uint_as_float(sr[h][i + 1]) - m_ref);
            sum += e0 + e1;
            pk[h * 16 + (i >> 1)] = pack_bf16x2(e0, e1);
          }
        l = l * corr + sum;
        // the O accumulator: rescaled by the warp when any of its rows moved its maximum (never on the first tile:
        // the first product overwrites the accumulator)
        const bool moved = m_new > m;
        m = m_new;
        if (c > 0 && __any_sync(0xffffffffu, moved)) {
#pragma unroll 1
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t orow[32];
            tmem_ld_32x32(o_addr + q4 * 32, orow);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
            tmem_st_32x32(o_addr + q4 * 32, orow);
          }
          tmem_st_wait();
        }
        // P row: 64 bf16 = eight 16-byte chunks, chunk index XOR (row % 8) within the 128-byte row
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 v = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(p_row + ((ch ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&p_full[t]);
      }
      if (ok) ok = mbar_wait(&o_full[t], 0, abort_flag, p.err, ERR_TIMEOUT_TMEM_FULL, wait_ns);
      if (__all_sync(0xffffffffu, ok)) {
        tc_fence_after();
        if (p.sinks) l += ex2_approx(p.sinks[ti.head] * 1.4426950408889634f - m);
        const float inv = (l > 0.f) ? 1.f / l : 0.f;
        __nv_bfloat16* orow_g = p.out + (static_cast<long long>(qstart + ti.row0 + row) * p.n_q_heads + ti.head) * kFaD;
#pragma unroll 1
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t orow[32];
          tmem_ld_32x32(o_addr + q4 * 32, orow);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(orow[i]) * inv, __uint_as_float(orow[i + 1]) * inv);
              w.y = pack_bf16x2(__uint_as_float(orow[i + 2]) * inv, __uint_as_float(orow[i + 3]) * inv);
              w.z = pack_bf16x2(__uint_as_float(orow[i + 4]) * inv, __uint_as_float(orow[i + 5]) * inv);
              w.w = pack_bf16x2(__uint_as_float(orow[i + 6]) * inv, __uint_as_float(orow[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow_g + q4 * 32 + i) = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, kFaTmemCols);
}

}  // namespace gllm

using namespace gllm;
extern "C" int* gllm_error_word();

// Causal (or bidirectional) flash attention over the paged bf16 KV cache for the query tokens of a prefill step.
// q / out: [total_tokens, n_q_heads, 128] bf16, contiguous. Same semantics as gllm_paged_prefill.
GLLM_API int gllm_paged_prefill_tc(const void* q, void* out, const void* kv_cache, int num_pages,
                                   const int* block_tables, int max_blocks, const int* q_start, const int* q_len,
                                   const int* ctx_lens, int num_seqs, int max_q_len, int total_tokens, int n_q_heads,
                                   int n_kv_heads, float scale, int causal, int window, const float* sinks,
                                   void* stream) {
  if (n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 || total_tokens <= 0) {
    set_last_error("paged_prefill_tc: heads %d / kv heads %d / tokens %d", n_q_heads, n_kv_heads, total_tokens);
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_last_error("paged_prefill_tc: q / out must be 16-byte aligned");
    return -1;
  }
  CUtensorMap tq, tkv;
  const uint64_t kv_rows = uint64_t(num_pages) * 2 * n_kv_heads * 16;
  if (make_tmap_2d(&tkv, kv_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kv_rows, kFaD, kFaD, 16, 64)) return -1;
  const uint64_t q_cols = uint64_t(n_q_heads) * kFaD;
  if (make_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, uint64_t(total_tokens), q_cols, q_cols, kFaRows, 64))
    return -1;
  FaParams p = {};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.q_start = q_start; p.q_len = q_len; p.ctx_lens = ctx_lens;
  p.block_tables = block_tables; p.max_blocks = max_blocks;
  p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.group = n_q_heads / n_kv_heads;
  p.pair_heads = (p.group % 2 == 0) ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_pages = num_pages; p.window = window; p.causal = causal; p.sinks = sinks;
  p.err = gllm_error_word();
  p.wait_ns = static_cast<unsigned long long>(settings().wait_ns);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(fa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem);
    if (e != cudaSuccess) { set_last_error("paged_prefill_tc: %s", cudaGetErrorString(e)); return -1; }
    attr_set[dev & 63] = true;
  }
  const int row_blocks = (max_q_len + kFaRows - 1) / kFaRows;
  dim3 grid(p.pair_heads ? row_blocks : (row_blocks + 1) / 2, p.pair_heads ? n_q_heads / 2 : n_q_heads, num_seqs);
  cudaError_t e = launch_kernel(fa_prefill_kernel, grid, dim3(kFaThreads), kFaSmem, (cudaStream_t)stream, true, 0, tq,
                                tkv, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_last_error("paged_prefill_tc launch: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}
