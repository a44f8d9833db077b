// Host-side plumbing shared by every kernel file: last-error string, per-device error word,
// tensor-map encoding (driver entry point fetched at run time) with a small cache, device queries.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

namespace gllm {

static thread_local char g_last_error[512] = {0};

RuntimeSettings& settings() {
  static RuntimeSettings s;
  return s;
}

const char* last_error() { return g_last_error; }

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

struct TmapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  int dt;
  int dev;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && dt == o.dt && dev == o.dev;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.rows);
    mix(k.cols);
    mix(k.ld);
    mix((uint64_t(k.box_rows) << 32) | k.box_cols);
    mix((uint64_t(k.dt) << 8) | uint64_t(k.dev));
    return h;
  }
};

static std::mutex g_tmap_mu;
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_size, uint64_t rows,
                 uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_last_error("tensor map base %p is not 16-byte aligned", base);
    return -1;
  }
  if ((ld * elem_size) % 16 != 0) {
    set_last_error("tensor map row pitch %llu bytes is not a multiple of 16", (unsigned long long)(ld * elem_size));
    return -1;
  }
  if (box_cols * elem_size != 128) {
    set_last_error("swizzle-128B box must be 128 bytes wide, got %u", box_cols * elem_size);
    return -1;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  TmapKey key{base, rows, cols, ld, box_rows, box_cols, int(dt), dev};
  {
    std::lock_guard<std::mutex> g(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return -1;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * uint64_t(elem_size)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (rows %llu cols %llu ld %llu box %ux%u)", int(r),
                   (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows, box_cols);
    return -1;
  }
  {
    std::lock_guard<std::mutex> g(g_tmap_mu);
    if (g_tmap_cache.size() > 8192) g_tmap_cache.clear();
    g_tmap_cache.emplace(key, *out);
  }
  return 0;
}

static int* g_err_words[64] = {nullptr};
static int g_sm_count[64] = {0};

}  // namespace gllm

using namespace gllm;

GLLM_API const char* gllm_last_error() { return last_error(); }

// Device error word for the current device: kernels write a status code there instead of trapping.
GLLM_API int* gllm_error_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_err_words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64);
    g_err_words[dev] = p;
  }
  return g_err_words[dev];
}

// Makes caller-owned device memory (at least 4 zeroed bytes, alive for the rest of the process) the error word of the
// current device, so that a host runtime can copy it back together with its own results instead of paying a separate
// synchronising read. Kernels launched (or graphs captured) before the call keep reporting to the old word.
GLLM_API int gllm_set_error_word(int* word) {
  int dev = 0;
  if (!word || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  g_err_words[dev] = word;
  return 0;
}

// Reads and clears the error word (synchronises the device).
GLLM_API int gllm_check_error() {
  int* w = gllm_error_word();
  if (!w) return -1;
  int v = 0;
  if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(w, 0, sizeof(int));
  return v;
}

GLLM_API int gllm_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!g_sm_count[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

GLLM_API int gllm_kernels_abi_version() { return 2; }

// Library settings by name (see RuntimeSettings in common.cuh). gllm_set_option returns the previous value, or
// LLONG_MIN for an unknown name; a change applies to launches made after it.
static long long* option_slot(const char* name, long long* tmp, int** as_int) {
  RuntimeSettings& s = settings();
  *as_int = nullptr;
  if (!strcmp(name, "wait_ns")) return reinterpret_cast<long long*>(&s.wait_ns);
  if (!strcmp(name, "peer_wait_ns")) return reinterpret_cast<long long*>(&s.peer_wait_ns);
  struct { const char* n; int* v; } ints[] = {
      {"pdl", &s.pdl}, {"park", &s.park}, {"cluster_sk", &s.cluster_sk}, {"ar_split", &s.ar_split},
      {"qkv_two_rows", &s.qkv_two_rows}, {"prefill_tc", &s.prefill_tc}, {"dec_tiles", &s.dec_tiles}, {"ar_drop_flags", &s.ar_drop_flags}, {"pair_max_m", &s.pair_max_m},
      {"pair_epi_mask", &s.pair_epi_mask}, {"pair_big_m", &s.pair_big_m}, {"ar_two_shot", &s.ar_two_shot}};
  for (auto& e : ints)
    if (!strcmp(name, e.n)) {
      *as_int = e.v;
      *tmp = *e.v;
      return tmp;
    }
  return nullptr;
}
GLLM_API long long gllm_get_option(const char* name) {
  long long tmp = 0;
  int* as_int = nullptr;
  long long* slot = name ? option_slot(name, &tmp, &as_int) : nullptr;
  return slot ? *slot : (-0x7fffffffffffffffLL - 1);
}
GLLM_API long long gllm_set_option(const char* name, long long value) {
  long long tmp = 0;
  int* as_int = nullptr;
  long long* slot = name ? option_slot(name, &tmp, &as_int) : nullptr;
  if (!slot) return -0x7fffffffffffffffLL - 1;
  const long long old = *slot;
  if (as_int) *as_int = static_cast<int>(value);
  else *slot = value;
  return old;
}
