// CPU dequantisation of GGML / GGUF block formats and the custom packed formats (AWQ4, GPTQ4, NVFP4)
// to fp32. This is the oracle for the fused-dequant GPU paths and the load-time conversion used when a
// checkpoint is expanded to bf16.
//
// Layouts follow the GGUF specification as the reference documents them
// (src/loader/gguf/types.rs:57-94,152-236; docs/domain-knowledge/quant-kquant-iq-proprietary.md:13-130;
// docs/domain-knowledge/gguf-classic-quant-layout.md:24-70). Block = fixed number of elements packed with
// their scales; all multi-byte fields are little endian; scales `d` are IEEE fp16.
#include <math.h>
#include <stdint.h>
#include <string.h>

#define API extern "C" __attribute__((visibility("default")))

namespace {

inline float fp16_to_fp32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal
      exp = 127 - 15 + 1;
      while ((man & 0x400) == 0) {
        man <<= 1;
        --exp;
      }
      man &= 0x3FF;
      bits = sign | (exp << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t rd16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
inline uint32_t rd32(const uint8_t* p) { return p[0] | (p[1] << 8) | (p[2] << 16) | (static_cast<uint32_t>(p[3]) << 24); }
inline float bf16_to_fp32(uint16_t h) {
  uint32_t bits = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline float e8m0_to_fp32(uint8_t e) {  // 2^(e-127); e == 255 is NaN
  if (e == 255) return NAN;
  if (e == 0) return ldexpf(1.0f, -127);
  return ldexpf(1.0f, static_cast<int>(e) - 127);
}
// unsigned e4m3 (OCP e4m3fn without the sign bit): bias 7, no infinities
inline float ue4m3_to_fp32(uint8_t v) {
  const int exp = (v >> 3) & 0xF, man = v & 7;
  if (exp == 0) return ldexpf(static_cast<float>(man), -9);
  if (exp == 15 && man == 7) return NAN;
  return ldexpf(1.0f + man / 8.0f, exp - 7);
}

const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
// e2m1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6} stored doubled, sign in bit 3
const int8_t kMxfp4x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// ---- 32-element blocks ----
void dq_q4_0(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b));
  const uint8_t* qs = b + 2;
  for (int j = 0; j < 16; ++j) {
    y[j] = ((qs[j] & 0xF) - 8) * d;
    y[j + 16] = ((qs[j] >> 4) - 8) * d;
  }
}
void dq_q4_1(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b)), m = fp16_to_fp32(rd16(b + 2));
  const uint8_t* qs = b + 4;
  for (int j = 0; j < 16; ++j) {
    y[j] = (qs[j] & 0xF) * d + m;
    y[j + 16] = (qs[j] >> 4) * d + m;
  }
}
void dq_q5_0(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b));
  const uint32_t qh = rd32(b + 2);
  const uint8_t* qs = b + 6;
  for (int j = 0; j < 16; ++j) {
    const uint8_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
    y[j] = (((qs[j] & 0xF) | h0) - 16) * d;
    y[j + 16] = (((qs[j] >> 4) | h1) - 16) * d;
  }
}
void dq_q5_1(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b)), m = fp16_to_fp32(rd16(b + 2));
  const uint32_t qh = rd32(b + 4);
  const uint8_t* qs = b + 8;
  for (int j = 0; j < 16; ++j) {
    const uint8_t h0 = ((qh >> j) << 4) & 0x10, h1 = (qh >> (j + 12)) & 0x10;
    y[j] = ((qs[j] & 0xF) | h0) * d + m;
    y[j + 16] = ((qs[j] >> 4) | h1) * d + m;
  }
}
void dq_q8_0(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b));
  const int8_t* qs = reinterpret_cast<const int8_t*>(b + 2);
  for (int j = 0; j < 32; ++j) y[j] = qs[j] * d;
}
void dq_q8_1(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b));
  const int8_t* qs = reinterpret_cast<const int8_t*>(b + 4);
  for (int j = 0; j < 32; ++j) y[j] = qs[j] * d;
}
void dq_iq4_nl(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b));
  const uint8_t* qs = b + 2;
  for (int j = 0; j < 16; ++j) {
    y[j] = d * kIq4nl[qs[j] & 0xF];
    y[j + 16] = d * kIq4nl[qs[j] >> 4];
  }
}
void dq_mxfp4(const uint8_t* b, float* y) {
  const float d = e8m0_to_fp32(b[0]) * 0.5f;
  const uint8_t* qs = b + 1;
  for (int j = 0; j < 16; ++j) {
    y[j] = kMxfp4x2[qs[j] & 0xF] * d;
    y[j + 16] = kMxfp4x2[qs[j] >> 4] * d;
  }
}

// ---- 256-element super blocks ----
void dq_q2_k(const uint8_t* b, float* y) {
  const uint8_t* scales = b;
  const uint8_t* q = b + 16;
  const float d = fp16_to_fp32(rd16(b + 80)), dmin = fp16_to_fp32(rd16(b + 82));
  int is = 0;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      uint8_t sc = scales[is++];
      float dl = d * (sc & 0xF), ml = dmin * (sc >> 4);
      for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l] >> shift) & 3) - ml;
      sc = scales[is++];
      dl = d * (sc & 0xF);
      ml = dmin * (sc >> 4);
      for (int l = 0; l < 16; ++l) *y++ = dl * ((q[l + 16] >> shift) & 3) - ml;
      shift += 2;
    }
    q += 32;
  }
}
void dq_q3_k(const uint8_t* b, float* y) {
  const uint8_t* hm = b;
  const uint8_t* q = b + 32;
  const float d_all = fp16_to_fp32(rd16(b + 108));
  const uint32_t kmask1 = 0x03030303, kmask2 = 0x0f0f0f0f;
  uint32_t aux[4];
  memcpy(aux, b + 96, 12);
  const uint32_t tmp = aux[2];
  aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
  aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
  aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
  aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
  const int8_t* scales = reinterpret_cast<const int8_t*>(aux);
  int is = 0;
  uint8_t m = 1;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      float dl = d_all * (scales[is++] - 32);
      for (int l = 0; l < 16; ++l)
        *y++ = dl * (static_cast<int8_t>((q[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4));
      dl = d_all * (scales[is++] - 32);
      for (int l = 0; l < 16; ++l)
        *y++ = dl * (static_cast<int8_t>((q[l + 16] >> shift) & 3) - ((hm[l + 16] & m) ? 0 : 4));
      shift += 2;
      m <<= 1;
    }
    q += 32;
  }
}
void dq_q4_k(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b)), dmin = fp16_to_fp32(rd16(b + 2));
  const uint8_t* scales = b + 4;
  const uint8_t* q = b + 16;
  int is = 0;
  uint8_t sc, m;
  for (int j = 0; j < 256; j += 64) {
    scale_min_k4(is, scales, &sc, &m);
    const float d1 = d * sc, m1 = dmin * m;
    scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * sc, m2 = dmin * m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 0xF) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
    q += 32;
    is += 2;
  }
}
void dq_q5_k(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b)), dmin = fp16_to_fp32(rd16(b + 2));
  const uint8_t* scales = b + 4;
  const uint8_t* qh = b + 16;
  const uint8_t* ql = b + 48;
  int is = 0;
  uint8_t sc, m, u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    scale_min_k4(is, scales, &sc, &m);
    const float d1 = d * sc, m1 = dmin * m;
    scale_min_k4(is + 1, scales, &sc, &m);
    const float d2 = d * sc, m2 = dmin * m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
    ql += 32;
    is += 2;
    u1 <<= 2;
    u2 <<= 2;
  }
}
void dq_q6_k(const uint8_t* b, float* y) {
  const uint8_t* ql = b;
  const uint8_t* qh = b + 128;
  const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
  const float d = fp16_to_fp32(rd16(b + 208));
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int8_t q1 = static_cast<int8_t>((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
      const int8_t q2 = static_cast<int8_t>((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int8_t q3 = static_cast<int8_t>((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int8_t q4 = static_cast<int8_t>((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l] = d * sc[is] * q1;
      y[l + 32] = d * sc[is + 2] * q2;
      y[l + 64] = d * sc[is + 4] * q3;
      y[l + 96] = d * sc[is + 6] * q4;
    }
    y += 128;
    ql += 64;
    qh += 32;
    sc += 8;
  }
}
void dq_q8_k(const uint8_t* b, float* y) {
  float d;
  memcpy(&d, b, 4);
  const int8_t* qs = reinterpret_cast<const int8_t*>(b + 4);
  for (int j = 0; j < 256; ++j) y[j] = d * qs[j];
}
void dq_iq4_xs(const uint8_t* b, float* y) {
  const float d = fp16_to_fp32(rd16(b));
  const uint16_t scales_h = rd16(b + 2);
  const uint8_t* scales_l = b + 4;
  const uint8_t* qs = b + 8;
  for (int ib = 0; ib < 8; ++ib) {
    const int ls = ((scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((scales_h >> (2 * ib)) & 3) << 4);
    const float dl = d * (ls - 32);
    for (int j = 0; j < 16; ++j) {
      y[j] = dl * kIq4nl[qs[j] & 0xF];
      y[j + 16] = dl * kIq4nl[qs[j] >> 4];
    }
    y += 32;
    qs += 16;
  }
}
void dq_tq1_0(const uint8_t* b, float* y) {  // 48 qs + 4 qh + d: five trits per byte (base-3, fixed point)
  const uint8_t* qs = b;
  const uint8_t* qh = b + 48;
  const float d = fp16_to_fp32(rd16(b + 52));
  static const uint8_t pow3[6] = {1, 3, 9, 27, 81, 243};
  for (int n = 0; n < 5; ++n)
    for (int m = 0; m < 32; ++m) {
      const uint8_t q = static_cast<uint8_t>(qs[m] * pow3[n]);
      *y++ = (static_cast<int16_t>((static_cast<uint16_t>(q) * 3) >> 8) - 1) * d;
    }
  for (int n = 0; n < 5; ++n)
    for (int m = 0; m < 16; ++m) {
      const uint8_t q = static_cast<uint8_t>(qs[32 + m] * pow3[n]);
      *y++ = (static_cast<int16_t>((static_cast<uint16_t>(q) * 3) >> 8) - 1) * d;
    }
  for (int n = 0; n < 4; ++n)
    for (int j = 0; j < 4; ++j) {
      const uint8_t q = static_cast<uint8_t>(qh[j] * pow3[n]);
      *y++ = (static_cast<int16_t>((static_cast<uint16_t>(q) * 3) >> 8) - 1) * d;
    }
}
void dq_tq2_0(const uint8_t* b, float* y) {
  const uint8_t* qs = b;
  const float d = fp16_to_fp32(rd16(b + 64));
  for (int j = 0; j < 64; j += 32)
    for (int l = 0; l < 4; ++l)
      for (int m = 0; m < 32; ++m) *y++ = (static_cast<int>((qs[j + m] >> (l * 2)) & 3) - 1) * d;
}

// ---- custom packed formats ----
// NVFP4: 64 elements = 4 unsigned-e4m3 scales (one per 16) + 32 bytes of e2m1 nibbles (low nibble first).
void dq_nvfp4(const uint8_t* b, float* y) {
  const uint8_t* qs = b + 4;
  for (int s = 0; s < 4; ++s) {
    const float d = ue4m3_to_fp32(b[s]) * 0.5f;
    for (int j = 0; j < 8; ++j) {
      const uint8_t v = qs[s * 8 + j];
      y[s * 16 + 2 * j] = kMxfp4x2[v & 0xF] * d;
      y[s * 16 + 2 * j + 1] = kMxfp4x2[v >> 4] * d;
    }
  }
}
// AWQ4 / GPTQ4 repacked: 128 elements = scale f16, pad, zero f16, pad, 16 x u32 (8 sequential nibbles each)
void dq_awq4(const uint8_t* b, float* y) {
  const float scale = fp16_to_fp32(rd16(b)), zero = fp16_to_fp32(rd16(b + 4));
  for (int w = 0; w < 16; ++w) {
    const uint32_t v = rd32(b + 8 + 4 * w);
    for (int i = 0; i < 8; ++i) y[w * 8 + i] = (static_cast<float>((v >> (4 * i)) & 0xF) - zero) * scale;
  }
}

struct TypeInfo {
  int id, block_elems, block_bytes;
  void (*fn)(const uint8_t*, float*);
};
// ids follow GGML's ggml_type numbering; 50..53 are the custom ids of the packed formats
const TypeInfo kTypes[] = {
    {2, 32, 18, dq_q4_0},   {3, 32, 20, dq_q4_1},   {6, 32, 22, dq_q5_0},   {7, 32, 24, dq_q5_1},
    {8, 32, 34, dq_q8_0},   {9, 32, 36, dq_q8_1},   {10, 256, 84, dq_q2_k}, {11, 256, 110, dq_q3_k},
    {12, 256, 144, dq_q4_k}, {13, 256, 176, dq_q5_k}, {14, 256, 210, dq_q6_k}, {15, 256, 292, dq_q8_k},
    {20, 32, 18, dq_iq4_nl}, {23, 256, 136, dq_iq4_xs}, {34, 256, 54, dq_tq1_0}, {35, 256, 66, dq_tq2_0},
    {39, 32, 17, dq_mxfp4}, {50, 128, 72, dq_awq4}, {51, 128, 72, dq_awq4}, {53, 64, 36, dq_nvfp4},
};

const TypeInfo* find_type(int id) {
  for (const TypeInfo& t : kTypes)
    if (t.id == id) return &t;
  return nullptr;
}

}  // namespace

// block geometry of a type id; returns 0 and fills the outputs, or -1 for an unknown / unsupported id
API int gllm_quant_block_info(int type_id, int* block_elems, int* block_bytes) {
  switch (type_id) {
    case 0: *block_elems = 1; *block_bytes = 4; return 0;   // F32
    case 1: *block_elems = 1; *block_bytes = 2; return 0;   // F16
    case 30: *block_elems = 1; *block_bytes = 2; return 0;  // BF16
    default: break;
  }
  const TypeInfo* t = find_type(type_id);
  if (!t) return -1;
  *block_elems = t->block_elems;
  *block_bytes = t->block_bytes;
  return 0;
}

// Dequantise `n_elems` (a multiple of the block size) from `src` into fp32 `dst`. Returns 0 or -1.
API int gllm_dequantize(int type_id, const void* src, long long n_elems, float* dst) {
  const uint8_t* s = static_cast<const uint8_t*>(src);
  if (type_id == 0) {
    memcpy(dst, src, static_cast<size_t>(n_elems) * 4);
    return 0;
  }
  if (type_id == 1) {
    for (long long i = 0; i < n_elems; ++i) dst[i] = fp16_to_fp32(rd16(s + 2 * i));
    return 0;
  }
  if (type_id == 30) {
    for (long long i = 0; i < n_elems; ++i) dst[i] = bf16_to_fp32(rd16(s + 2 * i));
    return 0;
  }
  const TypeInfo* t = find_type(type_id);
  if (!t || n_elems % t->block_elems != 0) return -1;
  const long long nb = n_elems / t->block_elems;
#pragma omp parallel for schedule(static) if (nb > 4096)
  for (long long b = 0; b < nb; ++b) t->fn(s + b * t->block_bytes, dst + b * t->block_elems);
  return 0;
}

// scalar codecs (OCP / IEEE conformant, round-to-nearest-even on encode)
API float gllm_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }
API float gllm_e8m0_to_fp32(uint8_t e) { return e8m0_to_fp32(e); }
API float gllm_ue4m3_to_fp32(uint8_t v) { return ue4m3_to_fp32(v); }
