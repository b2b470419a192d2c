// GGML block formats: geometry, scalar dequantisation, conversion to affine group quantisation and a
// set of encoders (Q8_0, Q4_0, Q4_K, Q6_K) for writing test / benchmark checkpoints.
//
// Type codes and block geometry follow the GGUF specification (reference table:
// eredu-gguf/src/format.rs:254-405). The affine mapping (which GGML type becomes how many bits and which
// group size) is the reference's (eredu-gguf/src/convert.rs:124-152): Q2_K(2,16) Q3_K(3,16)
// Q4_0/Q4_1/Q4_K(4,32) Q5_0/Q5_1/Q5_K(5,32) Q6_K(6,16) Q8_0(8,32), f16 scales and biases with
// w = scale * q + bias, codes packed as a little-endian bit stream in u32 words.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace eredu {

enum GgmlType : uint32_t {
  GGML_F32 = 0, GGML_F16 = 1, GGML_Q4_0 = 2, GGML_Q4_1 = 3, GGML_Q5_0 = 6, GGML_Q5_1 = 7, GGML_Q8_0 = 8,
  GGML_Q8_1 = 9, GGML_Q2_K = 10, GGML_Q3_K = 11, GGML_Q4_K = 12, GGML_Q5_K = 13, GGML_Q6_K = 14, GGML_Q8_K = 15,
  GGML_IQ2_XXS = 16, GGML_IQ2_XS = 17, GGML_IQ3_XXS = 18, GGML_IQ1_S = 19, GGML_IQ4_NL = 20, GGML_IQ3_S = 21,
  GGML_IQ2_S = 22, GGML_IQ4_XS = 23, GGML_I8 = 24, GGML_I16 = 25, GGML_I32 = 26, GGML_I64 = 27, GGML_F64 = 28,
  GGML_IQ1_M = 29, GGML_BF16 = 30, GGML_MXFP4 = 39,
};

struct GgmlGeometry {
  uint32_t block_elems;
  uint32_t block_bytes;
};

inline bool ggml_geometry(uint32_t type, GgmlGeometry* g) {
  switch (type) {
    case GGML_F32: *g = {1, 4}; return true;
    case GGML_F16: *g = {1, 2}; return true;
    case GGML_BF16: *g = {1, 2}; return true;
    case GGML_F64: *g = {1, 8}; return true;
    case GGML_I8: *g = {1, 1}; return true;
    case GGML_I16: *g = {1, 2}; return true;
    case GGML_I32: *g = {1, 4}; return true;
    case GGML_I64: *g = {1, 8}; return true;
    case GGML_Q4_0: *g = {32, 18}; return true;
    case GGML_Q4_1: *g = {32, 20}; return true;
    case GGML_Q5_0: *g = {32, 22}; return true;
    case GGML_Q5_1: *g = {32, 24}; return true;
    case GGML_Q8_0: *g = {32, 34}; return true;
    case GGML_Q8_1: *g = {32, 36}; return true;
    case GGML_Q2_K: *g = {256, 84}; return true;
    case GGML_Q3_K: *g = {256, 110}; return true;
    case GGML_Q4_K: *g = {256, 144}; return true;
    case GGML_Q5_K: *g = {256, 176}; return true;
    case GGML_Q6_K: *g = {256, 210}; return true;
    case GGML_Q8_K: *g = {256, 292}; return true;
    case GGML_IQ2_XXS: *g = {256, 66}; return true;
    case GGML_IQ2_XS: *g = {256, 74}; return true;
    case GGML_IQ3_XXS: *g = {256, 98}; return true;
    case GGML_IQ1_S: *g = {256, 50}; return true;
    case GGML_IQ4_NL: *g = {32, 18}; return true;
    case GGML_IQ3_S: *g = {256, 110}; return true;
    case GGML_IQ2_S: *g = {256, 82}; return true;
    case GGML_IQ4_XS: *g = {256, 136}; return true;
    case GGML_IQ1_M: *g = {256, 56}; return true;
    case GGML_MXFP4: *g = {32, 17}; return true;
    default: return false;
  }
}

inline const char* ggml_type_name(uint32_t t) {
  switch (t) {
    case GGML_F32: return "F32"; case GGML_F16: return "F16"; case GGML_BF16: return "BF16"; case GGML_F64: return "F64";
    case GGML_I8: return "I8"; case GGML_I16: return "I16"; case GGML_I32: return "I32"; case GGML_I64: return "I64";
    case GGML_Q4_0: return "Q4_0"; case GGML_Q4_1: return "Q4_1"; case GGML_Q5_0: return "Q5_0";
    case GGML_Q5_1: return "Q5_1"; case GGML_Q8_0: return "Q8_0"; case GGML_Q8_1: return "Q8_1";
    case GGML_Q2_K: return "Q2_K"; case GGML_Q3_K: return "Q3_K"; case GGML_Q4_K: return "Q4_K";
    case GGML_Q5_K: return "Q5_K"; case GGML_Q6_K: return "Q6_K"; case GGML_Q8_K: return "Q8_K";
    case GGML_IQ2_XXS: return "IQ2_XXS"; case GGML_IQ2_XS: return "IQ2_XS"; case GGML_IQ3_XXS: return "IQ3_XXS";
    case GGML_IQ1_S: return "IQ1_S"; case GGML_IQ4_NL: return "IQ4_NL"; case GGML_IQ3_S: return "IQ3_S";
    case GGML_IQ2_S: return "IQ2_S"; case GGML_IQ4_XS: return "IQ4_XS"; case GGML_IQ1_M: return "IQ1_M";
    case GGML_MXFP4: return "MXFP4";
    default: return "UNKNOWN";
  }
}

// ---------------------------------------------------------------------------------------- half / bf16
inline float half_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t float_to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = static_cast<int32_t>((x >> 23) & 0xFFu) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFFu) == 0xFFu) return static_cast<uint16_t>(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half_man = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
    return static_cast<uint16_t>(sign | half_man);
  }
  uint32_t half = sign | (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(half);
}

inline float bf16_to_float(uint16_t b) {
  uint32_t bits = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t float_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((x >> 16) | 0x40u);
  x += 0x7FFFu + ((x >> 16) & 1u);
  return static_cast<uint16_t>(x >> 16);
}

inline uint16_t rd16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }

// ---------------------------------------------------------------------------------------- K-quant helpers
// 6-bit (scale, min) pair j of a Q4_K / Q5_K super-block's 12-byte scale field.
inline void k4_scale_min(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = static_cast<uint8_t>((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
    *mn = static_cast<uint8_t>((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

// Q3_K: sixteen 6-bit scales packed in 12 bytes.
inline void q3k_scales(const uint8_t* s, int8_t out[16]) {
  for (int i = 0; i < 16; ++i) {
    const int lo = (i < 8) ? (s[i] & 0xF) : (s[i - 8] >> 4);
    const int hi = (s[8 + (i % 4)] >> (2 * (i / 4))) & 3;
    out[i] = static_cast<int8_t>((lo | (hi << 4)) - 32);
  }
}

static const int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static const float kE2m1Values[16] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

inline float e8m0_to_float(uint8_t e) {
  if (e == 0) return std::ldexp(1.0f, -127);
  return std::ldexp(1.0f, static_cast<int>(e) - 127);
}

// Dequantise `nblocks` blocks of `type` into fp32. Returns false for types without a scalar decoder here.
bool ggml_dequantize(uint32_t type, const uint8_t* src, size_t nblocks, float* dst);

struct AffineTensor {
  int bits = 0;
  int group_size = 0;
  std::vector<uint32_t> packed;   // rows * cols * bits / 32 words
  std::vector<uint16_t> scales;   // f16, rows * cols / group
  std::vector<uint16_t> biases;   // f16
};

// (bits, group) of the affine form of a GGML type, false when the type has none.
bool ggml_affine_config(uint32_t type, int* bits, int* group);
// Convert rows x cols elements of a GGML quantised tensor to the affine form.
void ggml_to_affine(uint32_t type, const uint8_t* src, size_t rows, size_t cols, AffineTensor* out);

// Little-endian bit-stream packing of `n` codes of `bits` bits, appended to `out`.
void pack_codes(const uint8_t* codes, size_t n, int bits, std::vector<uint32_t>* out);
void unpack_codes(const uint32_t* words, size_t n, int bits, uint8_t* codes);

// Encoders (row-major fp32 in, n a multiple of the block size).
void quantize_q8_0(const float* x, size_t n, uint8_t* dst);
void quantize_q4_0(const float* x, size_t n, uint8_t* dst);
void quantize_q4_k(const float* x, size_t n, uint8_t* dst);
void quantize_q6_k(const float* x, size_t n, uint8_t* dst);

}  // namespace eredu
