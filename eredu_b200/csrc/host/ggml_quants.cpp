// Scalar decoders, affine conversion and encoders for GGML block formats (see ggml_quants.h).
// Block layouts are those of the GGUF specification; the scalar decode of Q4_K / Q6_K mirrors what the
// reference uses as its CPU oracle (safemlx/src/native_quantization.rs:3445-3541).
#include "ggml_quants.h"

#include <algorithm>
#include <cfloat>

namespace eredu {

// ------------------------------------------------------------------------------------------ dequantise
static void dq_q4_0(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b));
  for (int j = 0; j < 16; ++j) {
    y[j] = d * static_cast<float>((b[2 + j] & 0xF) - 8);
    y[j + 16] = d * static_cast<float>((b[2 + j] >> 4) - 8);
  }
}
static void dq_q4_1(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b)), m = half_to_float(rd16(b + 2));
  for (int j = 0; j < 16; ++j) {
    y[j] = d * static_cast<float>(b[4 + j] & 0xF) + m;
    y[j + 16] = d * static_cast<float>(b[4 + j] >> 4) + m;
  }
}
static void dq_q5_0(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b));
  uint32_t qh;
  std::memcpy(&qh, b + 2, 4);
  for (int j = 0; j < 16; ++j) {
    const int h0 = ((qh >> j) & 1) << 4, h1 = ((qh >> (j + 16)) & 1) << 4;
    y[j] = d * static_cast<float>(((b[6 + j] & 0xF) | h0) - 16);
    y[j + 16] = d * static_cast<float>(((b[6 + j] >> 4) | h1) - 16);
  }
}
static void dq_q5_1(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b)), m = half_to_float(rd16(b + 2));
  uint32_t qh;
  std::memcpy(&qh, b + 4, 4);
  for (int j = 0; j < 16; ++j) {
    const int h0 = ((qh >> j) & 1) << 4, h1 = ((qh >> (j + 16)) & 1) << 4;
    y[j] = d * static_cast<float>((b[8 + j] & 0xF) | h0) + m;
    y[j + 16] = d * static_cast<float>((b[8 + j] >> 4) | h1) + m;
  }
}
static void dq_q8_0(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b));
  for (int j = 0; j < 32; ++j) y[j] = d * static_cast<float>(static_cast<int8_t>(b[2 + j]));
}
static void dq_q2_k(const uint8_t* b, float* y) {
  const uint8_t* scales = b;
  const uint8_t* q = b + 16;
  const float d = half_to_float(rd16(b + 80)), dmin = half_to_float(rd16(b + 82));
  int is = 0;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      for (int half = 0; half < 2; ++half) {
        const uint8_t sc = scales[is++];
        const float dl = d * static_cast<float>(sc & 0xF), ml = dmin * static_cast<float>(sc >> 4);
        for (int l = 0; l < 16; ++l) *y++ = dl * static_cast<float>((q[l + 16 * half] >> shift) & 3) - ml;
      }
      shift += 2;
    }
    q += 32;
  }
}
static void dq_q3_k(const uint8_t* b, float* y) {
  const uint8_t* hm = b;
  const uint8_t* q = b + 32;
  int8_t sc[16];
  q3k_scales(b + 96, sc);
  const float d_all = half_to_float(rd16(b + 108));
  int is = 0;
  uint8_t m = 1;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      for (int half = 0; half < 2; ++half) {
        const float dl = d_all * static_cast<float>(sc[is++]);
        for (int l = 0; l < 16; ++l) {
          const int idx = l + 16 * half;
          const int v = ((q[idx] >> shift) & 3) - ((hm[idx] & m) ? 0 : 4);
          *y++ = dl * static_cast<float>(v);
        }
      }
      shift += 2;
      m <<= 1;
    }
    q += 32;
  }
}
static void dq_q4_k(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b)), dmin = half_to_float(rd16(b + 2));
  const uint8_t* scales = b + 4;
  const uint8_t* q = b + 16;
  int is = 0;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    k4_scale_min(is, scales, &sc, &m);
    const float d1 = d * sc, m1 = dmin * m;
    k4_scale_min(is + 1, scales, &sc, &m);
    const float d2 = d * sc, m2 = dmin * m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * static_cast<float>(q[l] & 0xF) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * static_cast<float>(q[l] >> 4) - m2;
    q += 32;
    is += 2;
  }
}
static void dq_q5_k(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b)), dmin = half_to_float(rd16(b + 2));
  const uint8_t* scales = b + 4;
  const uint8_t* qh = b + 16;
  const uint8_t* ql = b + 48;
  int is = 0;
  uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    k4_scale_min(is, scales, &sc, &m);
    const float d1 = d * sc, m1 = dmin * m;
    k4_scale_min(is + 1, scales, &sc, &m);
    const float d2 = d * sc, m2 = dmin * m;
    for (int l = 0; l < 32; ++l) *y++ = d1 * static_cast<float>((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
    for (int l = 0; l < 32; ++l) *y++ = d2 * static_cast<float>((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
    ql += 32;
    is += 2;
    u1 <<= 2;
    u2 <<= 2;
  }
}
static void dq_q6_k(const uint8_t* b, float* y) {
  const uint8_t* ql = b;
  const uint8_t* qh = b + 128;
  const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
  const float d = half_to_float(rd16(b + 208));
  for (int n = 0; n < 256; n += 128) {
    for (int l = 0; l < 32; ++l) {
      const int is = l / 16;
      const int q1 = static_cast<int>((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
      const int q2 = static_cast<int>((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
      const int q3 = static_cast<int>((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      const int q4 = static_cast<int>((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
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
static void dq_iq4_nl(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b));
  for (int j = 0; j < 16; ++j) {
    y[j] = d * kIq4nlValues[b[2 + j] & 0xF];
    y[j + 16] = d * kIq4nlValues[b[2 + j] >> 4];
  }
}
static void dq_iq4_xs(const uint8_t* b, float* y) {
  const float d = half_to_float(rd16(b));
  const uint16_t scales_h = rd16(b + 2);
  const uint8_t* scales_l = b + 4;
  const uint8_t* q = b + 8;
  for (int ib = 0; ib < 8; ++ib) {
    const int ls = ((scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((scales_h >> (2 * ib)) & 3) << 4);
    const float dl = d * static_cast<float>(ls - 32);
    for (int j = 0; j < 16; ++j) {
      y[j] = dl * kIq4nlValues[q[j] & 0xF];
      y[j + 16] = dl * kIq4nlValues[q[j] >> 4];
    }
    y += 32;
    q += 16;
  }
}
static void dq_mxfp4(const uint8_t* b, float* y) {
  const float d = e8m0_to_float(b[0]) * 0.5f;  // ggml stores E2M1 values doubled (integers 0..12)
  for (int j = 0; j < 16; ++j) {
    y[j] = d * 2.0f * kE2m1Values[b[1 + j] & 0xF];
    y[j + 16] = d * 2.0f * kE2m1Values[b[1 + j] >> 4];
  }
}

bool ggml_dequantize(uint32_t type, const uint8_t* src, size_t nblocks, float* dst) {
  GgmlGeometry g;
  if (!ggml_geometry(type, &g)) return false;
  void (*fn)(const uint8_t*, float*) = nullptr;
  switch (type) {
    case GGML_Q4_0: fn = dq_q4_0; break;
    case GGML_Q4_1: fn = dq_q4_1; break;
    case GGML_Q5_0: fn = dq_q5_0; break;
    case GGML_Q5_1: fn = dq_q5_1; break;
    case GGML_Q8_0: fn = dq_q8_0; break;
    case GGML_Q2_K: fn = dq_q2_k; break;
    case GGML_Q3_K: fn = dq_q3_k; break;
    case GGML_Q4_K: fn = dq_q4_k; break;
    case GGML_Q5_K: fn = dq_q5_k; break;
    case GGML_Q6_K: fn = dq_q6_k; break;
    case GGML_IQ4_NL: fn = dq_iq4_nl; break;
    case GGML_IQ4_XS: fn = dq_iq4_xs; break;
    case GGML_MXFP4: fn = dq_mxfp4; break;
    case GGML_F32:
      std::memcpy(dst, src, nblocks * 4);
      return true;
    case GGML_F16:
      for (size_t i = 0; i < nblocks; ++i) dst[i] = half_to_float(rd16(src + 2 * i));
      return true;
    case GGML_BF16:
      for (size_t i = 0; i < nblocks; ++i) dst[i] = bf16_to_float(rd16(src + 2 * i));
      return true;
    case GGML_F64:
      for (size_t i = 0; i < nblocks; ++i) {
        double v;
        std::memcpy(&v, src + 8 * i, 8);
        dst[i] = static_cast<float>(v);
      }
      return true;
    default: return false;
  }
  for (size_t i = 0; i < nblocks; ++i) fn(src + i * g.block_bytes, dst + i * g.block_elems);
  return true;
}

// ------------------------------------------------------------------------------------------ packing
void pack_codes(const uint8_t* codes, size_t n, int bits, std::vector<uint32_t>* out) {
  const size_t words = (n * bits + 31) / 32;
  const size_t start = out->size();
  out->resize(start + words, 0u);
  uint32_t* w = out->data() + start;
  const uint32_t mask = (1u << bits) - 1;
  for (size_t i = 0; i < n; ++i) {
    const size_t off = i * bits;
    const size_t wi = off >> 5;
    const int s = static_cast<int>(off & 31);
    const uint32_t c = codes[i] & mask;
    w[wi] |= c << s;
    if (s + bits > 32) w[wi + 1] |= c >> (32 - s);
  }
}

void unpack_codes(const uint32_t* words, size_t n, int bits, uint8_t* codes) {
  const uint32_t mask = (1u << bits) - 1;
  for (size_t i = 0; i < n; ++i) {
    const size_t off = i * bits;
    const size_t wi = off >> 5;
    const int s = static_cast<int>(off & 31);
    uint32_t c = words[wi] >> s;
    if (s + bits > 32) c |= words[wi + 1] << (32 - s);
    codes[i] = static_cast<uint8_t>(c & mask);
  }
}

// ------------------------------------------------------------------------------------------ affine conversion
bool ggml_affine_config(uint32_t type, int* bits, int* group) {
  switch (type) {
    case GGML_Q2_K: *bits = 2; *group = 16; return true;
    case GGML_Q3_K: *bits = 3; *group = 16; return true;
    case GGML_Q4_0: case GGML_Q4_1: case GGML_Q4_K: *bits = 4; *group = 32; return true;
    case GGML_Q5_0: case GGML_Q5_1: case GGML_Q5_K: *bits = 5; *group = 32; return true;
    case GGML_Q6_K: *bits = 6; *group = 16; return true;
    case GGML_Q8_0: *bits = 8; *group = 32; return true;
    default: return false;
  }
}

namespace {
struct Emit {
  AffineTensor* out;
  std::vector<uint8_t> codes;  // one row's codes
  void group(float scale, float bias) {
    out->scales.push_back(float_to_half(scale));
    out->biases.push_back(float_to_half(bias));
  }
};

// Each block decoder appends `block_elems` codes and the (scale, bias) of each of its groups.
void af_q4_0(const uint8_t* b, Emit& e) {
  const float d = half_to_float(rd16(b));
  e.group(d, -8.f * d);
  for (int j = 0; j < 16; ++j) e.codes.push_back(b[2 + j] & 0xF);
  for (int j = 0; j < 16; ++j) e.codes.push_back(b[2 + j] >> 4);
}
void af_q4_1(const uint8_t* b, Emit& e) {
  e.group(half_to_float(rd16(b)), half_to_float(rd16(b + 2)));
  for (int j = 0; j < 16; ++j) e.codes.push_back(b[4 + j] & 0xF);
  for (int j = 0; j < 16; ++j) e.codes.push_back(b[4 + j] >> 4);
}
void af_q5_0(const uint8_t* b, Emit& e) {
  const float d = half_to_float(rd16(b));
  uint32_t qh;
  std::memcpy(&qh, b + 2, 4);
  e.group(d, -16.f * d);
  for (int j = 0; j < 16; ++j) e.codes.push_back(static_cast<uint8_t>((b[6 + j] & 0xF) | (((qh >> j) & 1) << 4)));
  for (int j = 0; j < 16; ++j) e.codes.push_back(static_cast<uint8_t>((b[6 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4)));
}
void af_q5_1(const uint8_t* b, Emit& e) {
  uint32_t qh;
  std::memcpy(&qh, b + 4, 4);
  e.group(half_to_float(rd16(b)), half_to_float(rd16(b + 2)));
  for (int j = 0; j < 16; ++j) e.codes.push_back(static_cast<uint8_t>((b[8 + j] & 0xF) | (((qh >> j) & 1) << 4)));
  for (int j = 0; j < 16; ++j) e.codes.push_back(static_cast<uint8_t>((b[8 + j] >> 4) | (((qh >> (j + 16)) & 1) << 4)));
}
void af_q8_0(const uint8_t* b, Emit& e) {
  const float d = half_to_float(rd16(b));
  e.group(d, -128.f * d);
  for (int j = 0; j < 32; ++j) e.codes.push_back(static_cast<uint8_t>(static_cast<int>(static_cast<int8_t>(b[2 + j])) + 128));
}
void af_q2_k(const uint8_t* b, Emit& e) {
  const uint8_t* scales = b;
  const uint8_t* q = b + 16;
  const float d = half_to_float(rd16(b + 80)), dmin = half_to_float(rd16(b + 82));
  int is = 0;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      for (int half = 0; half < 2; ++half) {
        const uint8_t sc = scales[is++];
        e.group(d * static_cast<float>(sc & 0xF), -dmin * static_cast<float>(sc >> 4));
        for (int l = 0; l < 16; ++l) e.codes.push_back((q[l + 16 * half] >> shift) & 3);
      }
      shift += 2;
    }
    q += 32;
  }
}
void af_q3_k(const uint8_t* b, Emit& e) {
  const uint8_t* hm = b;
  const uint8_t* q = b + 32;
  int8_t sc[16];
  q3k_scales(b + 96, sc);
  const float d_all = half_to_float(rd16(b + 108));
  int is = 0;
  uint8_t m = 1;
  for (int n = 0; n < 256; n += 128) {
    int shift = 0;
    for (int j = 0; j < 4; ++j) {
      for (int half = 0; half < 2; ++half) {
        const float dl = d_all * static_cast<float>(sc[is++]);
        e.group(dl, -4.f * dl);
        for (int l = 0; l < 16; ++l) {
          const int idx = l + 16 * half;
          e.codes.push_back(static_cast<uint8_t>(((q[idx] >> shift) & 3) | ((hm[idx] & m) ? 4 : 0)));
        }
      }
      shift += 2;
      m <<= 1;
    }
    q += 32;
  }
}
void af_q45_k(const uint8_t* b, Emit& e, bool q5) {
  const float d = half_to_float(rd16(b)), dmin = half_to_float(rd16(b + 2));
  const uint8_t* scales = b + 4;
  const uint8_t* qh = b + 16;
  const uint8_t* ql = q5 ? b + 48 : b + 16;
  int is = 0;
  uint8_t u1 = 1, u2 = 2;
  for (int j = 0; j < 256; j += 64) {
    uint8_t sc, m;
    k4_scale_min(is, scales, &sc, &m);
    e.group(d * sc, -dmin * m);
    for (int l = 0; l < 32; ++l) e.codes.push_back(static_cast<uint8_t>((ql[l] & 0xF) | ((q5 && (qh[l] & u1)) ? 16 : 0)));
    k4_scale_min(is + 1, scales, &sc, &m);
    e.group(d * sc, -dmin * m);
    for (int l = 0; l < 32; ++l) e.codes.push_back(static_cast<uint8_t>((ql[l] >> 4) | ((q5 && (qh[l] & u2)) ? 16 : 0)));
    ql += 32;
    is += 2;
    u1 <<= 2;
    u2 <<= 2;
  }
}
void af_q6_k(const uint8_t* b, Emit& e) {
  const uint8_t* ql = b;
  const uint8_t* qh = b + 128;
  const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
  const float d = half_to_float(rd16(b + 208));
  uint8_t codes[256];
  for (int n = 0, base = 0; n < 256; n += 128, base += 128) {
    for (int l = 0; l < 32; ++l) {
      codes[base + l] = static_cast<uint8_t>((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4));
      codes[base + l + 32] = static_cast<uint8_t>((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4));
      codes[base + l + 64] = static_cast<uint8_t>((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4));
      codes[base + l + 96] = static_cast<uint8_t>((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4));
    }
    ql += 64;
    qh += 32;
  }
  for (int gi = 0; gi < 16; ++gi) {
    const float s = d * static_cast<float>(sc[gi]);
    e.group(s, -32.f * s);
  }
  e.codes.insert(e.codes.end(), codes, codes + 256);
}
}  // namespace

void ggml_to_affine(uint32_t type, const uint8_t* src, size_t rows, size_t cols, AffineTensor* out) {
  int bits, group;
  GgmlGeometry g;
  if (!ggml_affine_config(type, &bits, &group) || !ggml_geometry(type, &g))
    throw std::runtime_error(std::string("no affine form for GGML type ") + ggml_type_name(type));
  if (cols % g.block_elems != 0) throw std::runtime_error("row length is not a multiple of the block size");
  out->bits = bits;
  out->group_size = group;
  out->packed.clear();
  out->scales.clear();
  out->biases.clear();
  out->packed.reserve(rows * cols * bits / 32);
  Emit e{out, {}};
  const size_t blocks_per_row = cols / g.block_elems;
  for (size_t r = 0; r < rows; ++r) {
    e.codes.clear();
    for (size_t bi = 0; bi < blocks_per_row; ++bi) {
      const uint8_t* b = src + (r * blocks_per_row + bi) * g.block_bytes;
      switch (type) {
        case GGML_Q4_0: af_q4_0(b, e); break;
        case GGML_Q4_1: af_q4_1(b, e); break;
        case GGML_Q5_0: af_q5_0(b, e); break;
        case GGML_Q5_1: af_q5_1(b, e); break;
        case GGML_Q8_0: af_q8_0(b, e); break;
        case GGML_Q2_K: af_q2_k(b, e); break;
        case GGML_Q3_K: af_q3_k(b, e); break;
        case GGML_Q4_K: af_q45_k(b, e, false); break;
        case GGML_Q5_K: af_q45_k(b, e, true); break;
        case GGML_Q6_K: af_q6_k(b, e); break;
        default: break;
      }
    }
    pack_codes(e.codes.data(), e.codes.size(), bits, &out->packed);
  }
}

// ------------------------------------------------------------------------------------------ encoders
void quantize_q8_0(const float* x, size_t n, uint8_t* dst) {
  for (size_t b = 0; b < n / 32; ++b) {
    const float* v = x + 32 * b;
    float amax = 0.f;
    for (int j = 0; j < 32; ++j) amax = std::max(amax, std::fabs(v[j]));
    const float d = amax / 127.f;
    const float id = d > 0.f ? 1.f / d : 0.f;
    uint8_t* o = dst + 34 * b;
    const uint16_t dh = float_to_half(d);
    o[0] = dh & 0xFF;
    o[1] = dh >> 8;
    for (int j = 0; j < 32; ++j) o[2 + j] = static_cast<uint8_t>(static_cast<int8_t>(std::lround(v[j] * id)));
  }
}

void quantize_q4_0(const float* x, size_t n, uint8_t* dst) {
  for (size_t b = 0; b < n / 32; ++b) {
    const float* v = x + 32 * b;
    float amax = 0.f, mx = 0.f;
    for (int j = 0; j < 32; ++j)
      if (std::fabs(v[j]) > amax) { amax = std::fabs(v[j]); mx = v[j]; }
    const float d = mx / -8.f;
    const float id = d != 0.f ? 1.f / d : 0.f;
    uint8_t* o = dst + 18 * b;
    const uint16_t dh = float_to_half(d);
    o[0] = dh & 0xFF;
    o[1] = dh >> 8;
    for (int j = 0; j < 16; ++j) {
      const int q0 = std::min(15, static_cast<int>(v[j] * id + 8.5f));
      const int q1 = std::min(15, static_cast<int>(v[j + 16] * id + 8.5f));
      o[2 + j] = static_cast<uint8_t>(std::max(0, q0) | (std::max(0, q1) << 4));
    }
  }
}

// Q4_K: per 32-value sub-block an affine fit (scale, min >= 0); the eight (scale, min) pairs are then
// quantised to 6 bits against the super-block maxima and the codes recomputed with the rounded pairs.
void quantize_q4_k(const float* x, size_t n, uint8_t* dst) {
  for (size_t b = 0; b < n / 256; ++b) {
    const float* v = x + 256 * b;
    float scales[8], mins[8];
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; ++j) {
      float lo = FLT_MAX, hi = -FLT_MAX;
      for (int l = 0; l < 32; ++l) {
        lo = std::min(lo, v[32 * j + l]);
        hi = std::max(hi, v[32 * j + l]);
      }
      if (lo > 0.f) lo = 0.f;
      scales[j] = (hi - lo) / 15.f;
      mins[j] = -lo;
      max_scale = std::max(max_scale, scales[j]);
      max_min = std::max(max_min, mins[j]);
    }
    const float inv_scale = max_scale > 0.f ? 63.f / max_scale : 0.f;
    const float inv_min = max_min > 0.f ? 63.f / max_min : 0.f;
    uint8_t* o = dst + 144 * b;
    const uint16_t dh = float_to_half(max_scale / 63.f), mh = float_to_half(max_min / 63.f);
    o[0] = dh & 0xFF; o[1] = dh >> 8; o[2] = mh & 0xFF; o[3] = mh >> 8;
    uint8_t* sc = o + 4;
    std::memset(sc, 0, 12);
    uint8_t ls[8], lm[8];
    for (int j = 0; j < 8; ++j) {
      ls[j] = static_cast<uint8_t>(std::min(63L, std::lround(inv_scale * scales[j])));
      lm[j] = static_cast<uint8_t>(std::min(63L, std::lround(inv_min * mins[j])));
      if (j < 4) {
        sc[j] = ls[j];
        sc[j + 4] = lm[j];
      } else {
        sc[j + 4] = static_cast<uint8_t>((ls[j] & 0xF) | ((lm[j] & 0xF) << 4));
        sc[j - 4] |= static_cast<uint8_t>((ls[j] >> 4) << 6);
        sc[j] |= static_cast<uint8_t>((lm[j] >> 4) << 6);
      }
    }
    const float d = half_to_float(dh), dm = half_to_float(mh);
    uint8_t L[256];
    for (int j = 0; j < 8; ++j) {
      const float dj = d * ls[j], mj = dm * lm[j];
      for (int l = 0; l < 32; ++l) {
        int q = dj > 0.f ? static_cast<int>(std::lround((v[32 * j + l] + mj) / dj)) : 0;
        L[32 * j + l] = static_cast<uint8_t>(std::max(0, std::min(15, q)));
      }
    }
    uint8_t* q = o + 16;
    for (int j = 0; j < 256; j += 64)
      for (int l = 0; l < 32; ++l) *q++ = static_cast<uint8_t>(L[j + l] | (L[j + l + 32] << 4));
  }
}

void quantize_q6_k(const float* x, size_t n, uint8_t* dst) {
  for (size_t b = 0; b < n / 256; ++b) {
    const float* v = x + 256 * b;
    float scales[16];
    float max_abs_scale = 0.f, max_scale = 0.f;
    for (int g = 0; g < 16; ++g) {
      float amax = 0.f, mx = 0.f;
      for (int l = 0; l < 16; ++l)
        if (std::fabs(v[16 * g + l]) > amax) { amax = std::fabs(v[16 * g + l]); mx = v[16 * g + l]; }
      scales[g] = mx / -32.f;
      if (std::fabs(scales[g]) > max_abs_scale) { max_abs_scale = std::fabs(scales[g]); max_scale = scales[g]; }
    }
    uint8_t* o = dst + 210 * b;
    std::memset(o, 0, 210);
    if (max_abs_scale == 0.f) continue;
    const float iscale = -128.f / max_scale;
    const uint16_t dh = float_to_half(1.f / iscale);
    o[208] = dh & 0xFF;
    o[209] = dh >> 8;
    const float d = half_to_float(dh);
    int8_t* sc = reinterpret_cast<int8_t*>(o + 192);
    uint8_t L[256];
    for (int g = 0; g < 16; ++g) {
      sc[g] = static_cast<int8_t>(std::min(127L, std::lround(iscale * scales[g])));
      const float dg = d * sc[g];
      for (int l = 0; l < 16; ++l) {
        int q = dg != 0.f ? static_cast<int>(std::lround(v[16 * g + l] / dg)) : 0;
        L[16 * g + l] = static_cast<uint8_t>(std::max(-32, std::min(31, q)) + 32);
      }
    }
    uint8_t* ql = o;
    uint8_t* qh = o + 128;
    for (int j = 0; j < 256; j += 128) {
      for (int l = 0; l < 32; ++l) {
        const uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF, q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
        ql[l] = static_cast<uint8_t>(q1 | (q3 << 4));
        ql[l + 32] = static_cast<uint8_t>(q2 | (q4 << 4));
        qh[l] = static_cast<uint8_t>((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) | ((L[j + l + 64] >> 4) << 4) |
                                     ((L[j + l + 96] >> 4) << 6));
      }
      ql += 64;
      qh += 32;
    }
  }
}

}  // namespace eredu
