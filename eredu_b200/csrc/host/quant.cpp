// CPU reference quantisers for the checkpoint formats the runtime serves: affine group quantisation
// (bits 2/3/4/5/6/8, group 16 or a multiple of 32; w ~ scale * q + bias; codes packed as a little-endian bit
// stream in u32 words, [out, in * bits / 32], scales / biases [out, in / group]) and MXFP4 (E2M1 x 32 with
// one E8M0 scale byte). Format contract: eredu/src/backend/mlx/runtime/checkpoint/quantization.rs:1-8,137-232,
// eredu-checkpoint/src/lib.rs:68-160; the scale / bias rule is the one MLX documents for `quantize`
// (edge-anchored: the group's larger-magnitude extreme is represented exactly).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <cmath>

#include "ggml_quants.h"

namespace py = pybind11;

namespace eredu {

static inline float round_to(float v, int mode) {  // 0: keep fp32, 1: bf16, 2: f16
  if (mode == 1) return bf16_to_float(float_to_bf16(v));
  if (mode == 2) return half_to_float(float_to_half(v));
  return v;
}

// Returns (packed u32 [rows, cols*bits/32], scales f32 [rows, cols/group], biases f32). `store` = dtype the
// scales and biases will be stored in ("f32" | "bf16" | "f16"): they are rounded to it before the codes are
// computed, so that dequantisation with the stored values reproduces the rounding decisions.
static py::tuple affine_quantize(py::array_t<float, py::array::c_style | py::array::forcecast> w, int bits, int group,
                                 const std::string& store) {
  if (w.ndim() != 2) throw std::runtime_error("affine_quantize expects a rank-2 array");
  if (!(bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8)) throw std::runtime_error("unsupported bit width");
  const int64_t rows = w.shape(0), cols = w.shape(1);
  if (!(group == 16 || group % 32 == 0) || cols % group != 0 || (cols * bits) % 32 != 0)
    throw std::runtime_error("group size must be 16 or a multiple of 32 and divide the row length");
  const int mode = store == "bf16" ? 1 : store == "f16" ? 2 : 0;
  const int64_t groups = cols / group;
  py::array_t<uint32_t> packed({rows, cols * bits / 32});
  py::array_t<float> scales({rows, groups}), biases({rows, groups});
  const float* src = w.data();
  uint32_t* pk = packed.mutable_data();
  float* sc = scales.mutable_data();
  float* bs = biases.mutable_data();
  const float n_bins = static_cast<float>((1 << bits) - 1);
  std::vector<uint8_t> codes(cols);
  std::vector<uint32_t> row_words;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < groups; ++g) {
      const float* v = src + r * cols + g * group;
      float lo = v[0], hi = v[0];
      for (int i = 1; i < group; ++i) {
        lo = std::min(lo, v[i]);
        hi = std::max(hi, v[i]);
      }
      const bool mask = std::fabs(lo) > std::fabs(hi);
      float scale = std::max((hi - lo) / n_bins, 1e-7f);
      scale = mask ? scale : -scale;
      const float edge = mask ? lo : hi;
      const float q0 = std::nearbyint(edge / scale);
      float bias = 0.f;
      if (q0 != 0.f) {
        scale = edge / q0;
        bias = edge;
      }
      scale = round_to(scale, mode);
      bias = round_to(bias, mode);
      sc[r * groups + g] = scale;
      bs[r * groups + g] = bias;
      for (int i = 0; i < group; ++i) {
        float q = scale != 0.f ? std::nearbyint((v[i] - bias) / scale) : 0.f;
        q = std::min(std::max(q, 0.f), n_bins);
        codes[g * group + i] = static_cast<uint8_t>(q);
      }
    }
    row_words.clear();
    pack_codes(codes.data(), static_cast<size_t>(cols), bits, &row_words);
    std::memcpy(pk + r * (cols * bits / 32), row_words.data(), row_words.size() * 4);
  }
  return py::make_tuple(packed, scales, biases);
}

static py::array_t<float> affine_dequantize(py::array_t<uint32_t, py::array::c_style | py::array::forcecast> packed,
                                            py::array_t<float, py::array::c_style | py::array::forcecast> scales,
                                            py::array_t<float, py::array::c_style | py::array::forcecast> biases, int bits,
                                            int group) {
  const int64_t rows = packed.shape(0);
  const int64_t cols = packed.shape(1) * 32 / bits;
  const int64_t groups = cols / group;
  py::array_t<float> out({rows, cols});
  std::vector<uint8_t> codes(cols);
  for (int64_t r = 0; r < rows; ++r) {
    unpack_codes(packed.data() + r * packed.shape(1), static_cast<size_t>(cols), bits, codes.data());
    for (int64_t c = 0; c < cols; ++c) {
      const int64_t g = c / group;
      out.mutable_data()[r * cols + c] = scales.data()[r * groups + g] * static_cast<float>(codes[c]) + biases.data()[r * groups + g];
    }
  }
  return out;
}

// MXFP4: returns (packed u32 [rows, cols/8], scales u8 [rows, cols/32]).
static py::tuple mxfp4_quantize(py::array_t<float, py::array::c_style | py::array::forcecast> w) {
  if (w.ndim() != 2 || w.shape(1) % 32 != 0) throw std::runtime_error("mxfp4_quantize expects [rows, cols] with cols % 32 == 0");
  const int64_t rows = w.shape(0), cols = w.shape(1);
  py::array_t<uint32_t> packed({rows, cols / 8});
  py::array_t<uint8_t> scales({rows, cols / 32});
  static const float grid[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  std::vector<uint8_t> codes(cols);
  std::vector<uint32_t> words;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t g = 0; g < cols / 32; ++g) {
      const float* v = w.data() + r * cols + g * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(v[i]));
      int e = amax > 0.f ? static_cast<int>(std::floor(std::log2(amax))) - 2 + 127 : 0;
      e = std::min(std::max(e, 0), 254);
      scales.mutable_data()[r * (cols / 32) + g] = static_cast<uint8_t>(e);
      const float inv = 1.f / e8m0_to_float(static_cast<uint8_t>(e));
      for (int i = 0; i < 32; ++i) {
        const float x = v[i] * inv;
        const float ax = std::fabs(x);
        int best = 0;
        for (int k = 1; k < 8; ++k)
          if (std::fabs(ax - grid[k]) < std::fabs(ax - grid[best]) ||
              (std::fabs(ax - grid[k]) == std::fabs(ax - grid[best]) && (k % 2 == 0)))
            best = k;
        codes[g * 32 + i] = static_cast<uint8_t>(best | (x < 0.f ? 8 : 0));
      }
    }
    words.clear();
    pack_codes(codes.data(), static_cast<size_t>(cols), 4, &words);
    std::memcpy(packed.mutable_data() + r * (cols / 8), words.data(), words.size() * 4);
  }
  return py::make_tuple(packed, scales);
}

static py::array_t<float> mxfp4_dequantize(py::array_t<uint32_t, py::array::c_style | py::array::forcecast> packed,
                                           py::array_t<uint8_t, py::array::c_style | py::array::forcecast> scales) {
  const int64_t rows = packed.shape(0), cols = packed.shape(1) * 8;
  py::array_t<float> out({rows, cols});
  std::vector<uint8_t> codes(cols);
  for (int64_t r = 0; r < rows; ++r) {
    unpack_codes(packed.data() + r * packed.shape(1), static_cast<size_t>(cols), 4, codes.data());
    for (int64_t c = 0; c < cols; ++c)
      out.mutable_data()[r * cols + c] = kE2m1Values[codes[c]] * e8m0_to_float(scales.data()[r * (cols / 32) + c / 32]);
  }
  return out;
}

static py::array_t<uint8_t> py_unpack_codes(py::array_t<uint32_t, py::array::c_style | py::array::forcecast> packed, int bits) {
  const int64_t rows = packed.shape(0), cols = packed.shape(1) * 32 / bits;
  py::array_t<uint8_t> out({rows, cols});
  for (int64_t r = 0; r < rows; ++r)
    unpack_codes(packed.data() + r * packed.shape(1), static_cast<size_t>(cols), bits, out.mutable_data() + r * cols);
  return out;
}

void bind_quant(py::module_& m) {
  m.def("unpack_codes", &py_unpack_codes, "u32 words [rows, cols*bits/32] -> codes u8 [rows, cols]");
  m.def("affine_quantize", &affine_quantize, py::arg("w"), py::arg("bits") = 4, py::arg("group_size") = 64,
        py::arg("store") = "f32");
  m.def("affine_dequantize", &affine_dequantize);
  m.def("mxfp4_quantize", &mxfp4_quantize);
  m.def("mxfp4_dequantize", &mxfp4_dequantize);
}

}  // namespace eredu
