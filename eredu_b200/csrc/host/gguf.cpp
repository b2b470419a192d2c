// GGUF v1-v3 container: memory-mapped reader (single file or "-00001-of-0000N.gguf" shard sets), writer,
// tensor dequantisation and conversion to affine group quantisation.
//
// Behavioural reference: eredu-gguf/src/reader.rs:567-905 (header limits, alignment, shard discovery via
// split.no / split.count / split.tensors.count), format.rs:254-437, writer.rs:30-175, convert.rs:124-545.
// Tensor shapes are reported row-major (GGUF stores ne[0] = innermost first; we reverse).
#include <fcntl.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <fstream>
#include <map>
#include <memory>

#include "ggml_quants.h"

namespace py = pybind11;

namespace eredu {

namespace {

constexpr uint32_t kMagicLE = 0x46554747u;  // "GGUF"
constexpr uint64_t kMaxStringBytes = 1ull << 30;
constexpr uint64_t kMaxArrayElems = 1ull << 31;
constexpr uint64_t kMaxTensors = 1ull << 24;
constexpr uint64_t kMaxKv = 1ull << 24;

enum ValueType : uint32_t { U8 = 0, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 };

struct Mapping {
  void* base = nullptr;
  size_t size = 0;
  ~Mapping() {
    if (base != nullptr && base != MAP_FAILED) munmap(base, size);
  }
};

struct Cursor {
  const uint8_t* p;
  const uint8_t* end;
  bool swap;  // big-endian file
  int version;
  void need(size_t n) const {
    if (static_cast<size_t>(end - p) < n) throw std::runtime_error("GGUF: truncated file");
  }
  template <typename T>
  T raw() {
    need(sizeof(T));
    T v;
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    if (swap) {
      uint8_t* b = reinterpret_cast<uint8_t*>(&v);
      std::reverse(b, b + sizeof(T));
    }
    return v;
  }
  uint64_t len() { return version == 1 ? raw<uint32_t>() : raw<uint64_t>(); }
  std::string str() {
    const uint64_t n = len();
    if (n > kMaxStringBytes) throw std::runtime_error("GGUF: string too long");
    need(n);
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    return s;
  }
};

py::object read_scalar(Cursor& c, uint32_t t) {
  switch (t) {
    case U8: return py::int_(c.raw<uint8_t>());
    case I8: return py::int_(c.raw<int8_t>());
    case U16: return py::int_(c.raw<uint16_t>());
    case I16: return py::int_(c.raw<int16_t>());
    case U32: return py::int_(c.raw<uint32_t>());
    case I32: return py::int_(c.raw<int32_t>());
    case F32: return py::float_(c.raw<float>());
    case BOOL: return py::bool_(c.raw<uint8_t>() != 0);
    case STRING: {
      std::string s = c.str();
      PyObject* o = PyUnicode_DecodeUTF8(s.data(), static_cast<Py_ssize_t>(s.size()), "replace");
      return py::reinterpret_steal<py::object>(o);
    }
    case U64: return py::int_(c.raw<uint64_t>());
    case I64: return py::int_(c.raw<int64_t>());
    case F64: return py::float_(c.raw<double>());
    default: throw std::runtime_error("GGUF: unknown metadata value type " + std::to_string(t));
  }
}

py::object read_value(Cursor& c, uint32_t t) {
  if (t != ARRAY) return read_scalar(c, t);
  const uint32_t et = c.raw<uint32_t>();
  const uint64_t n = c.len();
  if (n > kMaxArrayElems) throw std::runtime_error("GGUF: array too long");
  if (et == ARRAY) throw std::runtime_error("GGUF: nested arrays are not supported");
  py::list out;
  for (uint64_t i = 0; i < n; ++i) out.append(read_scalar(c, et));
  return std::move(out);
}

struct TensorInfo {
  std::string name;
  std::vector<uint64_t> ne;  // GGUF order (innermost first)
  uint32_t type = 0;
  uint64_t offset = 0;       // relative to the shard's data section
  uint64_t nbytes = 0;
  int shard = 0;
  uint64_t elems() const {
    uint64_t n = 1;
    for (uint64_t d : ne) n *= d;
    return n;
  }
  std::vector<uint64_t> shape() const { return std::vector<uint64_t>(ne.rbegin(), ne.rend()); }
};

struct Shard {
  std::string path;
  std::shared_ptr<Mapping> map;
  uint64_t data_offset = 0;
  bool big_endian = false;
  int version = 3;
};

}  // namespace

class GgufReader {
 public:
  explicit GgufReader(const std::string& path) {
    open_shard(path, true);
    // shard set?
    int count = 1;
    if (metadata_.contains("split.count")) count = metadata_["split.count"].cast<int>();
    if (count > 1) {
      const std::string marker = "-00001-of-";
      const size_t at = path.rfind(marker);
      if (at == std::string::npos) throw std::runtime_error("GGUF: split.count > 1 but the path is not a -00001-of-N shard");
      for (int i = 2; i <= count; ++i) {
        char buf[64];
        std::snprintf(buf, sizeof(buf), "-%05d-of-%05d.gguf", i, count);
        open_shard(path.substr(0, at) + buf, false);
      }
      if (metadata_.contains("split.tensors.count")) {
        const uint64_t want = metadata_["split.tensors.count"].cast<uint64_t>();
        if (want != tensors_.size())
          throw std::runtime_error("GGUF: shard set holds " + std::to_string(tensors_.size()) + " tensors, header says " +
                                   std::to_string(want));
      }
    }
  }

  py::dict metadata() const { return metadata_; }
  int version() const { return shards_.front().version; }
  bool big_endian() const { return shards_.front().big_endian; }
  uint32_t alignment() const { return alignment_; }
  size_t shard_count() const { return shards_.size(); }

  py::list tensors() const {
    py::list out;
    for (const TensorInfo& t : tensors_) {
      py::dict d;
      d["name"] = t.name;
      d["shape"] = t.shape();
      d["type"] = t.type;
      d["type_name"] = ggml_type_name(t.type);
      d["nbytes"] = t.nbytes;
      d["shard"] = t.shard;
      d["offset"] = t.offset;
      out.append(d);
    }
    return out;
  }

  bool has(const std::string& name) const { return index_.count(name) != 0; }

  const TensorInfo& info(const std::string& name) const {
    auto it = index_.find(name);
    if (it == index_.end()) throw std::runtime_error("GGUF: no tensor named " + name);
    return tensors_[it->second];
  }
  const uint8_t* data(const TensorInfo& t) const {
    const Shard& s = shards_[t.shard];
    return static_cast<const uint8_t*>(s.map->base) + s.data_offset + t.offset;
  }

  // Zero-copy view of the raw tensor bytes (kept alive by the reader).
  py::array raw(const std::string& name) {
    const TensorInfo& t = info(name);
    return py::array(py::dtype::of<uint8_t>(), {static_cast<py::ssize_t>(t.nbytes)}, {1}, data(t), py::cast(this));
  }

  py::array_t<float> dequantize(const std::string& name) {
    const TensorInfo& t = info(name);
    if (big_endian() && t.type != GGML_I8) throw std::runtime_error("GGUF: big-endian tensor payloads are not decoded here");
    GgmlGeometry g;
    if (!ggml_geometry(t.type, &g)) throw std::runtime_error("GGUF: unknown tensor type");
    std::vector<py::ssize_t> shape;
    for (uint64_t d : t.shape()) shape.push_back(static_cast<py::ssize_t>(d));
    py::array_t<float> out(shape);
    const uint64_t n = t.elems();
    if (!ggml_dequantize(t.type, data(t), n / g.block_elems, out.mutable_data()))
      throw std::runtime_error(std::string("GGUF: no scalar decoder for ") + ggml_type_name(t.type));
    return out;
  }

  // (packed u32 [rows, cols*bits/32], scales f16 bits [rows, cols/group], biases f16 bits, bits, group)
  py::tuple to_affine(const std::string& name) {
    const TensorInfo& t = info(name);
    if (t.ne.empty()) throw std::runtime_error("GGUF: scalar tensor");
    const uint64_t cols = t.ne[0];
    const uint64_t rows = t.elems() / cols;
    AffineTensor a;
    ggml_to_affine(t.type, data(t), rows, cols, &a);
    py::array_t<uint32_t> packed({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(cols * a.bits / 32)});
    std::memcpy(packed.mutable_data(), a.packed.data(), a.packed.size() * 4);
    py::array_t<uint16_t> scales({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(cols / a.group_size)});
    py::array_t<uint16_t> biases({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(cols / a.group_size)});
    std::memcpy(scales.mutable_data(), a.scales.data(), a.scales.size() * 2);
    std::memcpy(biases.mutable_data(), a.biases.data(), a.biases.size() * 2);
    return py::make_tuple(packed, scales, biases, a.bits, a.group_size);
  }

 private:
  void open_shard(const std::string& path, bool first) {
    Shard s;
    s.path = path;
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("GGUF: cannot open " + path);
    struct stat st;
    if (fstat(fd, &st) != 0) {
      ::close(fd);
      throw std::runtime_error("GGUF: cannot stat " + path);
    }
    s.map = std::make_shared<Mapping>();
    s.map->size = static_cast<size_t>(st.st_size);
    s.map->base = mmap(nullptr, s.map->size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (s.map->base == MAP_FAILED) throw std::runtime_error("GGUF: mmap failed for " + path);
    Cursor c{static_cast<const uint8_t*>(s.map->base), static_cast<const uint8_t*>(s.map->base) + s.map->size, false, 3};
    const uint32_t magic = c.raw<uint32_t>();
    if (magic != kMagicLE) throw std::runtime_error("GGUF: bad magic in " + path);
    uint32_t version = c.raw<uint32_t>();
    if (version > 0xFFFF) {  // byte-swapped version field: big-endian file
      c.swap = true;
      version = ((version & 0xFF) << 24) | ((version & 0xFF00) << 8) | ((version >> 8) & 0xFF00) | (version >> 24);
    }
    if (version < 1 || version > 3) throw std::runtime_error("GGUF: unsupported version " + std::to_string(version));
    c.version = static_cast<int>(version);
    s.version = c.version;
    s.big_endian = c.swap;
    const uint64_t n_tensors = c.len();
    const uint64_t n_kv = c.len();
    if (n_tensors > kMaxTensors || n_kv > kMaxKv) throw std::runtime_error("GGUF: header counts exceed limits");
    py::dict md;
    for (uint64_t i = 0; i < n_kv; ++i) {
      std::string key = c.str();
      const uint32_t t = c.raw<uint32_t>();
      md[py::str(key)] = read_value(c, t);
    }
    uint32_t alignment = 32;
    if (md.contains("general.alignment")) alignment = md["general.alignment"].cast<uint32_t>();
    if (alignment == 0 || (alignment & (alignment - 1)) != 0) throw std::runtime_error("GGUF: alignment must be a power of two");
    const int shard_index = static_cast<int>(shards_.size());
    std::vector<TensorInfo> local;
    for (uint64_t i = 0; i < n_tensors; ++i) {
      TensorInfo t;
      t.name = c.str();
      const uint32_t nd = c.raw<uint32_t>();
      if (nd > 8) throw std::runtime_error("GGUF: tensor rank too large");
      for (uint32_t d = 0; d < nd; ++d) t.ne.push_back(c.version == 1 ? c.raw<uint32_t>() : c.raw<uint64_t>());
      t.type = c.raw<uint32_t>();
      t.offset = c.raw<uint64_t>();
      GgmlGeometry g;
      if (!ggml_geometry(t.type, &g)) throw std::runtime_error("GGUF: unknown tensor type " + std::to_string(t.type) + " for " + t.name);
      const uint64_t n = t.elems();
      if (!t.ne.empty() && t.ne[0] % g.block_elems != 0) throw std::runtime_error("GGUF: row of " + t.name + " is not block aligned");
      t.nbytes = n / g.block_elems * g.block_bytes;
      if (t.offset % alignment != 0) throw std::runtime_error("GGUF: misaligned tensor " + t.name);
      t.shard = shard_index;
      local.push_back(std::move(t));
    }
    const uint64_t header_end = static_cast<uint64_t>(c.p - static_cast<const uint8_t*>(s.map->base));
    s.data_offset = (header_end + alignment - 1) / alignment * alignment;
    for (const TensorInfo& t : local) {
      if (s.data_offset + t.offset + t.nbytes > s.map->size) throw std::runtime_error("GGUF: tensor " + t.name + " runs past the end of " + path);
    }
    if (first) {
      metadata_ = md;
      alignment_ = alignment;
    }
    shards_.push_back(std::move(s));
    for (TensorInfo& t : local) {
      if (index_.count(t.name)) throw std::runtime_error("GGUF: duplicate tensor " + t.name);
      index_[t.name] = tensors_.size();
      tensors_.push_back(std::move(t));
    }
  }

  std::vector<Shard> shards_;
  std::vector<TensorInfo> tensors_;
  std::map<std::string, size_t> index_;
  py::dict metadata_;
  uint32_t alignment_ = 32;
};

// ------------------------------------------------------------------------------------------ writer
class GgufWriter {
 public:
  explicit GgufWriter(uint32_t alignment = 32) : alignment_(alignment) {}

  void add_metadata(const std::string& key, py::object value, const std::string& type_hint = "") {
    std::string buf;
    put_string(buf, key);
    put_value(buf, value, type_hint);
    kv_.push_back(std::move(buf));
  }

  // `data` holds the raw (already encoded) bytes; `shape` is row-major.
  void add_tensor(const std::string& name, const std::vector<uint64_t>& shape, uint32_t type, py::buffer data) {
    py::buffer_info bi = data.request();
    GgmlGeometry g;
    if (!ggml_geometry(type, &g)) throw std::runtime_error("GGUF writer: unknown type");
    uint64_t n = 1;
    for (uint64_t d : shape) n *= d;
    const uint64_t want = n / g.block_elems * g.block_bytes;
    const uint64_t have = static_cast<uint64_t>(bi.size) * static_cast<uint64_t>(bi.itemsize);
    if (want != have) throw std::runtime_error("GGUF writer: " + name + " needs " + std::to_string(want) + " bytes, got " + std::to_string(have));
    Pending p;
    p.name = name;
    p.shape = shape;
    p.type = type;
    p.bytes.assign(static_cast<const char*>(bi.ptr), static_cast<size_t>(have));
    tensors_.push_back(std::move(p));
  }

  void write(const std::string& path) {
    std::string head;
    put<uint32_t>(head, kMagicLE);
    put<uint32_t>(head, 3);
    put<uint64_t>(head, tensors_.size());
    put<uint64_t>(head, kv_.size());
    for (const std::string& kv : kv_) head += kv;
    uint64_t off = 0;
    std::vector<uint64_t> offsets;
    for (const Pending& t : tensors_) {
      offsets.push_back(off);
      off += (t.bytes.size() + alignment_ - 1) / alignment_ * alignment_;
    }
    for (size_t i = 0; i < tensors_.size(); ++i) {
      const Pending& t = tensors_[i];
      put_string(head, t.name);
      put<uint32_t>(head, static_cast<uint32_t>(t.shape.size()));
      for (auto it = t.shape.rbegin(); it != t.shape.rend(); ++it) put<uint64_t>(head, *it);
      put<uint32_t>(head, t.type);
      put<uint64_t>(head, offsets[i]);
    }
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) throw std::runtime_error("GGUF writer: cannot create " + path);
    f.write(head.data(), static_cast<std::streamsize>(head.size()));
    pad(f, head.size());
    for (const Pending& t : tensors_) {
      f.write(t.bytes.data(), static_cast<std::streamsize>(t.bytes.size()));
      pad(f, t.bytes.size());
    }
    if (!f) throw std::runtime_error("GGUF writer: short write to " + path);
  }

 private:
  struct Pending {
    std::string name;
    std::vector<uint64_t> shape;
    uint32_t type;
    std::string bytes;
  };
  template <typename T>
  static void put(std::string& b, T v) {
    b.append(reinterpret_cast<const char*>(&v), sizeof(T));
  }
  static void put_string(std::string& b, const std::string& s) {
    put<uint64_t>(b, s.size());
    b += s;
  }
  void pad(std::ofstream& f, size_t written) {
    const size_t rem = written % alignment_;
    if (rem) {
      std::string z(alignment_ - rem, '\0');
      f.write(z.data(), static_cast<std::streamsize>(z.size()));
    }
  }
  static uint32_t scalar_type(py::handle v, const std::string& hint) {
    if (hint == "u8") return U8; if (hint == "i8") return I8; if (hint == "u16") return U16; if (hint == "i16") return I16;
    if (hint == "u32") return U32; if (hint == "i32") return I32; if (hint == "f32") return F32; if (hint == "bool") return BOOL;
    if (hint == "u64") return U64; if (hint == "i64") return I64; if (hint == "f64") return F64; if (hint == "str") return STRING;
    if (py::isinstance<py::bool_>(v)) return BOOL;
    if (py::isinstance<py::int_>(v)) {
      const long long x = v.cast<long long>();
      return (x >= 0 && x <= 0xFFFFFFFFll) ? U32 : (x < 0 && x >= -0x80000000ll ? I32 : (x < 0 ? I64 : U64));
    }
    if (py::isinstance<py::float_>(v)) return F32;
    if (py::isinstance<py::str>(v)) return STRING;
    throw std::runtime_error("GGUF writer: unsupported metadata value");
  }
  static void put_scalar(std::string& b, py::handle v, uint32_t t) {
    switch (t) {
      case U8: put<uint8_t>(b, v.cast<uint8_t>()); break;
      case I8: put<int8_t>(b, v.cast<int8_t>()); break;
      case U16: put<uint16_t>(b, v.cast<uint16_t>()); break;
      case I16: put<int16_t>(b, v.cast<int16_t>()); break;
      case U32: put<uint32_t>(b, v.cast<uint32_t>()); break;
      case I32: put<int32_t>(b, v.cast<int32_t>()); break;
      case F32: put<float>(b, v.cast<float>()); break;
      case BOOL: put<uint8_t>(b, v.cast<bool>() ? 1 : 0); break;
      case STRING: put_string(b, v.cast<std::string>()); break;
      case U64: put<uint64_t>(b, v.cast<uint64_t>()); break;
      case I64: put<int64_t>(b, v.cast<int64_t>()); break;
      case F64: put<double>(b, v.cast<double>()); break;
      default: throw std::runtime_error("GGUF writer: bad scalar type");
    }
  }
  static void put_value(std::string& b, py::object v, const std::string& hint) {
    if (py::isinstance<py::list>(v) || py::isinstance<py::tuple>(v)) {
      py::sequence seq = v.cast<py::sequence>();
      const uint32_t et = seq.size() ? scalar_type(seq[0], hint) : (hint.empty() ? static_cast<uint32_t>(I32) : scalar_type(py::int_(0), hint));
      put<uint32_t>(b, ARRAY);
      put<uint32_t>(b, et);
      put<uint64_t>(b, seq.size());
      for (py::handle e : seq) put_scalar(b, e, et);
      return;
    }
    const uint32_t t = scalar_type(v, hint);
    put<uint32_t>(b, t);
    put_scalar(b, v, t);
  }

  uint32_t alignment_;
  std::vector<std::string> kv_;
  std::vector<Pending> tensors_;
};

// ------------------------------------------------------------------------------------------ free functions
static py::array_t<float> py_dequantize(uint32_t type, py::buffer raw, size_t n_elems) {
  py::buffer_info bi = raw.request();
  GgmlGeometry g;
  if (!ggml_geometry(type, &g)) throw std::runtime_error("unknown GGML type");
  const size_t nblocks = n_elems / g.block_elems;
  if (static_cast<size_t>(bi.size * bi.itemsize) < nblocks * g.block_bytes) throw std::runtime_error("buffer too small");
  py::array_t<float> out(static_cast<py::ssize_t>(n_elems));
  if (!ggml_dequantize(type, static_cast<const uint8_t*>(bi.ptr), nblocks, out.mutable_data()))
    throw std::runtime_error(std::string("no scalar decoder for ") + ggml_type_name(type));
  return out;
}

static py::tuple py_to_affine(uint32_t type, py::buffer raw, size_t rows, size_t cols) {
  py::buffer_info bi = raw.request();
  AffineTensor a;
  ggml_to_affine(type, static_cast<const uint8_t*>(bi.ptr), rows, cols, &a);
  py::array_t<uint32_t> packed({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(cols * a.bits / 32)});
  std::memcpy(packed.mutable_data(), a.packed.data(), a.packed.size() * 4);
  py::array_t<uint16_t> scales({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(cols / a.group_size)});
  py::array_t<uint16_t> biases({static_cast<py::ssize_t>(rows), static_cast<py::ssize_t>(cols / a.group_size)});
  std::memcpy(scales.mutable_data(), a.scales.data(), a.scales.size() * 2);
  std::memcpy(biases.mutable_data(), a.biases.data(), a.biases.size() * 2);
  return py::make_tuple(packed, scales, biases, a.bits, a.group_size);
}

static py::bytes py_quantize(uint32_t type, py::array_t<float, py::array::c_style | py::array::forcecast> x) {
  GgmlGeometry g;
  if (!ggml_geometry(type, &g)) throw std::runtime_error("unknown GGML type");
  const size_t n = static_cast<size_t>(x.size());
  if (n % g.block_elems != 0) throw std::runtime_error("element count is not a multiple of the block size");
  std::string out(n / g.block_elems * g.block_bytes, '\0');
  uint8_t* dst = reinterpret_cast<uint8_t*>(&out[0]);
  switch (type) {
    case GGML_Q8_0: quantize_q8_0(x.data(), n, dst); break;
    case GGML_Q4_0: quantize_q4_0(x.data(), n, dst); break;
    case GGML_Q4_K: quantize_q4_k(x.data(), n, dst); break;
    case GGML_Q6_K: quantize_q6_k(x.data(), n, dst); break;
    case GGML_F32: std::memcpy(dst, x.data(), n * 4); break;
    case GGML_F16:
      for (size_t i = 0; i < n; ++i) { const uint16_t h = float_to_half(x.data()[i]); std::memcpy(dst + 2 * i, &h, 2); }
      break;
    case GGML_BF16:
      for (size_t i = 0; i < n; ++i) { const uint16_t h = float_to_bf16(x.data()[i]); std::memcpy(dst + 2 * i, &h, 2); }
      break;
    default: throw std::runtime_error(std::string("no encoder for ") + ggml_type_name(type));
  }
  return py::bytes(out);
}

void bind_gguf(py::module_& m) {
  py::class_<GgufReader>(m, "GgufReader")
      .def(py::init<const std::string&>())
      .def_property_readonly("metadata", &GgufReader::metadata)
      .def_property_readonly("version", &GgufReader::version)
      .def_property_readonly("big_endian", &GgufReader::big_endian)
      .def_property_readonly("alignment", &GgufReader::alignment)
      .def_property_readonly("shard_count", &GgufReader::shard_count)
      .def("tensors", &GgufReader::tensors)
      .def("has", &GgufReader::has)
      .def("raw", &GgufReader::raw, py::keep_alive<0, 1>())
      .def("dequantize", &GgufReader::dequantize)
      .def("to_affine", &GgufReader::to_affine);
  py::class_<GgufWriter>(m, "GgufWriter")
      .def(py::init<uint32_t>(), py::arg("alignment") = 32)
      .def("add_metadata", &GgufWriter::add_metadata, py::arg("key"), py::arg("value"), py::arg("type_hint") = "")
      .def("add_tensor", &GgufWriter::add_tensor)
      .def("write", &GgufWriter::write);
  m.def("ggml_dequantize", &py_dequantize, "Decode raw GGML blocks to fp32");
  m.def("ggml_to_affine", &py_to_affine, "Convert GGML blocks to (packed, scales, biases, bits, group)");
  m.def("ggml_quantize", &py_quantize, "Encode fp32 values as GGML blocks (Q8_0, Q4_0, Q4_K, Q6_K, F32, F16, BF16)");
  m.def("ggml_block_geometry", [](uint32_t type) {
    GgmlGeometry g;
    if (!ggml_geometry(type, &g)) throw std::runtime_error("unknown GGML type");
    return py::make_tuple(g.block_elems, g.block_bytes);
  });
  m.def("ggml_type_name", [](uint32_t t) { return std::string(ggml_type_name(t)); });
}

}  // namespace eredu
