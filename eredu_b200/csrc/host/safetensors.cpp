// SafeTensors weight store: header-only inspection, lazily memory-mapped shards with a bounded
// mapped-shard cache, zero-copy tensor views, contiguous row-range selections for rank-selective
// (tensor-parallel) reads, and a writer.
//
// Behavioural reference: eredu/src/backend/mlx/runtime/checkpoint/store.rs:1374-1400 (mmap, bounded
// mapped shards, default 4), :314-360 (store contract), eredu-core/src/artifact.rs:709-861 (header-only
// inspection of `model.safetensors` / `model.safetensors.index.json` shard sets).
#include <fcntl.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <list>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace py = pybind11;

namespace eredu {

namespace {

struct StMapping {
  void* base = nullptr;
  size_t size = 0;
  ~StMapping() {
    if (base != nullptr && base != MAP_FAILED) munmap(base, size);
  }
};

struct StTensor {
  int shard;
  std::string dtype;
  std::vector<int64_t> shape;
  uint64_t begin, end;  // byte range inside the shard's data section
};

int dtype_bytes(const std::string& d) {
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
  if (d == "I8" || d == "U8" || d == "BOOL" || d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0") return 1;
  if (d == "F4") return 1;  // two E2M1 codes per byte: such a tensor is carried with its last axis counted in bytes
  throw std::runtime_error("safetensors: unknown dtype " + d);
}

// numpy dtype used to *carry* the bytes (bf16 / fp8 have no numpy type: same-width unsigned ints)
py::dtype carrier_dtype(const std::string& d) {
  if (d == "F64") return py::dtype("float64");
  if (d == "F32") return py::dtype("float32");
  if (d == "F16") return py::dtype("float16");
  if (d == "BF16" || d == "U16") return py::dtype("uint16");
  if (d == "I64") return py::dtype("int64");
  if (d == "U64") return py::dtype("uint64");
  if (d == "I32") return py::dtype("int32");
  if (d == "U32") return py::dtype("uint32");
  if (d == "I16") return py::dtype("int16");
  if (d == "I8") return py::dtype("int8");
  if (d == "BOOL") return py::dtype("bool");
  return py::dtype("uint8");
}

}  // namespace

class SafetensorsStore {
 public:
  SafetensorsStore(const std::string& path, int max_mapped) : max_mapped_(std::max(1, max_mapped)) {
    struct stat st;
    if (stat(path.c_str(), &st) != 0) throw std::runtime_error("safetensors: no such path " + path);
    if (S_ISDIR(st.st_mode)) {
      dir_ = path;
      const std::string index = path + "/model.safetensors.index.json";
      if (file_exists(index)) {
        py::object json = py::module_::import("json");
        py::dict idx = json.attr("loads")(read_text(index));
        py::dict wm = idx["weight_map"];
        std::map<std::string, int> shard_of;
        for (auto kv : wm) {
          const std::string file = kv.second.cast<std::string>();
          if (!shard_of.count(file)) {
            shard_of[file] = static_cast<int>(files_.size());
            files_.push_back(path + "/" + file);
          }
        }
      } else if (file_exists(path + "/model.safetensors")) {
        files_.push_back(path + "/model.safetensors");
      } else {
        py::object glob = py::module_::import("glob");
        py::list found = glob.attr("glob")(path + "/*.safetensors");
        std::vector<std::string> names;
        for (auto f : found) names.push_back(f.cast<std::string>());
        std::sort(names.begin(), names.end());
        files_ = names;
      }
    } else {
      files_.push_back(path);
    }
    if (files_.empty()) throw std::runtime_error("safetensors: no *.safetensors under " + path);
    data_offsets_.resize(files_.size());
    file_sizes_.resize(files_.size());
    metadata_.resize(files_.size());
    for (size_t i = 0; i < files_.size(); ++i) read_header(static_cast<int>(i));
  }

  std::vector<std::string> keys() const {
    std::vector<std::string> k;
    for (const auto& kv : tensors_) k.push_back(kv.first);
    return k;
  }
  bool has(const std::string& name) const { return tensors_.count(name) != 0; }
  py::dict info(const std::string& name) const {
    const StTensor& t = get(name);
    py::dict d;
    d["dtype"] = t.dtype;
    d["shape"] = t.shape;
    d["shard"] = files_[t.shard];
    d["nbytes"] = t.end - t.begin;
    return d;
  }
  py::dict metadata(int shard) const { return metadata_.at(shard); }

  // Zero-copy view; the mapping stays alive as long as the returned array does.
  py::array tensor(const std::string& name) { return view(get(name), 0, -1); }

  // Rows [start, stop) of the leading dimension: contiguous, still zero-copy.
  py::array rows(const std::string& name, int64_t start, int64_t stop) {
    const StTensor& t = get(name);
    if (t.shape.empty()) throw std::runtime_error("safetensors: rank-0 tensor has no rows");
    if (start < 0 || stop > t.shape[0] || start > stop) throw std::runtime_error("safetensors: row range out of bounds");
    return view(t, start, stop);
  }

  py::dict diagnostics() const {
    py::dict d;
    d["shards"] = files_.size();
    d["mapped_shards"] = lru_.size();
    d["max_mapped_shards"] = max_mapped_;
    d["map_events"] = map_events_;
    d["unmap_events"] = unmap_events_;
    d["header_bytes_read"] = header_bytes_;
    uint64_t mapped = 0;
    for (const auto& e : lru_) mapped += e.second->size;
    d["mapped_bytes"] = mapped;
    return d;
  }

 private:
  static bool file_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
  }
  static std::string read_text(const std::string& p) {
    std::ifstream f(p, std::ios::binary);
    return std::string((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  }
  const StTensor& get(const std::string& name) const {
    auto it = tensors_.find(name);
    if (it == tensors_.end()) throw std::runtime_error("safetensors: no tensor named " + name);
    return it->second;
  }

  void read_header(int shard) {
    const std::string& path = files_[shard];
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("safetensors: cannot open " + path);
    struct stat st;
    fstat(fd, &st);
    file_sizes_[shard] = static_cast<uint64_t>(st.st_size);
    uint64_t n = 0;
    if (pread(fd, &n, 8, 0) != 8) {
      ::close(fd);
      throw std::runtime_error("safetensors: truncated header in " + path);
    }
    if (n > (100ull << 20) || 8 + n > file_sizes_[shard]) {
      ::close(fd);
      throw std::runtime_error("safetensors: implausible header length in " + path);
    }
    std::string header(n, '\0');
    if (pread(fd, &header[0], n, 8) != static_cast<ssize_t>(n)) {
      ::close(fd);
      throw std::runtime_error("safetensors: short header read in " + path);
    }
    ::close(fd);
    header_bytes_ += 8 + n;
    data_offsets_[shard] = 8 + n;
    py::object json = py::module_::import("json");
    py::dict h = json.attr("loads")(py::bytes(header));
    const uint64_t data_size = file_sizes_[shard] - data_offsets_[shard];
    py::dict md;
    for (auto kv : h) {
      const std::string name = kv.first.cast<std::string>();
      if (name == "__metadata__") {
        md = kv.second.cast<py::dict>();
        continue;
      }
      py::dict e = kv.second.cast<py::dict>();
      StTensor t;
      t.shard = shard;
      t.dtype = e["dtype"].cast<std::string>();
      t.shape = e["shape"].cast<std::vector<int64_t>>();
      if (t.dtype == "F4") {
        // the header counts 4-bit elements; two share a byte along the last axis
        if (t.shape.empty() || t.shape.back() % 2 != 0)
          throw std::runtime_error("safetensors: F4 tensor " + name + " needs an even last dimension");
        t.shape.back() /= 2;
      }
      py::sequence off = e["data_offsets"];
      t.begin = off[0].cast<uint64_t>();
      t.end = off[1].cast<uint64_t>();
      uint64_t elems = 1;
      for (int64_t d : t.shape) elems *= static_cast<uint64_t>(d);
      if (t.end < t.begin || t.end > data_size || (t.end - t.begin) != elems * dtype_bytes(t.dtype))
        throw std::runtime_error("safetensors: bad extent for " + name + " in " + path);
      if (tensors_.count(name)) throw std::runtime_error("safetensors: duplicate tensor " + name);
      tensors_[name] = std::move(t);
    }
    metadata_[shard] = md;
  }

  std::shared_ptr<StMapping> mapping(int shard) {
    for (auto it = lru_.begin(); it != lru_.end(); ++it) {
      if (it->first == shard) {
        auto m = it->second;
        lru_.erase(it);
        lru_.emplace_front(shard, m);
        return m;
      }
    }
    const int fd = ::open(files_[shard].c_str(), O_RDONLY);
    if (fd < 0) throw std::runtime_error("safetensors: cannot open " + files_[shard]);
    auto m = std::make_shared<StMapping>();
    m->size = file_sizes_[shard];
    m->base = mmap(nullptr, m->size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m->base == MAP_FAILED) throw std::runtime_error("safetensors: mmap failed for " + files_[shard]);
    ++map_events_;
    lru_.emplace_front(shard, m);
    while (static_cast<int>(lru_.size()) > max_mapped_) {
      lru_.pop_back();  // outstanding views keep their own reference; the cache just forgets the shard
      ++unmap_events_;
    }
    return m;
  }

  py::array view(const StTensor& t, int64_t row0, int64_t row1) {
    auto m = mapping(t.shard);
    std::vector<py::ssize_t> shape(t.shape.begin(), t.shape.end());
    const int width = dtype_bytes(t.dtype);
    uint64_t row_bytes = width;
    for (size_t i = 1; i < t.shape.size(); ++i) row_bytes *= static_cast<uint64_t>(t.shape[i]);
    uint64_t begin = t.begin;
    if (row1 >= 0) {
      begin += static_cast<uint64_t>(row0) * row_bytes;
      shape[0] = row1 - row0;
    }
    const uint8_t* p = static_cast<const uint8_t*>(m->base) + data_offsets_[t.shard] + begin;
    auto* keep = new std::shared_ptr<StMapping>(m);
    py::capsule owner(keep, [](void* q) { delete static_cast<std::shared_ptr<StMapping>*>(q); });
    py::dtype dt = carrier_dtype(t.dtype);
    std::vector<py::ssize_t> strides(shape.size());
    py::ssize_t s = width;
    for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) {
      strides[i] = s;
      s *= shape[i];
    }
    py::array a(dt, shape, strides, p, owner);
    // read-only: the mapping is PROT_READ
    py::detail::array_proxy(a.ptr())->flags &= ~py::detail::npy_api::NPY_ARRAY_WRITEABLE_;
    return a;
  }

  std::string dir_;
  std::vector<std::string> files_;
  std::vector<uint64_t> data_offsets_, file_sizes_;
  std::vector<py::dict> metadata_;
  std::map<std::string, StTensor> tensors_;
  std::list<std::pair<int, std::shared_ptr<StMapping>>> lru_;
  int max_mapped_;
  uint64_t map_events_ = 0, unmap_events_ = 0, header_bytes_ = 0;
};

// tensors: list of (name, dtype string, shape, contiguous buffer); metadata: str -> str
static void write_safetensors(const std::string& path, py::list tensors, py::dict metadata) {
  py::object json = py::module_::import("json");
  py::dict header;
  if (py::len(metadata) > 0) header["__metadata__"] = metadata;
  uint64_t off = 0;
  std::vector<py::buffer_info> bufs;
  for (auto item : tensors) {
    py::tuple t = item.cast<py::tuple>();
    const std::string name = t[0].cast<std::string>();
    const std::string dtype = t[1].cast<std::string>();
    std::vector<int64_t> shape = t[2].cast<std::vector<int64_t>>();
    py::buffer_info bi = t[3].cast<py::buffer>().request();
    uint64_t elems = 1;
    for (int64_t d : shape) elems *= static_cast<uint64_t>(d);
    const uint64_t nbytes = elems * dtype_bytes(dtype);
    if (static_cast<uint64_t>(bi.size * bi.itemsize) != nbytes)
      throw std::runtime_error("safetensors writer: " + name + " has the wrong byte count");
    py::dict e;
    e["dtype"] = dtype;
    e["shape"] = shape;
    e["data_offsets"] = py::make_tuple(off, off + nbytes);
    header[py::str(name)] = e;
    off += nbytes;
    bufs.push_back(std::move(bi));
  }
  std::string h = json.attr("dumps")(header, py::arg("separators") = py::make_tuple(",", ":")).cast<std::string>();
  while ((h.size() + 8) % 8 != 0) h.push_back(' ');
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f) throw std::runtime_error("safetensors writer: cannot create " + path);
  const uint64_t n = h.size();
  f.write(reinterpret_cast<const char*>(&n), 8);
  f.write(h.data(), static_cast<std::streamsize>(h.size()));
  for (const py::buffer_info& bi : bufs) f.write(static_cast<const char*>(bi.ptr), bi.size * bi.itemsize);
  if (!f) throw std::runtime_error("safetensors writer: short write to " + path);
}

void bind_safetensors(py::module_& m) {
  py::class_<SafetensorsStore>(m, "SafetensorsStore")
      .def(py::init<const std::string&, int>(), py::arg("path"), py::arg("max_mapped_shards") = 4)
      .def("keys", &SafetensorsStore::keys)
      .def("has", &SafetensorsStore::has)
      .def("info", &SafetensorsStore::info)
      .def("metadata", &SafetensorsStore::metadata, py::arg("shard") = 0)
      .def("tensor", &SafetensorsStore::tensor)
      .def("rows", &SafetensorsStore::rows)
      .def("diagnostics", &SafetensorsStore::diagnostics);
  m.def("write_safetensors", &write_safetensors, py::arg("path"), py::arg("tensors"), py::arg("metadata") = py::dict());
}

}  // namespace eredu
