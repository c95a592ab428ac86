// Byte-exact binary encoding used by checkpoint files and by the CPU socket
// transport.
//
// Wire rules (they reproduce kraken/common/serialize.h:42-395 and
// kraken/common/deserialize.h of the reference so files interchange):
//   * little-endian PODs, no padding, no magic, no version;
//   * vector<POD> / string = u64 count + raw elements;
//   * enums = u8, except StateType = u32;
//   * Tensor = u8 layout; dense: dims(vector<i64>) + u8 dtype + raw bytes;
//              COO: Tensor indices + Tensor values + dims;
//   * map = u64 count + (key, value) pairs.  The reference writes maps in
//     unordered_map order; this writer always emits ascending keys and the
//     reader accepts any order.
#pragma once

#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "types.h"

namespace kb {

// ---------------------------------------------------------------- sinks / sources
class ByteSink {
 public:
  virtual ~ByteSink() = default;
  virtual void Write(const void* p, size_t n) = 0;
};

class ByteSource {
 public:
  virtual ~ByteSource() = default;
  // Returns false when fewer than n bytes remain.
  virtual bool Read(void* p, size_t n) = 0;
};

// Growable in-memory buffer (factor 1.5, like the reference's MemBuffer,
// kraken/common/mem_buffer.cc:74-98).
class MemSink : public ByteSink {
 public:
  void Write(const void* p, size_t n) override {
    if (len_ + n > buf_.size()) {
      size_t cap = buf_.size() < 64 ? 64 : buf_.size();
      while (cap < len_ + n) cap += cap / 2;
      buf_.resize(cap);
    }
    std::memcpy(buf_.data() + len_, p, n);
    len_ += n;
  }
  const uint8_t* data() const { return buf_.data(); }
  size_t size() const { return len_; }
  std::string str() const { return std::string(reinterpret_cast<const char*>(buf_.data()), len_); }

 private:
  std::vector<uint8_t> buf_;
  size_t len_ = 0;
};

// Bounds-checked cursor over borrowed memory (kraken/common/mem_reader.cc:11-20).
class MemSource : public ByteSource {
 public:
  MemSource(const void* p, size_t n) : p_(static_cast<const uint8_t*>(p)), n_(n) {}
  bool Read(void* dst, size_t n) override {
    if (off_ + n > n_) return false;
    std::memcpy(dst, p_ + off_, n);
    off_ += n;
    return true;
  }
  size_t offset() const { return off_; }
  size_t remaining() const { return n_ - off_; }

 private:
  const uint8_t* p_;
  size_t n_;
  size_t off_ = 0;
};

class FileSink : public ByteSink {
 public:
  explicit FileSink(const std::string& path) : f_(std::fopen(path.c_str(), "wb")) {
    if (f_) std::setvbuf(f_, nullptr, _IOFBF, 8 << 20);
  }
  ~FileSink() override { Close(); }
  bool IsOpen() const { return f_ != nullptr; }
  void Write(const void* p, size_t n) override {
    if (n == 0) return;
    KB_CHECK(f_ && std::fwrite(p, 1, n, f_) == n, err::kCheckpointIO, "short write");
  }
  void Close() {
    if (f_) {
      std::fclose(f_);
      f_ = nullptr;
    }
  }

 private:
  FILE* f_;
};

class FileSource : public ByteSource {
 public:
  explicit FileSource(const std::string& path) : f_(std::fopen(path.c_str(), "rb")) {
    if (f_) std::setvbuf(f_, nullptr, _IOFBF, 8 << 20);
  }
  ~FileSource() override {
    if (f_) std::fclose(f_);
  }
  bool IsOpen() const { return f_ != nullptr; }
  bool Read(void* p, size_t n) override { return n == 0 || (f_ && std::fread(p, 1, n, f_) == n); }
  bool AtEnd() {
    if (!f_) return true;
    int c = std::fgetc(f_);
    if (c == EOF) return true;
    std::ungetc(c, f_);
    return false;
  }

 private:
  FILE* f_;
};

// ---------------------------------------------------------------- value types
// Host-side tensor POD: enough structure for checkpoint I/O and the CPU shard.
struct HostTensor {
  Layout layout = Layout::kStride;
  std::vector<int64_t> dims;
  DType dtype = DType::kFloat32;
  std::vector<uint8_t> data;            // dense payload
  std::shared_ptr<HostTensor> indices;  // COO only
  std::shared_ptr<HostTensor> values;   // COO only

  // Product of dims; 0 for rank-0 (kraken/t/shape.cc:95-98 has the same quirk).
  int64_t Numel() const {
    if (dims.empty()) return 0;
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
  size_t NumBytes() const { return static_cast<size_t>(Numel()) * DTypeBytes(dtype); }
  float* f32() { return reinterpret_cast<float*>(data.data()); }
  const float* f32() const { return reinterpret_cast<const float*>(data.data()); }

  static HostTensor F32(std::vector<int64_t> d) {
    HostTensor t;
    t.dims = std::move(d);
    t.dtype = DType::kFloat32;
    t.data.assign(t.NumBytes(), 0);
    return t;
  }
};

struct Value {
  HostTensor val;
  std::map<uint32_t, HostTensor> states;
  std::map<uint32_t, int64_t> states_i;
};

struct TableMeta {
  uint64_t id = 0;
  std::string name;
  TableType table_type = TableType::kDense;
  DType element_type = DType::kFloat32;
  std::vector<int64_t> shape;  // dense only
  int64_t dimension = 0;       // sparse only
  InitializerType init_type = InitializerType::kConstant;
  Conf init_conf;
};

struct ModelMeta {
  std::string name;
  OptimType optim_type = OptimType::kSGD;
  Conf optim_conf;
  std::map<uint64_t, TableMeta> tables;
};

// ---------------------------------------------------------------- writer
class Writer {
 public:
  explicit Writer(ByteSink* s) : s_(s) {}

  template <typename T>
  void Pod(const T& v) {
    static_assert(std::is_trivially_copyable<T>::value, "POD only");
    s_->Write(&v, sizeof(T));
  }
  void Raw(const void* p, size_t n) { s_->Write(p, n); }
  void Str(const std::string& v) {
    Pod<uint64_t>(v.size());
    s_->Write(v.data(), v.size());
  }
  template <typename T>
  void Vec(const std::vector<T>& v) {
    Pod<uint64_t>(v.size());
    s_->Write(v.data(), v.size() * sizeof(T));
  }
  void ConfMap(const Conf& c) {
    Pod<uint64_t>(c.size());
    for (auto& kv : c) {
      Str(kv.first);
      Str(kv.second);
    }
  }
  void Tensor(const HostTensor& t) {
    Pod<uint8_t>(static_cast<uint8_t>(t.layout));
    if (t.layout == Layout::kStride) {
      Vec(t.dims);
      Pod<uint8_t>(static_cast<uint8_t>(t.dtype));
      s_->Write(t.data.data(), t.NumBytes());
    } else {
      KB_CHECK(t.indices && t.values, err::kSerializeRequest, "COO tensor without parts");
      Tensor(*t.indices);
      Tensor(*t.values);
      Vec(t.dims);
    }
  }
  // Dense f32 vector of `dim` elements straight from a row pointer: the hot
  // path of sparse-table export (no HostTensor temporaries).
  void RowF32(const float* row, int64_t dim) {
    Pod<uint8_t>(0);
    Pod<uint64_t>(1);
    Pod<int64_t>(dim);
    Pod<uint8_t>(static_cast<uint8_t>(DType::kFloat32));
    s_->Write(row, static_cast<size_t>(dim) * 4);
  }
  void Val(const Value& v) {
    Tensor(v.val);
    Pod<uint64_t>(v.states.size());
    for (auto& kv : v.states) {
      Pod<uint32_t>(kv.first);
      Tensor(kv.second);
    }
    Pod<uint64_t>(v.states_i.size());
    for (auto& kv : v.states_i) {
      Pod<uint32_t>(kv.first);
      Pod<int64_t>(kv.second);
    }
  }
  void Table(const TableMeta& m) {
    Pod<uint64_t>(m.id);
    Str(m.name);
    Pod<uint8_t>(static_cast<uint8_t>(m.table_type));
    Pod<uint8_t>(static_cast<uint8_t>(m.element_type));
    Vec(m.shape);
    Pod<int64_t>(m.dimension);
    Pod<uint8_t>(static_cast<uint8_t>(m.init_type));
    ConfMap(m.init_conf);
  }
  void Model(const ModelMeta& m) {
    Str(m.name);
    Pod<uint8_t>(static_cast<uint8_t>(m.optim_type));
    ConfMap(m.optim_conf);
    Pod<uint64_t>(m.tables.size());
    for (auto& kv : m.tables) {
      Pod<uint64_t>(kv.first);
      Table(kv.second);
    }
  }

 private:
  ByteSink* s_;
};

// ---------------------------------------------------------------- reader
class Reader {
 public:
  explicit Reader(ByteSource* s) : s_(s) {}

  template <typename T>
  T Pod() {
    T v;
    KB_CHECK(s_->Read(&v, sizeof(T)), err::kDeserializeReply, "truncated input");
    return v;
  }
  void Raw(void* p, size_t n) { KB_CHECK(s_->Read(p, n), err::kDeserializeReply, "truncated input"); }
  std::string Str() {
    uint64_t n = Pod<uint64_t>();
    KB_CHECK(n < (1ull << 32), err::kDeserializeReply, "implausible string length");
    std::string v(n, '\0');
    Raw(&v[0], n);
    return v;
  }
  template <typename T>
  std::vector<T> Vec() {
    uint64_t n = Pod<uint64_t>();
    KB_CHECK(n < (1ull << 40) / sizeof(T), err::kDeserializeReply, "implausible vector length");
    std::vector<T> v(n);
    Raw(v.data(), n * sizeof(T));
    return v;
  }
  Conf ConfMap() {
    Conf c;
    uint64_t n = Pod<uint64_t>();
    for (uint64_t i = 0; i < n; ++i) {
      std::string k = Str();
      c[k] = Str();
    }
    return c;
  }
  HostTensor Tensor() {
    HostTensor t;
    uint8_t layout = Pod<uint8_t>();
    KB_CHECK(layout <= 1, err::kDeserializeReply, "bad tensor layout byte");
    t.layout = static_cast<Layout>(layout);
    if (t.layout == Layout::kStride) {
      t.dims = Vec<int64_t>();
      t.dtype = static_cast<DType>(Pod<uint8_t>());
      KB_CHECK(DTypeBytes(t.dtype) > 0 || t.Numel() == 0, err::kDeserializeReply, "bad dtype byte");
      t.data.resize(t.NumBytes());
      Raw(t.data.data(), t.data.size());
    } else {
      t.indices = std::make_shared<HostTensor>(Tensor());
      t.values = std::make_shared<HostTensor>(Tensor());
      t.dims = Vec<int64_t>();
      t.dtype = t.values->dtype;
    }
    return t;
  }
  Value Val() {
    Value v;
    v.val = Tensor();
    uint64_t ns = Pod<uint64_t>();
    for (uint64_t i = 0; i < ns; ++i) {
      uint32_t k = Pod<uint32_t>();
      v.states[k] = Tensor();
    }
    uint64_t ni = Pod<uint64_t>();
    for (uint64_t i = 0; i < ni; ++i) {
      uint32_t k = Pod<uint32_t>();
      v.states_i[k] = Pod<int64_t>();
    }
    return v;
  }
  TableMeta Table() {
    TableMeta m;
    m.id = Pod<uint64_t>();
    m.name = Str();
    m.table_type = static_cast<TableType>(Pod<uint8_t>());
    m.element_type = static_cast<DType>(Pod<uint8_t>());
    m.shape = Vec<int64_t>();
    m.dimension = Pod<int64_t>();  // garbage for dense tables written by the reference: never validated
    m.init_type = static_cast<InitializerType>(Pod<uint8_t>());
    m.init_conf = ConfMap();
    return m;
  }
  ModelMeta Model() {
    ModelMeta m;
    m.name = Str();
    m.optim_type = static_cast<OptimType>(Pod<uint8_t>());
    m.optim_conf = ConfMap();
    uint64_t n = Pod<uint64_t>();
    for (uint64_t i = 0; i < n; ++i) {
      uint64_t k = Pod<uint64_t>();
      m.tables[k] = Table();
    }
    return m;
  }

 private:
  ByteSource* s_;
};

}  // namespace kb
