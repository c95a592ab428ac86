#include "checkpoint.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdio>
#include <ctime>
#include <filesystem>
#include <fstream>
#include <numeric>
#include <sstream>
#include <thread>

#include "hash.h"

namespace fs = std::filesystem;

namespace kb {
namespace ckpt {

namespace {

const char* kRouterJson = "router.json";
const char* kRouterBin = "router.binary";
const char* kModelJson = "model.json";
const char* kModelBin = "model.binary";
const char* kDenseSuffix = ".dense";
const char* kSparseSuffix = ".sparse";
const char* kShardPrefix = "shard_";

const char* OptimName(OptimType t) {
  switch (t) {
    case OptimType::kAdagrad: return "Adagrad";
    case OptimType::kAdam: return "Adam";
    case OptimType::kRMSprop: return "RMSprop";
    case OptimType::kSGD: return "SGD";
  }
  return "UnKnow";
}

const char* InitName(InitializerType t) {
  switch (t) {
    case InitializerType::kConstant: return "Constant";
    case InitializerType::kUniform: return "Uniform";
    case InitializerType::kNormal: return "Normal";
    case InitializerType::kXavierUniform: return "XavierUniform";
    case InitializerType::kXavierNormal: return "XavierNormal";
  }
  return "UnKnow";
}

std::string JsonStr(const std::string& s) {
  std::string o = "\"";
  for (char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\t': o += "\\t"; break;
      default:
        if (static_cast<unsigned char>(c) < 0x20) {
          char b[8];
          std::snprintf(b, sizeof(b), "\\u%04x", c);
          o += b;
        } else {
          o += c;
        }
    }
  }
  return o + "\"";
}

std::string JsonConf(const Conf& c, const std::string& ind) {
  if (c.empty()) return "{}";
  std::string o = "{\n";
  size_t i = 0;
  for (auto& kv : c) {
    o += ind + "    " + JsonStr(kv.first) + ": " + JsonStr(kv.second);
    o += (++i < c.size()) ? ",\n" : "\n";
  }
  return o + ind + "}";
}

void WriteText(const std::string& path, const std::string& text) {
  std::ofstream f(path);
  KB_CHECK(f.is_open(), err::kCheckpointIO, "cannot open " + path);
  f << text << std::endl;
}

}  // namespace

bool RowFilter::Keep(uint64_t id) const {
  switch (mode) {
    case kAll: return true;
    case kModulo: return OwnerOf(table_salt, id, world) == rank;
    case kRing: return ring->Hit(Mix64(table_id, id)) == node;
  }
  return true;
}

std::string TimestampDirName() {
  std::time_t tt = std::time(nullptr);
  std::tm local{};
  localtime_r(&tt, &local);
  char buf[80];
  std::strftime(buf, sizeof(buf), "%Y-%m-%d-%H-%M-%S", &local);
  return buf;
}

bool ParseTimestampDir(const std::string& name, int64_t* key) {
  int v[6];
  char tail;
  if (std::sscanf(name.c_str(), "%d-%d-%d-%d-%d-%d%c", &v[0], &v[1], &v[2], &v[3], &v[4], &v[5], &tail) != 6)
    return false;
  if (v[1] < 1 || v[1] > 12 || v[2] < 1 || v[2] > 31 || v[3] > 23 || v[4] > 59 || v[5] > 60) return false;
  for (int x : v)
    if (x < 0) return false;
  *key = ((((static_cast<int64_t>(v[0]) * 13 + v[1]) * 32 + v[2]) * 24 + v[3]) * 60 + v[4]) * 61 + v[5];
  return true;
}

std::string PrepareSaveDir(const std::string& saved_dir, uint64_t shard, size_t max_save_count) {
  fs::path shard_dir = fs::path(saved_dir) / (kShardPrefix + std::to_string(shard));
  std::error_code ec;
  fs::create_directories(shard_dir, ec);
  KB_CHECK(!ec, err::kCheckpointIO, "cannot create " + shard_dir.string());

  std::vector<std::pair<int64_t, fs::path>> stamped;
  for (auto& e : fs::directory_iterator(shard_dir)) {
    int64_t key;
    if (e.is_directory() && ParseTimestampDir(e.path().filename().string(), &key)) stamped.push_back({key, e.path()});
  }
  std::sort(stamped.begin(), stamped.end());
  size_t first = 0;
  if (max_save_count > 0) {
    while (stamped.size() - first >= max_save_count) fs::remove_all(stamped[first++].second);
  }

  // Two saves inside one second would collide: wait for the next tick.
  std::string name = TimestampDirName();
  fs::path dir = shard_dir / name;
  for (int tries = 0; fs::exists(dir) && tries < 50; ++tries) {
    struct timespec ts{0, 100 * 1000 * 1000};
    nanosleep(&ts, nullptr);
    name = TimestampDirName();
    dir = shard_dir / name;
  }
  fs::create_directories(dir, ec);
  KB_CHECK(!ec, err::kCheckpointIO, "cannot create " + dir.string());
  return dir.string();
}

std::map<uint64_t, std::string> LatestShardDirs(const std::string& load_dir) {
  std::map<uint64_t, std::string> out;
  if (!fs::is_directory(load_dir)) return out;
  for (auto& e : fs::directory_iterator(load_dir)) {
    std::string fname = e.path().filename().string();
    if (!e.is_directory() || fname.rfind(kShardPrefix, 0) != 0) continue;
    uint64_t shard;
    try {
      size_t used = 0;
      shard = std::stoull(fname.substr(std::string(kShardPrefix).size()), &used);
      if (used != fname.size() - std::string(kShardPrefix).size()) continue;
    } catch (...) {
      continue;
    }
    int64_t best_key = -1;
    std::string best;
    for (auto& t : fs::directory_iterator(e.path())) {
      int64_t key;
      if (t.is_directory() && ParseTimestampDir(t.path().filename().string(), &key) && key > best_key) {
        best_key = key;
        best = t.path().string();
      }
    }
    if (best_key >= 0) out[shard] = best;
  }
  return out;
}

void SaveRouter(const std::string& dir, const Router& r) {
  std::ostringstream j;
  j << "[";
  for (size_t i = 0; i < r.nodes().size(); ++i) {
    const auto& n = r.nodes()[i];
    j << (i ? ",\n" : "\n") << "    {\n        \"id\": " << n.id << ",\n        \"name\": " << JsonStr(n.name)
      << ",\n        \"virtual_nodes\": [";
    for (size_t k = 0; k < n.vnodes.size(); ++k) {
      std::string vname;
      for (const auto& v : r.ring())
        if (v.hash_v == n.vnodes[k]) vname = v.name;
      j << (k ? ",\n" : "\n") << "            {\n                \"hash_v\": " << n.vnodes[k]
        << ",\n                \"name\": " << JsonStr(vname) << "\n            }";
    }
    j << "\n        ]\n    }";
  }
  j << "\n]";
  WriteText((fs::path(dir) / kRouterJson).string(), j.str());

  FileSink sink((fs::path(dir) / kRouterBin).string());
  KB_CHECK(sink.IsOpen(), err::kCheckpointIO, "cannot open router.binary in " + dir);
  Writer w(&sink);
  r.Save(&w);
}

Router LoadRouter(const std::string& dir) {
  FileSource src((fs::path(dir) / kRouterBin).string());
  KB_CHECK(src.IsOpen(), err::kCheckpointIO, "cannot open router.binary in " + dir);
  Reader r(&src);
  return Router::Load(&r);
}

void SaveModel(const std::string& dir, const ModelMeta& m) {
  std::ostringstream j;
  j << "{\n    \"name\": " << JsonStr(m.name) << ",\n    \"optim_type\": " << JsonStr(OptimName(m.optim_type))
    << ",\n    \"optim_conf\": " << JsonConf(m.optim_conf, "    ") << ",\n    \"tables\": [";
  size_t i = 0;
  for (auto& kv : m.tables) {
    const TableMeta& t = kv.second;
    j << (i++ ? ",\n" : "\n") << "        {\n            \"id\": " << t.id << ",\n            \"name\": "
      << JsonStr(t.name) << ",\n            \"table_type\": "
      << (t.table_type == TableType::kDense ? "\"Dense\"" : "\"Sparse\"") << ",\n            \"element_type\": "
      << JsonStr(DTypeName(t.element_type));
    if (t.table_type == TableType::kDense) {
      j << ",\n            \"shape\": [";
      for (size_t k = 0; k < t.shape.size(); ++k) j << (k ? ", " : "") << t.shape[k];
      j << "]";
    } else {
      j << ",\n            \"dimension\": " << t.dimension << ",\n            \"init_type\": "
        << JsonStr(InitName(t.init_type)) << ",\n            \"init_conf\": " << JsonConf(t.init_conf, "            ");
    }
    j << "\n        }";
  }
  j << "\n    ]\n}";
  WriteText((fs::path(dir) / kModelJson).string(), j.str());

  FileSink sink((fs::path(dir) / kModelBin).string());
  KB_CHECK(sink.IsOpen(), err::kCheckpointIO, "cannot open model.binary in " + dir);
  Writer w(&sink);
  w.Model(m);
}

ModelMeta LoadModel(const std::string& dir) {
  FileSource src((fs::path(dir) / kModelBin).string());
  KB_CHECK(src.IsOpen(), err::kCheckpointIO, "cannot open model.binary in " + dir);
  Reader r(&src);
  return r.Model();
}

void SaveDense(const std::string& dir, uint64_t id, const std::string& name, const Value& v) {
  FileSink sink((fs::path(dir) / (name + kDenseSuffix)).string());
  KB_CHECK(sink.IsOpen(), err::kCheckpointIO, "cannot open dense file for " + name);
  Writer w(&sink);
  w.Pod<uint8_t>(static_cast<uint8_t>(TableType::kDense));
  w.Pod<uint64_t>(id);
  w.Str(name);
  w.Val(v);
}

bool LoadDense(const std::string& dir, const std::string& name, uint64_t* id, Value* v) {
  fs::path p = fs::path(dir) / (name + kDenseSuffix);
  if (!fs::exists(p)) return false;
  FileSource src(p.string());
  KB_CHECK(src.IsOpen(), err::kCheckpointIO, "cannot open " + p.string());
  Reader r(&src);
  KB_CHECK(r.Pod<uint8_t>() == static_cast<uint8_t>(TableType::kDense), err::kTableTypeUnCompatible,
           p.string() + " is not a dense table file");
  *id = r.Pod<uint64_t>();
  std::string stored = r.Str();
  (void)stored;
  *v = r.Val();
  return true;
}

void SaveSparse(const std::string& dir, const SparseHeader& h, const SparseColumns& c) {
  const size_t n = c.ids.size();
  const int64_t d = h.dim;
  KB_CHECK(c.vals.size() == n * static_cast<size_t>(d), err::kBadArgument, "vals size does not match ids");
  for (auto& kv : c.states)
    KB_CHECK(kv.second.size() == n * static_cast<size_t>(d), err::kBadArgument, "state size does not match ids");
  for (auto& kv : c.states_i) KB_CHECK(kv.second.size() == n, err::kBadArgument, "state_i size does not match ids");

  std::vector<uint64_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::sort(order.begin(), order.end(), [&](uint64_t a, uint64_t b) {
    uint64_t sa = c.ids[a] % kSlotCount, sb = c.ids[b] % kSlotCount;
    return sa != sb ? sa < sb : c.ids[a] < c.ids[b];
  });
  uint64_t per_slot[kSlotCount] = {0};
  for (uint64_t id : c.ids) per_slot[id % kSlotCount]++;

  FileSink sink((fs::path(dir) / (h.name + kSparseSuffix)).string());
  KB_CHECK(sink.IsOpen(), err::kCheckpointIO, "cannot open sparse file for " + h.name);
  Writer w(&sink);
  w.Pod<uint8_t>(static_cast<uint8_t>(TableType::kSparse));
  w.Pod<uint64_t>(h.id);
  w.Str(h.name);
  w.Pod<int64_t>(h.dim);
  w.Pod<uint8_t>(static_cast<uint8_t>(h.dtype));
  w.Pod<uint8_t>(static_cast<uint8_t>(h.init_type));
  w.ConfMap(h.init_conf);
  w.Pod<uint64_t>(kSlotCount);

  size_t pos = 0;
  for (uint64_t s = 0; s < kSlotCount; ++s) {
    w.Pod<uint64_t>(per_slot[s]);
    for (uint64_t k = 0; k < per_slot[s]; ++k, ++pos) {
      const uint64_t r = order[pos];
      w.Pod<uint64_t>(c.ids[r]);
      w.RowF32(c.vals.data() + r * d, d);
      w.Pod<uint64_t>(c.states.size());
      for (auto& kv : c.states) {
        w.Pod<uint32_t>(kv.first);
        w.RowF32(kv.second.data() + r * d, d);
      }
      w.Pod<uint64_t>(c.states_i.size());
      for (auto& kv : c.states_i) {
        w.Pod<uint32_t>(kv.first);
        w.Pod<int64_t>(kv.second[r]);
      }
    }
  }
}

bool LoadSparse(const std::string& dir, const std::string& name, const RowFilter& filter, SparseHeader* h,
                SparseColumns* c) {
  fs::path p = fs::path(dir) / (name + kSparseSuffix);
  if (!fs::exists(p)) return false;
  FileSource src(p.string());
  KB_CHECK(src.IsOpen(), err::kCheckpointIO, "cannot open " + p.string());
  Reader r(&src);
  KB_CHECK(r.Pod<uint8_t>() == static_cast<uint8_t>(TableType::kSparse), err::kTableTypeUnCompatible,
           p.string() + " is not a sparse table file");
  h->id = r.Pod<uint64_t>();
  h->name = r.Str();
  h->dim = r.Pod<int64_t>();
  h->dtype = static_cast<DType>(r.Pod<uint8_t>());
  h->init_type = static_cast<InitializerType>(r.Pod<uint8_t>());
  h->init_conf = r.ConfMap();
  KB_CHECK(h->dtype == DType::kFloat32, err::kSparseTableUnCompatible, "only Float32 sparse tables are supported");
  KB_CHECK(h->dim > 0 && h->dim < (1 << 20), err::kSparseDimensionUnCompatible, "implausible dimension");
  if (c->dim == 0) c->dim = h->dim;
  KB_CHECK(c->dim == h->dim, err::kSparseDimensionUnCompatible, "dimension differs between shard files");
  const size_t d = static_cast<size_t>(h->dim);

  const uint64_t slots = r.Pod<uint64_t>();
  KB_CHECK(slots < (1u << 16), err::kDeserializeReply, "implausible slot count");
  for (uint64_t s = 0; s < slots; ++s) {
    const uint64_t n = r.Pod<uint64_t>();
    for (uint64_t k = 0; k < n; ++k) {
      const uint64_t id = r.Pod<uint64_t>();
      Value v = r.Val();
      if (!filter.Keep(id)) continue;
      KB_CHECK(static_cast<size_t>(v.val.Numel()) == d && v.val.dtype == DType::kFloat32,
               err::kSparseDimensionUnCompatible, "row shape differs from table dimension");
      const size_t row = c->ids.size();
      c->ids.push_back(id);
      c->vals.insert(c->vals.end(), v.val.f32(), v.val.f32() + d);
      // A state the row does not carry means "never updated": zeros / step 0.
      for (auto& kv : v.states) {
        auto& col = c->states[kv.first];
        col.resize(row * d, 0.f);
        if (static_cast<size_t>(kv.second.Numel()) == d && kv.second.dtype == DType::kFloat32)
          col.insert(col.end(), kv.second.f32(), kv.second.f32() + d);
      }
      for (auto& kv : c->states) kv.second.resize((row + 1) * d, 0.f);
      for (auto& kv : v.states_i) {
        auto& col = c->states_i[kv.first];
        col.resize(row, 0);
        col.push_back(kv.second);
      }
      for (auto& kv : c->states_i) kv.second.resize(row + 1, 0);
    }
  }
  return true;
}

// ------------------------------------------------------------------ streamed save / fast load
namespace {

constexpr size_t kTensorHead = 1 + 8 + 8 + 1;  // layout, ndims, dim, dtype

size_t RowBytes(int64_t d, size_t n_states, size_t n_int) {
  const size_t tensor = kTensorHead + static_cast<size_t>(d) * 4;
  return 8 + tensor + 8 + n_states * (4 + tensor) + 8 + n_int * 12;
}

inline char* PutTensorHead(char* p, int64_t d) {
  *p++ = 0;
  const uint64_t one = 1;
  std::memcpy(p, &one, 8);
  p += 8;
  std::memcpy(p, &d, 8);
  p += 8;
  *p++ = static_cast<char>(DType::kFloat32);
  return p;
}

void PwriteAll(int fd, const char* buf, size_t n, uint64_t off) {
  while (n > 0) {
    const ssize_t w = ::pwrite(fd, buf, n, static_cast<off_t>(off));
    KB_CHECK(w > 0, err::kCheckpointIO, "write to the checkpoint file failed");
    buf += w;
    n -= static_cast<size_t>(w);
    off += static_cast<uint64_t>(w);
  }
}

}  // namespace

SparseStreamWriter::SparseStreamWriter(const std::string& dir, const SparseHeader& h, std::vector<uint32_t> state_types,
                                       std::vector<uint32_t> int_state_types, int threads)
    : dim_(h.dim), st_(std::move(state_types)), sti_(std::move(int_state_types)),
      row_bytes_(RowBytes(h.dim, st_.size(), sti_.size())), threads_(threads < 1 ? 1 : threads) {
  path_ = (fs::path(dir) / (h.name + kSparseSuffix)).string();
  MemSink head;
  Writer w(&head);
  w.Pod<uint8_t>(static_cast<uint8_t>(TableType::kSparse));
  w.Pod<uint64_t>(h.id);
  w.Str(h.name);
  w.Pod<int64_t>(h.dim);
  w.Pod<uint8_t>(static_cast<uint8_t>(h.dtype));
  w.Pod<uint8_t>(static_cast<uint8_t>(h.init_type));
  w.ConfMap(h.init_conf);
  w.Pod<uint64_t>(kSlotCount);
  const char* mode = std::getenv("KRAKEN_CKPT_WRITE");  // "pwrite": buffered writes instead of the shared mapping
  map_mode_ = mode == nullptr || std::string(mode) != "pwrite";
  fd_ = ::open(path_.c_str(), O_CREAT | O_TRUNC | (map_mode_ ? O_RDWR : O_WRONLY), 0644);
  KB_CHECK(fd_ >= 0, err::kCheckpointIO, "cannot open sparse file for " + h.name);
  PwriteAll(fd_, reinterpret_cast<const char*>(head.data()), head.size(), 0);
  offset_ = head.size();
}

SparseStreamWriter::~SparseStreamWriter() {
  Unmap();
  if (fd_ >= 0) ::close(fd_);
}

void SparseStreamWriter::Unmap() {
  if (map_ != nullptr) ::munmap(map_, map_len_);
  map_ = nullptr;
  map_len_ = 0;
}

void SparseStreamWriter::BeginSlot(uint64_t rows) {
  KB_CHECK(slot_left_ == 0 && slots_begun_ < static_cast<int>(kSlotCount), err::kBadArgument,
           "a slot was begun before the previous one was complete");
  PwriteAll(fd_, reinterpret_cast<const char*>(&rows), 8, offset_);
  offset_ += 8;
  slot_left_ = rows;
  ++slots_begun_;
  if (map_mode_ && rows > 0) {
    // the slot's byte range is known now: extend the file and map the range, so that the formatting threads
    // store rows straight into the page cache, each faulting its own pages, instead of queueing on the one
    // lock that buffered writes into a single file take
    const uint64_t end = offset_ + rows * row_bytes_;
    const uint64_t page = static_cast<uint64_t>(::sysconf(_SC_PAGESIZE));
    if (::ftruncate(fd_, static_cast<off_t>(end)) == 0) {
      map_file_off_ = offset_ / page * page;
      map_len_ = static_cast<size_t>(end - map_file_off_);
      void* m = ::mmap(nullptr, map_len_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, static_cast<off_t>(map_file_off_));
      map_ = m == MAP_FAILED ? nullptr : static_cast<char*>(m);  // no mapping: this slot goes through pwrite
      if (map_ == nullptr) map_len_ = 0;
    }
  }
}

void SparseStreamWriter::Append(const uint64_t* ids, const float* vals, const float* const* states,
                                const int64_t* const* states_i, size_t n) {
  KB_CHECK(n <= slot_left_, err::kBadArgument, "more rows appended than the slot was begun with");
  if (n == 0) return;
  const size_t d = static_cast<size_t>(dim_);
  const size_t R = row_bytes_;
  const uint64_t base = offset_;
  const int T = static_cast<int>(std::min<size_t>(threads_, (n + 4095) / 4096));
  std::vector<std::thread> pool;
  std::atomic<bool> failed{false};
  auto format = [&](size_t a, size_t b, char* p) {  // rows [a, b) of this call, back to back at p
    for (size_t r = a; r < b; ++r) {
      std::memcpy(p, &ids[r], 8);
      p += 8;
      p = PutTensorHead(p, dim_);
      std::memcpy(p, vals + r * d, d * 4);
      p += d * 4;
      const uint64_t ns = st_.size();
      std::memcpy(p, &ns, 8);
      p += 8;
      for (size_t k = 0; k < st_.size(); ++k) {
        std::memcpy(p, &st_[k], 4);
        p += 4;
        p = PutTensorHead(p, dim_);
        std::memcpy(p, states[k] + r * d, d * 4);
        p += d * 4;
      }
      const uint64_t ni = sti_.size();
      std::memcpy(p, &ni, 8);
      p += 8;
      for (size_t k = 0; k < sti_.size(); ++k) {
        std::memcpy(p, &sti_[k], 4);
        p += 4;
        std::memcpy(p, &states_i[k][r], 8);
        p += 8;
      }
    }
  };
  auto work = [&](size_t lo, size_t hi) {
    try {
      if (map_ != nullptr) {
        format(lo, hi, map_ + (base - map_file_off_) + lo * R);
        return;
      }
      constexpr size_t kBatch = 8192;  // rows formatted per pwrite
      std::vector<char> buf(kBatch * R);
      for (size_t a = lo; a < hi; a += kBatch) {
        const size_t b = std::min(hi, a + kBatch);
        format(a, b, buf.data());
        PwriteAll(fd_, buf.data(), (b - a) * R, base + a * R);
      }
    } catch (...) {
      failed = true;
    }
  };
  const size_t per = (n + T - 1) / T;
  for (int t = 1; t < T; ++t) pool.emplace_back(work, std::min(n, t * per), std::min(n, (t + 1) * per));
  work(0, std::min(n, per));
  for (auto& th : pool) th.join();
  KB_CHECK(!failed, err::kCheckpointIO, "write to the checkpoint file failed");
  offset_ += n * R;
  slot_left_ -= n;
  if (slot_left_ == 0) Unmap();
}

void SparseStreamWriter::Close() {
  KB_CHECK(slot_left_ == 0 && slots_begun_ == static_cast<int>(kSlotCount), err::kBadArgument,
           "the sparse file is incomplete: not all slots were written");
  Unmap();
  if (fd_ >= 0) {
    KB_CHECK(::close(fd_) == 0, err::kCheckpointIO, "closing the checkpoint file failed");
    fd_ = -1;
  }
}

// ------------------------------------------------------------------ chunked reader
namespace {

bool PreadAll(int fd, char* buf, size_t n, uint64_t off) {
  while (n > 0) {
    const ssize_t got = ::pread(fd, buf, n, static_cast<off_t>(off));
    if (got < 0 && errno == EINTR) continue;
    if (got <= 0) return false;
    buf += got;
    off += static_cast<uint64_t>(got);
    n -= static_cast<size_t>(got);
  }
  return true;
}

}  // namespace

SparseChunkReader::SparseChunkReader(const std::string& dir, const std::string& name, int threads)
    : threads_(threads < 1 ? 1 : threads) {
  fs::path p = fs::path(dir) / (name + kSparseSuffix);
  if (!fs::exists(p)) return;
  exists_ = true;
  fd_ = ::open(p.string().c_str(), O_RDONLY);
  KB_CHECK(fd_ >= 0, err::kCheckpointIO, "cannot open " + p.string());
  const uint64_t size = static_cast<uint64_t>(fs::file_size(p));

  // header: a few hundred bytes at most (name + initializer conf); 1 MiB is read to be safe
  std::vector<char> head(static_cast<size_t>(std::min<uint64_t>(size, 1u << 20)));
  KB_CHECK(PreadAll(fd_, head.data(), head.size(), 0), err::kCheckpointIO, "cannot read " + p.string());
  MemSource src(head.data(), head.size());
  Reader r(&src);
  KB_CHECK(r.Pod<uint8_t>() == static_cast<uint8_t>(TableType::kSparse), err::kTableTypeUnCompatible,
           p.string() + " is not a sparse table file");
  h_.id = r.Pod<uint64_t>();
  h_.name = r.Str();
  h_.dim = r.Pod<int64_t>();
  h_.dtype = static_cast<DType>(r.Pod<uint8_t>());
  h_.init_type = static_cast<InitializerType>(r.Pod<uint8_t>());
  h_.init_conf = r.ConfMap();
  if (h_.dtype != DType::kFloat32 || h_.dim <= 0 || h_.dim >= (1 << 20)) return;
  if (r.Pod<uint64_t>() != kSlotCount) return;
  uint64_t pos = src.offset();

  row_start_.assign(1, 0);
  for (uint64_t s = 0; s < kSlotCount; ++s) {
    uint64_t n = 0;
    if (pos + 8 > size || !PreadAll(fd_, reinterpret_cast<char*>(&n), 8, pos)) return;
    pos += 8;
    if (n > 0 && row_bytes_ == 0) {
      // the first row of the file fixes the layout: which state entries, in which order
      // no row carries more than 8 float and 8 integer state entries (the StateType codes are 0..7)
      std::vector<char> one(static_cast<size_t>(std::min<uint64_t>(size - pos, RowBytes(h_.dim, 8, 8))));
      if (!PreadAll(fd_, one.data(), one.size(), pos)) return;
      MemSource first(one.data(), one.size());
      Reader rr(&first);
      try {
        rr.Pod<uint64_t>();
        Value v = rr.Val();
        const size_t d = static_cast<size_t>(h_.dim);
        if (static_cast<size_t>(v.val.Numel()) != d || v.val.dtype != DType::kFloat32) return;
        for (auto& kv : v.states) {
          if (static_cast<size_t>(kv.second.Numel()) != d || kv.second.dtype != DType::kFloat32) return;
          st_.push_back(kv.first);
        }
        for (auto& kv : v.states_i) sti_.push_back(kv.first);
      } catch (const KrakenError&) {
        return;
      }
      row_bytes_ = RowBytes(h_.dim, st_.size(), sti_.size());
      if (first.offset() != row_bytes_) return;  // entries not in ascending type order, or another encoding
    }
    if (n > 0 && n > (size - pos) / row_bytes_) return;
    segs_.emplace_back(pos, n);
    pos += n * row_bytes_;
    total_ += n;
    row_start_.push_back(total_);
  }
  if (pos != size) return;

  tmpl_.assign(row_bytes_, 0);
  if (row_bytes_) {
    const size_t d = static_cast<size_t>(h_.dim);
    char* q = tmpl_.data() + 8;
    q = PutTensorHead(q, h_.dim) + d * 4;
    const uint64_t ns = st_.size();
    std::memcpy(q, &ns, 8);
    q += 8;
    for (uint32_t k : st_) {
      std::memcpy(q, &k, 4);
      q = PutTensorHead(q + 4, h_.dim) + d * 4;
    }
    const uint64_t ni = sti_.size();
    std::memcpy(q, &ni, 8);
    q += 8;
    for (uint32_t k : sti_) {
      std::memcpy(q, &k, 4);
      q += 12;
    }
  }
  bufs_.resize(static_cast<size_t>(threads_));
  fast_ = true;
}

SparseChunkReader::~SparseChunkReader() {
  if (fd_ >= 0) ::close(fd_);
}

bool SparseChunkReader::Read(uint64_t lo, uint64_t n, uint64_t* ids, float* vals, float* const* states,
                             int64_t* const* states_i) {
  KB_CHECK(fast_, err::kBadArgument, "the file does not have the fixed layout");
  KB_CHECK(lo + n <= total_, err::kBadArgument, "row range beyond the end of the file");
  if (n == 0) return true;
  const size_t d = static_cast<size_t>(h_.dim);
  const size_t R = row_bytes_;
  constexpr uint64_t kBatch = 8192;  // rows per pread
  std::atomic<bool> ok{true};
  auto work = [&](int tid, uint64_t a, uint64_t b) {  // global rows [a, b), written at index (row - lo)
    std::vector<char>& buf = bufs_[static_cast<size_t>(tid)];
    if (buf.size() < kBatch * R) buf.resize(kBatch * R);
    size_t seg = 0;
    const char* t = tmpl_.data();
    while (a < b && ok) {
      while (a >= row_start_[seg + 1]) ++seg;
      const uint64_t take = std::min<uint64_t>({kBatch, b - a, row_start_[seg + 1] - a});
      if (!PreadAll(fd_, buf.data(), take * R, segs_[seg].first + (a - row_start_[seg]) * R)) {
        ok = false;
        return;
      }
      for (uint64_t k = 0; k < take; ++k) {
        const char* q = buf.data() + k * R;
        const size_t out = static_cast<size_t>(a + k - lo);
        std::memcpy(&ids[out], q, 8);
        size_t o = 8;
        if (std::memcmp(q + o, t + o, kTensorHead) != 0) { ok = false; return; }
        o += kTensorHead;
        std::memcpy(vals + out * d, q + o, d * 4);
        o += d * 4;
        if (std::memcmp(q + o, t + o, 8) != 0) { ok = false; return; }
        o += 8;
        for (size_t c = 0; c < st_.size(); ++c) {
          if (std::memcmp(q + o, t + o, 4 + kTensorHead) != 0) { ok = false; return; }
          o += 4 + kTensorHead;
          std::memcpy(states[c] + out * d, q + o, d * 4);
          o += d * 4;
        }
        if (std::memcmp(q + o, t + o, 8) != 0) { ok = false; return; }
        o += 8;
        for (size_t c = 0; c < sti_.size(); ++c) {
          if (std::memcmp(q + o, t + o, 4) != 0) { ok = false; return; }
          std::memcpy(&states_i[c][out], q + o + 4, 8);
          o += 12;
        }
      }
      a += take;
    }
  };
  const int T = static_cast<int>(std::max<uint64_t>(1, std::min<uint64_t>(threads_, (n + kBatch - 1) / kBatch)));
  const uint64_t per = (n + T - 1) / T;
  std::vector<std::thread> pool;
  for (int t = 1; t < T; ++t)
    pool.emplace_back(work, t, lo + std::min<uint64_t>(n, t * per), lo + std::min<uint64_t>(n, (t + 1) * per));
  work(0, lo, lo + std::min<uint64_t>(n, per));
  for (auto& th : pool) th.join();
  return ok;
}

}  // namespace ckpt
}  // namespace kb
