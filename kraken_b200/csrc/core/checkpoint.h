// Checkpoint files in the reference's layout, readable and writable by both.
//
//   <saved_dir>/shard_<node_id>/<YYYY-MM-DD-HH-MM-SS>/
//       router.json  router.binary  model.json  model.binary
//       <table>.dense    u8 0, u64 id, string name, Value
//       <table>.sparse   u8 1, u64 id, string name, i64 dim, u8 dtype, u8 init_type, conf,
//                        u64 slot_count(=8), per slot: u64 n, n x {u64 id, Value}
//                        (slot = id % 8, ids ascending inside a slot)
//
// Format source: kraken/checkpoint/checkpoint.cc:17-23,55-63,288-510 and
// kraken/checkpoint/checkpoint_exec.cc:246-377 (save, retention) / :379-521 (load).
// Differences on purpose: maps are written in ascending key order, unused
// metadata fields are zero instead of uninitialised, and every row carries its
// optimizer-state entries.  The reader accepts the reference's variants (any
// map order, rows without state entries, garbage in unused fields).
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "router.h"
#include "serialize.h"

namespace kb {
namespace ckpt {

constexpr uint64_t kSlotCount = 8;

// Columnar image of one shard's part of a sparse table (what device export
// produces and device import consumes).
struct SparseColumns {
  int64_t dim = 0;
  std::vector<uint64_t> ids;                       // [n]
  std::vector<float> vals;                         // [n, dim]
  std::map<uint32_t, std::vector<float>> states;   // StateType -> [n, dim]
  std::map<uint32_t, std::vector<int64_t>> states_i;  // StateType -> [n]
};

struct SparseHeader {
  uint64_t id = 0;
  std::string name;
  int64_t dim = 0;
  DType dtype = DType::kFloat32;
  InitializerType init_type = InitializerType::kConstant;
  Conf init_conf;
};

// Row filter applied while loading a sparse file.
struct RowFilter {
  enum Mode { kAll = 0, kModulo = 1, kRing = 2 } mode = kAll;
  uint64_t table_salt = 0;  // kModulo: OwnerOf(table_salt, id, world) == rank
  uint32_t world = 1;
  uint32_t rank = 0;
  const Router* ring = nullptr;  // kRing: ring->Hit(Mix64(table_id) ^ Mix64(id)) == node
  uint64_t table_id = 0;
  uint64_t node = 0;
  bool Keep(uint64_t id) const;
};

std::string TimestampDirName();                       // local time, %Y-%m-%d-%H-%M-%S
bool ParseTimestampDir(const std::string& name, int64_t* key);  // sortable key, false if not a timestamp

// Creates <saved_dir>/shard_<shard>/<timestamp>/ after deleting the oldest
// timestamp dirs while their count >= max_save_count; returns the new dir.
std::string PrepareSaveDir(const std::string& saved_dir, uint64_t shard, size_t max_save_count);
// shard id -> newest timestamp dir below load_dir/shard_<id>/.
std::map<uint64_t, std::string> LatestShardDirs(const std::string& load_dir);

void SaveRouter(const std::string& dir, const Router& r);  // router.json + router.binary
Router LoadRouter(const std::string& dir);
void SaveModel(const std::string& dir, const ModelMeta& m);  // model.json + model.binary
ModelMeta LoadModel(const std::string& dir);

void SaveDense(const std::string& dir, uint64_t id, const std::string& name, const Value& v);
// Returns false if the file does not exist.
bool LoadDense(const std::string& dir, const std::string& name, uint64_t* id, Value* v);

// Rows may be passed in any order; they are written slot by slot, ascending.
// `order` (optional) receives the permutation used, for callers that cache it.
void SaveSparse(const std::string& dir, const SparseHeader& h, const SparseColumns& cols);
// Appends the kept rows of <dir>/<name>.sparse to *cols; false if the file does not exist.
bool LoadSparse(const std::string& dir, const std::string& name, const RowFilter& filter, SparseHeader* h,
                SparseColumns* cols);

// ---- large tables: streamed, multi-threaded save and load of the same file format ----
//
// Every row of a table written by this framework has the same byte length (same dimension, same
// state entries in ascending type order), so a row's file offset follows from its index.  The
// stream writer formats rows that arrive in chunks, already in file order (slot by slot, ids
// ascending as unsigned numbers inside a slot), with several threads that each store their part into a
// shared mapping of the slot's byte range (buffered writes into one file queue on the file's lock);
// no sort and no whole-table copy happens on the host.  The chunked reader below checks that every row
// matches the fixed layout of the file's first row while it extracts the columns with several threads;
// a file that does not match (written by the reference with per-row state sets, say) is left to LoadSparse.
class SparseStreamWriter {
 public:
  // state_types / int_state_types: StateType codes in ascending order, one column each in Append.
  SparseStreamWriter(const std::string& dir, const SparseHeader& h, std::vector<uint32_t> state_types,
                     std::vector<uint32_t> int_state_types, int threads = 8);
  ~SparseStreamWriter();
  void BeginSlot(uint64_t rows);  // slots 0..7 in order; `rows` rows follow through Append
  void Append(const uint64_t* ids, const float* vals, const float* const* states, const int64_t* const* states_i,
              size_t n);
  void Close();  // all 8 slots must be complete
  uint64_t bytes_written() const { return offset_; }
  size_t row_bytes() const { return row_bytes_; }

 private:
  int fd_ = -1;
  int64_t dim_;
  std::vector<uint32_t> st_, sti_;
  size_t row_bytes_;
  uint64_t offset_ = 0, slot_left_ = 0;
  int slots_begun_ = 0, threads_;
  std::string path_;
  // rows are stored through a shared mapping of the slot's byte range (KRAKEN_CKPT_WRITE=pwrite: buffered writes)
  bool map_mode_ = false;
  char* map_ = nullptr;
  size_t map_len_ = 0;
  uint64_t map_file_off_ = 0;
  void Unmap();
};

// Chunked reader of a fixed-layout sparse file, for tables larger than the host wants to hold twice: the file
// is opened once (header, the 8 slot counts and the first row's layout are read with pread), then Read()
// extracts any row range [lo, lo + n) of the file order straight into caller-owned column arrays - pinned
// staging buffers that are reused for every chunk, so that neither the file (no mapping) nor the destination
// pays a page fault per 4 KiB in steady state.  Each thread preads its rows in batches into a buffer it keeps.
class SparseChunkReader {
 public:
  SparseChunkReader(const std::string& dir, const std::string& name, int threads = 8);
  ~SparseChunkReader();
  SparseChunkReader(const SparseChunkReader&) = delete;
  SparseChunkReader& operator=(const SparseChunkReader&) = delete;
  bool exists() const { return exists_; }
  bool fast() const { return fast_; }  // false: not the fixed layout (or not float32): use LoadSparse
  const SparseHeader& header() const { return h_; }
  uint64_t rows() const { return total_; }
  const std::vector<uint32_t>& state_types() const { return st_; }
  const std::vector<uint32_t>& int_state_types() const { return sti_; }
  // False when a row deviates from the first row's layout (nothing can be trusted then: use LoadSparse).
  bool Read(uint64_t lo, uint64_t n, uint64_t* ids, float* vals, float* const* states, int64_t* const* states_i);

 private:
  int fd_ = -1;
  bool exists_ = false, fast_ = false;
  SparseHeader h_;
  uint64_t total_ = 0;
  size_t row_bytes_ = 0;
  int threads_;
  std::vector<uint32_t> st_, sti_;
  std::vector<std::pair<uint64_t, uint64_t>> segs_;  // (file offset of the first row, rows) per slot
  std::vector<uint64_t> row_start_;                  // first global row of each slot, plus the total
  std::vector<char> tmpl_;                           // a row with every fixed byte in place
  std::vector<std::vector<char>> bufs_;              // one batch buffer per thread
};

}  // namespace ckpt
}  // namespace kb
