// CPU parameter shard: the executable specification of the server semantics
// and the storage engine of the CPU (gloo / socket) backend.
//
// Semantics reproduced from the reference's server side:
//   * pulling an unseen sparse id creates the row with the table's initializer
//     (kraken/ps/sparse_table.cc:33-75);
//   * pushing to an unseen id is kSparseIdNotExist and aborts the rest of the
//     request (kraken/ps/sparse_table.cc:77-108);
//   * a dense table is one Value updated as a whole, a COO gradient is
//     scattered (added) into zeros first and an empty COO is a no-op
//     (kraken/ps/dense_table.cc:31-43, kraken/ps/optim/sgd.cc:26-39);
//   * optimizer state lives beside each row / table and is created on first use.
// Storage is columnar (row index -> slabs), the same shape the GPU shard
// exports, so checkpoints and resharding share one code path.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../core/checkpoint.h"
#include "../core/optim_math.h"
#include "../core/serialize.h"

namespace kb {

OptimPOD ParseOptim(OptimType type, const Conf& conf);
InitPOD ParseInit(InitializerType type, const Conf& conf);
// StateType of slab i (0..2) for an optimizer, see optim_math.h.
uint32_t SlabStateType(const OptimPOD& o, int slab);

class CpuShard {
 public:
  explicit CpuShard(uint64_t seed = 0) : seed_(seed) {}

  // Idempotent; a second call with another optimizer is kModelAlreadyInitialized.
  void InitModel(const std::string& name, OptimType type, const Conf& conf);
  bool model_initialized() const { return model_init_; }
  const ModelMeta& meta() const { return meta_; }

  void CreateDenseTable(uint64_t id, const std::string& name, const std::vector<int64_t>& shape, const float* val);
  void CreateSparseTable(uint64_t id, const std::string& name, int64_t dim, InitializerType init_type,
                         const Conf& init_conf);
  bool HasTable(uint64_t id) const;

  int64_t DenseNumel(uint64_t id) const;
  void PullDense(uint64_t id, float* out) const;
  void PushDense(uint64_t id, const float* grad, int64_t n, float lr);
  void PushDenseCoo(uint64_t id, const int64_t* idx, const float* vals, int64_t nnz, float lr);

  int64_t SparseDim(uint64_t id) const;
  int64_t SparseSize(uint64_t id) const;
  void PullSparse(uint64_t id, const uint64_t* ids, int64_t n, float* out);
  // ids must be unique inside one call (the client sums duplicates first).
  int32_t PushSparse(uint64_t id, const uint64_t* ids, int64_t n, const float* grads, float lr);

  // Checkpoint / resharding.
  Value ExportDense(uint64_t id) const;
  void ImportDense(uint64_t id, const std::string& name, const Value& v);
  ckpt::SparseColumns ExportSparse(uint64_t id) const;
  // overwrite = false keeps the rows the table already holds (a row that arrived earlier is newer).
  void ImportSparse(uint64_t id, const ckpt::SparseColumns& cols, bool overwrite = true);
  // out[i] = 1 if the table holds ids[i].
  void ContainsSparse(uint64_t id, const uint64_t* ids, int64_t n, uint8_t* out) const;
  // Value, optimizer state and step count of those of the given ids that the table holds (others are skipped).
  ckpt::SparseColumns ExportSparseRows(uint64_t id, const uint64_t* ids, int64_t n) const;
  // Drops the rows for which keep(id) is false; returns how many were dropped.
  int64_t FilterSparse(uint64_t id, const ckpt::RowFilter& keep);

 private:
  struct Dense {
    std::string name;
    std::vector<int64_t> shape;
    std::vector<float> val, s[3];
    int64_t steps = 0;
    bool touched = false;
    mutable std::mutex mu;
  };
  struct Sparse {
    std::string name;
    int64_t dim = 0;
    InitPOD init;
    uint64_t seed_key = 0;
    std::unordered_map<uint64_t, int64_t> index;
    std::vector<uint64_t> ids;
    std::vector<float> val, s[3];
    std::vector<int64_t> steps;
    mutable std::mutex mu;
    int64_t AddRow(uint64_t id, const OptimPOD& o);
  };

  Dense& dense(uint64_t id);
  const Dense& dense(uint64_t id) const;
  Sparse& sparse(uint64_t id);
  const Sparse& sparse(uint64_t id) const;
  void UpdateDense(Dense& t, const float* g, float lr);

  uint64_t seed_;
  bool model_init_ = false;
  ModelMeta meta_;
  OptimPOD optim_;
  mutable std::mutex mu_;
  std::map<uint64_t, std::unique_ptr<Dense>> dense_;
  std::map<uint64_t, std::unique_ptr<Sparse>> sparse_;
};

}  // namespace kb
