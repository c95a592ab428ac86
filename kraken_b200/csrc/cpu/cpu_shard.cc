#include "cpu_shard.h"

#include <algorithm>
#include <cstring>

namespace kb {

namespace {

bool GetFloat(const Conf& c, const char* key, float* v) {
  auto it = c.find(key);
  if (it == c.end()) return false;
  try {
    *v = std::stof(it->second);
  } catch (...) {
    return false;
  }
  return true;
}

bool GetBool(const Conf& c, const char* key, bool* v) {
  auto it = c.find(key);
  if (it == c.end()) return false;
  std::string s = it->second;
  std::transform(s.begin(), s.end(), s.begin(), ::tolower);
  *v = (s == "true" || s == "1");
  return true;
}

}  // namespace

// Keys and defaults as parsed by the reference's factory (kraken/ps/optim/optim.cc:18-105).
OptimPOD ParseOptim(OptimType type, const Conf& conf) {
  OptimPOD o;
  o.type = static_cast<uint8_t>(type);
  o.has_weight_decay = GetFloat(conf, "weight_decay", &o.weight_decay);
  switch (type) {
    case OptimType::kAdagrad:
      o.eps = 1e-10f;
      GetFloat(conf, "eps", &o.eps);
      GetFloat(conf, "initial_accumulator_value", &o.initial_accumulator_value);
      break;
    case OptimType::kAdam:
      o.eps = 1e-8f;
      GetFloat(conf, "beta1", &o.beta1);
      GetFloat(conf, "beta2", &o.beta2);
      GetFloat(conf, "eps", &o.eps);
      GetBool(conf, "amsgrad", &o.amsgrad);
      break;
    case OptimType::kRMSprop:
      o.eps = 1e-8f;
      o.has_momentum = GetFloat(conf, "momentum", &o.momentum);
      GetFloat(conf, "alpha", &o.alpha);
      GetFloat(conf, "eps", &o.eps);
      GetBool(conf, "centered", &o.centered);
      break;
    case OptimType::kSGD:
      o.has_momentum = GetFloat(conf, "momentum", &o.momentum);
      o.has_dampening = GetFloat(conf, "dampening", &o.dampening);
      GetBool(conf, "nesterov", &o.nesterov);
      break;
  }
  return o;
}

// Keys and defaults of kraken/ps/initializer/initializer.cc:22-61.
InitPOD ParseInit(InitializerType type, const Conf& conf) {
  InitPOD p;
  p.type = static_cast<uint8_t>(type);
  switch (type) {
    case InitializerType::kConstant:
      p.a = 0.f;
      GetFloat(conf, "value", &p.a);
      break;
    case InitializerType::kUniform:
      p.a = 0.f;
      p.b = 1.f;
      GetFloat(conf, "lower", &p.a);
      GetFloat(conf, "upper", &p.b);
      break;
    case InitializerType::kNormal:
      p.a = 0.f;
      p.b = 1.f;
      GetFloat(conf, "mean", &p.a);
      GetFloat(conf, "stddev", &p.b);
      break;
    case InitializerType::kXavierUniform:
    case InitializerType::kXavierNormal:
      p.a = 1.f;
      GetFloat(conf, "gain", &p.a);
      break;
  }
  return p;
}

uint32_t SlabStateType(const OptimPOD& o, int slab) {
  static const uint32_t kMap[4][3] = {
      {2, 0, 0},  // Adagrad: StateSum
      {3, 4, 5},  // Adam: FirstMoment, SecondMoment, SecondMomentMax
      {6, 7, 1},  // RMSprop: SquareAverage, GAve, MomentumBuffer
      {1, 0, 0},  // SGD: MomentumBuffer
  };
  return kMap[o.type][slab];
}

void CpuShard::InitModel(const std::string& name, OptimType type, const Conf& conf) {
  std::lock_guard<std::mutex> g(mu_);
  if (model_init_) {
    KB_CHECK(meta_.optim_type == type, err::kModelAlreadyInitialized, "model already initialized with another optimizer");
    return;
  }
  meta_.name = name;
  meta_.optim_type = type;
  meta_.optim_conf = conf;
  optim_ = ParseOptim(type, conf);
  model_init_ = true;
}

CpuShard::Dense& CpuShard::dense(uint64_t id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = dense_.find(id);
  KB_CHECK(it != dense_.end(), sparse_.count(id) ? err::kTableTypeUnCompatible : err::kTableNotExist,
           "dense table " + std::to_string(id));
  return *it->second;
}
const CpuShard::Dense& CpuShard::dense(uint64_t id) const { return const_cast<CpuShard*>(this)->dense(id); }

CpuShard::Sparse& CpuShard::sparse(uint64_t id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = sparse_.find(id);
  KB_CHECK(it != sparse_.end(), dense_.count(id) ? err::kTableTypeUnCompatible : err::kTableNotExist,
           "sparse table " + std::to_string(id));
  return *it->second;
}
const CpuShard::Sparse& CpuShard::sparse(uint64_t id) const { return const_cast<CpuShard*>(this)->sparse(id); }

bool CpuShard::HasTable(uint64_t id) const {
  std::lock_guard<std::mutex> g(mu_);
  return dense_.count(id) || sparse_.count(id);
}

void CpuShard::CreateDenseTable(uint64_t id, const std::string& name, const std::vector<int64_t>& shape,
                                const float* val) {
  KB_CHECK(model_init_, err::kModelNotInitialized, "create dense table before init_model");
  std::lock_guard<std::mutex> g(mu_);
  KB_CHECK(!sparse_.count(id), err::kTableTypeUnCompatible, "id already names a sparse table");
  if (dense_.count(id)) return;  // idempotent (kraken/ps/ps.cc:644-649)
  auto t = std::make_unique<Dense>();
  t->name = name;
  t->shape = shape;
  int64_t n = 1;
  for (auto d : shape) n *= d;
  t->val.assign(val, val + n);
  dense_[id] = std::move(t);
  TableMeta m;
  m.id = id;
  m.name = name;
  m.table_type = TableType::kDense;
  m.shape = shape;
  meta_.tables[id] = m;
}

void CpuShard::CreateSparseTable(uint64_t id, const std::string& name, int64_t dim, InitializerType init_type,
                                 const Conf& init_conf) {
  KB_CHECK(model_init_, err::kModelNotInitialized, "create sparse table before init_model");
  KB_CHECK(dim > 0, err::kSparseDimensionUnCompatible, "dimension must be positive");
  std::lock_guard<std::mutex> g(mu_);
  KB_CHECK(!dense_.count(id), err::kTableTypeUnCompatible, "id already names a dense table");
  if (sparse_.count(id)) {
    KB_CHECK(sparse_[id]->dim == dim, err::kSparseDimensionUnCompatible, "sparse table exists with another dimension");
    return;
  }
  auto t = std::make_unique<Sparse>();
  t->name = name;
  t->dim = dim;
  t->init = ParseInit(init_type, init_conf);
  t->seed_key = SeedKey(seed_, id);
  sparse_[id] = std::move(t);
  TableMeta m;
  m.id = id;
  m.name = name;
  m.table_type = TableType::kSparse;
  m.dimension = dim;
  m.init_type = init_type;
  m.init_conf = init_conf;
  meta_.tables[id] = m;
}

int64_t CpuShard::DenseNumel(uint64_t id) const { return static_cast<int64_t>(dense(id).val.size()); }

void CpuShard::PullDense(uint64_t id, float* out) const {
  const Dense& t = dense(id);
  std::lock_guard<std::mutex> g(t.mu);
  std::memcpy(out, t.val.data(), t.val.size() * sizeof(float));
}

namespace {

// One optimizer update over a contiguous span.  The optimizer type is a template constant, so the
// per-element switch folds away and the loop vectorises; slabs the optimizer does not use point at
// a scratch block (in pieces of kSpanBlock elements) instead of being tested per element.
constexpr int64_t kSpanBlock = 256;

template <int TYPE>
void UpdateSpanT(OptimPOD o, float lr, const float* g, int64_t n, int64_t step, float* w, float* s0, float* s1,
                 float* s2) {
  o.type = TYPE;
  const AdamBias ab = TYPE == 1 ? AdamBiasAt(o, step) : AdamBias{1.f, 1.f};
  float scratch[3][kSpanBlock];
  for (int64_t base = 0; base < n; base += kSpanBlock) {
    const int64_t m = n - base < kSpanBlock ? n - base : kSpanBlock;
    float* a0 = s0 ? s0 + base : scratch[0];
    float* a1 = s1 ? s1 + base : scratch[1];
    float* a2 = s2 ? s2 + base : scratch[2];
    if (!s0) for (int64_t j = 0; j < m; ++j) a0[j] = 0.f;
    if (!s1) for (int64_t j = 0; j < m; ++j) a1[j] = 0.f;
    if (!s2) for (int64_t j = 0; j < m; ++j) a2[j] = 0.f;
    const float* gg = g + base;
    float* ww = w + base;
    for (int64_t j = 0; j < m; ++j) UpdateElem(o, lr, gg[j], step, ab, ww[j], a0[j], a1[j], a2[j]);
  }
}

void UpdateSpan(const OptimPOD& o, float lr, const float* g, int64_t n, int64_t step, float* w, float* s0, float* s1,
                float* s2) {
  switch (o.type) {
    case 0: UpdateSpanT<0>(o, lr, g, n, step, w, s0, s1, s2); break;
    case 1: UpdateSpanT<1>(o, lr, g, n, step, w, s0, s1, s2); break;
    case 2: UpdateSpanT<2>(o, lr, g, n, step, w, s0, s1, s2); break;
    default: UpdateSpanT<3>(o, lr, g, n, step, w, s0, s1, s2); break;
  }
}

}  // namespace

void CpuShard::UpdateDense(Dense& t, const float* g, float lr) {
  const size_t n = t.val.size();
  for (int k = 0; k < 3; ++k)
    if (optim_.SlabUsed(k) && t.s[k].size() != n)
      t.s[k].assign(n, (optim_.type == 0 && k == 0) ? optim_.initial_accumulator_value : 0.f);
  const int64_t step = ++t.steps;
  t.touched = true;
  float* s0 = t.s[0].empty() ? nullptr : t.s[0].data();
  float* s1 = t.s[1].empty() ? nullptr : t.s[1].data();
  float* s2 = t.s[2].empty() ? nullptr : t.s[2].data();
  UpdateSpan(optim_, lr, g, static_cast<int64_t>(n), step, t.val.data(), s0, s1, s2);
}

void CpuShard::PushDense(uint64_t id, const float* grad, int64_t n, float lr) {
  Dense& t = dense(id);
  std::lock_guard<std::mutex> g(t.mu);
  KB_CHECK(static_cast<size_t>(n) == t.val.size(), err::kGradientUnCompatible, "dense gradient size mismatch");
  UpdateDense(t, grad, lr);
}

void CpuShard::PushDenseCoo(uint64_t id, const int64_t* idx, const float* vals, int64_t nnz, float lr) {
  if (nnz == 0) return;
  Dense& t = dense(id);
  std::lock_guard<std::mutex> g(t.mu);
  std::vector<float> full(t.val.size(), 0.f);
  for (int64_t i = 0; i < nnz; ++i) {
    KB_CHECK(idx[i] >= 0 && static_cast<size_t>(idx[i]) < full.size(), err::kGradientUnCompatible,
             "COO index out of range");
    full[idx[i]] += vals[i];
  }
  UpdateDense(t, full.data(), lr);
}

int64_t CpuShard::SparseDim(uint64_t id) const { return sparse(id).dim; }

int64_t CpuShard::SparseSize(uint64_t id) const {
  const Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  return static_cast<int64_t>(t.ids.size());
}

int64_t CpuShard::Sparse::AddRow(uint64_t id, const OptimPOD& o) {
  const int64_t row = static_cast<int64_t>(ids.size());
  ids.push_back(id);
  index.emplace(id, row);
  val.resize((row + 1) * dim);
  InitRow(init, seed_key, id, static_cast<uint32_t>(dim), val.data() + row * dim);
  for (int k = 0; k < 3; ++k)
    if (o.SlabUsed(k)) s[k].resize((row + 1) * dim, (o.type == 0 && k == 0) ? o.initial_accumulator_value : 0.f);
  steps.push_back(0);
  return row;
}

void CpuShard::PullSparse(uint64_t id, const uint64_t* ids, int64_t n, float* out) {
  Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  for (int64_t i = 0; i < n; ++i) {
    auto it = t.index.find(ids[i]);
    const int64_t row = it != t.index.end() ? it->second : t.AddRow(ids[i], optim_);
    std::memcpy(out + i * t.dim, t.val.data() + row * t.dim, t.dim * sizeof(float));
  }
}

int32_t CpuShard::PushSparse(uint64_t id, const uint64_t* ids, int64_t n, const float* grads, float lr) {
  Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  for (int64_t i = 0; i < n; ++i) {
    auto it = t.index.find(ids[i]);
    if (it == t.index.end()) return err::kSparseIdNotExist;
    const int64_t row = it->second;
    const int64_t step = ++t.steps[row];
    const int64_t e = row * t.dim;
    UpdateSpan(optim_, lr, grads + i * t.dim, t.dim, step, t.val.data() + e, t.s[0].empty() ? nullptr : t.s[0].data() + e,
               t.s[1].empty() ? nullptr : t.s[1].data() + e, t.s[2].empty() ? nullptr : t.s[2].data() + e);
  }
  return err::kSuccess;
}

Value CpuShard::ExportDense(uint64_t id) const {
  const Dense& t = dense(id);
  std::lock_guard<std::mutex> g(t.mu);
  Value v;
  v.val = HostTensor::F32(t.shape);
  std::memcpy(v.val.data.data(), t.val.data(), t.val.size() * 4);
  if (t.touched) {
    for (int k = 0; k < 3; ++k) {
      if (t.s[k].empty()) continue;
      HostTensor s = HostTensor::F32(t.shape);
      std::memcpy(s.data.data(), t.s[k].data(), t.s[k].size() * 4);
      v.states[SlabStateType(optim_, k)] = std::move(s);
    }
    if (optim_.NeedsSteps()) v.states_i[static_cast<uint32_t>(StateType::kSteps)] = t.steps;
  }
  return v;
}

void CpuShard::ImportDense(uint64_t id, const std::string& name, const Value& v) {
  KB_CHECK(model_init_, err::kModelNotInitialized, "import before init_model");
  KB_CHECK(v.val.dtype == DType::kFloat32, err::kDenseTableUnCompatible, "only Float32 dense tables are supported");
  CreateDenseTable(id, name, v.val.dims, v.val.f32());
  Dense& t = dense(id);
  std::lock_guard<std::mutex> g(t.mu);
  std::memcpy(t.val.data(), v.val.f32(), t.val.size() * 4);
  for (int k = 0; k < 3; ++k) {
    auto it = v.states.find(SlabStateType(optim_, k));
    if (!optim_.SlabUsed(k) || it == v.states.end()) continue;
    KB_CHECK(static_cast<size_t>(it->second.Numel()) == t.val.size(), err::kDenseTableUnCompatible,
             "state size differs from value size");
    t.s[k].assign(it->second.f32(), it->second.f32() + t.val.size());
    t.touched = true;
  }
  auto si = v.states_i.find(static_cast<uint32_t>(StateType::kSteps));
  if (si != v.states_i.end()) {
    t.steps = si->second;
    t.touched = true;
  }
}

ckpt::SparseColumns CpuShard::ExportSparse(uint64_t id) const {
  const Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  ckpt::SparseColumns c;
  c.dim = t.dim;
  c.ids = t.ids;
  c.vals = t.val;
  for (int k = 0; k < 3; ++k)
    if (!t.s[k].empty() || (optim_.SlabUsed(k) && t.ids.empty())) c.states[SlabStateType(optim_, k)] = t.s[k];
  if (optim_.NeedsSteps()) c.states_i[static_cast<uint32_t>(StateType::kSteps)] = t.steps;
  return c;
}

void CpuShard::ContainsSparse(uint64_t id, const uint64_t* ids, int64_t n, uint8_t* out) const {
  const Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  for (int64_t i = 0; i < n; ++i) out[i] = t.index.find(ids[i]) != t.index.end() ? 1 : 0;
}

ckpt::SparseColumns CpuShard::ExportSparseRows(uint64_t id, const uint64_t* ids, int64_t n) const {
  const Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  ckpt::SparseColumns c;
  c.dim = t.dim;
  std::vector<int64_t> rows;
  for (int64_t i = 0; i < n; ++i) {
    auto it = t.index.find(ids[i]);
    if (it == t.index.end()) continue;
    c.ids.push_back(ids[i]);
    rows.push_back(it->second);
  }
  c.vals.resize(rows.size() * t.dim);
  for (size_t r = 0; r < rows.size(); ++r) std::memcpy(c.vals.data() + r * t.dim, t.val.data() + rows[r] * t.dim, t.dim * 4);
  for (int k = 0; k < 3; ++k) {
    if (t.s[k].empty() && !(optim_.SlabUsed(k) && rows.empty())) continue;
    std::vector<float>& dst = c.states[SlabStateType(optim_, k)];
    dst.resize(rows.size() * t.dim);
    for (size_t r = 0; r < rows.size(); ++r) std::memcpy(dst.data() + r * t.dim, t.s[k].data() + rows[r] * t.dim, t.dim * 4);
  }
  if (optim_.NeedsSteps()) {
    std::vector<int64_t>& st = c.states_i[static_cast<uint32_t>(StateType::kSteps)];
    st.resize(rows.size());
    for (size_t r = 0; r < rows.size(); ++r) st[r] = t.steps[rows[r]];
  }
  return c;
}

void CpuShard::ImportSparse(uint64_t id, const ckpt::SparseColumns& c, bool overwrite) {
  Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  KB_CHECK(c.dim == t.dim || c.ids.empty(), err::kSparseDimensionUnCompatible, "imported rows have another dimension");
  auto steps_it = c.states_i.find(static_cast<uint32_t>(StateType::kSteps));
  for (size_t i = 0; i < c.ids.size(); ++i) {
    auto it = t.index.find(c.ids[i]);
    if (it != t.index.end() && !overwrite) continue;
    const int64_t row = it != t.index.end() ? it->second : t.AddRow(c.ids[i], optim_);
    std::memcpy(t.val.data() + row * t.dim, c.vals.data() + i * t.dim, t.dim * 4);
    for (int k = 0; k < 3; ++k) {
      if (!optim_.SlabUsed(k)) continue;
      auto st = c.states.find(SlabStateType(optim_, k));
      if (st == c.states.end() || st->second.size() < (i + 1) * t.dim) continue;
      std::memcpy(t.s[k].data() + row * t.dim, st->second.data() + i * t.dim, t.dim * 4);
    }
    if (steps_it != c.states_i.end() && i < steps_it->second.size()) t.steps[row] = steps_it->second[i];
  }
}

int64_t CpuShard::FilterSparse(uint64_t id, const ckpt::RowFilter& keep) {
  Sparse& t = sparse(id);
  std::lock_guard<std::mutex> g(t.mu);
  const int64_t n = static_cast<int64_t>(t.ids.size());
  int64_t w = 0;
  for (int64_t r = 0; r < n; ++r) {
    if (!keep.Keep(t.ids[r])) continue;
    if (w != r) {
      t.ids[w] = t.ids[r];
      t.steps[w] = t.steps[r];
      std::memmove(t.val.data() + w * t.dim, t.val.data() + r * t.dim, t.dim * 4);
      for (int k = 0; k < 3; ++k)
        if (!t.s[k].empty()) std::memmove(t.s[k].data() + w * t.dim, t.s[k].data() + r * t.dim, t.dim * 4);
    }
    ++w;
  }
  t.ids.resize(w);
  t.steps.resize(w);
  t.val.resize(w * t.dim);
  for (int k = 0; k < 3; ++k)
    if (!t.s[k].empty()) t.s[k].resize(w * t.dim);
  t.index.clear();
  for (int64_t r = 0; r < w; ++r) t.index.emplace(t.ids[r], r);
  return n - w;
}

}  // namespace kb
