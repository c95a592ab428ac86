// Python bindings (`kraken_b200._C`).  Thin: every function converts torch
// tensors to raw pointers and forwards to the host core (core/, cpu/) or to
// the kernel launchers (cuda/kernels.h) on the current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <cstring>
#include <map>

#include "core/checkpoint.h"
#include "core/hash.h"
#include "core/net.h"
#include "core/router.h"
#include "core/serialize.h"
#include "core/snappy_codec.h"
#include "core/task_queue.h"
#include "cpu/cpu_ops.h"
#include "cpu/cpu_shard.h"
#include "cuda/kernels.h"

namespace py = pybind11;
using namespace kb;

namespace {

#define CUDA_OK(expr)                                                                                   \
  do {                                                                                                  \
    cudaError_t e__ = (expr);                                                                           \
    if (e__ != cudaSuccess) throw std::runtime_error(std::string(#expr) + ": " + cudaGetErrorString(e__)); \
  } while (0)

cudaStream_t cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <typename T>
T* ptr(const torch::Tensor& t) {
  return t.defined() && t.numel() > 0 ? reinterpret_cast<T*>(t.data_ptr()) : nullptr;
}
template <typename T>
T* optr(const c10::optional<torch::Tensor>& t) {
  return t.has_value() ? ptr<T>(*t) : nullptr;
}

// The channel control block (cuda/kernels.h: Ctrl) lives in an int32 CUDA tensor of at least kCtrlInts elements.
cu::Ctrl* ctrl_ptr(const torch::Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kInt32 && t.numel() >= cu::kCtrlInts,
              "ctrl must be a contiguous int32 CUDA tensor of at least ", cu::kCtrlInts, " elements");
  return reinterpret_cast<cu::Ctrl*>(t.data_ptr());
}

void need_cuda(const torch::Tensor& t, const char* name, c10::ScalarType st) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.scalar_type() == st, name, " has the wrong dtype");
}
void need_cpu(const torch::Tensor& t, const char* name, c10::ScalarType st) {
  TORCH_CHECK(!t.is_cuda(), name, " must be a CPU tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.scalar_type() == st, name, " has the wrong dtype");
}

// ------------------------------------------------------------------ tensors <-> HostTensor
DType dtype_of(const torch::Tensor& t) {
  switch (t.scalar_type()) {
    case torch::kBool: return DType::kBool;
    case torch::kUInt8: return DType::kUint8;
    case torch::kInt8: return DType::kInt8;
    case torch::kInt16: return DType::kInt16;
    case torch::kInt32: return DType::kInt32;
    case torch::kInt64: return DType::kInt64;
    case torch::kFloat16: return DType::kFloat16;
    case torch::kFloat32: return DType::kFloat32;
    case torch::kFloat64: return DType::kFloat64;
    default: throw KrakenError(err::kBadArgument, "unsupported torch dtype");
  }
}

c10::ScalarType scalar_of(DType d) {
  switch (d) {
    case DType::kBool: return torch::kBool;
    case DType::kUint8: return torch::kUInt8;
    case DType::kInt8: return torch::kInt8;
    case DType::kInt16: return torch::kInt16;
    case DType::kUint16: return torch::kInt16;
    case DType::kInt32: return torch::kInt32;
    case DType::kUint32: return torch::kInt32;
    case DType::kInt64: return torch::kInt64;
    case DType::kUint64: return torch::kInt64;
    case DType::kFloat16: return torch::kFloat16;
    case DType::kFloat32: return torch::kFloat32;
    case DType::kFloat64: return torch::kFloat64;
    default: throw KrakenError(err::kBadArgument, "unsupported element type");
  }
}

HostTensor to_host(const torch::Tensor& t_in) {
  torch::Tensor t = t_in.detach().cpu().contiguous();
  HostTensor h;
  h.dtype = dtype_of(t);
  h.dims.assign(t.sizes().begin(), t.sizes().end());
  h.data.resize(static_cast<size_t>(t.numel()) * t.element_size());
  if (!h.data.empty()) std::memcpy(h.data.data(), t.data_ptr(), h.data.size());
  return h;
}

torch::Tensor from_host(const HostTensor& h) {
  if (h.layout == Layout::kCoo) {
    // densify: zeros then add at the flat indices
    torch::Tensor idx = from_host(*h.indices).to(torch::kInt64).reshape({-1});
    torch::Tensor val = from_host(*h.values).reshape({-1});
    int64_t n = 1;
    for (auto d : h.dims) n *= d;
    torch::Tensor out = torch::zeros({n}, val.options());
    out.index_add_(0, idx, val);
    return out.reshape(h.dims);
  }
  torch::Tensor t = torch::empty(h.dims, torch::TensorOptions().dtype(scalar_of(h.dtype)));
  if (t.numel() > 0) std::memcpy(t.data_ptr(), h.data.data(), std::min<size_t>(h.data.size(), t.nbytes()));
  return t;
}

py::dict value_to_py(const Value& v) {
  py::dict d, st, sti;
  d["val"] = from_host(v.val);
  for (auto& kv : v.states) st[py::int_(kv.first)] = from_host(kv.second);
  for (auto& kv : v.states_i) sti[py::int_(kv.first)] = kv.second;
  d["states"] = st;
  d["states_i"] = sti;
  return d;
}

Value value_from_py(const py::dict& d) {
  Value v;
  v.val = to_host(d["val"].cast<torch::Tensor>());
  if (d.contains("states"))
    for (auto kv : d["states"].cast<py::dict>()) v.states[kv.first.cast<uint32_t>()] = to_host(kv.second.cast<torch::Tensor>());
  if (d.contains("states_i"))
    for (auto kv : d["states_i"].cast<py::dict>()) v.states_i[kv.first.cast<uint32_t>()] = kv.second.cast<int64_t>();
  return v;
}

py::dict columns_to_py(const ckpt::SparseColumns& c) {
  py::dict d, st, sti;
  const int64_t n = static_cast<int64_t>(c.ids.size());
  torch::Tensor ids = torch::empty({n}, torch::kInt64);
  if (n) std::memcpy(ids.data_ptr(), c.ids.data(), n * 8);
  torch::Tensor vals = torch::empty({n, c.dim}, torch::kFloat32);
  if (n) std::memcpy(vals.data_ptr(), c.vals.data(), c.vals.size() * 4);
  for (auto& kv : c.states) {
    torch::Tensor s = torch::zeros({n, c.dim}, torch::kFloat32);
    if (!kv.second.empty()) std::memcpy(s.data_ptr(), kv.second.data(), std::min<size_t>(kv.second.size() * 4, s.nbytes()));
    st[py::int_(kv.first)] = s;
  }
  for (auto& kv : c.states_i) {
    torch::Tensor s = torch::zeros({n}, torch::kInt64);
    if (!kv.second.empty()) std::memcpy(s.data_ptr(), kv.second.data(), std::min<size_t>(kv.second.size() * 8, s.nbytes()));
    sti[py::int_(kv.first)] = s;
  }
  d["dim"] = c.dim;
  d["ids"] = ids;
  d["vals"] = vals;
  d["states"] = st;
  d["states_i"] = sti;
  return d;
}

ckpt::SparseColumns columns_from_py(int64_t dim, const torch::Tensor& ids, const torch::Tensor& vals,
                                    const py::dict& states, const py::dict& states_i) {
  ckpt::SparseColumns c;
  c.dim = dim;
  torch::Tensor i = ids.detach().cpu().contiguous();
  need_cpu(i, "ids", torch::kInt64);
  const int64_t n = i.numel();
  c.ids.resize(n);
  if (n) std::memcpy(c.ids.data(), i.data_ptr(), n * 8);
  torch::Tensor v = vals.detach().cpu().contiguous().to(torch::kFloat32);
  TORCH_CHECK(v.numel() == n * dim, "vals must be [n, dim]");
  c.vals.resize(n * dim);
  if (n) std::memcpy(c.vals.data(), v.data_ptr(), n * dim * 4);
  for (auto kv : states) {
    torch::Tensor s = kv.second.cast<torch::Tensor>().detach().cpu().contiguous().to(torch::kFloat32);
    TORCH_CHECK(s.numel() == n * dim, "state must be [n, dim]");
    auto& col = c.states[kv.first.cast<uint32_t>()];
    col.resize(n * dim);
    if (n) std::memcpy(col.data(), s.data_ptr(), n * dim * 4);
  }
  for (auto kv : states_i) {
    torch::Tensor s = kv.second.cast<torch::Tensor>().detach().cpu().contiguous().to(torch::kInt64);
    TORCH_CHECK(s.numel() == n, "state_i must be [n]");
    auto& col = c.states_i[kv.first.cast<uint32_t>()];
    col.resize(n);
    if (n) std::memcpy(col.data(), s.data_ptr(), n * 8);
  }
  return c;
}

ckpt::RowFilter make_filter(int mode, uint64_t salt, uint32_t world, uint32_t rank, const Router* ring, uint64_t table_id,
                            uint64_t node) {
  ckpt::RowFilter f;
  f.mode = static_cast<ckpt::RowFilter::Mode>(mode);
  f.table_salt = salt;
  f.world = world;
  f.rank = rank;
  f.ring = ring;
  f.table_id = table_id;
  f.node = node;
  return f;
}

// ------------------------------------------------------------------ symmetric heap
// One cudaMalloc'd arena per rank, exported with a CUDA IPC handle and mapped by
// every peer of the same box.
struct SymHeap {
  void* local = nullptr;
  size_t bytes = 0;
  int rank = 0, world = 1;
  std::vector<void*> bases;
  std::vector<bool> opened;

  // alias_peers: every peer pointer is the local arena.  Lets one GPU run the multi-rank kernels
  // against itself (peers that never answer), which is how the bounded waits are tested.
  SymHeap(size_t nbytes, int r, int w, bool alias_peers) : bytes(nbytes), rank(r), world(w) {
    TORCH_CHECK(w >= 1 && w <= cu::kMaxWorldHost, "world size must be 1..16");
    CUDA_OK(cudaMalloc(&local, nbytes));
    CUDA_OK(cudaMemset(local, 0, nbytes));
    bases.assign(w, alias_peers ? local : nullptr);
    opened.assign(w, false);
    bases[r] = local;
  }
  ~SymHeap() { Close(); }
  py::bytes Handle() const {
    cudaIpcMemHandle_t h;
    CUDA_OK(cudaIpcGetMemHandle(&h, local));
    return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
  }
  void Open(const std::vector<std::string>& handles) {
    TORCH_CHECK(static_cast<int>(handles.size()) == world, "need one handle per rank");
    for (int p = 0; p < world; ++p) {
      if (p == rank) continue;
      TORCH_CHECK(handles[p].size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
      cudaIpcMemHandle_t h;
      std::memcpy(&h, handles[p].data(), sizeof(h));
      CUDA_OK(cudaIpcOpenMemHandle(&bases[p], h, cudaIpcMemLazyEnablePeerAccess));
      opened[p] = true;
    }
  }
  void Close() {
    for (int p = 0; p < static_cast<int>(bases.size()); ++p)
      if (opened[p]) {
        cudaIpcCloseMemHandle(bases[p]);
        opened[p] = false;
      }
    if (local) {
      cudaFree(local);
      local = nullptr;
    }
  }
  cu::SymHost View() const {
    cu::SymHost s{};
    for (int p = 0; p < world; ++p) s.base[p] = bases[p];
    s.rank = rank;
    s.world = world;
    return s;
  }
  // Typed window into the local arena (no ownership: the heap must outlive it).
  torch::Tensor Window(size_t off, std::vector<int64_t> shape, py::object dtype) const {
    auto st = torch::python::detail::py_object_to_dtype(dtype);
    int64_t n = 1;
    for (auto d : shape) n *= d;
    TORCH_CHECK(off + static_cast<size_t>(n) * c10::elementSize(st) <= bytes, "window exceeds the heap");
    int dev;
    CUDA_OK(cudaGetDevice(&dev));
    return torch::from_blob(static_cast<char*>(local) + off, shape,
                            torch::TensorOptions().dtype(st).device(torch::kCUDA, dev));
  }
};

cu::TableHost make_table(const torch::Tensor& keys, const torch::Tensor& val, const c10::optional<torch::Tensor>& s0,
                         const c10::optional<torch::Tensor>& s1, const c10::optional<torch::Tensor>& s2,
                         const c10::optional<torch::Tensor>& steps, const c10::optional<torch::Tensor>& lead,
                         const torch::Tensor& size, const torch::Tensor& status, uint32_t bits, int dim, int init_type,
                         float init_a, float init_b, uint64_t seed_key) {
  need_cuda(keys, "keys", torch::kInt64);
  need_cuda(val, "val", torch::kFloat32);
  TORCH_CHECK(keys.numel() == (1ll << bits), "keys must have 1 << bits elements");
  TORCH_CHECK(val.numel() == keys.numel() * dim, "val must be [cap, dim]");
  cu::TableHost t{};
  t.keys = keys.data_ptr();
  t.val = ptr<float>(val);
  t.s[0] = optr<float>(s0);
  t.s[1] = optr<float>(s1);
  t.s[2] = optr<float>(s2);
  t.steps = optr<int>(steps);
  t.lead = lead.has_value() ? lead->data_ptr() : nullptr;
  t.size = ptr<int>(size);
  t.status = ptr<int>(status);
  t.bits = bits;
  t.dim = dim;
  t.init.type = static_cast<uint8_t>(init_type);
  t.init.a = init_a;
  t.init.b = init_b;
  t.seed_key = seed_key;
  return t;
}

}  // namespace

void bind_dense(py::module_& m);  // bindings_dense.cc

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::register_exception<KrakenError>(m, "KrakenError");
  m.attr("CTRL_INTS") = cu::kCtrlInts;

  py::enum_<OptimType>(m, "OptimType")
      .value("kAdagrad", OptimType::kAdagrad)
      .value("kAdam", OptimType::kAdam)
      .value("kRMSprop", OptimType::kRMSprop)
      .value("kSGD", OptimType::kSGD);
  py::enum_<InitializerType>(m, "InitializerType")
      .value("kConstant", InitializerType::kConstant)
      .value("kUniform", InitializerType::kUniform)
      .value("kNormal", InitializerType::kNormal)
      .value("kXavierUniform", InitializerType::kXavierUniform)
      .value("kXavierNormal", InitializerType::kXavierNormal);
  py::enum_<EmitterType>(m, "EmitterType").value("kDefault", EmitterType::kDefault).value("kDCT", EmitterType::kDCT);
  py::enum_<TableType>(m, "TableType").value("kDense", TableType::kDense).value("kSparse", TableType::kSparse);

  m.def("mix64", [](uint64_t v) { return Mix64(v); });
  m.def("mix64_pair", [](uint64_t a, uint64_t b) { return Mix64(a, b); });
  m.def("owner_of", [](uint64_t salt, uint64_t id, uint32_t world) { return OwnerOf(salt, id, world); });
  m.def("table_salt", [](uint64_t table_id) { return TableSalt(table_id); });
  m.def("seed_key", [](uint64_t seed, uint64_t table_id) { return SeedKey(seed, table_id); });
  m.def("error_message", [](int32_t c) { return std::string(err::Msg(c)); });
  m.def("init_row", [](int init_type, float a, float b, uint64_t seed_key, uint64_t id, int dim) {
    InitPOD ip;
    ip.type = static_cast<uint8_t>(init_type);
    ip.a = a;
    ip.b = b;
    torch::Tensor t = torch::empty({dim}, torch::kFloat32);
    InitRow(ip, seed_key, id, dim, t.data_ptr<float>());
    return t;
  });

  // ---------------- router
  py::class_<Router>(m, "Router")
      .def(py::init<>())
      .def("add", &Router::Add)
      .def("remove", &Router::Remove)
      .def("empty", &Router::Empty)
      .def("contains", &Router::Contains)
      .def("version", &Router::version)
      .def("hit", &Router::Hit)
      .def("node_ids",
           [](const Router& r) {
             std::vector<uint64_t> v;
             for (auto& n : r.nodes()) v.push_back(n.id);
             return v;
           })
      .def("node_name",
           [](const Router& r, uint64_t id) {
             for (auto& n : r.nodes())
               if (n.id == id) return n.name;
             throw KrakenError(err::kBadArgument, "no such node");
           })
      .def("vnodes",
           [](const Router& r) {
             std::vector<std::tuple<uint64_t, uint64_t, std::string>> v;
             for (auto& x : r.ring()) v.emplace_back(x.hash_v, x.node_id, x.name);
             return v;
           })
      .def("node_hash_ranges",
           [](const Router& r, uint64_t id) {
             std::vector<std::pair<uint64_t, uint64_t>> v;
             for (auto& x : r.NodeHashRanges(id)) v.emplace_back(x.start, x.end);
             return v;
           })
      .def("intersect_nodes",
           [](const Router& r, uint64_t start, uint64_t end) {
             auto s = r.IntersectNodes({start, end});
             return std::vector<uint64_t>(s.begin(), s.end());
           })
      .def("__eq__", [](const Router& a, const Router& b) { return a == b; })
      .def("__str__", &Router::Str)
      .def("to_bytes",
           [](const Router& r) {
             MemSink s;
             Writer w(&s);
             r.Save(&w);
             return py::bytes(s.str());
           })
      .def_static("from_bytes",
                  [](const std::string& b) {
                    MemSource s(b.data(), b.size());
                    Reader r(&s);
                    return Router::Load(&r);
                  })
      .def_static("for_ranks", &Router::ForRanks);

  // ---------------- metadata
  py::class_<TableMeta>(m, "TableMeta")
      .def(py::init<>())
      .def_readwrite("id", &TableMeta::id)
      .def_readwrite("name", &TableMeta::name)
      .def_readwrite("table_type", &TableMeta::table_type)
      .def_readwrite("shape", &TableMeta::shape)
      .def_readwrite("dimension", &TableMeta::dimension)
      .def_readwrite("init_type", &TableMeta::init_type)
      .def_readwrite("init_conf", &TableMeta::init_conf);
  py::class_<ModelMeta>(m, "ModelMeta")
      .def(py::init<>())
      .def_readwrite("name", &ModelMeta::name)
      .def_readwrite("optim_type", &ModelMeta::optim_type)
      .def_readwrite("optim_conf", &ModelMeta::optim_conf)
      .def_readwrite("tables", &ModelMeta::tables)
      .def("to_bytes",
           [](const ModelMeta& mm) {
             MemSink s;
             Writer w(&s);
             w.Model(mm);
             return py::bytes(s.str());
           })
      .def_static("from_bytes", [](const std::string& b) {
        MemSource s(b.data(), b.size());
        Reader r(&s);
        return r.Model();
      });

  // ---------------- message bodies of the socket transport: u32 json_len | json | u32 n | n x (u64 len | tensor)
  // One allocation and one copy per tensor in each direction (the per-tensor calls below copy four times).
  m.def("rpc_pack_body", [](const std::string& json, const std::vector<torch::Tensor>& tensors) {
    std::vector<torch::Tensor> keep;
    keep.reserve(tensors.size());
    size_t total = 4 + json.size() + 4;
    for (auto& t_in : tensors) {
      torch::Tensor t = t_in.detach();
      KB_CHECK(!t.is_cuda(), err::kSerializeRequest, "message tensors live on the host");
      if (t.dim() == 0) t = t.reshape({1});
      t = t.contiguous();
      dtype_of(t);  // throws for a dtype the wire format has no code for
      total += 8 + 1 + 8 + 8 * static_cast<size_t>(t.dim()) + 1 + static_cast<size_t>(t.nbytes());
      keep.push_back(std::move(t));
    }
    KB_CHECK(json.size() <= 0xFFFFFFFFu && keep.size() <= 0xFFFFFFFFu, err::kSerializeRequest, "message too large");
    py::bytes out = py::reinterpret_steal<py::bytes>(PyBytes_FromStringAndSize(nullptr, static_cast<Py_ssize_t>(total)));
    KB_CHECK(out.ptr() != nullptr, err::kSerializeRequest, "cannot allocate the message body");
    char* p = PyBytes_AS_STRING(out.ptr());
    auto put = [&p](const void* src, size_t n) {
      std::memcpy(p, src, n);
      p += n;
    };
    const uint32_t jl = static_cast<uint32_t>(json.size()), n = static_cast<uint32_t>(keep.size());
    put(&jl, 4);
    put(json.data(), json.size());
    put(&n, 4);
    for (auto& t : keep) {
      const uint64_t nd = static_cast<uint64_t>(t.dim());
      const uint64_t len = 1 + 8 + 8 * nd + 1 + static_cast<uint64_t>(t.nbytes());
      const uint8_t layout = static_cast<uint8_t>(Layout::kStride), dt = static_cast<uint8_t>(dtype_of(t));
      put(&len, 8);
      put(&layout, 1);
      put(&nd, 8);
      for (int64_t d : t.sizes()) put(&d, 8);
      put(&dt, 1);
      if (t.nbytes()) put(t.data_ptr(), static_cast<size_t>(t.nbytes()));
    }
    return out;
  });
  m.def("rpc_unpack_body", [](const std::string& b) {
    size_t pos = 0;
    auto need = [&](size_t n) {
      KB_CHECK(n <= b.size() - pos, err::kDeserializeRequest, "message body is truncated");
    };
    auto u32 = [&]() {
      need(4);
      uint32_t v;
      std::memcpy(&v, b.data() + pos, 4);
      pos += 4;
      return v;
    };
    const uint32_t jl = u32();
    need(jl);
    py::bytes json(b.data() + pos, jl);
    pos += jl;
    const uint32_t n = u32();
    py::list tensors;
    for (uint32_t i = 0; i < n; ++i) {
      need(8);
      uint64_t len;
      std::memcpy(&len, b.data() + pos, 8);
      pos += 8;
      need(len);
      const char* q = b.data() + pos;
      if (len >= 1 && static_cast<uint8_t>(q[0]) == static_cast<uint8_t>(Layout::kStride)) {
        // dense: straight from the message into the tensor's storage
        MemSource one(q + 1, len - 1);
        Reader rr(&one);
        std::vector<int64_t> dims = rr.Vec<int64_t>();
        const DType dt = static_cast<DType>(rr.Pod<uint8_t>());
        // the shape comes off the wire: it must describe exactly the bytes that follow BEFORE anything is allocated
        const uint64_t payload = len - 1 - one.offset();
        uint64_t bytes = DTypeBytes(dt);
        KB_CHECK(bytes > 0, err::kDeserializeRequest, "tensor of a type without a size");
        for (int64_t d : dims) {
          KB_CHECK(d >= 0, err::kDeserializeRequest, "negative tensor extent");
          KB_CHECK(d == 0 || bytes <= payload / static_cast<uint64_t>(d), err::kDeserializeRequest,
                   "tensor payload does not match its shape");
          bytes *= static_cast<uint64_t>(d);
        }
        KB_CHECK(bytes == payload, err::kDeserializeRequest, "tensor payload does not match its shape");
        torch::Tensor t = torch::empty(dims, torch::TensorOptions().dtype(scalar_of(dt)));
        if (t.nbytes()) std::memcpy(t.data_ptr(), q + 1 + one.offset(), static_cast<size_t>(t.nbytes()));
        tensors.append(t);
      } else {
        MemSource one(q, len);
        Reader rr(&one);
        tensors.append(from_host(rr.Tensor()));
      }
      pos += len;
    }
    return py::make_tuple(json, tensors);
  });

  // ---------------- the reference's own message bodies (ZeroMQ front end): a vector<Tensor> of n rows of one width,
  // as its servers answer a sparse pull and its workers send sparse gradients (kraken/common/serialize.h:156-217:
  // u64 count, then per tensor u8 layout = 0, Shape = u64 rank + i64 dims, u8 dtype, raw data)
  m.def("wire_rows_to_tensor_list", [](const torch::Tensor& rows_in) {
    torch::Tensor rows = rows_in.detach().contiguous();
    need_cpu(rows, "rows", torch::kFloat32);
    TORCH_CHECK(rows.dim() == 2, "rows must be [n, dim]");
    const uint64_t n = static_cast<uint64_t>(rows.size(0));
    const int64_t dim = rows.size(1);
    const size_t per = 1 + 8 + 8 + 1 + static_cast<size_t>(dim) * 4;
    py::bytes out = py::reinterpret_steal<py::bytes>(PyBytes_FromStringAndSize(nullptr, static_cast<Py_ssize_t>(8 + n * per)));
    KB_CHECK(out.ptr() != nullptr, err::kSerializeReply, "cannot allocate the reply");
    char* p = PyBytes_AS_STRING(out.ptr());
    std::memcpy(p, &n, 8);
    p += 8;
    const uint64_t rank = 1;
    const uint8_t f32 = static_cast<uint8_t>(DType::kFloat32);
    const float* src = rows.data_ptr<float>();
    for (uint64_t i = 0; i < n; ++i) {
      *p++ = 0;
      std::memcpy(p, &rank, 8);
      std::memcpy(p + 8, &dim, 8);
      p[16] = static_cast<char>(f32);
      std::memcpy(p + 17, src + i * dim, static_cast<size_t>(dim) * 4);
      p += 17 + static_cast<size_t>(dim) * 4;
    }
    return out;
  });
  m.def("wire_tensor_list_to_rows", [](const std::string& b, uint64_t offset) {
    // (rows [n, dim] float32, offset behind the list); every tensor must be a dense float32 vector of one width
    auto fail = [] { throw KrakenError(err::kDeserializeRequest, "malformed list of row tensors"); };
    size_t pos = static_cast<size_t>(offset);
    if (pos + 8 > b.size()) fail();
    uint64_t n;
    std::memcpy(&n, b.data() + pos, 8);
    pos += 8;
    int64_t dim = 0;
    torch::Tensor rows;
    for (uint64_t i = 0; i < n; ++i) {
      if (pos + 18 > b.size()) fail();
      uint64_t rank;
      int64_t d;
      std::memcpy(&rank, b.data() + pos + 1, 8);
      if (b[pos] != 0 || rank != 1) fail();
      if (pos + 18 > b.size()) fail();
      std::memcpy(&d, b.data() + pos + 9, 8);
      if (static_cast<uint8_t>(b[pos + 17]) != static_cast<uint8_t>(DType::kFloat32) || d < 0) fail();
      if (i == 0) {
        dim = d;
        if (n > (b.size() - pos) / (18 + static_cast<size_t>(dim) * 4 == 0 ? 1 : 18 + static_cast<size_t>(dim) * 4)) fail();
        rows = torch::empty({static_cast<int64_t>(n), dim}, torch::kFloat32);
      }
      if (d != dim || pos + 18 + static_cast<size_t>(dim) * 4 > b.size()) fail();
      std::memcpy(rows.data_ptr<float>() + i * dim, b.data() + pos + 18, static_cast<size_t>(dim) * 4);
      pos += 18 + static_cast<size_t>(dim) * 4;
    }
    if (n == 0) rows = torch::empty({0, 0}, torch::kFloat32);
    return py::make_tuple(rows, static_cast<uint64_t>(pos));
  });

  // ---------------- serializer (tests, socket transport)
  m.def("serialize_tensor", [](const torch::Tensor& t) {
    MemSink s;
    Writer w(&s);
    w.Tensor(to_host(t));
    return py::bytes(s.str());
  });
  m.def("serialize_coo", [](const torch::Tensor& indices, const torch::Tensor& values, std::vector<int64_t> shape) {
    HostTensor t;
    t.layout = Layout::kCoo;
    t.indices = std::make_shared<HostTensor>(to_host(indices));
    t.values = std::make_shared<HostTensor>(to_host(values));
    t.dims = shape;
    MemSink s;
    Writer w(&s);
    w.Tensor(t);
    return py::bytes(s.str());
  });
  m.def("deserialize_tensor", [](const std::string& b) {
    MemSource s(b.data(), b.size());
    Reader r(&s);
    return from_host(r.Tensor());
  });
  // RPC body compression in the Snappy block format (kraken/common/compress.h:18-91)
  m.def("snappy_compress", [](const std::string& b) {
    std::string out;
    {
      py::gil_scoped_release nogil;
      snappy_codec::Compress(b.data(), b.size(), &out);
    }
    return py::bytes(out);
  });
  m.def("snappy_uncompress", [](const std::string& b) {
    std::string out;
    bool ok;
    {
      py::gil_scoped_release nogil;
      ok = snappy_codec::Uncompress(b.data(), b.size(), &out);
    }
    KB_CHECK(ok, err::kSnappyUncompress, "malformed Snappy stream");
    return py::bytes(out);
  });
  m.def("serialize_value", [](const py::dict& d) {
    MemSink s;
    Writer w(&s);
    w.Val(value_from_py(d));
    return py::bytes(s.str());
  });
  m.def("deserialize_value", [](const std::string& b) {
    MemSource s(b.data(), b.size());
    Reader r(&s);
    return value_to_py(r.Val());
  });
  m.def("serialize_string", [](const std::string& v) {
    MemSink s;
    Writer w(&s);
    w.Str(v);
    return py::bytes(s.str());
  });
  m.def("serialize_conf", [](const Conf& c) {
    MemSink s;
    Writer w(&s);
    w.ConfMap(c);
    return py::bytes(s.str());
  });

  // ---------------- checkpoint
  m.def("ckpt_timestamp_dir_name", &ckpt::TimestampDirName);
  m.def("ckpt_parse_timestamp", [](const std::string& n) {
    int64_t k = -1;
    bool ok = ckpt::ParseTimestampDir(n, &k);
    return std::make_pair(ok, k);
  });
  m.def("ckpt_prepare_save_dir", &ckpt::PrepareSaveDir);
  m.def("ckpt_latest_shard_dirs", &ckpt::LatestShardDirs);
  m.def("ckpt_save_router", &ckpt::SaveRouter);
  m.def("ckpt_load_router", &ckpt::LoadRouter);
  m.def("ckpt_save_model", &ckpt::SaveModel);
  m.def("ckpt_load_model", &ckpt::LoadModel);
  m.def("ckpt_save_dense", [](const std::string& dir, uint64_t id, const std::string& name, const py::dict& v) {
    ckpt::SaveDense(dir, id, name, value_from_py(v));
  });
  m.def("ckpt_load_dense", [](const std::string& dir, const std::string& name) -> py::object {
    uint64_t id;
    Value v;
    if (!ckpt::LoadDense(dir, name, &id, &v)) return py::none();
    py::dict d = value_to_py(v);
    d["id"] = id;
    return d;
  });
  m.def("ckpt_save_sparse",
        [](const std::string& dir, uint64_t id, const std::string& name, int64_t dim, InitializerType init_type,
           const Conf& init_conf, const torch::Tensor& ids, const torch::Tensor& vals, const py::dict& states,
           const py::dict& states_i) {
          ckpt::SparseHeader h;
          h.id = id;
          h.name = name;
          h.dim = dim;
          h.init_type = init_type;
          h.init_conf = init_conf;
          ckpt::SparseColumns c = columns_from_py(dim, ids, vals, states, states_i);
          py::gil_scoped_release nogil;
          ckpt::SaveSparse(dir, h, c);
        });
  m.def(
      "ckpt_load_sparse",
      [](const std::string& dir, const std::string& name, int filter_mode, uint64_t salt, uint32_t world, uint32_t rank,
         const Router* ring, uint64_t table_id, uint64_t node) -> py::object {
        ckpt::SparseHeader h;
        ckpt::SparseColumns c;
        bool ok;
        {
          py::gil_scoped_release nogil;
          ok = ckpt::LoadSparse(dir, name, make_filter(filter_mode, salt, world, rank, ring, table_id, node), &h, &c);
        }
        if (!ok) return py::none();
        py::dict d = columns_to_py(c);
        d["id"] = h.id;
        d["name"] = h.name;
        d["init_type"] = h.init_type;
        d["init_conf"] = h.init_conf;
        return d;
      },
      py::arg("dir"), py::arg("name"), py::arg("filter_mode") = 0, py::arg("salt") = 0, py::arg("world") = 1,
      py::arg("rank") = 0, py::arg("ring") = nullptr, py::arg("table_id") = 0, py::arg("node") = 0);

  // streamed save of a large table: rows arrive in chunks, already in file order (slot by slot, ids ascending
  // as unsigned numbers inside a slot); CPU tensors (pinned or not), float32 / int64, contiguous
  py::class_<ckpt::SparseStreamWriter>(m, "SparseStreamWriter")
      .def(py::init([](const std::string& dir, uint64_t id, const std::string& name, int64_t dim, InitializerType init_type,
                       const Conf& init_conf, std::vector<uint32_t> state_types, std::vector<uint32_t> int_state_types,
                       int threads) {
             ckpt::SparseHeader h;
             h.id = id;
             h.name = name;
             h.dim = dim;
             h.init_type = init_type;
             h.init_conf = init_conf;
             return new ckpt::SparseStreamWriter(dir, h, std::move(state_types), std::move(int_state_types), threads);
           }),
           py::arg("dir"), py::arg("id"), py::arg("name"), py::arg("dim"), py::arg("init_type"), py::arg("init_conf"),
           py::arg("state_types"), py::arg("int_state_types"), py::arg("threads") = 8)
      .def("begin_slot", &ckpt::SparseStreamWriter::BeginSlot)
      .def("append",
           [](ckpt::SparseStreamWriter& w, const torch::Tensor& ids, const torch::Tensor& vals,
              const std::vector<torch::Tensor>& states, const std::vector<torch::Tensor>& states_i) {
             need_cpu(ids, "ids", torch::kInt64);
             need_cpu(vals, "vals", torch::kFloat32);
             const size_t n = static_cast<size_t>(ids.numel());
             std::vector<const float*> sp;
             std::vector<const int64_t*> ip;
             for (auto& t : states) {
               need_cpu(t, "state", torch::kFloat32);
               TORCH_CHECK(t.numel() == vals.numel(), "a state column differs in size from the values");
               sp.push_back(t.data_ptr<float>());
             }
             for (auto& t : states_i) {
               need_cpu(t, "int state", torch::kInt64);
               TORCH_CHECK(static_cast<size_t>(t.numel()) == n, "an integer state column differs in size from the ids");
               ip.push_back(t.data_ptr<int64_t>());
             }
             py::gil_scoped_release nogil;
             w.Append(reinterpret_cast<const uint64_t*>(ids.data_ptr<int64_t>()), vals.data_ptr<float>(), sp.data(),
                      ip.data(), n);
           })
      .def("close", &ckpt::SparseStreamWriter::Close)
      .def("bytes_written", &ckpt::SparseStreamWriter::bytes_written)
      .def("row_bytes", &ckpt::SparseStreamWriter::row_bytes);
  m.def(
      "ckpt_load_sparse_fast",
      [](const std::string& dir, const std::string& name, int threads) -> py::object {
        // None: no such file; False: the file is not in the fixed layout (use ckpt_load_sparse); else all rows,
        // extracted by `threads` threads straight into the tensors that are returned
        ckpt::SparseChunkReader r(dir, name, threads);
        if (!r.exists()) return py::none();
        if (!r.fast()) return py::bool_(false);
        const int64_t n = static_cast<int64_t>(r.rows()), dim = r.header().dim;
        torch::Tensor ids = torch::empty({n}, torch::kInt64), vals = torch::empty({n, dim}, torch::kFloat32);
        std::vector<torch::Tensor> st, sti;
        std::vector<float*> sp;
        std::vector<int64_t*> ip;
        for (size_t k = 0; k < r.state_types().size(); ++k) {
          st.push_back(torch::empty({n, dim}, torch::kFloat32));
          sp.push_back(st.back().data_ptr<float>());
        }
        for (size_t k = 0; k < r.int_state_types().size(); ++k) {
          sti.push_back(torch::empty({n}, torch::kInt64));
          ip.push_back(sti.back().data_ptr<int64_t>());
        }
        bool ok;
        {
          py::gil_scoped_release nogil;
          ok = r.Read(0, r.rows(), reinterpret_cast<uint64_t*>(ids.data_ptr<int64_t>()), vals.data_ptr<float>(), sp.data(),
                      ip.data());
        }
        if (!ok) return py::bool_(false);
        py::dict d, ds, di;
        for (size_t k = 0; k < st.size(); ++k) ds[py::int_(r.state_types()[k])] = st[k];
        for (size_t k = 0; k < sti.size(); ++k) di[py::int_(r.int_state_types()[k])] = sti[k];
        d["dim"] = dim;
        d["ids"] = ids;
        d["vals"] = vals;
        d["states"] = ds;
        d["states_i"] = di;
        d["id"] = r.header().id;
        d["name"] = r.header().name;
        d["init_type"] = r.header().init_type;
        d["init_conf"] = r.header().init_conf;
        return d;
      },
      py::arg("dir"), py::arg("name"), py::arg("threads") = 8);

  // chunked load of a large table: rows [lo, lo + n) of the file order into caller-owned CPU tensors
  // (pinned staging buffers that are reused for every chunk)
  py::class_<ckpt::SparseChunkReader>(m, "SparseChunkReader")
      .def(py::init<const std::string&, const std::string&, int>(), py::arg("dir"), py::arg("name"),
           py::arg("threads") = 8)
      .def_property_readonly("exists", &ckpt::SparseChunkReader::exists)
      .def_property_readonly("fast", &ckpt::SparseChunkReader::fast)
      .def_property_readonly("rows", &ckpt::SparseChunkReader::rows)
      .def_property_readonly("dim", [](const ckpt::SparseChunkReader& r) { return r.header().dim; })
      .def_property_readonly("id", [](const ckpt::SparseChunkReader& r) { return r.header().id; })
      .def_property_readonly("name", [](const ckpt::SparseChunkReader& r) { return r.header().name; })
      .def_property_readonly("init_type", [](const ckpt::SparseChunkReader& r) { return r.header().init_type; })
      .def_property_readonly("init_conf", [](const ckpt::SparseChunkReader& r) { return r.header().init_conf; })
      .def_property_readonly("state_types", &ckpt::SparseChunkReader::state_types)
      .def_property_readonly("int_state_types", &ckpt::SparseChunkReader::int_state_types)
      .def("read_into",
           [](ckpt::SparseChunkReader& r, uint64_t lo, uint64_t n, torch::Tensor ids, torch::Tensor vals,
              std::vector<torch::Tensor> states, std::vector<torch::Tensor> states_i) {
             need_cpu(ids, "ids", torch::kInt64);
             need_cpu(vals, "vals", torch::kFloat32);
             const int64_t d = r.header().dim;
             TORCH_CHECK(static_cast<uint64_t>(ids.numel()) >= n && static_cast<uint64_t>(vals.numel()) >= n * d,
                         "read_into: the destination holds fewer than n rows");
             TORCH_CHECK(states.size() == r.state_types().size() && states_i.size() == r.int_state_types().size(),
                         "read_into: one tensor per state column of the file is needed");
             std::vector<float*> sp;
             std::vector<int64_t*> ip;
             for (auto& t : states) {
               need_cpu(t, "state", torch::kFloat32);
               TORCH_CHECK(static_cast<uint64_t>(t.numel()) >= n * d, "read_into: a state column is too small");
               sp.push_back(t.data_ptr<float>());
             }
             for (auto& t : states_i) {
               need_cpu(t, "int state", torch::kInt64);
               TORCH_CHECK(static_cast<uint64_t>(t.numel()) >= n, "read_into: an integer state column is too small");
               ip.push_back(t.data_ptr<int64_t>());
             }
             py::gil_scoped_release nogil;
             return r.Read(lo, n, reinterpret_cast<uint64_t*>(ids.data_ptr<int64_t>()), vals.data_ptr<float>(), sp.data(),
                           ip.data());
           },
           "False: a row deviates from the fixed layout (load the file with ckpt_load_sparse instead)");

  // ---------------- TCP transport of the multi-process deployment (framing, compression, client, server)
  m.def(
      "net_send_frame",
      [](int fd, uint64_t stamp, int32_t code, const std::string& body, uint8_t compress) {
        py::gil_scoped_release nogil;
        return net::SendFrame(fd, stamp, code, body, compress);
      },
      py::arg("fd"), py::arg("stamp"), py::arg("code"), py::arg("body"), py::arg("compress") = 0);
  m.def(
      "net_recv_frame",
      [](int fd, int timeout_ms) -> py::object {
        // (stamp, code, body, compress), or the reason as a string: "closed", "timeout", "bad frame"
        net::Frame f;
        net::RecvStatus st;
        {
          py::gil_scoped_release nogil;
          st = net::RecvFrame(fd, timeout_ms, &f);
        }
        switch (st) {
          case net::RecvStatus::kOk: return py::make_tuple(f.stamp, f.code, py::bytes(f.body), f.compress);
          case net::RecvStatus::kClosed: return py::str("closed");
          case net::RecvStatus::kTimeout: return py::str("timeout");
          default: return py::str("bad frame");
        }
      },
      py::arg("fd"), py::arg("timeout_ms") = -1);
  py::class_<net::Connecter>(m, "NetConnecter")
      .def(py::init<const std::string&, int, int, uint8_t>(), py::arg("host"), py::arg("port"),
           py::arg("timeout_ms") = 5000, py::arg("compress") = 0, py::call_guard<py::gil_scoped_release>())
      .def(
          "call",
          [](net::Connecter& c, uint32_t type, const std::string& body, int timeout_ms) {
            // (0, reply code, reply body), or (kTimeout | kConnection, 0, message) when no reply was had
            std::pair<int32_t, std::string> r;
            int32_t transport = 0;
            {
              py::gil_scoped_release nogil;
              try {
                r = c.Call(type, body, timeout_ms);
              } catch (const KrakenError& e) {
                transport = e.code;
                r = {0, e.what()};
              }
            }
            return py::make_tuple(transport, r.first, py::bytes(r.second));
          },
          py::arg("type"), py::arg("body"), py::arg("timeout_ms") = 0)
      .def("close", &net::Connecter::Close, py::call_guard<py::gil_scoped_release>());
  py::class_<net::Station>(m, "NetStation")
      .def(py::init([](const std::string& host, int port, py::function fn) {
             // the callable is released under the GIL, whichever thread drops the last reference
             auto held = std::shared_ptr<py::function>(new py::function(std::move(fn)), [](py::function* p) {
               py::gil_scoped_acquire g;
               delete p;
             });
             net::Handler h = [held](uint32_t type, const std::string& body) -> std::pair<int32_t, std::string> {
               py::gil_scoped_acquire g;
               try {
                 py::tuple out = (*held)(type, py::bytes(body)).cast<py::tuple>();
                 return {out[0].cast<int32_t>(), out[1].cast<std::string>()};
               } catch (py::error_already_set& e) {
                 return {err::kUnknown, std::string(e.what())};
               }
             };
             return new net::Station(host, port, std::move(h));
           }),
           py::arg("host"), py::arg("port"), py::arg("handler"))
      .def_property_readonly("port", &net::Station::port)
      .def("start", &net::Station::Start)
      .def("stop", &net::Station::Stop, py::call_guard<py::gil_scoped_release>());

  // ---------------- CPU shard
  py::class_<CpuShard>(m, "CpuShard")
      .def(py::init<uint64_t>(), py::arg("seed") = 0)
      .def("init_model", &CpuShard::InitModel)
      .def("model_initialized", &CpuShard::model_initialized)
      .def("meta", &CpuShard::meta)
      .def("has_table", &CpuShard::HasTable)
      .def("create_dense_table",
           [](CpuShard& s, uint64_t id, const std::string& name, const torch::Tensor& val) {
             torch::Tensor v = val.detach().cpu().contiguous().to(torch::kFloat32);
             s.CreateDenseTable(id, name, std::vector<int64_t>(v.sizes().begin(), v.sizes().end()), v.data_ptr<float>());
           })
      .def("create_sparse_table", &CpuShard::CreateSparseTable)
      .def("pull_dense",
           [](CpuShard& s, uint64_t id) {
             torch::Tensor out = torch::empty({s.DenseNumel(id)}, torch::kFloat32);
             {
               py::gil_scoped_release nogil;   // the shard locks per table: other connections' handlers run meanwhile
               s.PullDense(id, out.data_ptr<float>());
             }
             return out;
           })
      .def("push_dense",
           [](CpuShard& s, uint64_t id, const torch::Tensor& grad, float lr) {
             torch::Tensor g = grad.detach().cpu().contiguous().to(torch::kFloat32);
             py::gil_scoped_release nogil;
             s.PushDense(id, g.data_ptr<float>(), g.numel(), lr);
           })
      .def("push_dense_coo",
           [](CpuShard& s, uint64_t id, const torch::Tensor& idx, const torch::Tensor& vals, float lr) {
             torch::Tensor i = idx.detach().cpu().contiguous().to(torch::kInt64).reshape({-1});
             torch::Tensor v = vals.detach().cpu().contiguous().to(torch::kFloat32).reshape({-1});
             TORCH_CHECK(i.numel() == v.numel(), "COO indices and values differ in length");
             py::gil_scoped_release nogil;
             s.PushDenseCoo(id, i.data_ptr<int64_t>(), v.data_ptr<float>(), i.numel(), lr);
           })
      .def("sparse_dim", &CpuShard::SparseDim)
      .def("sparse_size", &CpuShard::SparseSize)
      .def("pull_sparse",
           [](CpuShard& s, uint64_t id, const torch::Tensor& ids) {
             torch::Tensor i = ids.detach().cpu().contiguous().to(torch::kInt64).reshape({-1});
             torch::Tensor out = torch::empty({i.numel(), s.SparseDim(id)}, torch::kFloat32);
             {
               py::gil_scoped_release nogil;
               s.PullSparse(id, reinterpret_cast<const uint64_t*>(i.data_ptr<int64_t>()), i.numel(), out.data_ptr<float>());
             }
             return out;
           })
      .def("push_sparse",
           [](CpuShard& s, uint64_t id, const torch::Tensor& ids, const torch::Tensor& grads, float lr) {
             torch::Tensor i = ids.detach().cpu().contiguous().to(torch::kInt64).reshape({-1});
             torch::Tensor g = grads.detach().cpu().contiguous().to(torch::kFloat32);
             TORCH_CHECK(g.numel() == i.numel() * s.SparseDim(id), "grads must be [n, dim]");
             py::gil_scoped_release nogil;
             return s.PushSparse(id, reinterpret_cast<const uint64_t*>(i.data_ptr<int64_t>()), i.numel(),
                                 g.data_ptr<float>(), lr);
           })
      .def("export_dense", [](CpuShard& s, uint64_t id) { return value_to_py(s.ExportDense(id)); })
      .def("import_dense", [](CpuShard& s, uint64_t id, const std::string& name,
                              const py::dict& v) { s.ImportDense(id, name, value_from_py(v)); })
      .def("export_sparse", [](CpuShard& s, uint64_t id) { return columns_to_py(s.ExportSparse(id)); })
      .def("import_sparse",
           [](CpuShard& s, uint64_t id, const torch::Tensor& ids, const torch::Tensor& vals, const py::dict& states,
              const py::dict& states_i, bool overwrite) {
             s.ImportSparse(id, columns_from_py(s.SparseDim(id), ids, vals, states, states_i), overwrite);
           },
           py::arg("id"), py::arg("ids"), py::arg("vals"), py::arg("states"), py::arg("states_i"),
           py::arg("overwrite") = true)
      .def("contains_sparse",
           [](CpuShard& s, uint64_t id, const torch::Tensor& ids) {
             need_cpu(ids, "ids", torch::kInt64);
             auto out = torch::zeros({ids.numel()}, torch::kUInt8);
             s.ContainsSparse(id, reinterpret_cast<const uint64_t*>(ids.data_ptr<int64_t>()), ids.numel(),
                              out.data_ptr<uint8_t>());
             return out;
           })
      .def("export_sparse_rows",
           [](CpuShard& s, uint64_t id, const torch::Tensor& ids) {
             need_cpu(ids, "ids", torch::kInt64);
             return columns_to_py(s.ExportSparseRows(id, reinterpret_cast<const uint64_t*>(ids.data_ptr<int64_t>()),
                                                     ids.numel()));
           })
      .def("filter_sparse", [](CpuShard& s, uint64_t id, int mode, uint64_t salt, uint32_t world, uint32_t rank,
                               const Router* ring, uint64_t node) {
        return s.FilterSparse(id, make_filter(mode, salt, world, rank, ring, id, node));
      });

  m.def("parse_optim", [](OptimType t, const Conf& c) {
    OptimPOD o = ParseOptim(t, c);
    py::dict d;
    d["type"] = o.type;
    d["has_weight_decay"] = o.has_weight_decay;
    d["weight_decay"] = o.weight_decay;
    d["has_momentum"] = o.has_momentum;
    d["momentum"] = o.momentum;
    d["has_dampening"] = o.has_dampening;
    d["dampening"] = o.dampening;
    d["nesterov"] = o.nesterov;
    d["amsgrad"] = o.amsgrad;
    d["centered"] = o.centered;
    d["beta1"] = o.beta1;
    d["beta2"] = o.beta2;
    d["alpha"] = o.alpha;
    d["eps"] = o.eps;
    d["initial_accumulator_value"] = o.initial_accumulator_value;
    d["slabs"] = std::vector<bool>{o.SlabUsed(0), o.SlabUsed(1), o.SlabUsed(2)};
    d["needs_steps"] = o.NeedsSteps();
    d["slab_state_types"] = std::vector<uint32_t>{SlabStateType(o, 0), SlabStateType(o, 1), SlabStateType(o, 2)};
    return d;
  });
  m.def("parse_init", [](InitializerType t, const Conf& c) {
    InitPOD p = ParseInit(t, c);
    return std::make_tuple(static_cast<int>(p.type), p.a, p.b);
  });

  // ---------------- CPU client-side ops
  // Worker side of the TCP deployment: which ring node owns every (table, id), grouped by node.  Returns
  // (nodes ascending, positions of the ids grouped in that node order, how many per node); with one node
  // the positions are simply 0..n-1.  hash = Mix64(table) ^ Mix64(id), owner = first virtual node at or after
  // it on the ring (kraken/common/router.cc:262-277, kraken/worker/emitter.cc:123-183).
  m.def("route_partition", [](const torch::Tensor& ids, uint64_t table_id, const torch::Tensor& vhash,
                              const torch::Tensor& vnode) {
    need_cpu(ids, "ids", torch::kInt64);
    TORCH_CHECK(vhash.is_contiguous() && vnode.is_contiguous() && vhash.numel() == vnode.numel() && vhash.numel() > 0 &&
                    vhash.element_size() == 8 && vnode.scalar_type() == torch::kInt64,
                "route_partition: the ring is two equally long arrays of 64-bit numbers");
    const int64_t n = ids.numel(), v = vhash.numel();
    const uint64_t* id = reinterpret_cast<const uint64_t*>(ids.data_ptr<int64_t>());
    const uint64_t* vh = reinterpret_cast<const uint64_t*>(vhash.data_ptr());
    const int64_t* vn = vnode.data_ptr<int64_t>();
    const uint64_t salt = Mix64(table_id);
    std::vector<int64_t> owner(static_cast<size_t>(n));
    std::map<int64_t, int64_t> count;
    for (int64_t i = 0; i < n; ++i) {
      const uint64_t h = salt ^ Mix64(id[i]);
      int64_t k = std::lower_bound(vh, vh + v, h) - vh;
      if (k == v) k = 0;
      owner[static_cast<size_t>(i)] = vn[k];
      ++count[vn[k]];
    }
    std::vector<int64_t> nodes, counts;
    std::map<int64_t, int64_t> cursor;
    int64_t at = 0;
    for (auto& kv : count) {
      nodes.push_back(kv.first);
      counts.push_back(kv.second);
      cursor[kv.first] = at;
      at += kv.second;
    }
    torch::Tensor order = torch::empty({n}, torch::kInt64);
    int64_t* o = order.data_ptr<int64_t>();
    if (nodes.size() == 1) {
      for (int64_t i = 0; i < n; ++i) o[i] = i;
    } else {
      for (int64_t i = 0; i < n; ++i) o[cursor[owner[static_cast<size_t>(i)]]++] = i;
    }
    return py::make_tuple(nodes, order, counts);
  });
  m.def("cpu_dedup", [](const torch::Tensor& ids) {
    torch::Tensor i = ids.detach().cpu().contiguous().to(torch::kInt64).reshape({-1});
    std::vector<uint64_t> uniq;
    std::vector<int64_t> inv;
    cpu::Dedup(reinterpret_cast<const uint64_t*>(i.data_ptr<int64_t>()), i.numel(), &uniq, &inv);
    torch::Tensor u = torch::empty({static_cast<int64_t>(uniq.size())}, torch::kInt64);
    if (!uniq.empty()) std::memcpy(u.data_ptr(), uniq.data(), uniq.size() * 8);
    torch::Tensor v = torch::empty({i.numel()}, torch::kInt64);
    if (!inv.empty()) std::memcpy(v.data_ptr(), inv.data(), inv.size() * 8);
    return std::make_pair(u, v);
  });
  m.def("cpu_segment_sum", [](const torch::Tensor& grads, const torch::Tensor& inverse, int64_t num_uniq) {
    torch::Tensor g = grads.detach().cpu().contiguous().to(torch::kFloat32);
    torch::Tensor inv = inverse.detach().cpu().contiguous().to(torch::kInt64);
    const int64_t n = inv.numel();
    const int64_t dim = n ? g.numel() / n : 0;
    torch::Tensor out = torch::zeros({num_uniq, dim}, torch::kFloat32);
    cpu::SegmentSum(g.data_ptr<float>(), inv.data_ptr<int64_t>(), n, dim, num_uniq, out.data_ptr<float>());
    return out;
  });
  m.def("kth_largest_abs", [](const torch::Tensor& x, int64_t k) {
    torch::Tensor v = x.detach().cpu().contiguous().to(torch::kFloat32).reshape({-1});
    return cpu::KthLargestAbs(v.data_ptr<float>(), v.numel(), k);
  });
  py::class_<cpu::DctState>(m, "DctState")
      .def(py::init<>())
      .def_readwrite("tau", &cpu::DctState::tau)
      .def_readwrite("step", &cpu::DctState::step)
      .def("residual", [](const cpu::DctState& s) {
        torch::Tensor t = torch::empty({static_cast<int64_t>(s.e.size())}, torch::kFloat32);
        if (!s.e.empty()) std::memcpy(t.data_ptr(), s.e.data(), s.e.size() * 4);
        return t;
      });
  m.def("cpu_dct_compress",
        [](const torch::Tensor& grad, int64_t life_span, float eta, cpu::DctState& st) -> py::object {
          torch::Tensor g = grad.detach().cpu().contiguous().to(torch::kFloat32).reshape({-1});
          std::vector<int64_t> idx;
          std::vector<float> vals;
          if (!cpu::DctCompress(g.data_ptr<float>(), g.numel(), life_span, eta, &st, &idx, &vals)) return py::none();
          torch::Tensor i = torch::empty({static_cast<int64_t>(idx.size())}, torch::kInt64);
          torch::Tensor v = torch::empty({static_cast<int64_t>(vals.size())}, torch::kFloat32);
          if (!idx.empty()) {
            std::memcpy(i.data_ptr(), idx.data(), idx.size() * 8);
            std::memcpy(v.data_ptr(), vals.data(), vals.size() * 4);
          }
          return py::make_tuple(i, v);
        });

  // ---------------- jagged ops (CPU and CUDA), API of the reference's kraken_native
  auto jagged_fwd = [](const torch::Tensor& values, const torch::Tensor& offsets, float patch_value,
                       const c10::optional<torch::Tensor>& weights, bool mean) {
    TORCH_CHECK(values.dim() >= 1, "values must have at least one dimension");
    torch::Tensor v = values.contiguous().to(torch::kFloat32);
    torch::Tensor o = offsets.contiguous().to(torch::kInt64);
    const int64_t k = o.numel() - 1;
    TORCH_CHECK(k >= 0, "offsets must have at least one element");
    const int64_t R = v.size(0);
    const int64_t dim = R ? v.numel() / R : (v.dim() > 1 ? v.numel() : 1);
    std::vector<int64_t> shape(v.sizes().begin(), v.sizes().end());
    shape[0] = k;
    torch::Tensor out = torch::empty(shape, v.options());
    c10::optional<torch::Tensor> w;
    if (weights.has_value()) w = weights->contiguous().to(torch::kFloat32);
    int64_t d = 1;
    for (size_t i = 1; i < shape.size(); ++i) d *= shape[i];
    (void)dim;
    if (v.is_cuda()) {
      c10::cuda::CUDAGuard guard(v.device());
      TORCH_CHECK(o.is_cuda(), "offsets must live on the same device as values");
      cu::jagged_forward(ptr<float>(v), optr<float>(w), ptr<int64_t>(o), k, d, mean, patch_value, ptr<float>(out),
                         cur_stream());
      check_launch("jagged_forward");
    } else {
      cpu::JaggedForward(ptr<float>(v), optr<float>(w), ptr<int64_t>(o), k, d, mean, patch_value, ptr<float>(out));
    }
    return out;
  };
  auto jagged_bwd = [](const torch::Tensor& offsets, const torch::Tensor& grads,
                       const c10::optional<torch::Tensor>& weights, bool mean) {
    torch::Tensor g = grads.contiguous().to(torch::kFloat32);
    torch::Tensor o = offsets.contiguous().to(torch::kInt64);
    const int64_t k = o.numel() - 1;
    TORCH_CHECK(k >= 0 && g.size(0) == k, "grads must have one row per bag");
    const int64_t R = k > 0 ? o.cpu()[k].item<int64_t>() : 0;
    std::vector<int64_t> shape(g.sizes().begin(), g.sizes().end());
    shape[0] = R;
    torch::Tensor out = torch::zeros(shape, g.options());
    int64_t d = 1;
    for (size_t i = 1; i < shape.size(); ++i) d *= shape[i];
    c10::optional<torch::Tensor> w;
    if (weights.has_value()) w = weights->contiguous().to(torch::kFloat32);
    if (g.is_cuda()) {
      c10::cuda::CUDAGuard guard(g.device());
      TORCH_CHECK(o.is_cuda(), "offsets must live on the same device as grads");
      cu::jagged_backward(ptr<float>(g), optr<float>(w), ptr<int64_t>(o), k, d, mean, ptr<float>(out), cur_stream());
      check_launch("jagged_backward");
    } else {
      cpu::JaggedBackward(ptr<float>(g), optr<float>(w), ptr<int64_t>(o), k, d, mean, ptr<float>(out));
    }
    return out;
  };
  m.def(
      "jagged_sum_forward",
      [jagged_fwd](const torch::Tensor& v, const torch::Tensor& o, float p, const c10::optional<torch::Tensor>& w) {
        return jagged_fwd(v, o, p, w, false);
      },
      py::arg("values"), py::arg("offsets"), py::arg("patch_value"), py::arg("weights") = py::none());
  m.def(
      "jagged_mean_forward",
      [jagged_fwd](const torch::Tensor& v, const torch::Tensor& o, float p, const c10::optional<torch::Tensor>& w) {
        return jagged_fwd(v, o, p, w, true);
      },
      py::arg("values"), py::arg("offsets"), py::arg("patch_value"), py::arg("weights") = py::none());
  m.def(
      "jagged_sum_backward",
      [jagged_bwd](const torch::Tensor& o, const torch::Tensor& g, const c10::optional<torch::Tensor>& w) {
        return jagged_bwd(o, g, w, false);
      },
      py::arg("offsets"), py::arg("grads"), py::arg("weights") = py::none());
  m.def(
      "jagged_mean_backward",
      [jagged_bwd](const torch::Tensor& o, const torch::Tensor& g, const c10::optional<torch::Tensor>& w) {
        return jagged_bwd(o, g, w, true);
      },
      py::arg("offsets"), py::arg("grads"), py::arg("weights") = py::none());

  // ---------------- symmetric heap + device structs
  py::class_<SymHeap>(m, "SymHeap")
      .def(py::init<size_t, int, int, bool>(), py::arg("bytes"), py::arg("rank"), py::arg("world"),
           py::arg("alias_peers") = false)
      .def("handle", &SymHeap::Handle)
      .def("open", &SymHeap::Open)
      .def("close", &SymHeap::Close)
      .def("window", &SymHeap::Window)
      .def_readonly("bytes", &SymHeap::bytes)
      .def_readonly("rank", &SymHeap::rank)
      .def_readonly("world", &SymHeap::world)
      .def("local_ptr", [](const SymHeap& h) { return reinterpret_cast<uintptr_t>(h.local); })
      .def("peer_ptr", [](const SymHeap& h, int p) { return reinterpret_cast<uintptr_t>(h.bases.at(p)); });

  py::class_<cu::ChanLayout>(m, "ChanLayout")
      .def(py::init<>())
      .def_readwrite("inbox_ids", &cu::ChanLayout::inbox_ids)
      .def_readwrite("inbox_meta", &cu::ChanLayout::inbox_meta)
      .def_readwrite("rows_recv", &cu::ChanLayout::rows_recv)
      .def_readwrite("inbox_grad", &cu::ChanLayout::inbox_grad)
      .def_readwrite("flag_req", &cu::ChanLayout::flag_req)
      .def_readwrite("flag_rsp", &cu::ChanLayout::flag_rsp)
      .def_readwrite("flag_push", &cu::ChanLayout::flag_push)
      .def_readwrite("inbox_tcnt", &cu::ChanLayout::inbox_tcnt)
      .def_readwrite("capS", &cu::ChanLayout::capS)
      .def_readwrite("capU", &cu::ChanLayout::capU);

  py::class_<cu::TableHost>(m, "TableHost");
  m.def("make_table", &make_table, py::arg("keys"), py::arg("val"), py::arg("s0"), py::arg("s1"), py::arg("s2"),
        py::arg("steps"), py::arg("lead"), py::arg("size"), py::arg("status"), py::arg("bits"), py::arg("dim"),
        py::arg("init_type"), py::arg("init_a"), py::arg("init_b"), py::arg("seed_key"));

  py::class_<OptimPOD>(m, "OptimPOD");
  m.def("make_optim", [](OptimType t, const Conf& c) { return ParseOptim(t, c); });

  // ---------------- sparse kernels
  m.def("dedup_bucketize", [](const torch::Tensor& ids, int world, uint64_t salt, const torch::Tensor& hkeys,
                              const torch::Tensor& slot_of, uint32_t hbits, const torch::Tensor& cnt, const torch::Tensor& off,
                              const torch::Tensor& uniq, const torch::Tensor& inv, const torch::Tensor& status,
                              int cap_u, const SymHeap* heap, const cu::ChanLayout* lay,
                              const c10::optional<torch::Tensor>& ctrl, int owner_world) {
    if (owner_world <= 0 || owner_world > world) owner_world = world;
    need_cuda(ids, "ids", torch::kInt64);
    need_cuda(hkeys, "hkeys", torch::kInt64);
    const int n = static_cast<int>(ids.numel());
    TORCH_CHECK(hkeys.dim() == 2 && hkeys.size(0) == (1ll << hbits) && hkeys.size(1) == 2 && hkeys.is_contiguous() &&
                    (1ll << hbits) >= 2ll * n,
                "dedup scratch must be a contiguous int64 [1 << hbits, 2] tensor with at least 2 n slots");
    if (cap_u <= 0) cap_u = static_cast<int>(uniq.numel());
    TORCH_CHECK(slot_of.numel() >= n && inv.numel() >= n && uniq.numel() >= cap_u, "dedup outputs too small");
    TORCH_CHECK(cnt.numel() >= world && off.numel() >= world + 1, "cnt/off too small");
    c10::cuda::CUDAGuard guard(ids.device());
    cu::DedupScratch sc{hkeys.data_ptr(), ptr<int>(slot_of), hbits};
    if (heap != nullptr && lay != nullptr && ctrl.has_value()) {
      // with a channel: the dedup's second kernel also dispatches the unique ids to their owners
      cu::dedup_bucketize_dispatch(ptr<int64_t>(ids), n, world, owner_world, salt, sc, ptr<int>(cnt), ptr<int>(off),
                                   ptr<int64_t>(uniq), ptr<int>(inv), cap_u, ptr<int>(status), heap->View(), *lay,
                                   ctrl_ptr(*ctrl), cur_stream());
    } else {
      cu::dedup_bucketize(ptr<int64_t>(ids), n, world, owner_world, salt, sc, ptr<int>(cnt), ptr<int>(off), ptr<int64_t>(uniq),
                          ptr<int>(inv), cap_u, ptr<int>(status), cur_stream());
    }
    check_launch("dedup_bucketize");
  }, py::arg("ids"), py::arg("world"), py::arg("salt"), py::arg("hkeys"), py::arg("slot_of"), py::arg("hbits"), py::arg("cnt"), py::arg("off"), py::arg("uniq"), py::arg("inv"),
     py::arg("status"), py::arg("cap_u") = 0, py::arg("heap") = nullptr, py::arg("layout") = nullptr,
     py::arg("ctrl") = py::none(), py::arg("owner_world") = 0);
  m.def("pull_dispatch", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                            const torch::Tensor& uniq, const torch::Tensor& off, int max_n) {
    cu::pull_dispatch(h.View(), lay, ctrl_ptr(ctrl), ptr<int64_t>(uniq), ptr<int>(off),
                      max_n, cur_stream());
    check_launch("pull_dispatch");
  });
  m.def("pull_probe", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                         const cu::TableHost& table, const torch::Tensor& slot_cache, bool insert, uint32_t spin) {
    cu::pull_probe(h.View(), lay, ctrl_ptr(ctrl), table, ptr<int>(slot_cache), insert,
                   spin, cur_stream());
    check_launch("pull_probe");
  });
  m.def("pull_gather", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                          const cu::TableHost& table, const torch::Tensor& slot_cache) {
    cu::pull_gather(h.View(), lay, ctrl_ptr(ctrl), table, ptr<int>(slot_cache),
                    cur_stream());
    check_launch("pull_gather");
  });
  m.def("pull_combine",
        [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl, const torch::Tensor& inv, int n,
           int dim, const c10::optional<torch::Tensor>& bag_offsets, const c10::optional<torch::Tensor>& weights,
           bool mean, const c10::optional<torch::Tensor>& bag_mean, float patch_value, const torch::Tensor& out,
           uint32_t spin) {
          const int k = bag_offsets.has_value() ? static_cast<int>(bag_offsets->numel()) - 1 : 0;
          need_cuda(out, "out", torch::kFloat32);
          TORCH_CHECK(out.numel() == static_cast<int64_t>(bag_offsets.has_value() ? k : n) * dim, "out has the wrong size");
          cu::pull_combine(h.View(), lay, ctrl_ptr(ctrl), ptr<int>(inv), n, dim,
                           optr<int64_t>(bag_offsets), k, optr<float>(weights), mean, optr<uint8_t>(bag_mean),
                           patch_value, ptr<float>(out), spin, cur_stream());
          check_launch("pull_combine");
        });
  m.def("push_scatter",
        [](const torch::Tensor& grads, const torch::Tensor& inv, int n, int dim,
           const c10::optional<torch::Tensor>& bag_offsets, const c10::optional<torch::Tensor>& weights, bool mean,
           const c10::optional<torch::Tensor>& bag_mean, const torch::Tensor& ugrad) {
          need_cuda(grads, "grads", torch::kFloat32);
          const int k = bag_offsets.has_value() ? static_cast<int>(bag_offsets->numel()) - 1 : 0;
          TORCH_CHECK(grads.numel() == static_cast<int64_t>(bag_offsets.has_value() ? k : n) * dim,
                      "grads has the wrong size");
          cu::push_scatter(ptr<float>(grads), ptr<int>(inv), n, dim, optr<int64_t>(bag_offsets), k, optr<float>(weights),
                           mean, optr<uint8_t>(bag_mean), ptr<float>(ugrad), cur_stream());
          check_launch("push_scatter");
        });
  m.def("push_dispatch", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                            const torch::Tensor& ugrad, const torch::Tensor& off, int max_n, int dim) {
    cu::push_dispatch(h.View(), lay, ctrl_ptr(ctrl), ptr<float>(ugrad), ptr<int>(off),
                      max_n, dim, cur_stream());
    check_launch("push_dispatch");
  });
  m.def("push_apply", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                         const cu::TableHost& table, const torch::Tensor& slot_cache, const OptimPOD& optim,
                         const torch::Tensor& lr, uint32_t spin) {
    need_cuda(lr, "lr", torch::kFloat32);
    cu::push_apply(h.View(), lay, ctrl_ptr(ctrl), table, ptr<int>(slot_cache), optim,
                   ptr<float>(lr), spin, cur_stream());
    check_launch("push_apply");
  });

  // ---------------- one exchange for several tables of one row width
  m.def("group_table_views", [](const std::vector<cu::TableHost>& tables) {
    // the tables' device-side descriptors as one CPU byte tensor; the caller copies it to the device
    const int T = static_cast<int>(tables.size());
    auto out = torch::zeros({static_cast<int64_t>(T * cu::group_table_view_bytes())}, torch::kUInt8);
    cu::group_table_views(tables.data(), T, out.data_ptr());
    return out;
  });
  m.def("group_dedup_dispatch",
        [](const torch::Tensor& ids, const torch::Tensor& occ_start, const torch::Tensor& region_base,
           const torch::Tensor& region_bits, const torch::Tensor& salts, int world, const torch::Tensor& hkeys,
           const torch::Tensor& slot_of, const torch::Tensor& cnt, const torch::Tensor& off, const torch::Tensor& uniq,
           const torch::Tensor& inv, const torch::Tensor& status, int cap_u, const SymHeap& heap,
           const cu::ChanLayout& lay, const torch::Tensor& ctrl, int owner_world) {
          if (owner_world <= 0 || owner_world > world) owner_world = world;
          need_cuda(ids, "ids", torch::kInt64);
          need_cuda(occ_start, "occ_start", torch::kInt32);
          need_cuda(region_base, "region_base", torch::kInt32);
          need_cuda(region_bits, "region_bits", torch::kInt32);
          need_cuda(salts, "salts", torch::kInt64);
          need_cuda(hkeys, "hkeys", torch::kInt64);
          const int T = static_cast<int>(region_base.numel());
          const int n = static_cast<int>(ids.numel());
          TORCH_CHECK(T >= 1 && T <= 4096 && occ_start.numel() == T + 1 && region_bits.numel() == T && salts.numel() == T,
                      "group descriptors differ in length");
          TORCH_CHECK(static_cast<size_t>(4) * (T + 1 + 2 * world * T + 256) <= 48 * 1024,
                      "too many tables in one group for the kernels' shared memory");
          TORCH_CHECK(slot_of.numel() >= n && inv.numel() >= n && cnt.numel() >= static_cast<int64_t>(world) * T &&
                          off.numel() >= world + 1 && uniq.numel() >= cap_u,
                      "group dedup buffers too small");
          c10::cuda::CUDAGuard guard(ids.device());
          cu::GroupDesc d{T, owner_world, ptr<int>(occ_start), ptr<int>(region_base), ptr<int>(region_bits),
                          reinterpret_cast<const unsigned long long*>(salts.data_ptr())};
          cu::DedupScratch sc{hkeys.data_ptr(), ptr<int>(slot_of), 0};
          cu::group_dedup_dispatch(ptr<int64_t>(ids), n, d, world, sc, ptr<int>(cnt), ptr<int>(off), ptr<int64_t>(uniq),
                                   ptr<int>(inv), cap_u, ptr<int>(status), heap.View(), lay, ctrl_ptr(ctrl), cur_stream());
          check_launch("group_dedup_dispatch");
        });
  m.def("group_probe", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                          const torch::Tensor& table_views, int T, int dim, const torch::Tensor& snap_t,
                          const torch::Tensor& slot_cache, const torch::Tensor& ttab, bool insert, uint32_t spin) {
    need_cuda(table_views, "table_views", torch::kUInt8);
    need_cuda(snap_t, "snap_t", torch::kInt32);
    need_cuda(ttab, "ttab", torch::kInt16);
    TORCH_CHECK(table_views.numel() >= static_cast<int64_t>(T * cu::group_table_view_bytes()), "table_views too small");
    TORCH_CHECK(snap_t.numel() >= static_cast<int64_t>(h.world) * (T + 1), "snap_t too small");
    cu::group_probe(h.View(), lay, ctrl_ptr(ctrl), table_views.data_ptr(), T, dim, ptr<int>(snap_t), ptr<int>(slot_cache),
                    ptr<int16_t>(ttab), insert, spin, cur_stream());
    check_launch("group_probe");
  });
  m.def("group_gather", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                           const torch::Tensor& table_views, int dim, const torch::Tensor& slot_cache,
                           const torch::Tensor& ttab) {
    cu::group_gather(h.View(), lay, ctrl_ptr(ctrl), table_views.data_ptr(), dim, ptr<int>(slot_cache), ptr<int16_t>(ttab),
                     cur_stream());
    check_launch("group_gather");
  });
  m.def("group_push_apply", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl,
                               const torch::Tensor& table_views, int dim, const torch::Tensor& slot_cache,
                               const torch::Tensor& ttab, const OptimPOD& optim, const torch::Tensor& lr, uint32_t spin) {
    need_cuda(lr, "lr", torch::kFloat32);
    cu::group_push_apply(h.View(), lay, ctrl_ptr(ctrl), table_views.data_ptr(), dim, ptr<int>(slot_cache),
                         ptr<int16_t>(ttab), optim, ptr<float>(lr), spin, cur_stream());
    check_launch("group_push_apply");
  });

  // ---------------- fused DeepFM front end
  m.def("pull_wait", [](const SymHeap& h, const cu::ChanLayout& lay, const torch::Tensor& ctrl, uint32_t spin) {
    cu::pull_wait(h.View(), lay, ctrl_ptr(ctrl), spin, cur_stream());
    check_launch("pull_wait");
  });
  m.def("deepfm_pack_forward",
        [](const torch::Tensor& rows2, const torch::Tensor& inv2, const c10::optional<torch::Tensor>& rows1,
           const c10::optional<torch::Tensor>& inv1, const torch::Tensor& dense, int B, int F, int D,
           const torch::Tensor& x, const torch::Tensor& fm_logit, const c10::optional<torch::Tensor>& slots2,
           const c10::optional<torch::Tensor>& slots1, const c10::optional<torch::Tensor>& ssum) {
          need_cuda(rows2, "rows2", torch::kFloat32);
          need_cuda(dense, "dense", torch::kFloat32);
          need_cuda(x, "x", torch::kBFloat16);
          need_cuda(fm_logit, "fm_logit", torch::kFloat32);
          const int RD = rows2.size(1), ND = dense.size(1), ldx = x.size(1);
          TORCH_CHECK(D % 4 == 0 && RD % 4 == 0 && RD >= D, "row widths must be multiples of 4");
          TORCH_CHECK(((D / 4) & (D / 4 - 1)) == 0 && D <= 128, "D / 4 must be a power of two, D <= 128");
          if (ssum.has_value()) {
            need_cuda(*ssum, "ssum", torch::kFloat32);
            TORCH_CHECK(ssum->numel() == static_cast<int64_t>(B) * D, "ssum must be [B, D]");
          }
          if (rows1.has_value()) {
            need_cuda(*rows1, "rows1", torch::kFloat32);
            TORCH_CHECK(rows1->size(1) == 1 && inv1.has_value() && inv1->numel() >= static_cast<int64_t>(B) * F,
                        "first-order table must have dim 1 and its own occurrence map");
          } else {
            TORCH_CHECK(RD >= D + 1, "folded layout needs a column for the first-order weight");
          }
          TORCH_CHECK(inv2.numel() >= static_cast<int64_t>(B) * F, "occurrence map too small");
          TORCH_CHECK(x.size(0) == B && ldx >= F * D + ND && ldx % 4 == 0 && dense.size(0) == B && fm_logit.numel() == B,
                      "deepfm_pack_forward: shape mismatch");
          cu::deepfm_pack_forward(ptr<float>(rows2), ptr<int>(inv2), optr<int>(slots2), optr<float>(rows1), optr<int>(inv1),
                                  optr<int>(slots1), ptr<float>(dense), B, F, D, RD, ND, reinterpret_cast<__nv_bfloat16*>(x.data_ptr()), ldx,
                                  ptr<float>(fm_logit), optr<float>(ssum), cur_stream());
          check_launch("deepfm_pack_forward");
        },
        py::arg("rows2"), py::arg("inv2"), py::arg("rows1"), py::arg("inv1"), py::arg("dense"), py::arg("B"), py::arg("F"),
        py::arg("D"), py::arg("x"), py::arg("fm_logit"), py::arg("slots2") = py::none(), py::arg("slots1") = py::none(),
        py::arg("ssum") = py::none());
  m.def("deepfm_pack_backward",
        [](const torch::Tensor& rows2, const torch::Tensor& inv2, const c10::optional<torch::Tensor>& inv1,
           const c10::optional<torch::Tensor>& dx, const torch::Tensor& dlogit, int B, int F, int D,
           const torch::Tensor& ugrad2, const c10::optional<torch::Tensor>& ugrad1,
           const c10::optional<torch::Tensor>& slots2, const torch::Tensor& ssum) {
          need_cuda(rows2, "rows2", torch::kFloat32);
          need_cuda(ssum, "ssum", torch::kFloat32);
          TORCH_CHECK(ssum.numel() == static_cast<int64_t>(B) * D && ((D / 4) & (D / 4 - 1)) == 0 && D <= 128,
                      "ssum must be [B, D] with D / 4 a power of two");
          need_cuda(dlogit, "dlogit", torch::kFloat32);
          need_cuda(ugrad2, "ugrad2", torch::kFloat32);
          const int RD = rows2.size(1);
          TORCH_CHECK(ugrad2.size(1) == RD && D % 4 == 0 && RD % 4 == 0, "gradient buffer must match the row width");
          if (ugrad1.has_value()) {
            need_cuda(*ugrad1, "ugrad1", torch::kFloat32);
            TORCH_CHECK(inv1.has_value(), "separate first-order table needs its occurrence map");
          } else {
            TORCH_CHECK(RD >= D + 1, "folded layout needs a column for the first-order weight");
          }
          const __nv_bfloat16* dxp = nullptr;
          int lddx = 0;
          if (dx.has_value()) {
            need_cuda(*dx, "dx", torch::kBFloat16);
            TORCH_CHECK(dx->size(0) == B && dx->size(1) >= F * D && dx->size(1) % 4 == 0, "dx has the wrong shape");
            dxp = reinterpret_cast<const __nv_bfloat16*>(dx->data_ptr());
            lddx = dx->size(1);
          }
          TORCH_CHECK(dlogit.numel() == B, "deepfm_pack_backward: shape mismatch");
          cu::deepfm_pack_backward(ptr<float>(rows2), ptr<int>(inv2), optr<int>(slots2), optr<int>(inv1), dxp, lddx,
                                   ptr<float>(dlogit), ptr<float>(ssum), B, F, D, RD, ptr<float>(ugrad2),
                                   optr<float>(ugrad1), cur_stream());
          check_launch("deepfm_pack_backward");
        },
        py::arg("rows2"), py::arg("inv2"), py::arg("inv1"), py::arg("dx"), py::arg("dlogit"), py::arg("B"), py::arg("F"),
        py::arg("D"), py::arg("ugrad2"), py::arg("ugrad1"), py::arg("slots2"), py::arg("ssum"));

  m.def("owner_of_cuda", [](const torch::Tensor& ids, uint64_t salt, int world) {
    need_cuda(ids, "ids", torch::kInt64);
    torch::Tensor out = torch::empty({ids.numel()}, ids.options().dtype(torch::kInt32));
    cu::owner_of(ptr<int64_t>(ids), static_cast<int>(ids.numel()), salt, world, ptr<int>(out), cur_stream());
    check_launch("owner_of");
    return out;
  });

  // ---------------- table maintenance
  m.def("table_clear", [](const cu::TableHost& t) {
    cu::table_clear(t, cur_stream());
    check_launch("table_clear");
  });
  m.def("table_import", [](const cu::TableHost& t, const torch::Tensor& ids, const torch::Tensor& vals,
                           const c10::optional<torch::Tensor>& s0, const c10::optional<torch::Tensor>& s1,
                           const c10::optional<torch::Tensor>& s2, const c10::optional<torch::Tensor>& steps) {
    need_cuda(ids, "ids", torch::kInt64);
    need_cuda(vals, "vals", torch::kFloat32);
    TORCH_CHECK(vals.numel() == ids.numel() * t.dim, "vals must be [n, dim]");
    cu::table_import(t, ptr<int64_t>(ids), ptr<float>(vals), optr<float>(s0), optr<float>(s1), optr<float>(s2),
                     optr<int>(steps), static_cast<int>(ids.numel()), cur_stream());
    check_launch("table_import");
  });
  m.def("table_lookup", [](const cu::TableHost& t, const torch::Tensor& ids) {
    need_cuda(ids, "ids", torch::kInt64);
    torch::Tensor rows = torch::empty({ids.numel(), t.dim}, ids.options().dtype(torch::kFloat32));
    torch::Tensor found = torch::empty({ids.numel()}, ids.options().dtype(torch::kUInt8));
    cu::table_lookup(t, ptr<int64_t>(ids), static_cast<int>(ids.numel()), ptr<float>(rows), ptr<uint8_t>(found),
                     cur_stream());
    check_launch("table_lookup");
    return std::make_pair(rows, found);
  });
  m.def("table_export",
        [](const cu::TableHost& t, int filter_mode, uint64_t salt, int world, int rank, int min_steps,
           const c10::optional<torch::Tensor>& out_ids, const c10::optional<torch::Tensor>& out_vals,
           const c10::optional<torch::Tensor>& s0, const c10::optional<torch::Tensor>& s1,
           const c10::optional<torch::Tensor>& s2, const c10::optional<torch::Tensor>& steps,
           const torch::Tensor& out_count) {
          const int cap = out_ids.has_value() ? static_cast<int>(out_ids->numel()) : 0;
          cu::table_export(t, filter_mode, salt, world, rank, min_steps, optr<int64_t>(out_ids), optr<float>(out_vals),
                           optr<float>(s0), optr<float>(s1), optr<float>(s2), optr<int>(steps), ptr<int>(out_count), cap,
                           cur_stream());
          check_launch("table_export");
        });

  // ---------------- model kernels
  m.def("fm_forward", [](const torch::Tensor& emb) {
    need_cuda(emb, "emb", torch::kFloat32);
    TORCH_CHECK(emb.dim() == 3, "emb must be [B, F, D]");
    c10::cuda::CUDAGuard guard(emb.device());
    torch::Tensor out = torch::empty({emb.size(0)}, emb.options());
    cu::fm_forward(ptr<float>(emb), emb.size(0), emb.size(1), emb.size(2), ptr<float>(out), cur_stream());
    check_launch("fm_forward");
    return out;
  });
  m.def("fm_backward", [](const torch::Tensor& emb, const torch::Tensor& gout) {
    need_cuda(emb, "emb", torch::kFloat32);
    need_cuda(gout, "gout", torch::kFloat32);
    c10::cuda::CUDAGuard guard(emb.device());
    torch::Tensor g = torch::empty_like(emb);
    cu::fm_backward(ptr<float>(emb), ptr<float>(gout), emb.size(0), emb.size(1), emb.size(2), ptr<float>(g), cur_stream());
    check_launch("fm_backward");
    return g;
  });
  m.def("bce_with_logits", [](const torch::Tensor& logits, const torch::Tensor& labels, bool want_grad) {
    need_cuda(logits, "logits", torch::kFloat32);
    need_cuda(labels, "labels", torch::kFloat32);
    TORCH_CHECK(logits.numel() == labels.numel(), "logits and labels differ in size");
    c10::cuda::CUDAGuard guard(logits.device());
    torch::Tensor loss = torch::zeros({}, logits.options());
    torch::Tensor grad = want_grad ? torch::empty_like(logits) : torch::Tensor();
    cu::bce_forward_backward(ptr<float>(logits), ptr<float>(labels), static_cast<int>(logits.numel()), ptr<float>(loss),
                             want_grad ? ptr<float>(grad) : nullptr, cur_stream());
    check_launch("bce_with_logits");
    return std::make_pair(loss, grad);
  });

  bind_dense(m);
}
