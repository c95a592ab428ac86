#include "router.h"

#include <algorithm>
#include <functional>
#include <limits>
#include <random>
#include <sstream>

namespace kb {

namespace {
uint64_t RandomStep(uint64_t hi) {
  static thread_local std::mt19937_64 rng(0x6b72616b656eull);
  if (hi <= 1) return 1;
  return 1 + rng() % (hi - 1);
}
}  // namespace

const Router::Node* Router::FindNode(uint64_t id) const {
  auto it = std::lower_bound(nodes_.begin(), nodes_.end(), id,
                             [](const Node& n, uint64_t v) { return n.id < v; });
  return (it != nodes_.end() && it->id == id) ? &*it : nullptr;
}

const Router::VNode* Router::FindVNode(uint64_t hash_v) const {
  auto it = std::lower_bound(ring_.begin(), ring_.end(), hash_v,
                             [](const VNode& n, uint64_t v) { return n.hash_v < v; });
  return (it != ring_.end() && it->hash_v == hash_v) ? &*it : nullptr;
}

bool Router::Add(uint64_t id, const std::string& name) {
  if (!nodes_.empty() && nodes_.back().id >= id) return false;

  const uint64_t kMax = std::numeric_limits<uint64_t>::max();
  const uint64_t interval = ring_.empty() ? kMax : kMax / ring_.size();

  Node node{id, name, {}};
  for (size_t i = 0; i < kVirtualNodes; ++i) {
    std::string vname = name + "#" + std::to_string(i);
    uint64_t hv = static_cast<uint64_t>(std::hash<std::string>{}(vname));
    while (FindVNode(hv) != nullptr ||
           std::find(node.vnodes.begin(), node.vnodes.end(), hv) != node.vnodes.end()) {
      hv += RandomStep(interval);  // wrap-around is fine
    }
    node.vnodes.push_back(hv);
    ring_.push_back(VNode{hv, id, vname});
    std::sort(ring_.begin(), ring_.end(), [](const VNode& a, const VNode& b) { return a.hash_v < b.hash_v; });
  }
  nodes_.push_back(std::move(node));
  ++version_;
  return true;
}

bool Router::Remove(uint64_t id) {
  if (FindNode(id) == nullptr) return false;
  ring_.erase(std::remove_if(ring_.begin(), ring_.end(), [id](const VNode& v) { return v.node_id == id; }),
              ring_.end());
  nodes_.erase(std::remove_if(nodes_.begin(), nodes_.end(), [id](const Node& n) { return n.id == id; }),
               nodes_.end());
  ++version_;
  return true;
}

uint64_t Router::Hit(uint64_t hv) const {
  if (ring_.empty()) return std::numeric_limits<uint64_t>::max();
  auto it = std::lower_bound(ring_.begin(), ring_.end(), hv,
                             [](const VNode& n, uint64_t v) { return n.hash_v < v; });
  return it == ring_.end() ? ring_.front().node_id : it->node_id;
}

std::vector<Router::Range> Router::NodeHashRanges(uint64_t id) const {
  std::vector<Range> out;
  const Node* node = FindNode(id);
  if (!node) return out;
  for (uint64_t hv : node->vnodes) {
    const VNode* v = FindVNode(hv);
    if (!v) continue;
    if (v == &ring_.front()) {
      // The first ring entry also owns everything past the last one.
      out.push_back({0, v->hash_v});
      out.push_back({0, 0});
      out.push_back({ring_.back().hash_v, std::numeric_limits<uint64_t>::max()});
    } else {
      out.push_back({(v - 1)->hash_v, v->hash_v});
    }
  }
  return out;
}

std::unordered_set<uint64_t> Router::IntersectNodes(const Range& r) const {
  std::unordered_set<uint64_t> ids;
  for (const auto& n : nodes_) {
    for (const auto& o : NodeHashRanges(n.id)) {
      if (r.start < o.end && r.end > o.start) ids.insert(n.id);
    }
  }
  return ids;
}

bool Router::operator==(const Router& o) const {
  if (version_ != o.version_ || nodes_.size() != o.nodes_.size() || ring_.size() != o.ring_.size()) return false;
  for (size_t i = 0; i < nodes_.size(); ++i) {
    if (nodes_[i].id != o.nodes_[i].id || nodes_[i].name != o.nodes_[i].name ||
        nodes_[i].vnodes != o.nodes_[i].vnodes)
      return false;
  }
  for (size_t i = 0; i < ring_.size(); ++i) {
    if (ring_[i].hash_v != o.ring_[i].hash_v || ring_[i].node_id != o.ring_[i].node_id ||
        ring_[i].name != o.ring_[i].name)
      return false;
  }
  return true;
}

std::string Router::Str() const {
  std::ostringstream s;
  s << "Version:" << version_ << ", Nodes:[";
  for (const auto& n : nodes_) {
    s << "id:" << n.id << ", name:" << n.name << ", vnode_list:";
    for (auto v : n.vnodes) s << v << ", ";
  }
  s << "], Ring:[";
  for (const auto& v : ring_) s << v.node_id << ", ";
  s << "]";
  return s.str();
}

void Router::Save(Writer* w) const {
  w->Pod<uint64_t>(version_);
  w->Pod<uint64_t>(nodes_.size());
  for (const auto& n : nodes_) {
    w->Pod<uint64_t>(n.id);
    w->Str(n.name);
    w->Vec(n.vnodes);
  }
  w->Pod<uint64_t>(ring_.size());
  for (const auto& v : ring_) {
    w->Pod<uint64_t>(v.hash_v);
    w->Pod<uint64_t>(v.node_id);
    w->Str(v.name);
  }
}

Router Router::Load(Reader* r) {
  Router out;
  out.version_ = r->Pod<uint64_t>();
  uint64_t nn = r->Pod<uint64_t>();
  KB_CHECK(nn < (1u << 20), err::kDeserializeReply, "implausible node count");
  for (uint64_t i = 0; i < nn; ++i) {
    Node n;
    n.id = r->Pod<uint64_t>();
    n.name = r->Str();
    n.vnodes = r->Vec<uint64_t>();
    out.nodes_.push_back(std::move(n));
  }
  uint64_t nv = r->Pod<uint64_t>();
  KB_CHECK(nv < (1u << 24), err::kDeserializeReply, "implausible vnode count");
  for (uint64_t i = 0; i < nv; ++i) {
    VNode v;
    v.hash_v = r->Pod<uint64_t>();
    v.node_id = r->Pod<uint64_t>();
    v.name = r->Str();
    out.ring_.push_back(std::move(v));
  }
  return out;
}

Router Router::ForRanks(uint32_t world) {
  Router r;
  for (uint32_t i = 0; i < world; ++i) r.Add(i, "rank" + std::to_string(i));
  return r;
}

}  // namespace kb
