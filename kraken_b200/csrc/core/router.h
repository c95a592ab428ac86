// Consistent-hash ring that places tables and sparse rows on shards.
//
// On the GPU data path rows are placed by OwnerOf() (hash.h), which is a plain
// modulo; the ring exists for what has to interoperate with reference
// checkpoints: `router.binary`, resharding loads and the CPU socket backend.
// Behaviour matched (kraken/common/router.cc:12-277): three virtual nodes per
// shard, vnode hash = std::hash<std::string>(name + "#" + i) with a random
// re-probe on collision, strictly increasing node ids, lookup by lower_bound
// with wrap-around, version bumped by every Add/Remove.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_set>
#include <vector>

#include "serialize.h"

namespace kb {

class Router {
 public:
  struct Range {  // (start, end]
    uint64_t start;
    uint64_t end;
  };
  struct Node {
    uint64_t id;
    std::string name;
    std::vector<uint64_t> vnodes;
  };
  struct VNode {
    uint64_t hash_v;
    uint64_t node_id;
    std::string name;
  };

  static constexpr size_t kVirtualNodes = 3;

  bool Add(uint64_t id, const std::string& name);
  bool Remove(uint64_t id);
  bool Empty() const { return nodes_.empty(); }
  bool Contains(uint64_t id) const { return FindNode(id) != nullptr; }
  uint64_t version() const { return version_; }
  const std::vector<Node>& nodes() const { return nodes_; }
  const std::vector<VNode>& ring() const { return ring_; }

  // Owner of hash value hv; uint64(-1) on an empty ring.
  uint64_t Hit(uint64_t hv) const;
  std::vector<Range> NodeHashRanges(uint64_t id) const;
  std::unordered_set<uint64_t> IntersectNodes(const Range& r) const;

  bool operator==(const Router& o) const;
  bool operator!=(const Router& o) const { return !(*this == o); }
  std::string Str() const;

  void Save(Writer* w) const;
  static Router Load(Reader* r);

  // Ring of `world` shards named "rank<r>": what GPU shards write into router.binary.
  static Router ForRanks(uint32_t world);

 private:
  const Node* FindNode(uint64_t id) const;
  const VNode* FindVNode(uint64_t hash_v) const;

  uint64_t version_ = 0;
  std::vector<Node> nodes_;  // ascending id
  std::vector<VNode> ring_;  // ascending hash_v
};

}  // namespace kb
