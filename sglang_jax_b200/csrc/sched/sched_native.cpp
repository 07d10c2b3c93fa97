// Host-side scheduler structures that sit on the per-step critical path: the paged KV slot
// allocator and the radix-tree prefix index.  Python keeps the policy (what to insert, when to
// evict); the token comparisons, node splits, LRU eviction and free-list bookkeeping run here.
//
// Semantics mirror `mem_cache/allocator.py: PagedTokenToKVPoolAllocator` and
// `mem_cache/radix_cache.py: RadixCache` (keys namespaced, page-granular matching and splitting,
// unlocked leaves evicted least-recently-used first).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <thread>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <queue>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace py = pybind11;
using i32arr = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;
using i64arr = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

// ------------------------------------------------------------------------------------ allocator
class PagedAllocator {
 public:
  PagedAllocator(int64_t size, int page_size) : page_(page_size), num_pages_(size / page_size) { clear(); }

  void clear() {
    free_.clear();
    for (int32_t p = 1; p <= num_pages_; ++p) free_.push_back(p);
    in_group_ = false;
    group_.clear();
  }
  int64_t available_size() const { return (int64_t)free_.size() * page_; }
  int64_t num_free_pages() const { return (int64_t)free_.size(); }

  py::object alloc(int64_t need) {
    if (need % page_) throw std::invalid_argument("paged alloc() needs a page-aligned size");
    int64_t n = need / page_;
    if (n > (int64_t)free_.size()) return py::none();
    i32arr out(need);
    int32_t* o = out.mutable_data();
    for (int64_t i = 0; i < n; ++i) {
      int32_t p = free_.front();
      free_.pop_front();
      for (int r = 0; r < page_; ++r) *o++ = p * page_ + r;
    }
    return out;
  }

  // Slots for tokens prefix_len..seq_len of each request; `last_loc[i]` is the slot of the last
  // prefix token (or -1): rows left in that page are used before new pages are taken.
  py::object alloc_extend(i64arr prefix_lens, i64arr seq_lens, i64arr last_loc, int64_t extend_num_tokens) {
    const int64_t B = prefix_lens.size();
    const int64_t *pre = prefix_lens.data(), *seq = seq_lens.data(), *last = last_loc.data();
    int64_t need = 0, total = 0;
    for (int64_t i = 0; i < B; ++i) {
      int64_t ext = seq[i] - pre[i];
      int64_t room = pre[i] % page_ == 0 ? 0 : page_ - pre[i] % page_;
      int64_t in_old = std::min(room, ext);
      need += (ext - in_old + page_ - 1) / page_;
      total += ext;
    }
    if (total != extend_num_tokens) throw std::invalid_argument("extend_num_tokens does not match the lengths");
    if (need > (int64_t)free_.size()) return py::none();
    i32arr out(total);
    int32_t* o = out.mutable_data();
    for (int64_t i = 0; i < B; ++i) {
      int64_t ext = seq[i] - pre[i];
      if (ext == 0) continue;
      int64_t room = pre[i] % page_ == 0 ? 0 : page_ - pre[i] % page_;
      int64_t in_old = std::min(room, ext);
      for (int64_t j = 0; j < in_old; ++j) *o++ = (int32_t)(last[i] + 1 + j);
      int64_t rest = ext - in_old;
      while (rest > 0) {
        int32_t p = free_.front();
        free_.pop_front();
        for (int r = 0; r < page_ && rest > 0; ++r, --rest) *o++ = p * page_ + r;
      }
    }
    return out;
  }

  // One slot per request for token index seq_len - 1.
  py::object alloc_decode(i64arr seq_lens, i64arr last_loc) {
    const int64_t B = seq_lens.size();
    const int64_t *seq = seq_lens.data(), *last = last_loc.data();
    int64_t need = 0;
    for (int64_t i = 0; i < B; ++i) need += ((seq[i] - 1) % page_ == 0);
    if (need > (int64_t)free_.size()) return py::none();
    i32arr out(B);
    int32_t* o = out.mutable_data();
    for (int64_t i = 0; i < B; ++i) {
      if ((seq[i] - 1) % page_ == 0) {
        o[i] = free_.front() * page_;
        free_.pop_front();
      } else {
        o[i] = (int32_t)(last[i] + 1);
      }
    }
    return out;
  }

  // One decode step's batch metadata in one call (the per-request Python loops of the scheduler's hot path):
  // for every row r with `kv_lens[i]` committed tokens, take the slot of token `kv_lens[i]` (the next slot of the
  // row's last page, or the first slot of a fresh page when that page is full), write it into the request ->
  // slot table, and return everything the worker batch needs:
  //   (out_cache_loc, new_lens, positions, placeholder_ids, delta_rows, delta_pos, delta_ids)
  // `placeholder_ids[i] = -(row + 1)` are the overlap scheduler's future-token references; the deltas are the
  // page-table entries this step created.  Returns None, and changes nothing, if the pool lacks the pages.
  // Counterpart of the reference's prepare_for_decode + get_model_worker_batch arithmetic
  // (python/sgl_jax/srt/managers/schedule_batch.py:1680-1811, :3034-3293).
  py::object build_decode_step(py::array_t<int32_t, py::array::c_style> table, i32arr rows, i32arr kv_lens) {
    const int64_t B = rows.size();
    if (kv_lens.size() != B || table.ndim() != 2) throw std::invalid_argument("build_decode_step: bad shapes");
    const int64_t width = table.shape(1), nrows = table.shape(0);
    int32_t* tab = table.mutable_data();
    const int32_t *r = rows.data(), *len = kv_lens.data();
    int64_t need = 0;
    for (int64_t i = 0; i < B; ++i) {
      if (r[i] < 0 || r[i] >= nrows || len[i] < 1 || len[i] >= width) throw std::out_of_range("build_decode_step: row / length");
      need += (len[i] % page_ == 0);
    }
    if (need > (int64_t)free_.size()) return py::none();
    i32arr out(B), new_lens(B), positions(B), placeholders(B), d_rows(need), d_pos(need), d_ids(need);
    int32_t *o = out.mutable_data(), *nl = new_lens.mutable_data(), *ps = positions.mutable_data(),
            *ph = placeholders.mutable_data(), *dr = d_rows.mutable_data(), *dp = d_pos.mutable_data(),
            *di = d_ids.mutable_data();
    int64_t nd = 0;
    for (int64_t i = 0; i < B; ++i) {
      int32_t* row = tab + (int64_t)r[i] * width;
      int32_t slot;
      if (len[i] % page_ == 0) {
        const int32_t page = free_.front();
        free_.pop_front();
        slot = page * page_;
        dr[nd] = r[i];
        dp[nd] = len[i] / page_;
        di[nd] = page;
        ++nd;
      } else {
        slot = row[len[i] - 1] + 1;
      }
      row[len[i]] = slot;
      o[i] = slot;
      nl[i] = len[i] + 1;
      ps[i] = len[i];
      ph[i] = -(r[i] + 1);
    }
    return py::make_tuple(out, new_lens, positions, placeholders, d_rows, d_pos, d_ids);
  }

  void free_slots(i32arr idx) {
    if (idx.size() == 0) return;
    if (in_group_) {
      group_.insert(group_.end(), idx.data(), idx.data() + idx.size());
      return;
    }
    release(idx.data(), idx.size());
  }
  void free_group_begin() { in_group_ = true; group_.clear(); }
  void free_group_end() {
    in_group_ = false;
    if (!group_.empty()) release(group_.data(), (int64_t)group_.size());
    group_.clear();
  }
  i32arr backup_state() const {
    i32arr out((int64_t)free_.size());
    std::copy(free_.begin(), free_.end(), out.mutable_data());
    return out;
  }
  void restore_state(i32arr st) { free_.assign(st.data(), st.data() + st.size()); }

 private:
  void release(const int32_t* idx, int64_t n) {
    if (page_ == 1) {  // single-slot pages: slots go back in the order they were released
      for (int64_t i = 0; i < n; ++i)
        if (idx[i] > 0) free_.push_back(idx[i]);
      return;
    }
    std::vector<int32_t> pages(n);
    for (int64_t i = 0; i < n; ++i) pages[i] = idx[i] / page_;
    std::sort(pages.begin(), pages.end());
    pages.erase(std::unique(pages.begin(), pages.end()), pages.end());
    for (int32_t p : pages)
      if (p > 0) free_.push_back(p);
  }
  int page_;
  int64_t num_pages_;
  std::deque<int32_t> free_;
  bool in_group_ = false;
  std::vector<int32_t> group_;
};

// ------------------------------------------------------------------------------------ radix tree
struct Node {
  int64_t id = 0;
  Node* parent = nullptr;
  std::unordered_map<std::string, Node*> children;
  std::vector<int64_t> key;
  std::vector<int32_t> value;
  int lock_ref = 0;
  uint64_t last_access = 0;
  int ns = 0;
  std::string child_key;
};

class RadixTree {
 public:
  explicit RadixTree(int page_size) : page_(page_size) { reset(); }
  ~RadixTree() { destroy(root_); }

  void reset() {
    if (root_) destroy(root_);
    by_id_.clear();
    evictable_.clear();
    protected_.clear();
    next_id_ = 0;
    root_ = make();
    root_->lock_ref = 1;
  }
  int64_t root_id() const { return root_->id; }

  // -> (values of the matched prefix, id of the deepest matched node)
  py::tuple match(i64arr tokens, int ns) {
    const int64_t* t = tokens.data();
    int64_t n = tokens.size() / page_ * page_;
    std::vector<int32_t> out;
    Node* node = root_;
    uint64_t now = ++clock_;
    node->last_access = now;
    int64_t pos = 0;
    while (pos < n) {
      auto it = node->children.find(child_key(t + pos, ns, node == root_));
      if (it == node->children.end()) break;
      Node* child = it->second;
      child->last_access = now;
      int64_t m = match_len(child->key, t + pos, n - pos);
      if (m < (int64_t)child->key.size()) {
        if (m == 0) break;
        child = split(child, m);
        out.insert(out.end(), child->value.begin(), child->value.end());
        node = child;
        break;
      }
      out.insert(out.end(), child->value.begin(), child->value.end());
      node = child;
      pos += m;
    }
    i32arr vals((int64_t)out.size());
    std::copy(out.begin(), out.end(), vals.mutable_data());
    return py::make_tuple(vals, node->id);
  }

  // -> (tokens that already existed, id of a newly created node or -1, its parent id, its length)
  py::tuple insert(i64arr tokens, i32arr values, int ns) {
    const int64_t* t = tokens.data();
    const int32_t* v = values.data();
    int64_t n = std::min<int64_t>(tokens.size(), values.size()) / page_ * page_;
    Node* node = root_;
    uint64_t now = ++clock_;
    int64_t pos = 0, existed = 0;
    while (pos < n) {
      auto it = node->children.find(child_key(t + pos, ns, node == root_));
      if (it == node->children.end()) break;
      Node* child = it->second;
      child->last_access = now;
      int64_t m = match_len(child->key, t + pos, n - pos);
      if (m == 0) break;
      if (m < (int64_t)child->key.size()) child = split(child, m);
      existed += m;
      node = child;
      pos += m;
    }
    int64_t new_id = -1, parent_id = -1, new_len = 0;
    if (pos < n) {
      Node* nn = make();
      nn->ns = ns;
      nn->parent = node;
      nn->key.assign(t + pos, t + n);
      nn->value.assign(v + pos, v + n);
      nn->last_access = ++clock_;  // younger than the siblings this insert touched on its way down
      nn->child_key = child_key(t + pos, ns, node == root_);
      node->children[nn->child_key] = nn;
      evictable_[ns] += n - pos;
      new_id = nn->id;
      parent_id = node->id;
      new_len = n - pos;
    }
    return py::make_tuple(existed, new_id, parent_id, new_len);
  }

  // Evict unlocked leaves, least recently used first, until `num_tokens` slots are released.
  // `ns_filter` empty = every namespace.  -> list of (ns, node id, slots).
  py::list evict(int64_t num_tokens, std::vector<int> ns_filter) {
    py::list out;
    if (num_tokens <= 0) return out;
    auto allowed = [&](int ns) {
      return ns_filter.empty() || std::find(ns_filter.begin(), ns_filter.end(), ns) != ns_filter.end();
    };
    using Item = std::pair<uint64_t, Node*>;
    std::priority_queue<Item, std::vector<Item>, std::greater<Item>> heap;
    std::vector<Node*> stack{root_};
    while (!stack.empty()) {
      Node* n = stack.back();
      stack.pop_back();
      if (n != root_ && n->children.empty() && n->lock_ref == 0 && allowed(n->ns)) heap.push({n->last_access, n});
      for (auto& kv : n->children) stack.push_back(kv.second);
    }
    int64_t freed = 0;
    while (freed < num_tokens && !heap.empty()) {
      Node* n = heap.top().second;
      heap.pop();
      if (n->lock_ref > 0) continue;
      i32arr vals((int64_t)n->value.size());
      std::copy(n->value.begin(), n->value.end(), vals.mutable_data());
      out.append(py::make_tuple(n->ns, n->id, vals));
      freed += (int64_t)n->value.size();
      evictable_[n->ns] -= (int64_t)n->value.size();
      Node* p = n->parent;
      p->children.erase(n->child_key);
      by_id_.erase(n->id);
      delete n;
      if (p != root_ && p->lock_ref == 0 && p->children.empty()) heap.push({p->last_access, p});
    }
    return out;
  }

  int64_t inc_lock(int64_t id) {
    int64_t delta = 0;
    for (Node* n = get(id); n && n != root_; n = n->parent) {
      if (n->lock_ref == 0) {
        int64_t k = (int64_t)n->value.size();
        evictable_[n->ns] -= k;
        protected_[n->ns] += k;
        delta -= k;
      }
      ++n->lock_ref;
    }
    return delta;
  }
  int64_t dec_lock(int64_t id) {
    int64_t delta = 0;
    for (Node* n = get(id); n && n != root_; n = n->parent) {
      if (n->lock_ref == 1) {
        int64_t k = (int64_t)n->value.size();
        evictable_[n->ns] += k;
        protected_[n->ns] -= k;
        delta += k;
      }
      if (--n->lock_ref < 0) throw std::runtime_error("radix node unlocked more often than locked");
    }
    return delta;
  }

  std::map<int, int64_t> evictable() const { return evictable_; }
  std::map<int, int64_t> protected_sizes() const { return protected_; }
  int64_t total_size() const {
    int64_t t = 0;
    for (auto& kv : by_id_)
      if (kv.second != root_) t += (int64_t)kv.second->value.size();
    return t;
  }
  i32arr all_values() const {
    std::vector<int32_t> v;
    for (auto& kv : by_id_)
      if (kv.second != root_) v.insert(v.end(), kv.second->value.begin(), kv.second->value.end());
    i32arr out((int64_t)v.size());
    std::copy(v.begin(), v.end(), out.mutable_data());
    return out;
  }
  // (parent id, child ids, lock_ref, ns, key length, last access tick) of a node; raises for ids that no longer exist
  py::tuple info(int64_t id) const {
    Node* n = get(id);
    if (!n) throw py::key_error("radix node " + std::to_string(id) + " no longer exists");
    std::vector<int64_t> ch;
    for (auto& kv : n->children) ch.push_back(kv.second->id);
    std::sort(ch.begin(), ch.end());
    return py::make_tuple(n->parent ? n->parent->id : -1, ch, n->lock_ref, n->ns, (int64_t)n->key.size(), n->last_access);
  }
  py::tuple key_value(int64_t id) const {
    Node* n = get(id);
    if (!n) throw py::key_error("radix node " + std::to_string(id) + " no longer exists");
    i64arr k((int64_t)n->key.size());
    std::copy(n->key.begin(), n->key.end(), k.mutable_data());
    i32arr v((int64_t)n->value.size());
    std::copy(n->value.begin(), n->value.end(), v.mutable_data());
    return py::make_tuple(k, v);
  }
  bool alive(int64_t id) const { return by_id_.count(id) != 0; }
  int64_t num_nodes() const { return (int64_t)by_id_.size() - 1; }

 private:
  Node* make() {
    Node* n = new Node();
    n->id = next_id_++;
    n->last_access = clock_;
    by_id_[n->id] = n;
    return n;
  }
  Node* get(int64_t id) const {
    auto it = by_id_.find(id);
    return it == by_id_.end() ? nullptr : it->second;
  }
  void destroy(Node* n) {
    if (!n) return;
    for (auto& kv : n->children) destroy(kv.second);
    delete n;
  }
  std::string child_key(const int64_t* t, int ns, bool at_root) const {
    std::string k;
    k.reserve(sizeof(int64_t) * page_ + sizeof(int));
    if (at_root) k.append(reinterpret_cast<const char*>(&ns), sizeof(int));
    k.append(reinterpret_cast<const char*>(t), sizeof(int64_t) * page_);
    return k;
  }
  int64_t match_len(const std::vector<int64_t>& key, const int64_t* t, int64_t avail) const {
    int64_t n = std::min<int64_t>((int64_t)key.size(), avail), i = 0;
    while (i + page_ <= n && std::memcmp(key.data() + i, t + i, sizeof(int64_t) * page_) == 0) i += page_;
    return i;
  }
  // Cut `child` at `m` tokens; returns the new upper node.
  Node* split(Node* child, int64_t m) {
    Node* parent = child->parent;
    Node* upper = make();
    upper->ns = child->ns;
    upper->parent = parent;
    upper->key.assign(child->key.begin(), child->key.begin() + m);
    upper->value.assign(child->value.begin(), child->value.begin() + m);
    upper->lock_ref = child->lock_ref;
    upper->last_access = child->last_access;
    upper->child_key = child->child_key;
    parent->children[upper->child_key] = upper;
    child->parent = upper;
    child->key.erase(child->key.begin(), child->key.begin() + m);
    child->value.erase(child->value.begin(), child->value.begin() + m);
    child->child_key = child_key(child->key.data(), child->ns, false);
    upper->children[child->child_key] = child;
    return upper;
  }

  int page_;
  Node* root_ = nullptr;
  int64_t next_id_ = 0;
  uint64_t clock_ = 0;
  std::unordered_map<int64_t, Node*> by_id_;
  std::map<int, int64_t> evictable_, protected_;
};


// ------------------------------------------------------------------------------------ step ring
// Single-producer / multi-consumer message ring in POSIX shared memory: tensor rank 0 publishes each
// step's batch (a fixed-layout block of integers, or a pickled control message) and the follower
// ranks of the node read it, without a socket round-trip or a host collective per step.
//
//   header   : magic | slots | slot_bytes | consumers | write_seq (atomic) | closed | read_seq[consumers]
//   slot i   : length (u32) | kind (u32) | payload
// The producer may run at most `slots` messages ahead of the slowest consumer; a push that finds the ring
// full, or a pop that finds it empty, waits (GIL released) up to its timeout and then reports failure, which
// is how a dead peer shows up on the host.  Counterpart of the reference's request mirror over ZMQ PUB/SUB
// (python/sgl_jax/srt/managers/scheduler.py:625-676).
class StepRing {
 public:
  static constexpr uint64_t kMagic = 0x53474c4252494e47ull;   // "SGLBRING"
  static constexpr int kMaxConsumers = 64;
  struct alignas(64) Header {
    uint64_t magic;
    uint32_t slots, slot_bytes, consumers, pad;
    alignas(64) std::atomic<uint64_t> write_seq;
    alignas(64) std::atomic<uint32_t> closed;
    struct alignas(64) Cursor { std::atomic<uint64_t> seq; } read_seq[kMaxConsumers];
  };

  // consumer < 0: create (producer side); otherwise attach as that consumer
  StepRing(const std::string& name, int slots, int slot_bytes, int consumers, int consumer)
      : name_(name), consumer_(consumer), owner_(consumer < 0) {
    if (consumers < 1 || consumers > kMaxConsumers) throw std::invalid_argument("StepRing: bad consumer count");
    const size_t slot_stride = (static_cast<size_t>(slot_bytes) + 8 + 63) / 64 * 64;
    bytes_ = sizeof(Header) + slot_stride * slots;
    int fd = -1;
    if (owner_) {
      ::shm_unlink(name.c_str());
      fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
      if (fd < 0 || ::ftruncate(fd, bytes_) != 0) throw std::runtime_error("StepRing: cannot create " + name);
    } else {
      fd = ::shm_open(name.c_str(), O_RDWR, 0600);
      if (fd < 0) throw std::runtime_error("StepRing: cannot open " + name);
    }
    void* p = ::mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (p == MAP_FAILED) throw std::runtime_error("StepRing: mmap failed");
    h_ = static_cast<Header*>(p);
    data_ = static_cast<uint8_t*>(p) + sizeof(Header);
    stride_ = slot_stride;
    if (owner_) {
      std::memset(p, 0, sizeof(Header));
      h_->slots = slots;
      h_->slot_bytes = slot_bytes;
      h_->consumers = consumers;
      h_->write_seq.store(0, std::memory_order_relaxed);
      std::atomic_thread_fence(std::memory_order_release);
      h_->magic = kMagic;
    } else if (h_->magic != kMagic || (int)h_->slots != slots || (int)h_->slot_bytes != slot_bytes ||
               consumer >= (int)h_->consumers) {
      throw std::runtime_error("StepRing: header mismatch for " + name);
    }
  }
  ~StepRing() {
    if (h_ != nullptr) ::munmap(h_, bytes_);
    if (owner_) ::shm_unlink(name_.c_str());
  }

  int slot_bytes() const { return h_->slot_bytes; }
  uint64_t written() const { return h_->write_seq.load(std::memory_order_acquire); }
  uint64_t consumed(int c) const { return h_->read_seq[c].seq.load(std::memory_order_acquire); }
  void close_ring() { h_->closed.store(1, std::memory_order_release); }
  bool closed() const { return h_->closed.load(std::memory_order_acquire) != 0; }

  // index of the slowest consumer and how many messages it is behind
  std::pair<int, uint64_t> slowest() const {
    const uint64_t w = written();
    int who = 0;
    uint64_t lag = 0;
    for (uint32_t c = 0; c < h_->consumers; ++c) {
      const uint64_t l = w - consumed(c);
      if (l >= lag) { lag = l; who = c; }
    }
    return {who, lag};
  }

  // producer: false = ring still full after `timeout_s` (a consumer stopped reading)
  bool push(py::bytes payload, uint32_t kind, double timeout_s) {
    char* buf;
    Py_ssize_t len;
    if (PyBytes_AsStringAndSize(payload.ptr(), &buf, &len) != 0) throw py::error_already_set();
    return push_raw(reinterpret_cast<const uint8_t*>(buf), static_cast<size_t>(len), kind, timeout_s);
  }
  bool push_ints(i32arr arr, uint32_t kind, double timeout_s) {
    return push_raw(reinterpret_cast<const uint8_t*>(arr.data()), static_cast<size_t>(arr.size()) * 4, kind, timeout_s);
  }
  bool push_raw(const uint8_t* src, size_t len, uint32_t kind, double timeout_s) {
    if (!owner_) throw std::runtime_error("StepRing: only the creator may push");
    if (len > h_->slot_bytes) throw std::length_error("StepRing: message larger than a slot");
    const uint64_t w = h_->write_seq.load(std::memory_order_relaxed);
    {
      py::gil_scoped_release nogil;
      const auto t0 = std::chrono::steady_clock::now();
      unsigned spins = 0;
      for (;;) {
        uint64_t min_read = w;
        for (uint32_t c = 0; c < h_->consumers; ++c) min_read = std::min(min_read, consumed(c));
        if (w - min_read < h_->slots) break;
        if ((++spins & 0x3f) == 0) {
          if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) return false;
          std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
      }
      uint8_t* slot = data_ + (w % h_->slots) * stride_;
      reinterpret_cast<uint32_t*>(slot)[0] = static_cast<uint32_t>(len);
      reinterpret_cast<uint32_t*>(slot)[1] = kind;
      std::memcpy(slot + 8, src, len);
    }
    h_->write_seq.store(w + 1, std::memory_order_release);
    return true;
  }

  // consumer: (kind, payload) or None after `timeout_s` without a message / once the ring is closed and drained
  py::object pop(double timeout_s, bool as_ints) {
    if (consumer_ < 0) throw std::runtime_error("StepRing: the creator does not pop");
    auto& cur = h_->read_seq[consumer_].seq;
    const uint64_t r = cur.load(std::memory_order_relaxed);
    bool got = false;
    {
      py::gil_scoped_release nogil;
      const auto t0 = std::chrono::steady_clock::now();
      unsigned spins = 0;
      for (;;) {
        if (h_->write_seq.load(std::memory_order_acquire) > r) { got = true; break; }
        if (closed()) break;
        if ((++spins & 0xff) == 0) {
          const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
          if (dt > timeout_s) break;
          if (dt > 0.002) std::this_thread::sleep_for(std::chrono::microseconds(dt > 0.1 ? 200 : 20));
        }
      }
    }
    if (!got) return py::none();
    const uint8_t* slot = data_ + (r % h_->slots) * stride_;
    const uint32_t len = reinterpret_cast<const uint32_t*>(slot)[0];
    const uint32_t kind = reinterpret_cast<const uint32_t*>(slot)[1];
    py::object payload;
    if (as_ints && kind != 0) {
      i32arr out(len / 4);
      std::memcpy(out.mutable_data(), slot + 8, len / 4 * 4);
      payload = std::move(out);
    } else {
      payload = py::bytes(reinterpret_cast<const char*>(slot + 8), len);
    }
    cur.store(r + 1, std::memory_order_release);
    return py::make_tuple(kind, payload);
  }

 private:
  std::string name_;
  int consumer_;
  bool owner_;
  size_t bytes_ = 0, stride_ = 0;
  Header* h_ = nullptr;
  uint8_t* data_ = nullptr;
};

PYBIND11_MODULE(_sched_native, m) {
  m.doc() = "paged KV slot allocator and radix-tree prefix index";
  py::class_<PagedAllocator>(m, "PagedAllocator")
      .def(py::init<int64_t, int>())
      .def("clear", &PagedAllocator::clear)
      .def("available_size", &PagedAllocator::available_size)
      .def("num_free_pages", &PagedAllocator::num_free_pages)
      .def("alloc", &PagedAllocator::alloc)
      .def("alloc_extend", &PagedAllocator::alloc_extend)
      .def("alloc_decode", &PagedAllocator::alloc_decode)
      .def("build_decode_step", &PagedAllocator::build_decode_step)
      .def("free", &PagedAllocator::free_slots)
      .def("free_group_begin", &PagedAllocator::free_group_begin)
      .def("free_group_end", &PagedAllocator::free_group_end)
      .def("backup_state", &PagedAllocator::backup_state)
      .def("restore_state", &PagedAllocator::restore_state);
  py::class_<RadixTree>(m, "RadixTree")
      .def(py::init<int>())
      .def("reset", &RadixTree::reset)
      .def("root_id", &RadixTree::root_id)
      .def("match", &RadixTree::match)
      .def("insert", &RadixTree::insert)
      .def("evict", &RadixTree::evict)
      .def("inc_lock", &RadixTree::inc_lock)
      .def("dec_lock", &RadixTree::dec_lock)
      .def("evictable", &RadixTree::evictable)
      .def("protected_sizes", &RadixTree::protected_sizes)
      .def("total_size", &RadixTree::total_size)
      .def("all_values", &RadixTree::all_values)
      .def("info", &RadixTree::info)
      .def("key_value", &RadixTree::key_value)
      .def("alive", &RadixTree::alive)
      .def("num_nodes", &RadixTree::num_nodes);
  py::class_<StepRing>(m, "StepRing")
      .def(py::init<const std::string&, int, int, int, int>(), py::arg("name"), py::arg("slots"),
           py::arg("slot_bytes"), py::arg("consumers"), py::arg("consumer") = -1)
      .def("push", &StepRing::push, py::arg("payload"), py::arg("kind") = 0, py::arg("timeout_s") = 60.0)
      .def("push_ints", &StepRing::push_ints, py::arg("ints"), py::arg("kind") = 1, py::arg("timeout_s") = 60.0)
      .def("pop", &StepRing::pop, py::arg("timeout_s") = 60.0, py::arg("as_ints") = true)
      .def("written", &StepRing::written)
      .def("consumed", &StepRing::consumed)
      .def("slowest", &StepRing::slowest)
      .def("close", &StepRing::close_ring)
      .def("closed", &StepRing::closed)
      .def("slot_bytes", &StepRing::slot_bytes);
}
