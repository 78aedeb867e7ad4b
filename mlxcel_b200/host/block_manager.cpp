// Host runtime: paged KV block manager, prefix (automatic prompt cache) index and the
// per-step page-table / slot-mapping builder.
//
// One block id names the same slot in every layer's slab, so there is a single free list and a
// single table per sequence (the reference keeps one table per layer,
// src/lib/mlxcel-core/src/cache/paged.rs:212-260, and has to balance per-layer free lists).
// Blocks are reference counted; full blocks are registered under a chained 128-bit content hash
// (parent hash, token ids, salt) like the reference's APC index
// (src/server/prompt_cache/block_hash.rs:71); unreferenced registered blocks stay resident in an
// LRU list and are evicted only when the free list runs dry. A write into a shared block forks
// it first (copy-on-write), reported to the caller as (src, dst) block copies.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <list>
#include <stdexcept>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

namespace {

struct Hash128 {
  uint64_t a = 0, b = 0;
  bool operator==(const Hash128& o) const { return a == o.a && b == o.b; }
};
struct Hash128Hasher {
  size_t operator()(const Hash128& h) const { return static_cast<size_t>(h.a ^ (h.b * 0x9E3779B97F4A7C15ull)); }
};

inline uint64_t mix64(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

Hash128 chain_hash(const Hash128& parent, const int32_t* tokens, int n, uint64_t salt) {
  uint64_t a = parent.a ^ 0x243F6A8885A308D3ull ^ salt;
  uint64_t b = parent.b ^ 0x13198A2E03707344ull ^ (salt * 0x9E3779B97F4A7C15ull);
  for (int i = 0; i < n; ++i) {
    const uint64_t t = static_cast<uint32_t>(tokens[i]);
    a = mix64(a ^ (t + 0x9E3779B97F4A7C15ull + (a << 6) + (a >> 2)));
    b = mix64(b + t * 0xC2B2AE3D27D4EB4Full + (b << 7) + 0x165667B19E3779F9ull);
  }
  return Hash128{a, b};
}

struct Block {
  int ref = 0;
  bool hashed = false;
  Hash128 hash;
  std::list<int>::iterator lru_it;  // valid when ref == 0 && hashed
  bool in_lru = false;
};

struct Sequence {
  std::vector<int> blocks;
  int num_tokens = 0;       // tokens with KV slots reserved
  int num_hashed = 0;       // leading full blocks already registered
  Hash128 last_hash;        // hash of block num_hashed - 1
  uint64_t salt = 0;
  int front_released = 0;   // leading table entries given back by release_front (stored as -1)
  // Context shift: `shifted` tokens (whole blocks) were cut out of the table behind the first
  // `keep_tokens` tokens. Callers keep counting tokens absolutely; positions >= keep_tokens + shifted
  // live at table index (pos - shifted) / block_size.
  int shifted = 0;
  int keep_tokens = 0;
};

class BlockManager {
 public:
  BlockManager(int num_blocks, int block_size, bool prefix_cache, double watermark)
      : num_blocks_(num_blocks), block_size_(block_size), prefix_cache_(prefix_cache),
        blocks_(num_blocks) {
    if (num_blocks <= 0 || block_size <= 0) throw std::invalid_argument("bad pool geometry");
    free_.reserve(num_blocks);
    for (int i = num_blocks - 1; i >= 0; --i) free_.push_back(i);
    watermark_blocks_ = static_cast<int>(watermark * num_blocks);
  }

  int block_size() const { return block_size_; }
  int num_blocks() const { return num_blocks_; }
  int num_free() const { return static_cast<int>(free_.size() + lru_.size()); }
  int num_cached() const { return static_cast<int>(lru_.size()); }
  int watermark_blocks() const { return watermark_blocks_; }
  bool has_seq(int64_t id) const { return seqs_.count(id) != 0; }
  int seq_len(int64_t id) const { return get(id).num_tokens; }
  int shifted(int64_t id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? 0 : it->second.shifted;
  }
  std::vector<int> seq_blocks(int64_t id) const { return get(id).blocks; }

  int blocks_needed(int64_t id, int total_tokens) const {
    auto it = seqs_.find(id);
    const int have = it == seqs_.end() ? 0 : static_cast<int>(it->second.blocks.size());
    const int cut = it == seqs_.end() ? 0 : it->second.shifted;
    const int need = (std::max(0, total_tokens - cut) + block_size_ - 1) / block_size_;
    return std::max(0, need - have);
  }

  // Admission test: room for `n` more blocks while leaving the watermark untouched.
  bool can_allocate(int n, bool respect_watermark) const {
    return num_free() - (respect_watermark ? watermark_blocks_ : 0) >= n;
  }

  void create(int64_t id, uint64_t salt) {
    if (seqs_.count(id)) throw std::invalid_argument("sequence exists");
    Sequence s;
    s.salt = salt;
    seqs_.emplace(id, std::move(s));
  }

  // Adopt the longest registered prefix of `tokens` (whole blocks, and never the whole prompt:
  // at least one token is left to compute so that the step produces logits).
  int match_prefix(int64_t id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens) {
    Sequence& s = get(id);
    if (!prefix_cache_ || !s.blocks.empty()) return 0;
    const int n = static_cast<int>(tokens.size());
    const int32_t* t = tokens.data();
    const int max_full = (n - 1) / block_size_;
    Hash128 h;
    int matched = 0;
    for (int b = 0; b < max_full; ++b) {
      Hash128 nh = chain_hash(h, t + b * block_size_, block_size_, s.salt);
      auto it = index_.find(nh);
      if (it == index_.end()) break;
      const int blk = it->second;
      retain(blk);
      s.blocks.push_back(blk);
      h = nh;
      ++matched;
    }
    s.num_tokens = matched * block_size_;
    s.num_hashed = matched;
    s.last_hash = h;
    hits_ += matched;
    queries_ += max_full;
    return s.num_tokens;
  }

  // Reserve slots so that the sequence can hold `total_tokens`. Returns false (and changes
  // nothing) when the pool cannot provide the blocks.
  bool reserve(int64_t id, int total_tokens) {
    Sequence& s = get(id);
    const int need = blocks_needed(id, total_tokens);
    if (need > num_free()) return false;
    for (int i = 0; i < need; ++i) s.blocks.push_back(take_block());
    s.num_tokens = std::max(s.num_tokens, total_tokens);
    return true;
  }

  // Register the full blocks covered by the first `num_computed` tokens.
  void commit(int64_t id, py::array_t<int32_t, py::array::c_style | py::array::forcecast> tokens,
              int num_computed) {
    if (!prefix_cache_) return;
    Sequence& s = get(id);
    if (s.shifted > 0) return;          // the block chain has a hole: nothing more of it is shareable
    const int32_t* t = tokens.data();
    const int n = std::min<int>(num_computed, static_cast<int>(tokens.size()));
    const int full = std::min<int>(n / block_size_, static_cast<int>(s.blocks.size()));
    for (int b = s.num_hashed; b < full; ++b) {
      Hash128 nh = chain_hash(s.last_hash, t + b * block_size_, block_size_, s.salt);
      const int blk = s.blocks[b];
      auto it = index_.find(nh);
      if (it == index_.end()) {
        if (!blocks_[blk].hashed) {
          blocks_[blk].hashed = true;
          blocks_[blk].hash = nh;
          index_.emplace(nh, blk);
        }
      }
      s.last_hash = nh;
      s.num_hashed = b + 1;
    }
  }

  // Make the block that holds position `pos` private to the sequence. Returns (src, dst) when a
  // copy of the block's contents is required, (-1, -1) otherwise.
  std::pair<int, int> ensure_writable(int64_t id, int pos) {
    Sequence& s = get(id);
    const int bi = pos / block_size_;
    if (bi >= static_cast<int>(s.blocks.size())) throw std::out_of_range("position not reserved");
    const int blk = s.blocks[bi];
    if (blocks_[blk].ref <= 1 && !blocks_[blk].hashed) return {-1, -1};
    if (blocks_[blk].ref <= 1 && blocks_[blk].hashed) {
      // Sole owner of a registered block: unregister instead of copying.
      index_.erase(blocks_[blk].hash);
      blocks_[blk].hashed = false;
      if (bi < s.num_hashed) truncate_hash(s, bi);
      return {-1, -1};
    }
    if (num_free() < 1) throw std::runtime_error("no block for copy-on-write");
    const int nb = take_block();
    release(blk);
    s.blocks[bi] = nb;
    if (bi < s.num_hashed) truncate_hash(s, bi);
    ++cow_copies_;
    return {blk, nb};
  }

  // Share all blocks of `src` with a new sequence `dst` (beam / n>1 sampling / speculative fork).
  void fork(int64_t src, int64_t dst) {
    const Sequence& a = get(src);
    if (seqs_.count(dst)) throw std::invalid_argument("sequence exists");
    Sequence b = a;
    for (int blk : b.blocks) retain(blk);
    seqs_.emplace(dst, std::move(b));
  }

  // Drop trailing tokens (speculative rollback, lookahead teardown).
  void truncate(int64_t id, int new_len) {
    Sequence& s = get(id);
    if (new_len >= s.num_tokens) return;
    if (s.shifted > 0 && new_len < s.keep_tokens + s.shifted)
      throw std::invalid_argument("truncate below a context shift");
    const int keep = (new_len - s.shifted + block_size_ - 1) / block_size_;
    while (static_cast<int>(s.blocks.size()) > keep) {
      if (s.blocks.back() >= 0) release(s.blocks.back());
      s.blocks.pop_back();
    }
    s.front_released = std::min<int>(s.front_released, static_cast<int>(s.blocks.size()));
    s.num_tokens = new_len;
    const int full = new_len / block_size_;
    if (s.num_hashed > full) truncate_hash(s, full);
  }

  // Sliding-window pools: give back every block whose tokens all lie before `first_needed_token`
  // (they can never be attended again). The entries stay in the table as -1 so that positions keep
  // indexing it; fill_tables writes block 0 there (the kernels mask those positions). Returns the
  // number of blocks released. Not meant for pools with a prefix index (released blocks of a
  // shared prefix would break the chain); such pools never call it.
  int release_front(int64_t id, int first_needed_token) {
    Sequence& s = get(id);
    const int upto = std::min<int>(std::max(0, first_needed_token) / block_size_, static_cast<int>(s.blocks.size()));
    int n = 0;
    for (int b = s.front_released; b < upto; ++b) {
      if (s.blocks[b] >= 0) {
        release(s.blocks[b]);
        s.blocks[b] = -1;
        ++n;
      }
    }
    s.front_released = std::max(s.front_released, upto);
    front_released_ += n;
    return n;
  }

  // Context shift: cut whole blocks out of the table behind the first `keep_tokens` tokens (rounded
  // up to a block) so that at most `max_live` tokens stay, and give them back. The keys that stay
  // keep the rotary position they were written with, and the caller keeps counting tokens
  // absolutely (see Sequence::shifted). Returns the number of tokens cut. Such a sequence is no
  // longer registered in the prefix index (its block chain has a hole).
  int shift_front(int64_t id, int keep_tokens, int max_live) {
    Sequence& s = get(id);
    if (s.front_released > 0) throw std::invalid_argument("context shift on a sliding-window pool");
    const int live = s.num_tokens - s.shifted;
    if (live <= max_live) return 0;
    const int keep_blocks = s.shifted > 0 ? s.keep_tokens / block_size_
                                          : (std::max(0, keep_tokens) + block_size_ - 1) / block_size_;
    // never touch the block that is being written
    const int last_full = std::max(0, live - 1) / block_size_;
    const int drop = std::min((live - max_live + block_size_ - 1) / block_size_, last_full - keep_blocks);
    if (drop <= 0) return 0;
    if (s.num_hashed > keep_blocks) truncate_hash(s, keep_blocks);
    for (int b = keep_blocks; b < keep_blocks + drop; ++b) release(s.blocks[b]);
    s.blocks.erase(s.blocks.begin() + keep_blocks, s.blocks.begin() + keep_blocks + drop);
    if (s.shifted == 0) s.keep_tokens = keep_blocks * block_size_;
    s.shifted += drop * block_size_;
    shifted_tokens_ += static_cast<long long>(drop) * block_size_;
    return drop * block_size_;
  }

  void free_seq(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return;
    // Release from the tail so that leaf blocks are evicted before their parents.
    for (auto b = it->second.blocks.rbegin(); b != it->second.blocks.rend(); ++b)
      if (*b >= 0) release(*b);
    seqs_.erase(it);
  }

  // Drop every unreferenced cached block (cache reset). Returns the number dropped.
  int reset_prefix_cache() {
    int n = 0;
    while (!lru_.empty()) {
      evict_one();
      ++n;
    }
    return n;
  }

  // Fill block tables / context lens for a batch. tables: int32 [B, max_blocks] (padded with 0).
  void fill_tables(const std::vector<int64_t>& ids, py::array_t<int32_t, py::array::c_style> tables) {
    auto buf = tables.mutable_unchecked<2>();
    const int B = static_cast<int>(ids.size());
    if (buf.shape(0) < B) throw std::invalid_argument("table rows");
    const int width = static_cast<int>(buf.shape(1));
    for (int i = 0; i < B; ++i) {
      const Sequence& s = get(ids[i]);
      const int n = static_cast<int>(s.blocks.size());
      if (n > width) throw std::invalid_argument("table too narrow");
      int32_t* row = &buf(i, 0);
      std::memcpy(row, s.blocks.data(), sizeof(int32_t) * n);
      for (int b = 0; b < s.front_released && b < n; ++b) row[b] = 0;   // released by a sliding window
      if (n < width) std::memset(row + n, 0, sizeof(int32_t) * (width - n));
    }
  }

  // Slot indices (block * block_size + offset) of positions [start, start + count) of a sequence.
  void fill_slots(int64_t id, int start, int count, py::array_t<int32_t, py::array::c_style> out,
                  int out_offset) {
    const Sequence& s = get(id);
    auto buf = out.mutable_unchecked<1>();
    if (out_offset + count > buf.shape(0)) throw std::invalid_argument("slot buffer");
    for (int i = 0; i < count; ++i) {
      int pos = start + i;
      if (s.shifted > 0 && pos >= s.keep_tokens) {
        if (pos < s.keep_tokens + s.shifted) throw std::out_of_range("slot in a range cut by a context shift");
        pos -= s.shifted;
      }
      const int bi = pos / block_size_;
      if (bi >= static_cast<int>(s.blocks.size())) throw std::out_of_range("slot beyond reservation");
      if (s.blocks[bi] < 0) throw std::out_of_range("slot in a block released by the sliding window");
      buf(out_offset + i) = s.blocks[bi] * block_size_ + pos % block_size_;
    }
  }

  py::dict stats() const {
    py::dict d;
    d["num_blocks"] = num_blocks_;
    d["block_size"] = block_size_;
    d["free"] = static_cast<int>(free_.size());
    d["cached"] = static_cast<int>(lru_.size());
    d["registered"] = static_cast<int>(index_.size());
    d["sequences"] = static_cast<int>(seqs_.size());
    d["front_released"] = front_released_;
    d["shifted_tokens"] = shifted_tokens_;
    d["prefix_hits"] = hits_;
    d["prefix_queries"] = queries_;
    d["evictions"] = evictions_;
    d["cow_copies"] = cow_copies_;
    return d;
  }

 private:
  const Sequence& get(int64_t id) const {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) throw std::out_of_range("unknown sequence");
    return it->second;
  }
  Sequence& get(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) throw std::out_of_range("unknown sequence");
    return it->second;
  }
  void truncate_hash(Sequence& s, int full) {
    // Re-derive the chain tail lazily: hashes of blocks [0, full) stay valid; remember the
    // parent by walking the registered hashes of the kept blocks.
    s.num_hashed = std::min(s.num_hashed, full);
    s.last_hash = Hash128{};
    if (s.num_hashed > 0) {
      const int blk = s.blocks[s.num_hashed - 1];
      if (blocks_[blk].hashed) {
        s.last_hash = blocks_[blk].hash;
      } else {
        s.num_hashed = 0;  // chain broken: stop registering for this sequence
      }
    }
  }
  void retain(int blk) {
    Block& b = blocks_[blk];
    if (b.ref == 0 && b.in_lru) {
      lru_.erase(b.lru_it);
      b.in_lru = false;
    }
    ++b.ref;
  }
  void release(int blk) {
    Block& b = blocks_[blk];
    if (b.ref <= 0) throw std::logic_error("release of unreferenced block");
    if (--b.ref == 0) {
      if (b.hashed && prefix_cache_) {
        lru_.push_back(blk);
        b.lru_it = std::prev(lru_.end());
        b.in_lru = true;
      } else {
        free_.push_back(blk);
      }
    }
  }
  void evict_one() {
    const int blk = lru_.front();
    lru_.pop_front();
    Block& b = blocks_[blk];
    b.in_lru = false;
    if (b.hashed) {
      auto it = index_.find(b.hash);
      if (it != index_.end() && it->second == blk) index_.erase(it);
      b.hashed = false;
    }
    free_.push_back(blk);
    ++evictions_;
  }
  int take_block() {
    if (free_.empty()) {
      if (lru_.empty()) throw std::runtime_error("block pool exhausted");
      evict_one();
    }
    const int blk = free_.back();
    free_.pop_back();
    blocks_[blk].ref = 1;
    blocks_[blk].hashed = false;
    return blk;
  }

  int num_blocks_, block_size_;
  bool prefix_cache_;
  int watermark_blocks_ = 0;
  std::vector<Block> blocks_;
  std::vector<int> free_;
  std::list<int> lru_;
  std::unordered_map<Hash128, int, Hash128Hasher> index_;
  std::unordered_map<int64_t, Sequence> seqs_;
  long long hits_ = 0, queries_ = 0, evictions_ = 0, cow_copies_ = 0, front_released_ = 0, shifted_tokens_ = 0;
};

}  // namespace

void bind_scheduler(py::module_& m);

PYBIND11_MODULE(_mlxcel_host, m) {
  m.doc() = "mlxcel_b200 host runtime (C++): KV block manager, prefix index, batch tables, tick policy";
  py::class_<BlockManager>(m, "BlockManager")
      .def(py::init<int, int, bool, double>(), py::arg("num_blocks"), py::arg("block_size"),
           py::arg("prefix_cache") = true, py::arg("watermark") = 0.01)
      .def_property_readonly("block_size", &BlockManager::block_size)
      .def_property_readonly("num_blocks", &BlockManager::num_blocks)
      .def_property_readonly("num_free", &BlockManager::num_free)
      .def_property_readonly("num_cached", &BlockManager::num_cached)
      .def_property_readonly("watermark_blocks", &BlockManager::watermark_blocks)
      .def("has_seq", &BlockManager::has_seq)
      .def("seq_len", &BlockManager::seq_len)
      .def("seq_blocks", &BlockManager::seq_blocks)
      .def("blocks_needed", &BlockManager::blocks_needed)
      .def("can_allocate", &BlockManager::can_allocate, py::arg("n"), py::arg("respect_watermark") = true)
      .def("create", &BlockManager::create, py::arg("seq_id"), py::arg("salt") = 0)
      .def("match_prefix", &BlockManager::match_prefix)
      .def("reserve", &BlockManager::reserve)
      .def("commit", &BlockManager::commit)
      .def("ensure_writable", &BlockManager::ensure_writable)
      .def("fork", &BlockManager::fork)
      .def("truncate", &BlockManager::truncate)
      .def("free_seq", &BlockManager::free_seq)
      .def("release_front", &BlockManager::release_front)
      .def("shift_front", &BlockManager::shift_front, py::arg("seq_id"), py::arg("keep_tokens"), py::arg("max_live"))
      .def("shifted", &BlockManager::shifted)
      .def("reset_prefix_cache", &BlockManager::reset_prefix_cache)
      .def("fill_tables", &BlockManager::fill_tables)
      .def("fill_slots", &BlockManager::fill_slots)
      .def("stats", &BlockManager::stats);
  bind_scheduler(m);
}
