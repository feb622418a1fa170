// Host-side runtime of the generation engine and the trainer, exported with a C ABI:
//
//   * BlockManager  - paged KV-cache block pool with reference counts and a content-addressed
//                     prefix cache (hash chain over full blocks, salted per weight version).
//   * Scheduler     - continuous batching: admits waiting requests for prefill under a token
//                     budget, runs decode for everything admitted, preempts (recompute) the most
//                     recent request when the pool runs dry, supports pause (keep / abort).
//   * HashRing      - consistent hashing with virtual nodes for session-affine routing.
//   * bin packing   - balanced token-budget micro-batching and first-fit-decreasing packing.
//
// The roles match what the reference obtains from vLLM's scheduler/block manager and from the
// vllm-router binary; nothing here touches the GPU.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <numeric>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

inline uint64_t mix64(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return x;
}

inline uint64_t hash_tokens(uint64_t seed, const int32_t* t, int n) {
  uint64_t h = seed ^ 0x9e3779b97f4a7c15ULL;
  for (int i = 0; i < n; ++i) h = mix64(h ^ (static_cast<uint64_t>(static_cast<uint32_t>(t[i])) + 0x9e3779b97f4a7c15ULL + (h << 6)));
  return h;
}

// ------------------------------------------------------------------ BlockManager
class BlockManager {
 public:
  BlockManager(int num_blocks, int block_size, bool prefix_cache)
      : block_size_(block_size), prefix_(prefix_cache), ref_(num_blocks, 0), hash_of_(num_blocks, 0),
        cached_(num_blocks, 0) {
    for (int i = num_blocks - 1; i >= 0; --i) free_.push_back(i);
  }

  int num_free() const { return static_cast<int>(free_.size() + evictable_.size()); }
  int num_total() const { return static_cast<int>(ref_.size()); }
  int block_size() const { return block_size_; }

  // Allocates n blocks (evicting unreferenced cached blocks if needed). Returns false if impossible.
  bool alloc(int n, int32_t* out) {
    if (n > num_free()) return false;
    for (int i = 0; i < n; ++i) {
      int b;
      if (!free_.empty()) {
        b = free_.back();
        free_.pop_back();
      } else {
        b = evictable_.front();  // least recently released first
        evictable_.pop_front();
        drop_cache_entry(b);
      }
      ref_[b] = 1;
      out[i] = b;
    }
    return true;
  }

  void release(const int32_t* ids, int n) {
    for (int i = 0; i < n; ++i) {
      const int b = ids[i];
      if (b < 0 || b >= num_total() || ref_[b] <= 0) continue;
      if (--ref_[b] == 0) {
        if (cached_[b])
          evictable_.push_back(b);
        else
          free_.push_back(b);
      }
    }
  }

  // Longest cached prefix of full blocks. Takes a reference on each matched block.
  int match_prefix(const int32_t* tokens, int n_tokens, uint64_t salt, int32_t* out_blocks, int max_blocks) {
    if (!prefix_) return 0;
    int matched = 0;
    uint64_t h = salt;
    const int full = n_tokens / block_size_;
    for (int i = 0; i < full && i < max_blocks; ++i) {
      h = hash_tokens(h, tokens + static_cast<size_t>(i) * block_size_, block_size_);
      auto it = table_.find(h);
      if (it == table_.end()) break;
      const int b = it->second;
      if (ref_[b] == 0) {
        auto pos = std::find(evictable_.begin(), evictable_.end(), b);
        if (pos != evictable_.end()) evictable_.erase(pos);
      }
      ++ref_[b];
      out_blocks[matched++] = b;
    }
    hits_ += matched;
    queries_ += full;
    return matched;
  }

  // Hash chain of every full block of `tokens` (into `hashes`) and how many leading ones are cached right now.
  // Takes no references.
  int probe_prefix(const int32_t* tokens, int n_tokens, uint64_t salt, std::vector<uint64_t>& hashes) const {
    hashes.clear();
    if (!prefix_) return 0;
    uint64_t h = salt;
    const int full = n_tokens / block_size_;
    int cached = 0;
    bool run = true;
    for (int i = 0; i < full; ++i) {
      h = hash_tokens(h, tokens + static_cast<size_t>(i) * block_size_, block_size_);
      hashes.push_back(h);
      if (run && table_.find(h) != table_.end())
        ++cached;
      else
        run = false;
    }
    return cached;
  }
  bool prefix_enabled() const { return prefix_; }

  // Publishes the first n_full blocks of a sequence into the prefix cache.
  void register_prefix(const int32_t* tokens, int n_tokens, uint64_t salt, const int32_t* blocks, int n_blocks) {
    if (!prefix_) return;
    uint64_t h = salt;
    const int full = std::min(n_tokens / block_size_, n_blocks);
    for (int i = 0; i < full; ++i) {
      h = hash_tokens(h, tokens + static_cast<size_t>(i) * block_size_, block_size_);
      const int b = blocks[i];
      if (cached_[b]) continue;
      if (table_.find(h) != table_.end()) continue;  // another block already holds this content
      table_[h] = b;
      hash_of_[b] = h;
      cached_[b] = 1;
    }
  }

  void reset_prefix_cache() {
    for (int b : evictable_) {
      cached_[b] = 0;
      free_.push_back(b);
    }
    evictable_.clear();
    for (size_t b = 0; b < cached_.size(); ++b) cached_[b] = 0;
    table_.clear();
  }

  double hit_rate() const { return queries_ ? static_cast<double>(hits_) / queries_ : 0.0; }

 private:
  void drop_cache_entry(int b) {
    if (cached_[b]) {
      auto it = table_.find(hash_of_[b]);
      if (it != table_.end() && it->second == b) table_.erase(it);
      cached_[b] = 0;
    }
  }
  int block_size_;
  bool prefix_;
  std::vector<int> ref_;
  std::vector<uint64_t> hash_of_;
  std::vector<uint8_t> cached_;
  std::vector<int> free_;
  std::deque<int> evictable_;
  std::unordered_map<uint64_t, int> table_;
  uint64_t hits_ = 0, queries_ = 0;
};

// ------------------------------------------------------------------ Scheduler
enum SeqState { WAITING = 0, RUNNING = 1, FINISHED = 2, PREEMPTED = 3 };

struct Seq {
  int64_t id;
  std::vector<int32_t> tokens;  // prompt + generated
  int prompt_len;
  int max_total;      // prompt_len + max_new_tokens
  int num_computed;   // tokens whose KV is in the cache
  int num_cached;     // tokens served from the prefix cache at admission
  uint64_t salt;
  std::vector<int32_t> blocks;
  SeqState state;
  int64_t arrival;
};

struct StepPlan {
  int mode;  // 0 idle, 1 prefill, 2 decode
  std::vector<int64_t> seq_ids;
  std::vector<int32_t> starts;  // prefill: first token position to compute
  std::vector<int32_t> counts;  // prefill: number of tokens to compute
};

class Scheduler {
 public:
  Scheduler(int num_blocks, int block_size, int max_num_seqs, int max_batched_tokens, bool prefix_cache,
            bool reserve_full)
      : bm_(num_blocks, block_size, prefix_cache), max_seqs_(max_num_seqs), max_tokens_(max_batched_tokens),
        reserve_full_(reserve_full) {}

  BlockManager& bm() { return bm_; }

  int add(int64_t id, const int32_t* prompt, int prompt_len, int max_new, uint64_t salt) {
    if (seqs_.count(id)) return -1;
    Seq s;
    s.id = id;
    s.tokens.assign(prompt, prompt + prompt_len);
    s.prompt_len = prompt_len;
    s.max_total = prompt_len + max_new;
    s.num_computed = 0;
    s.num_cached = 0;
    s.salt = salt;
    s.state = WAITING;
    s.arrival = clock_++;
    seqs_[id] = std::move(s);
    waiting_.push_back(id);
    return 0;
  }

  int blocks_needed(int tokens) const { return (tokens + bm_.block_size() - 1) / bm_.block_size(); }

  // Ensures the sequence owns blocks for `tokens` positions. Preempts younger sequences if needed.
  bool ensure_blocks(Seq& s, int tokens, bool allow_preempt) {
    const int need = blocks_needed(tokens) - static_cast<int>(s.blocks.size());
    if (need <= 0) return true;
    while (bm_.num_free() < need) {
      if (!allow_preempt || !preempt_youngest(s.id)) return false;
    }
    const size_t old = s.blocks.size();
    s.blocks.resize(old + need);
    if (!bm_.alloc(need, s.blocks.data() + old)) {
      s.blocks.resize(old);
      return false;
    }
    return true;
  }

  bool preempt_youngest(int64_t except) {
    int64_t victim = -1, best = -1;
    for (int64_t id : running_) {
      if (id == except) continue;
      const Seq& s = seqs_[id];
      if (s.arrival > best) {
        best = s.arrival;
        victim = id;
      }
    }
    if (victim < 0) return false;
    Seq& v = seqs_[victim];
    bm_.release(v.blocks.data(), static_cast<int>(v.blocks.size()));
    v.blocks.clear();
    v.num_computed = 0;
    v.num_cached = 0;
    v.state = PREEMPTED;
    running_.erase(std::find(running_.begin(), running_.end(), victim));
    waiting_.push_front(victim);
    ++num_preemptions_;
    return true;
  }

  void plan(StepPlan& p) {
    p.mode = 0;
    p.seq_ids.clear();
    p.starts.clear();
    p.counts.clear();
    if (paused_) return;
    // 1. admit waiting requests for prefill under the token budget.  With the prefix cache on, a request whose next
    // uncached block is being computed by a request admitted in this very step (same prompt sampled n times) waits
    // one step instead of computing it again: after that step the blocks are published and it shares them.
    int budget = max_tokens_;
    std::unordered_set<uint64_t> in_flight;
    std::vector<uint64_t> chain;
    size_t wi = 0;
    while (wi < waiting_.size() && static_cast<int>(running_.size() + p.seq_ids.size()) < max_seqs_) {
      Seq& s = seqs_[waiting_[wi]];
      const int total = static_cast<int>(s.tokens.size());
      const bool fresh = s.blocks.empty() && s.num_computed == 0;
      if (fresh && bm_.prefix_enabled()) {
        const int have = bm_.probe_prefix(s.tokens.data(), total - 1, s.salt, chain);
        if (have < static_cast<int>(chain.size()) && in_flight.count(chain[have])) {
          ++wi;  // a request of this step computes that block: come back when it is published
          continue;
        }
      }
      if (fresh) {
        // prefix-cache lookup; never match the whole prompt (the last token must be computed)
        std::vector<int32_t> hit(blocks_needed(total));
        const int m = bm_.match_prefix(s.tokens.data(), total - 1, s.salt, hit.data(), static_cast<int>(hit.size()));
        s.blocks.assign(hit.begin(), hit.begin() + m);
        s.num_computed = s.num_cached = m * bm_.block_size();
      }
      const int todo = total - s.num_computed;
      if (todo > budget && !p.seq_ids.empty()) break;
      const int reserve = reserve_full_ ? s.max_total : total + 1;
      if (!ensure_blocks(s, reserve, /*allow_preempt=*/false)) {
        if (running_.empty() && p.seq_ids.empty() && wi == 0) {
          // nothing else can make progress: this request can never fit
          s.state = FINISHED;
          failed_.push_back(s.id);
          waiting_.erase(waiting_.begin() + wi);
          continue;
        }
        break;
      }
      if (fresh && bm_.prefix_enabled()) {
        bm_.probe_prefix(s.tokens.data(), total, s.salt, chain);
        for (size_t i = static_cast<size_t>(s.num_cached / bm_.block_size()); i < chain.size(); ++i) in_flight.insert(chain[i]);
      }
      p.seq_ids.push_back(s.id);
      p.starts.push_back(s.num_computed);
      p.counts.push_back(todo);
      budget -= todo;
      waiting_.erase(waiting_.begin() + wi);
      if (budget <= 0) break;
    }
    if (!p.seq_ids.empty()) {
      p.mode = 1;
      for (int64_t id : p.seq_ids) {
        seqs_[id].state = RUNNING;
        running_.push_back(id);
      }
      return;
    }
    // 2. decode everything that is running
    if (running_.empty()) return;
    std::vector<int64_t> order(running_.begin(), running_.end());
    for (int64_t id : order) {
      auto it = seqs_.find(id);
      if (it == seqs_.end() || it->second.state != RUNNING) continue;
      Seq& s = it->second;
      if (!ensure_blocks(s, static_cast<int>(s.tokens.size()) + 1, /*allow_preempt=*/true)) continue;
      if (s.state == RUNNING) p.seq_ids.push_back(id);
    }
    // drop sequences that were preempted while making room for others
    p.seq_ids.erase(std::remove_if(p.seq_ids.begin(), p.seq_ids.end(),
                                   [&](int64_t id) { return seqs_[id].state != RUNNING; }),
                    p.seq_ids.end());
    if (!p.seq_ids.empty()) p.mode = 2;
  }

  // Records that the KV of all current tokens is computed (after prefill) and publishes the prefix.
  void mark_prefilled(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return;
    Seq& s = it->second;
    s.num_computed = static_cast<int>(s.tokens.size());
    bm_.register_prefix(s.tokens.data(), s.num_computed, s.salt, s.blocks.data(), static_cast<int>(s.blocks.size()));
  }

  void append(int64_t id, int32_t token) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return;
    Seq& s = it->second;
    s.num_computed = static_cast<int>(s.tokens.size());
    s.tokens.push_back(token);
  }

  void finish(int64_t id, bool publish_prefix) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return;
    Seq& s = it->second;
    if (publish_prefix && !s.blocks.empty())
      bm_.register_prefix(s.tokens.data(), s.num_computed, s.salt, s.blocks.data(), static_cast<int>(s.blocks.size()));
    bm_.release(s.blocks.data(), static_cast<int>(s.blocks.size()));
    auto r = std::find(running_.begin(), running_.end(), id);
    if (r != running_.end()) running_.erase(r);
    auto w = std::find(waiting_.begin(), waiting_.end(), id);
    if (w != waiting_.end()) waiting_.erase(w);
    seqs_.erase(it);
  }

  Seq* get(int64_t id) {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? nullptr : &it->second;
  }

  void set_paused(bool p) { paused_ = p; }
  bool paused() const { return paused_; }
  int num_running() const { return static_cast<int>(running_.size()); }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_preemptions() const { return num_preemptions_; }
  const std::deque<int64_t>& running() const { return running_; }
  const std::deque<int64_t>& waiting() const { return waiting_; }
  std::vector<int64_t>& failed() { return failed_; }

  // Drops the cached KV of every sequence (weights changed): running sequences go back to waiting.
  void invalidate_all_kv() {
    std::vector<int64_t> ids(running_.begin(), running_.end());
    std::sort(ids.begin(), ids.end(), [&](int64_t a, int64_t b) { return seqs_[a].arrival > seqs_[b].arrival; });
    for (int64_t id : ids) {
      Seq& v = seqs_[id];
      bm_.release(v.blocks.data(), static_cast<int>(v.blocks.size()));
      v.blocks.clear();
      v.num_computed = v.num_cached = 0;
      v.state = PREEMPTED;
      waiting_.push_front(id);
    }
    running_.clear();
    for (int64_t id : waiting_) {
      Seq& v = seqs_[id];
      if (!v.blocks.empty()) {
        bm_.release(v.blocks.data(), static_cast<int>(v.blocks.size()));
        v.blocks.clear();
        v.num_computed = v.num_cached = 0;
      }
    }
    bm_.reset_prefix_cache();
  }

 private:
  BlockManager bm_;
  int max_seqs_, max_tokens_;
  bool reserve_full_;
  bool paused_ = false;
  int64_t clock_ = 0;
  int num_preemptions_ = 0;
  std::unordered_map<int64_t, Seq> seqs_;
  std::deque<int64_t> waiting_, running_;
  std::vector<int64_t> failed_;
};

// ------------------------------------------------------------------ HashRing
class HashRing {
 public:
  explicit HashRing(int vnodes) : vnodes_(vnodes) {}
  void add(int node) {
    for (int v = 0; v < vnodes_; ++v) ring_[mix64((static_cast<uint64_t>(node) << 32) ^ static_cast<uint64_t>(v) ^ 0xabcdef12345ULL)] = node;
  }
  void remove(int node) {
    for (auto it = ring_.begin(); it != ring_.end();) it = (it->second == node) ? ring_.erase(it) : std::next(it);
  }
  int lookup(const char* key, int len) const {
    if (ring_.empty()) return -1;
    uint64_t h = 0xcbf29ce484222325ULL;
    for (int i = 0; i < len; ++i) h = (h ^ static_cast<uint8_t>(key[i])) * 0x100000001b3ULL;
    h = mix64(h);
    auto it = ring_.lower_bound(h);
    if (it == ring_.end()) it = ring_.begin();
    return it->second;
  }
  int size() const { return static_cast<int>(ring_.size()) / std::max(1, vnodes_); }

 private:
  int vnodes_;
  std::map<uint64_t, int> ring_;
};

}  // namespace

extern "C" {

// ---- block manager -------------------------------------------------------
void* sbrt_bm_create(int num_blocks, int block_size, int prefix_cache) {
  return new BlockManager(num_blocks, block_size, prefix_cache != 0);
}
void sbrt_bm_destroy(void* h) { delete static_cast<BlockManager*>(h); }
int sbrt_bm_num_free(void* h) { return static_cast<BlockManager*>(h)->num_free(); }
int sbrt_bm_alloc(void* h, int n, int32_t* out) { return static_cast<BlockManager*>(h)->alloc(n, out) ? 0 : -1; }
void sbrt_bm_release(void* h, const int32_t* ids, int n) { static_cast<BlockManager*>(h)->release(ids, n); }
int sbrt_bm_match_prefix(void* h, const int32_t* tokens, int n, uint64_t salt, int32_t* out, int max_blocks) {
  return static_cast<BlockManager*>(h)->match_prefix(tokens, n, salt, out, max_blocks);
}
void sbrt_bm_register_prefix(void* h, const int32_t* tokens, int n, uint64_t salt, const int32_t* blocks, int nb) {
  static_cast<BlockManager*>(h)->register_prefix(tokens, n, salt, blocks, nb);
}
void sbrt_bm_reset_prefix_cache(void* h) { static_cast<BlockManager*>(h)->reset_prefix_cache(); }
double sbrt_bm_hit_rate(void* h) { return static_cast<BlockManager*>(h)->hit_rate(); }

// ---- scheduler -----------------------------------------------------------
void* sbrt_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_batched_tokens, int prefix_cache,
                        int reserve_full) {
  return new Scheduler(num_blocks, block_size, max_num_seqs, max_batched_tokens, prefix_cache != 0, reserve_full != 0);
}
void sbrt_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }
int sbrt_sched_add(void* h, int64_t id, const int32_t* prompt, int n, int max_new, uint64_t salt) {
  return static_cast<Scheduler*>(h)->add(id, prompt, n, max_new, salt);
}
// Fills ids/starts/counts (capacity cap). Returns the number of sequences; *mode: 0 idle, 1 prefill, 2 decode.
int sbrt_sched_plan(void* h, int* mode, int64_t* ids, int32_t* starts, int32_t* counts, int cap) {
  StepPlan p;
  static_cast<Scheduler*>(h)->plan(p);
  *mode = p.mode;
  const int n = std::min<int>(cap, static_cast<int>(p.seq_ids.size()));
  for (int i = 0; i < n; ++i) {
    ids[i] = p.seq_ids[i];
    starts[i] = p.mode == 1 ? p.starts[i] : 0;
    counts[i] = p.mode == 1 ? p.counts[i] : 1;
  }
  return n;
}
void sbrt_sched_mark_prefilled(void* h, int64_t id) { static_cast<Scheduler*>(h)->mark_prefilled(id); }
void sbrt_sched_append(void* h, int64_t id, int32_t token) { static_cast<Scheduler*>(h)->append(id, token); }
void sbrt_sched_finish(void* h, int64_t id, int publish) { static_cast<Scheduler*>(h)->finish(id, publish != 0); }
int sbrt_sched_seq_len(void* h, int64_t id) {
  Seq* s = static_cast<Scheduler*>(h)->get(id);
  return s ? static_cast<int>(s->tokens.size()) : -1;
}
int sbrt_sched_seq_cached(void* h, int64_t id) {
  Seq* s = static_cast<Scheduler*>(h)->get(id);
  return s ? s->num_cached : -1;
}
int sbrt_sched_seq_tokens(void* h, int64_t id, int32_t* out, int cap) {
  Seq* s = static_cast<Scheduler*>(h)->get(id);
  if (!s) return -1;
  const int n = std::min<int>(cap, static_cast<int>(s->tokens.size()));
  std::memcpy(out, s->tokens.data(), sizeof(int32_t) * n);
  return n;
}
int sbrt_sched_seq_blocks(void* h, int64_t id, int32_t* out, int cap) {
  Seq* s = static_cast<Scheduler*>(h)->get(id);
  if (!s) return -1;
  const int n = std::min<int>(cap, static_cast<int>(s->blocks.size()));
  std::memcpy(out, s->blocks.data(), sizeof(int32_t) * n);
  return n;
}
void sbrt_sched_set_paused(void* h, int p) { static_cast<Scheduler*>(h)->set_paused(p != 0); }
int sbrt_sched_num_running(void* h) { return static_cast<Scheduler*>(h)->num_running(); }
int sbrt_sched_num_waiting(void* h) { return static_cast<Scheduler*>(h)->num_waiting(); }
int sbrt_sched_num_free_blocks(void* h) { return static_cast<Scheduler*>(h)->bm().num_free(); }
int sbrt_sched_num_preemptions(void* h) { return static_cast<Scheduler*>(h)->num_preemptions(); }
double sbrt_sched_prefix_hit_rate(void* h) { return static_cast<Scheduler*>(h)->bm().hit_rate(); }
void sbrt_sched_reset_prefix_cache(void* h) { static_cast<Scheduler*>(h)->bm().reset_prefix_cache(); }
void sbrt_sched_invalidate_all_kv(void* h) { static_cast<Scheduler*>(h)->invalidate_all_kv(); }
int sbrt_sched_pop_failed(void* h, int64_t* out, int cap) {
  auto& f = static_cast<Scheduler*>(h)->failed();
  const int n = std::min<int>(cap, static_cast<int>(f.size()));
  for (int i = 0; i < n; ++i) out[i] = f[i];
  f.erase(f.begin(), f.begin() + n);
  return n;
}
int sbrt_sched_list(void* h, int which, int64_t* out, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  const auto& q = which == 0 ? s->waiting() : s->running();
  int n = 0;
  for (int64_t id : q) {
    if (n >= cap) break;
    out[n++] = id;
  }
  return n;
}

// ---- consistent-hash ring -------------------------------------------------
void* sbrt_ring_create(int vnodes) { return new HashRing(vnodes); }
void sbrt_ring_destroy(void* h) { delete static_cast<HashRing*>(h); }
void sbrt_ring_add(void* h, int node) { static_cast<HashRing*>(h)->add(node); }
void sbrt_ring_remove(void* h, int node) { static_cast<HashRing*>(h)->remove(node); }
int sbrt_ring_lookup(void* h, const char* key, int len) { return static_cast<HashRing*>(h)->lookup(key, len); }

// ---- bin packing ----------------------------------------------------------
// Balanced partition of `n` sequence lengths into micro-batches of at most `budget` tokens: the number of
// bins is the minimum feasible for longest-first greedy; items go to the currently lightest bin that fits.
// out_bin[i] receives the bin of item i. Returns the number of bins (or -1 if an item exceeds the budget).
int sbrt_balanced_bins(const int32_t* lens, int n, int budget, int32_t* out_bin) {
  if (n <= 0) return 0;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lens[a] > lens[b]; });
  if (lens[order[0]] > budget) return -1;
  int64_t total = 0;
  for (int i = 0; i < n; ++i) total += lens[i];
  int bins = static_cast<int>((total + budget - 1) / budget);
  if (bins < 1) bins = 1;
  for (;; ++bins) {
    std::vector<int64_t> load(bins, 0);
    bool ok = true;
    for (int idx : order) {
      int best = -1;
      for (int b = 0; b < bins; ++b)
        if (load[b] + lens[idx] <= budget && (best < 0 || load[b] < load[best])) best = b;
      if (best < 0) {
        ok = false;
        break;
      }
      load[best] += lens[idx];
      out_bin[idx] = best;
    }
    if (ok) return bins;
  }
}

// First-fit-decreasing packing into bins of `capacity` tokens (sequence packing for SFT).
int sbrt_ffd_pack(const int32_t* lens, int n, int capacity, int32_t* out_bin) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lens[a] > lens[b]; });
  std::vector<int64_t> load;
  for (int idx : order) {
    const int L = std::min(lens[idx], capacity);
    int b = 0;
    for (; b < static_cast<int>(load.size()); ++b)
      if (load[b] + L <= capacity) break;
    if (b == static_cast<int>(load.size())) load.push_back(0);
    load[b] += L;
    out_bin[idx] = b;
  }
  return static_cast<int>(load.size());
}

const char* sbrt_version() { return "skyrl_b200-runtime 1"; }

}  // extern "C"
