// Host-side serving scheduler: page allocator, per-request block tables, page-granular prefix
// index, decode-first continuous batcher with chunked prefill, admission policy.
//
// Capability parity with the reference's scheduler layer (all unit-testable without a GPU, as there:
// src/scheduler/mod.rs:1-5):
//   BlockAllocator      src/scheduler/allocator.rs:5-52          FIFO free list of physical page ids
//   PrefixIndex         src/scheduler/prefix_index.rs:9-84        longest shared prompt prefix -> pages
//   PagedScheduler      src/scheduler/paged_scheduler.rs:85-620   block tables, prefix reuse, rollback
//   ContinuousBatcher   src/scheduler/batcher.rs:149-607          decode first, then prefill backfill
//   AbsolutePolicy      src/scheduler/policy.rs:5-125             batch cap / admission / forced swap-out
//
// Design differences (deliberate): pages are shared only when completely filled (a partially
// filled page is never aliased, so a writer can never touch a reader's tokens); shared pages are
// reference counted and stay cached after their last user finishes until the allocator needs them
// (LRU); running sequences own a stable slot index so a CUDA-graph decode step can address
// per-sequence state by slot.
#pragma once
#include <cstdint>
#include <deque>
#include <list>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace gsched {

constexpr int kNoPage = -1;

// ---------------------------------------------------------------------------------------------
class BlockAllocator {
 public:
  explicit BlockAllocator(int num_blocks);
  int allocate();                 // kNoPage when exhausted; new page has refcount 1
  void retain(int page);          // +1
  bool release(int page);         // -1; returns true when the page went back to the free list
  int refcount(int page) const { return refs_[page]; }
  int num_free() const { return static_cast<int>(free_.size()); }
  int num_total() const { return static_cast<int>(refs_.size()); }
  double fragmentation(int used_tokens, int page_size) const;

 private:
  std::deque<int> free_;
  std::vector<int> refs_;
};

// ---------------------------------------------------------------------------------------------
// Page-granular radix tree over token chunks. Each node stands for one full page of tokens and
// pins that page (one reference) while it is cached.
class PrefixIndex {
 public:
  PrefixIndex(BlockAllocator* alloc, int page_size) : alloc_(alloc), page_size_(page_size) {}
  ~PrefixIndex();
  // Longest cached prefix of `tokens`, in whole pages; appends page ids to `pages` (not retained).
  int find_longest_prefix(const int32_t* tokens, int n, std::vector<int>* pages);
  // Register the first n_pages full pages of `tokens` (pages[i] holds tokens [i*ps, (i+1)*ps)).
  void insert(const int32_t* tokens, int n_tokens, const int* pages, int n_pages);
  // Drop least-recently-used leaf pages that only the cache still references; returns pages freed.
  int evict(int want_pages);
  int cached_pages() const { return cached_; }
  uint64_t hits() const { return hits_; }
  uint64_t lookups() const { return lookups_; }

 private:
  struct Node {
    std::vector<int32_t> chunk;
    int page = kNoPage;
    Node* parent = nullptr;
    uint64_t last_use = 0;
    std::unordered_map<uint64_t, std::vector<std::unique_ptr<Node>>> children;
    int n_children = 0;
  };
  static uint64_t hash_chunk(const int32_t* t, int n);
  Node* find_child(Node* n, const int32_t* t);
  void collect_leaves(Node* n, std::vector<Node*>* out);
  Node root_;
  BlockAllocator* alloc_;
  int page_size_;
  int cached_ = 0;
  uint64_t clock_ = 0, hits_ = 0, lookups_ = 0;
};

// ---------------------------------------------------------------------------------------------
enum class SeqState : int { Waiting = 0, Prefilling = 1, Running = 2, Paused = 3, Finished = 4, Swapped = 5 };
enum class FinishReason : int { None = 0, Eos = 1, Length = 2, Aborted = 3, Veto = 4 };
enum class OrderPolicy : int { StrictRequestId = 0, Fifo = 1 };

struct SamplingParams {
  float temperature = 0.7f;
  int top_k = 0;
  float top_p = 1.0f;
  int max_new_tokens = 256;
  std::vector<int32_t> eos_ids;
};

struct Sequence {
  int64_t id = 0;
  uint64_t arrival = 0;
  std::vector<int32_t> tokens;  // prompt followed by generated tokens
  int prompt_len = 0;
  int num_computed = 0;  // tokens whose KV is in the cache
  int num_cached_prefix = 0;  // tokens served from the prefix cache at admission
  std::vector<int> block_table;
  SeqState state = SeqState::Waiting;
  FinishReason finish = FinishReason::None;
  int slot = -1;
  SamplingParams sp;
  int preemptions = 0;
  std::string session;
  int num_generated() const { return static_cast<int>(tokens.size()) - prompt_len; }
};

struct PolicyConfig {
  int max_batch_size = 256;          // running-sequence cap (the reference defaults to 32)
  int max_batch_tokens = 4096;       // token budget of one step
  int prefill_chunk = 2048;          // upper bound of one prefill chunk
  int min_prefill_chunk = 64;
  double decode_ratio_cap = 1.0;     // share of the budget decode may take (reference: 0.6 interleaved)
  double emergency_pressure = 0.9;   // above: no new prefill, force swap-outs
  double defrag_threshold = 0.5;
  int watermark_pages = 2;           // keep this many pages free when admitting
  bool enable_prefix_cache = true;
  bool phase_isolated = true;        // decode batch and prefill chunk are separate launches
  int order = 0;                     // OrderPolicy
  // Preemption of a running (fully prefilled) sequence: false = recompute (pages go back, the sequence is prefilled
  // again later); true = swap (the plan lists the victim's pages in `swap_out`, the caller copies them to host memory
  // before the step runs, the sequence keeps its position and comes back through `swap_in` when pages are free).
  bool preempt_swap = false;
  // Prefill chunk size from the share of free pages: under a quarter free the smallest chunk, above three quarters the
  // largest, linear in between (the reference's adaptive chunk: src/scheduler/vllm2024.rs:24-68).
  bool adaptive_chunk = false;
};

struct SystemState {
  double memory_pressure = 0, kv_fragmentation = 0, logits_entropy = 0, attention_sparsity = 0;
  int waiting = 0, running = 0;
};

struct PolicyDecision {
  int max_batch_size = 0;
  bool admit_new_prefill = true;
  int force_swap_out_count = 0;
};

PolicyDecision policy_decide(const PolicyConfig& cfg, const SystemState& st);

// A sequence leaving for / returning from host memory: its pages in logical order and the tokens they cover.
struct SwapItem {
  int64_t seq_id;
  std::vector<int> pages;
  int num_tokens;
};

// One prefill work item: a chunk of one sequence.
struct PrefillItem {
  int64_t seq_id;
  int slot;
  int start;    // first token position of the chunk
  int len;      // tokens in the chunk
  bool last;    // chunk reaches the end of the known tokens -> sample
};

struct StepPlan {
  // decode part, indexed by slot (dense arrays of max_slots entries)
  int num_decode = 0;
  std::vector<int32_t> dec_tokens, dec_positions, dec_slot_mapping, dec_ctx_lens;  // [max_slots]
  std::vector<int64_t> dec_seq_ids;                                                 // [max_slots], -1 = empty
  // prefill part, flat tokens
  std::vector<PrefillItem> prefill;
  std::vector<int32_t> pf_tokens, pf_positions, pf_slot_mapping;  // [T]
  std::vector<int32_t> pf_q_start, pf_q_len, pf_ctx_lens, pf_slots;  // [S]
  std::vector<int32_t> pf_block_tables;  // [S, max_blocks]
  int max_blocks = 0;
  std::vector<int64_t> preempted;
  // swap-style preemption (PolicyConfig::preempt_swap): copy these pages out BEFORE, these in BEFORE the step's
  // kernels run (pages of a swapped-out sequence may already belong to another sequence of this same plan)
  std::vector<SwapItem> swap_out, swap_in;
  bool idle() const { return num_decode == 0 && prefill.empty() && swap_out.empty() && swap_in.empty(); }
};

struct FinishedSeq {
  int64_t id;
  std::vector<int32_t> tokens;  // generated tokens only
  int prompt_len;
  int finish;
  int cached_prefix;
  int preemptions;
};

class ContinuousBatcher {
 public:
  ContinuousBatcher(int num_pages, int page_size, int max_slots, int max_blocks_per_seq, PolicyConfig cfg);

  int64_t add_request(int64_t id, const std::vector<int32_t>& prompt, const SamplingParams& sp,
                      const std::string& session);
  bool abort(int64_t id);
  StepPlan schedule();
  // tokens sampled for the decode slots of the last plan (array of max_slots) and for the prefill
  // items that ended with `last` (in plan order).
  void commit(const StepPlan& plan, const int32_t* decode_tokens, const int32_t* prefill_tokens);
  std::vector<FinishedSeq> pop_finished();

  // speculative / MTP support: drop the last n tokens of a running sequence and their pages
  bool rollback(int64_t id, int n_tokens);
  // append externally verified tokens to a running sequence (speculative accept)
  bool append_tokens(int64_t id, const std::vector<int32_t>& toks);
  // speculative decoding: make sure a running sequence owns pages for its next `n_tokens` positions (no preemption;
  // false when the pool cannot give them), and commit tokens whose predecessors' KV a verify forward already wrote:
  // every committed token advances the computed position by one. Stops at EOS / the length limit.
  bool reserve_tokens(int64_t id, int n_tokens);
  bool commit_tokens(int64_t id, const std::vector<int32_t>& toks);

  const Sequence* find(int64_t id) const;
  std::vector<int32_t> block_table_of(int64_t id) const;
  // dense [max_slots, max_blocks] table of the running sequences (row = slot)
  const std::vector<int32_t>& slot_block_tables() const { return slot_tables_; }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_swapped() const { return static_cast<int>(swapped_.size()); }
  // Preferred victims of the next preemptions, best victim first (an eviction policy such as HGAL supplies it);
  // ids that are not running are skipped, and when the list runs out the youngest running sequence is taken.
  void set_victim_order(const std::vector<int64_t>& ids) { victim_order_ = ids; }
  int num_running() const { return static_cast<int>(running_.size()); }
  int num_free_pages() const { return alloc_.num_free(); }
  int num_total_pages() const { return alloc_.num_total(); }
  int cached_pages() const { return prefix_.cached_pages(); }
  uint64_t prefix_hits() const { return prefix_.hits(); }
  uint64_t prefix_lookups() const { return prefix_.lookups(); }
  double memory_pressure() const;
  double fragmentation() const;
  int max_slots() const { return max_slots_; }
  int max_blocks() const { return max_blocks_; }
  int page_size() const { return page_size_; }
  PolicyConfig& config() { return cfg_; }
  void set_system_state(const SystemState& s) { sys_ = s; }
  // sessions: keep the pages of a finished request alive for the next turn of the same session
  int session_cached_tokens(const std::string& session) const;
  // persistence of the prefix cache / sessions (snapshot to disk and back):
  std::vector<std::string> session_ids() const;
  std::vector<int32_t> session_tokens(const std::string& session) const;
  // pages that currently cache the longest whole-page prefix of `tokens` (empty when nothing is cached)
  std::vector<int> lookup_prefix_pages(const std::vector<int32_t>& tokens);
  // allocate pages for the whole-page prefix of `tokens`, register them in the prefix index and return them so
  // the caller can fill their contents; pages already cached are reused (-1 marks "already there, skip").
  std::vector<int> import_prefix(const std::vector<int32_t>& tokens, const std::string& session);

 private:
  bool ensure_pages(Sequence& s, int upto_tokens);
  int take_page();
  void free_sequence(Sequence& s, bool to_prefix_cache);
  void finish(Sequence& s, FinishReason why);
  bool preempt_one(int64_t protect_id);
  void write_slot_table(const Sequence& s);
  bool is_eos(const Sequence& s, int32_t tok) const;

  BlockAllocator alloc_;
  PrefixIndex prefix_;
  int page_size_, max_slots_, max_blocks_;
  PolicyConfig cfg_;
  SystemState sys_;
  uint64_t arrivals_ = 0;
  std::deque<int64_t> waiting_;
  std::deque<int64_t> swapped_;               // swapped-out sequences, oldest first
  std::vector<SwapItem> pending_swap_out_;    // filled by preempt_one during schedule()
  std::vector<int64_t> victim_order_;
  std::map<int64_t, int64_t> running_;  // order key -> id
  std::unordered_map<int64_t, std::unique_ptr<Sequence>> seqs_;
  std::vector<int64_t> slot_owner_;
  std::vector<int> free_slots_;
  std::vector<int32_t> slot_tables_;
  std::vector<FinishedSeq> finished_;
  struct SessionEntry {
    std::vector<int32_t> tokens;
    std::vector<int> pages;
  };
  std::unordered_map<std::string, SessionEntry> sessions_;
};

}  // namespace gsched
