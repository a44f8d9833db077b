#include "sched.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace gsched {

// ---------------------------------------------------------------------------------------------
// BlockAllocator
// ---------------------------------------------------------------------------------------------
BlockAllocator::BlockAllocator(int num_blocks) : refs_(static_cast<size_t>(num_blocks), 0) {
  for (int i = 0; i < num_blocks; ++i) free_.push_back(i);
}

int BlockAllocator::allocate() {
  if (free_.empty()) return kNoPage;
  int p = free_.front();
  free_.pop_front();
  refs_[p] = 1;
  return p;
}

void BlockAllocator::retain(int page) {
  if (page < 0 || page >= num_total() || refs_[page] <= 0) throw std::runtime_error("retain of a free page");
  ++refs_[page];
}

bool BlockAllocator::release(int page) {
  if (page < 0 || page >= num_total() || refs_[page] <= 0) throw std::runtime_error("release of a free page");
  if (--refs_[page] == 0) {
    free_.push_back(page);
    return true;
  }
  return false;
}

double BlockAllocator::fragmentation(int used_tokens, int page_size) const {
  const int used_pages = num_total() - num_free();
  if (used_pages <= 0) return 0.0;
  const double cap = static_cast<double>(used_pages) * page_size;
  return std::max(0.0, 1.0 - static_cast<double>(used_tokens) / cap);
}

// ---------------------------------------------------------------------------------------------
// PrefixIndex
// ---------------------------------------------------------------------------------------------
uint64_t PrefixIndex::hash_chunk(const int32_t* t, int n) {
  uint64_t h = 1469598103934665603ull;
  for (int i = 0; i < n; ++i) {
    h ^= static_cast<uint32_t>(t[i]);
    h *= 1099511628211ull;
  }
  return h;
}

PrefixIndex::Node* PrefixIndex::find_child(Node* n, const int32_t* t) {
  auto it = n->children.find(hash_chunk(t, page_size_));
  if (it == n->children.end()) return nullptr;
  for (auto& c : it->second)
    if (std::memcmp(c->chunk.data(), t, sizeof(int32_t) * page_size_) == 0) return c.get();
  return nullptr;
}

int PrefixIndex::find_longest_prefix(const int32_t* tokens, int n, std::vector<int>* pages) {
  ++lookups_;
  Node* cur = &root_;
  int matched = 0;
  while (matched + page_size_ <= n) {
    Node* c = find_child(cur, tokens + matched);
    if (!c) break;
    c->last_use = ++clock_;
    if (pages) pages->push_back(c->page);
    matched += page_size_;
    cur = c;
  }
  if (matched > 0) ++hits_;
  return matched;
}

void PrefixIndex::insert(const int32_t* tokens, int n_tokens, const int* pages, int n_pages) {
  Node* cur = &root_;
  for (int i = 0; i < n_pages && (i + 1) * page_size_ <= n_tokens; ++i) {
    const int32_t* t = tokens + i * page_size_;
    Node* c = find_child(cur, t);
    if (!c) {
      auto node = std::make_unique<Node>();
      node->chunk.assign(t, t + page_size_);
      node->page = pages[i];
      node->parent = cur;
      alloc_->retain(pages[i]);
      ++cached_;
      c = node.get();
      cur->children[hash_chunk(t, page_size_)].push_back(std::move(node));
      ++cur->n_children;
    }
    c->last_use = ++clock_;
    cur = c;
  }
}

void PrefixIndex::collect_leaves(Node* n, std::vector<Node*>* out) {
  for (auto& kv : n->children)
    for (auto& c : kv.second) {
      if (c->n_children == 0)
        out->push_back(c.get());
      else
        collect_leaves(c.get(), out);
    }
}

int PrefixIndex::evict(int want_pages) {
  int freed = 0;
  while (freed < want_pages) {
    std::vector<Node*> leaves;
    collect_leaves(&root_, &leaves);
    // only pages nobody but the cache references can actually be returned to the allocator
    leaves.erase(std::remove_if(leaves.begin(), leaves.end(),
                                [this](Node* l) { return alloc_->refcount(l->page) != 1; }),
                 leaves.end());
    if (leaves.empty()) break;
    std::sort(leaves.begin(), leaves.end(), [](Node* a, Node* b) { return a->last_use < b->last_use; });
    bool progress = false;
    for (Node* l : leaves) {
      if (freed >= want_pages) break;
      Node* parent = l->parent;
      const uint64_t h = hash_chunk(l->chunk.data(), page_size_);
      alloc_->release(l->page);
      --cached_;
      ++freed;
      progress = true;
      auto& vec = parent->children[h];
      vec.erase(std::remove_if(vec.begin(), vec.end(), [l](const std::unique_ptr<Node>& p) { return p.get() == l; }),
                vec.end());
      if (vec.empty()) parent->children.erase(h);
      --parent->n_children;
    }
    if (!progress) break;
  }
  return freed;
}

PrefixIndex::~PrefixIndex() {}

// ---------------------------------------------------------------------------------------------
// policy (src/scheduler/policy.rs:23-108)
// ---------------------------------------------------------------------------------------------
PolicyDecision policy_decide(const PolicyConfig& cfg, const SystemState& st) {
  PolicyDecision d;
  d.max_batch_size = cfg.max_batch_size;
  if (st.logits_entropy > 8.0) d.max_batch_size = std::max(1, std::min(d.max_batch_size, std::max(st.running, 1)));
  if (st.attention_sparsity > 0.7)
    d.max_batch_size = std::max(1, static_cast<int>(d.max_batch_size * (1.0 - 0.5 * st.attention_sparsity)));
  if (st.memory_pressure > cfg.emergency_pressure) {
    d.admit_new_prefill = false;
    d.force_swap_out_count = static_cast<int>(std::ceil(3.0 * st.memory_pressure));
  } else if (st.kv_fragmentation > cfg.defrag_threshold) {
    d.admit_new_prefill = false;
    d.force_swap_out_count = 1;
  }
  return d;
}

// ---------------------------------------------------------------------------------------------
// ContinuousBatcher
// ---------------------------------------------------------------------------------------------
ContinuousBatcher::ContinuousBatcher(int num_pages, int page_size, int max_slots, int max_blocks_per_seq,
                                     PolicyConfig cfg)
    : alloc_(num_pages),
      prefix_(&alloc_, page_size),
      page_size_(page_size),
      max_slots_(max_slots),
      max_blocks_(max_blocks_per_seq),
      cfg_(cfg),
      slot_owner_(static_cast<size_t>(max_slots), -1),
      slot_tables_(static_cast<size_t>(max_slots) * max_blocks_per_seq, 0) {
  for (int i = max_slots - 1; i >= 0; --i) free_slots_.push_back(i);
}

int64_t ContinuousBatcher::add_request(int64_t id, const std::vector<int32_t>& prompt, const SamplingParams& sp,
                                       const std::string& session) {
  if (prompt.empty()) throw std::invalid_argument("empty prompt");
  if (seqs_.count(id)) throw std::invalid_argument("duplicate request id");
  const long long total = static_cast<long long>(prompt.size()) + sp.max_new_tokens;
  if ((total + page_size_ - 1) / page_size_ > max_blocks_) throw std::length_error("SequenceTooLong");
  auto s = std::make_unique<Sequence>();
  s->id = id;
  s->arrival = arrivals_++;
  s->tokens = prompt;
  s->prompt_len = static_cast<int>(prompt.size());
  s->sp = sp;
  s->session = session;
  seqs_[id] = std::move(s);
  waiting_.push_back(id);
  return id;
}

bool ContinuousBatcher::is_eos(const Sequence& s, int32_t tok) const {
  for (int32_t e : s.sp.eos_ids)
    if (e == tok) return true;
  return false;
}

int ContinuousBatcher::take_page() {
  int p = alloc_.allocate();
  if (p == kNoPage && prefix_.evict(1) > 0) p = alloc_.allocate();
  return p;
}

bool ContinuousBatcher::ensure_pages(Sequence& s, int upto_tokens) {
  const int need = (upto_tokens + page_size_ - 1) / page_size_;
  if (need > max_blocks_) return false;
  std::vector<int> got;
  while (static_cast<int>(s.block_table.size()) + static_cast<int>(got.size()) < need) {
    int p = take_page();
    if (p == kNoPage) {
      for (int g : got) alloc_.release(g);
      return false;
    }
    got.push_back(p);
  }
  for (int g : got) s.block_table.push_back(g);
  return true;
}

void ContinuousBatcher::write_slot_table(const Sequence& s) {
  if (s.slot < 0) return;
  int32_t* row = slot_tables_.data() + static_cast<size_t>(s.slot) * max_blocks_;
  const int n = static_cast<int>(s.block_table.size());
  for (int i = 0; i < max_blocks_; ++i) row[i] = i < n ? s.block_table[i] : 0;
}

void ContinuousBatcher::free_sequence(Sequence& s, bool to_prefix_cache) {
  if (to_prefix_cache && cfg_.enable_prefix_cache && s.num_computed >= page_size_) {
    const int full = std::min<int>(s.num_computed / page_size_, static_cast<int>(s.block_table.size()));
    prefix_.insert(s.tokens.data(), s.num_computed, s.block_table.data(), full);
  }
  for (int p : s.block_table) alloc_.release(p);
  s.block_table.clear();
  if (s.slot >= 0) {
    slot_owner_[s.slot] = -1;
    free_slots_.push_back(s.slot);
    s.slot = -1;
  }
}

void ContinuousBatcher::finish(Sequence& s, FinishReason why) {
  s.finish = why;
  s.state = SeqState::Finished;
  FinishedSeq f;
  f.id = s.id;
  f.tokens.assign(s.tokens.begin() + s.prompt_len, s.tokens.end());
  f.prompt_len = s.prompt_len;
  f.finish = static_cast<int>(why);
  f.cached_prefix = s.num_cached_prefix;
  f.preemptions = s.preemptions;
  finished_.push_back(std::move(f));
  if (!s.session.empty()) {
    // next turn of the session finds the whole conversation through the prefix index
    SessionEntry e;
    e.tokens.assign(s.tokens.begin(), s.tokens.begin() + s.num_computed);
    sessions_[s.session] = std::move(e);
  }
  for (auto it = running_.begin(); it != running_.end(); ++it)
    if (it->second == s.id) {
      running_.erase(it);
      break;
    }
  free_sequence(s, true);
  seqs_.erase(s.id);
}

int ContinuousBatcher::session_cached_tokens(const std::string& session) const {
  auto it = sessions_.find(session);
  return it == sessions_.end() ? 0 : static_cast<int>(it->second.tokens.size());
}

std::vector<std::string> ContinuousBatcher::session_ids() const {
  std::vector<std::string> out;
  for (auto& kv : sessions_) out.push_back(kv.first);
  return out;
}

std::vector<int32_t> ContinuousBatcher::session_tokens(const std::string& session) const {
  auto it = sessions_.find(session);
  return it == sessions_.end() ? std::vector<int32_t>() : it->second.tokens;
}

std::vector<int> ContinuousBatcher::lookup_prefix_pages(const std::vector<int32_t>& tokens) {
  std::vector<int> pages;
  prefix_.find_longest_prefix(tokens.data(), static_cast<int>(tokens.size()), &pages);
  return pages;
}

std::vector<int> ContinuousBatcher::import_prefix(const std::vector<int32_t>& tokens, const std::string& session) {
  const int n_pages = static_cast<int>(tokens.size()) / page_size_;
  std::vector<int> have;
  prefix_.find_longest_prefix(tokens.data(), n_pages * page_size_, &have);
  std::vector<int> all(have.begin(), have.end()), out(have.size(), -1);
  for (int i = static_cast<int>(have.size()); i < n_pages; ++i) {
    const int p = take_page();
    if (p == kNoPage) break;
    all.push_back(p);
    out.push_back(p);
  }
  const int got = static_cast<int>(all.size());
  prefix_.insert(tokens.data(), got * page_size_, all.data(), got);
  // the index holds its own reference now; drop the allocation reference of the new pages
  for (size_t i = have.size(); i < all.size(); ++i) alloc_.release(all[i]);
  if (!session.empty()) {
    SessionEntry e;
    e.tokens.assign(tokens.begin(), tokens.begin() + got * page_size_);
    sessions_[session] = std::move(e);
  }
  return out;
}

bool ContinuousBatcher::abort(int64_t id) {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) return false;
  Sequence& s = *it->second;
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  swapped_.erase(std::remove(swapped_.begin(), swapped_.end(), id), swapped_.end());
  finish(s, FinishReason::Aborted);
  return true;
}

// Recompute-style preemption: the youngest running sequence gives its pages back and re-enters the
// waiting queue (front) with its generated tokens kept; it is re-prefilled later (the prefix cache
// usually turns that into a short tail). The reference pauses on OOM (src/scheduler/batcher.rs:250-252).
bool ContinuousBatcher::preempt_one(int64_t protect_id) {
  if (running_.empty()) return false;
  int64_t victim = -1;
  // the eviction policy's order first (best victim first) ...
  for (int64_t id : victim_order_) {
    if (id == protect_id) continue;
    auto it = seqs_.find(id);
    if (it == seqs_.end() || it->second->state != SeqState::Running) continue;
    victim = id;
    break;
  }
  // ... else the youngest running sequence
  uint64_t best = 0;
  if (victim < 0) {
    for (auto& kv : running_) {
      Sequence& s = *seqs_[kv.second];
      if (s.id == protect_id) continue;
      if (victim < 0 || s.arrival >= best) {
        victim = s.id;
        best = s.arrival;
      }
    }
  }
  if (victim < 0) return false;
  Sequence& v = *seqs_[victim];
  for (auto it = running_.begin(); it != running_.end(); ++it)
    if (it->second == victim) {
      running_.erase(it);
      break;
    }
  ++v.preemptions;
  if (cfg_.preempt_swap && v.state == SeqState::Running && v.num_computed > 0) {
    // swap: the caller copies these pages to host memory before the step runs; the position is kept
    SwapItem item;
    item.seq_id = victim;
    item.pages.assign(v.block_table.begin(), v.block_table.end());
    item.num_tokens = v.num_computed;
    pending_swap_out_.push_back(std::move(item));
    free_sequence(v, false);
    v.state = SeqState::Swapped;
    swapped_.push_back(victim);
    return true;
  }
  free_sequence(v, true);
  v.state = SeqState::Paused;
  v.num_computed = 0;
  waiting_.push_front(victim);
  return true;
}

double ContinuousBatcher::memory_pressure() const {
  const int total = alloc_.num_total();
  if (total == 0) return 0.0;
  // pages only the prefix cache holds are reclaimable and do not count as pressure
  const int hard_used = total - alloc_.num_free() - prefix_.cached_pages();
  return std::max(0.0, static_cast<double>(hard_used) / total);
}

double ContinuousBatcher::fragmentation() const {
  long long used_tokens = 0;
  long long pages = 0;
  for (auto& kv : seqs_) {
    used_tokens += kv.second->num_computed;
    pages += static_cast<long long>(kv.second->block_table.size());
  }
  if (pages == 0) return 0.0;
  return std::max(0.0, 1.0 - static_cast<double>(used_tokens) / (static_cast<double>(pages) * page_size_));
}

StepPlan ContinuousBatcher::schedule() {
  StepPlan plan;
  plan.max_blocks = max_blocks_;
  plan.dec_tokens.assign(max_slots_, 0);
  plan.dec_positions.assign(max_slots_, 0);
  plan.dec_slot_mapping.assign(max_slots_, -1);
  plan.dec_ctx_lens.assign(max_slots_, 0);
  plan.dec_seq_ids.assign(max_slots_, -1);

  SystemState st = sys_;
  st.memory_pressure = memory_pressure();
  st.kv_fragmentation = fragmentation();
  st.waiting = num_waiting();
  st.running = num_running();
  const PolicyDecision dec = policy_decide(cfg_, st);
  for (int i = 0; i < dec.force_swap_out_count && static_cast<int>(running_.size()) > 1; ++i) {
    int64_t before = waiting_.empty() ? -1 : waiting_.front();
    if (!preempt_one(-1)) break;
    if (!waiting_.empty() && waiting_.front() != before) plan.preempted.push_back(waiting_.front());
  }

  int budget = cfg_.max_batch_tokens;

  // ---- 1. decode first: every running sequence advances by one token ----
  const int decode_cap = static_cast<int>(cfg_.decode_ratio_cap * cfg_.max_batch_tokens);
  std::vector<int64_t> order;
  for (auto& kv : running_) order.push_back(kv.second);
  for (int64_t id : order) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) continue;
    Sequence& s = *it->second;
    if (s.state != SeqState::Running) continue;
    if (plan.num_decode >= decode_cap || plan.num_decode >= dec.max_batch_size) break;
    // the token to feed is the last one; its KV lands at position num_computed
    while (!ensure_pages(s, s.num_computed + 1)) {
      if (!preempt_one(s.id)) break;
      plan.preempted.push_back(waiting_.front());
    }
    if (static_cast<int>(s.block_table.size()) * page_size_ < s.num_computed + 1) {
      // could not get a page even after preempting everyone else: pause this one too
      for (auto rit = running_.begin(); rit != running_.end(); ++rit)
        if (rit->second == s.id) {
          running_.erase(rit);
          break;
        }
      free_sequence(s, true);
      s.state = SeqState::Paused;
      s.num_computed = 0;
      ++s.preemptions;
      waiting_.push_front(s.id);
      plan.preempted.push_back(s.id);
      continue;
    }
    if (s.state != SeqState::Running) continue;  // it was the victim of its own growth
    write_slot_table(s);
    const int pos = s.num_computed;
    plan.dec_tokens[s.slot] = s.tokens.back();
    plan.dec_positions[s.slot] = pos;
    plan.dec_slot_mapping[s.slot] = s.block_table[pos / page_size_] * page_size_ + pos % page_size_;
    plan.dec_ctx_lens[s.slot] = pos + 1;
    plan.dec_seq_ids[s.slot] = s.id;
    ++plan.num_decode;
    --budget;
  }
  // sequences preempted above may still appear in the decode arrays: scrub them
  for (int sl = 0; sl < max_slots_; ++sl) {
    const int64_t id = plan.dec_seq_ids[sl];
    if (id < 0) continue;
    auto it = seqs_.find(id);
    if (it == seqs_.end() || it->second->state != SeqState::Running || it->second->slot != sl) {
      plan.dec_seq_ids[sl] = -1;
      plan.dec_ctx_lens[sl] = 0;
      plan.dec_slot_mapping[sl] = -1;
      --plan.num_decode;
      ++budget;
    }
  }

  // ---- 2. prefill backfill: sequences already prefilling continue, then admit from the queue ----
  std::vector<int64_t> pf_order;
  for (auto& kv : seqs_)
    if (kv.second->state == SeqState::Prefilling) pf_order.push_back(kv.first);
  std::sort(pf_order.begin(), pf_order.end(), [this](int64_t a, int64_t b) {
    return seqs_[a]->arrival < seqs_[b]->arrival;
  });

  auto add_chunk = [&](Sequence& s) -> bool {
    const int known = static_cast<int>(s.tokens.size());
    const int remaining = known - s.num_computed;
    if (remaining <= 0 || budget <= 0) return false;
    int cap = cfg_.prefill_chunk;
    if (cfg_.adaptive_chunk) {
      const double free_ratio = static_cast<double>(alloc_.num_free()) / std::max(1, num_total_pages());
      const int lo = std::min(cfg_.min_prefill_chunk, cfg_.prefill_chunk);
      if (free_ratio < 0.25) cap = lo;
      else if (free_ratio < 0.75) cap = lo + static_cast<int>((cfg_.prefill_chunk - lo) * (free_ratio - 0.25) / 0.5);
      cap = std::max(page_size_, cap / page_size_ * page_size_);      // whole pages
    }
    int chunk = std::min(remaining, std::min(budget, cap));
    // A sliver left over by the budget is not worth a launch, unless the step would otherwise be empty
    // (progress guarantee) or the configured chunk cap itself is that small.
    const int min_chunk = std::min(cfg_.min_prefill_chunk, cfg_.prefill_chunk);
    if (chunk < remaining && chunk < min_chunk && (plan.num_decode > 0 || !plan.prefill.empty())) return false;
    if (!ensure_pages(s, s.num_computed + chunk)) {
      // take what fits in the pages we can still get
      const int have = static_cast<int>(s.block_table.size()) * page_size_ - s.num_computed;
      if (have <= 0) return false;
      chunk = std::min(chunk, have);
    }
    PrefillItem item;
    item.seq_id = s.id;
    item.slot = s.slot;
    item.start = s.num_computed;
    item.len = chunk;
    item.last = (s.num_computed + chunk == known);
    const int q_start = static_cast<int>(plan.pf_tokens.size());
    for (int i = 0; i < chunk; ++i) {
      const int pos = s.num_computed + i;
      plan.pf_tokens.push_back(s.tokens[pos]);
      plan.pf_positions.push_back(pos);
      plan.pf_slot_mapping.push_back(s.block_table[pos / page_size_] * page_size_ + pos % page_size_);
    }
    plan.pf_q_start.push_back(q_start);
    plan.pf_q_len.push_back(chunk);
    plan.pf_ctx_lens.push_back(s.num_computed + chunk);
    plan.pf_slots.push_back(s.slot);
    const size_t off = plan.pf_block_tables.size();
    plan.pf_block_tables.resize(off + max_blocks_, 0);
    for (size_t i = 0; i < s.block_table.size(); ++i) plan.pf_block_tables[off + i] = s.block_table[i];
    plan.prefill.push_back(item);
    budget -= chunk;
    return true;
  };

  for (int64_t id : pf_order) {
    if (budget <= 0) break;
    add_chunk(*seqs_[id]);
  }

  // ---- 2b. swapped-out sequences come back (oldest first) as soon as their pages and a slot are free; they take the
  // pages now, the caller copies their KV back before the step runs, and they decode again from the next step on.
  // Sequences still paying for this step's preemptions never return in the same step.
  plan.swap_out = std::move(pending_swap_out_);
  pending_swap_out_.clear();
  while (!swapped_.empty() && plan.swap_out.empty()) {
    const int64_t id = swapped_.front();
    auto sit = seqs_.find(id);
    if (sit == seqs_.end()) {   // aborted while swapped out
      swapped_.pop_front();
      continue;
    }
    Sequence& s = *sit->second;
    const int need = (s.num_computed + 1 + page_size_ - 1) / page_size_;
    const int reclaimable = alloc_.num_free() + prefix_.cached_pages();
    if (free_slots_.empty() || need + cfg_.watermark_pages > reclaimable) break;
    if (!ensure_pages(s, s.num_computed + 1)) break;
    s.slot = free_slots_.back();
    free_slots_.pop_back();
    slot_owner_[s.slot] = s.id;
    s.state = SeqState::Running;
    const uint64_t key = static_cast<OrderPolicy>(cfg_.order) == OrderPolicy::StrictRequestId
                             ? static_cast<uint64_t>(s.id)
                             : s.arrival;
    running_[static_cast<int64_t>(key)] = s.id;
    write_slot_table(s);
    SwapItem item;
    item.seq_id = id;
    item.pages.assign(s.block_table.begin(), s.block_table.end());
    item.num_tokens = s.num_computed;
    plan.swap_in.push_back(std::move(item));
    swapped_.pop_front();
  }

  if (dec.admit_new_prefill && swapped_.empty()) {   // nobody new while a swapped-out sequence still waits
    if (static_cast<OrderPolicy>(cfg_.order) == OrderPolicy::StrictRequestId) {
      // paused sequences keep their place at the front; the rest is ordered by request id
      std::stable_sort(waiting_.begin(), waiting_.end(), [this](int64_t a, int64_t b) {
        const Sequence &sa = *seqs_[a], &sb = *seqs_[b];
        const bool pa = sa.state == SeqState::Paused, pb = sb.state == SeqState::Paused;
        if (pa != pb) return pa;
        return sa.id < sb.id;
      });
    }
    while (!waiting_.empty() && budget > 0) {
      if (free_slots_.empty()) break;
      if (static_cast<int>(running_.size()) + static_cast<int>(pf_order.size()) >= dec.max_batch_size) break;
      const int64_t id = waiting_.front();
      Sequence& s = *seqs_[id];
      const int known = static_cast<int>(s.tokens.size());
      // prefix reuse: bind shared full pages read-only; always leave at least one token to compute
      std::vector<int> shared;
      int matched = 0;
      if (cfg_.enable_prefix_cache && s.block_table.empty()) {
        matched = prefix_.find_longest_prefix(s.tokens.data(), known - 1, &shared);
      }
      const int first_chunk = std::min(known - matched, std::min(budget, cfg_.prefill_chunk));
      const int need_new = (matched + first_chunk + page_size_ - 1) / page_size_ - static_cast<int>(shared.size());
      const int reclaimable = alloc_.num_free() + prefix_.cached_pages() - static_cast<int>(shared.size());
      if (need_new + cfg_.watermark_pages > reclaimable) break;  // head-of-line blocks: keep order
      for (int p : shared) {
        alloc_.retain(p);
        s.block_table.push_back(p);
      }
      s.num_computed = matched;
      if (s.preemptions == 0) s.num_cached_prefix = matched;
      s.slot = free_slots_.back();
      free_slots_.pop_back();
      slot_owner_[s.slot] = s.id;
      s.state = SeqState::Prefilling;
      waiting_.pop_front();
      pf_order.push_back(id);
      if (!add_chunk(s)) {
        // no room after all: undo the admission
        for (int p : s.block_table) alloc_.release(p);
        s.block_table.clear();
        s.num_computed = 0;
        slot_owner_[s.slot] = -1;
        free_slots_.push_back(s.slot);
        s.slot = -1;
        s.state = s.preemptions ? SeqState::Paused : SeqState::Waiting;
        waiting_.push_front(id);
        pf_order.pop_back();
        break;
      }
    }
  }
  return plan;
}

void ContinuousBatcher::commit(const StepPlan& plan, const int32_t* decode_tokens, const int32_t* prefill_tokens) {
  // decode slots
  for (int sl = 0; sl < max_slots_; ++sl) {
    const int64_t id = plan.dec_seq_ids[sl];
    if (id < 0) continue;
    auto it = seqs_.find(id);
    if (it == seqs_.end()) continue;
    Sequence& s = *it->second;
    if (s.state != SeqState::Running) continue;
    s.num_computed += 1;
    const int32_t tok = decode_tokens[sl];
    s.tokens.push_back(tok);
    if (is_eos(s, tok))
      finish(s, FinishReason::Eos);
    else if (s.num_generated() >= s.sp.max_new_tokens)
      finish(s, FinishReason::Length);
  }
  // prefill items
  int k = 0;
  for (const PrefillItem& item : plan.prefill) {
    auto it = seqs_.find(item.seq_id);
    if (it == seqs_.end()) {
      if (item.last) ++k;
      continue;
    }
    Sequence& s = *it->second;
    s.num_computed = item.start + item.len;
    if (!item.last) continue;
    const int32_t tok = prefill_tokens[k++];
    // the prompt's full pages become shareable as soon as they are computed (batcher.rs:355-360)
    if (cfg_.enable_prefix_cache) {
      const int full = s.num_computed / page_size_;
      prefix_.insert(s.tokens.data(), s.num_computed, s.block_table.data(), full);
    }
    s.tokens.push_back(tok);
    s.state = SeqState::Running;
    const uint64_t key = static_cast<OrderPolicy>(cfg_.order) == OrderPolicy::StrictRequestId
                             ? static_cast<uint64_t>(s.id)
                             : s.arrival;
    running_[static_cast<int64_t>(key)] = s.id;
    write_slot_table(s);
    if (is_eos(s, tok))
      finish(s, FinishReason::Eos);
    else if (s.num_generated() >= s.sp.max_new_tokens)
      finish(s, FinishReason::Length);
  }
}

std::vector<FinishedSeq> ContinuousBatcher::pop_finished() {
  std::vector<FinishedSeq> out;
  out.swap(finished_);
  return out;
}

bool ContinuousBatcher::rollback(int64_t id, int n_tokens) {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) return false;
  Sequence& s = *it->second;
  if (n_tokens <= 0 || n_tokens > s.num_generated()) return false;
  s.tokens.resize(s.tokens.size() - n_tokens);
  s.num_computed = std::min<int>(s.num_computed, static_cast<int>(s.tokens.size()) - 1);
  const int keep = (s.num_computed + 1 + page_size_ - 1) / page_size_;
  while (static_cast<int>(s.block_table.size()) > keep) {
    alloc_.release(s.block_table.back());
    s.block_table.pop_back();
  }
  write_slot_table(s);
  return true;
}

bool ContinuousBatcher::append_tokens(int64_t id, const std::vector<int32_t>& toks) {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) return false;
  Sequence& s = *it->second;
  if (s.state != SeqState::Running) return false;
  for (int32_t t : toks) {
    s.tokens.push_back(t);
    if (is_eos(s, t)) {
      finish(s, FinishReason::Eos);
      return true;
    }
    if (s.num_generated() >= s.sp.max_new_tokens) {
      finish(s, FinishReason::Length);
      return true;
    }
  }
  return true;
}

bool ContinuousBatcher::reserve_tokens(int64_t id, int n_tokens) {
  auto it = seqs_.find(id);
  if (it == seqs_.end() || n_tokens <= 0) return false;
  Sequence& s = *it->second;
  if (s.state != SeqState::Running) return false;
  if (!ensure_pages(s, s.num_computed + n_tokens)) return false;
  write_slot_table(s);
  return true;
}

bool ContinuousBatcher::commit_tokens(int64_t id, const std::vector<int32_t>& toks) {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) return false;
  Sequence& s = *it->second;
  if (s.state != SeqState::Running) return false;
  for (int32_t t : toks) {
    s.num_computed += 1;       // the KV of the token before this one is in the cache
    s.tokens.push_back(t);
    if (is_eos(s, t)) {
      finish(s, FinishReason::Eos);
      return true;
    }
    if (s.num_generated() >= s.sp.max_new_tokens) {
      finish(s, FinishReason::Length);
      return true;
    }
  }
  return true;
}

const Sequence* ContinuousBatcher::find(int64_t id) const {
  auto it = seqs_.find(id);
  return it == seqs_.end() ? nullptr : it->second.get();
}

std::vector<int32_t> ContinuousBatcher::block_table_of(int64_t id) const {
  std::vector<int32_t> out;
  const Sequence* s = find(id);
  if (s) out.assign(s->block_table.begin(), s->block_table.end());
  return out;
}

}  // namespace gsched
