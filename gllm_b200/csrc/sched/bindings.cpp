// pybind11 surface of the host scheduler (module gllm_b200._lib._sched).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "sched.hpp"

namespace py = pybind11;
using namespace gsched;

template <typename T>
static py::array_t<T> to_array(const std::vector<T>& v) {
  py::array_t<T> a(static_cast<py::ssize_t>(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

template <typename T>
static py::array_t<T> to_array_2d(const std::vector<T>& v, py::ssize_t cols) {
  const py::ssize_t rows = cols > 0 ? static_cast<py::ssize_t>(v.size()) / cols : 0;
  py::array_t<T> a({rows, cols});
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

PYBIND11_MODULE(_sched, m) {
  m.doc() = "gllm_b200 host scheduler: paged KV allocator, prefix index, continuous batcher";

  py::class_<BlockAllocator>(m, "BlockAllocator")
      .def(py::init<int>())
      .def("allocate", &BlockAllocator::allocate)
      .def("retain", &BlockAllocator::retain)
      .def("release", &BlockAllocator::release)
      .def("refcount", &BlockAllocator::refcount)
      .def_property_readonly("num_free", &BlockAllocator::num_free)
      .def_property_readonly("num_total", &BlockAllocator::num_total)
      .def("fragmentation", &BlockAllocator::fragmentation);

  py::class_<PrefixIndex>(m, "PrefixIndex")
      .def(py::init<BlockAllocator*, int>(), py::keep_alive<1, 2>())
      .def("find_longest_prefix",
           [](PrefixIndex& self, const std::vector<int32_t>& toks) {
             std::vector<int> pages;
             int n = self.find_longest_prefix(toks.data(), static_cast<int>(toks.size()), &pages);
             return py::make_tuple(n, pages);
           })
      .def("insert",
           [](PrefixIndex& self, const std::vector<int32_t>& toks, const std::vector<int>& pages) {
             self.insert(toks.data(), static_cast<int>(toks.size()), pages.data(), static_cast<int>(pages.size()));
           })
      .def("evict", &PrefixIndex::evict)
      .def_property_readonly("cached_pages", &PrefixIndex::cached_pages)
      .def_property_readonly("hits", &PrefixIndex::hits)
      .def_property_readonly("lookups", &PrefixIndex::lookups);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def(py::init([](float t, int k, float p, int n, std::vector<int32_t> eos) {
             SamplingParams s;
             s.temperature = t;
             s.top_k = k;
             s.top_p = p;
             s.max_new_tokens = n;
             s.eos_ids = std::move(eos);
             return s;
           }),
           py::arg("temperature") = 0.7f, py::arg("top_k") = 0, py::arg("top_p") = 1.0f,
           py::arg("max_new_tokens") = 256, py::arg("eos_ids") = std::vector<int32_t>{})
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("max_new_tokens", &SamplingParams::max_new_tokens)
      .def_readwrite("eos_ids", &SamplingParams::eos_ids);

  py::class_<PolicyConfig>(m, "PolicyConfig")
      .def(py::init<>())
      .def_readwrite("max_batch_size", &PolicyConfig::max_batch_size)
      .def_readwrite("max_batch_tokens", &PolicyConfig::max_batch_tokens)
      .def_readwrite("prefill_chunk", &PolicyConfig::prefill_chunk)
      .def_readwrite("min_prefill_chunk", &PolicyConfig::min_prefill_chunk)
      .def_readwrite("decode_ratio_cap", &PolicyConfig::decode_ratio_cap)
      .def_readwrite("emergency_pressure", &PolicyConfig::emergency_pressure)
      .def_readwrite("defrag_threshold", &PolicyConfig::defrag_threshold)
      .def_readwrite("watermark_pages", &PolicyConfig::watermark_pages)
      .def_readwrite("enable_prefix_cache", &PolicyConfig::enable_prefix_cache)
      .def_readwrite("preempt_swap", &PolicyConfig::preempt_swap)
      .def_readwrite("adaptive_chunk", &PolicyConfig::adaptive_chunk)
      .def_readwrite("phase_isolated", &PolicyConfig::phase_isolated)
      .def_readwrite("order", &PolicyConfig::order);

  py::class_<SystemState>(m, "SystemState")
      .def(py::init<>())
      .def_readwrite("memory_pressure", &SystemState::memory_pressure)
      .def_readwrite("kv_fragmentation", &SystemState::kv_fragmentation)
      .def_readwrite("logits_entropy", &SystemState::logits_entropy)
      .def_readwrite("attention_sparsity", &SystemState::attention_sparsity)
      .def_readwrite("waiting", &SystemState::waiting)
      .def_readwrite("running", &SystemState::running);

  py::class_<PolicyDecision>(m, "PolicyDecision")
      .def_readonly("max_batch_size", &PolicyDecision::max_batch_size)
      .def_readonly("admit_new_prefill", &PolicyDecision::admit_new_prefill)
      .def_readonly("force_swap_out_count", &PolicyDecision::force_swap_out_count);
  m.def("policy_decide", &policy_decide);

  py::class_<PrefillItem>(m, "PrefillItem")
      .def_readonly("seq_id", &PrefillItem::seq_id)
      .def_readonly("slot", &PrefillItem::slot)
      .def_readonly("start", &PrefillItem::start)
      .def_readonly("len", &PrefillItem::len)
      .def_readonly("last", &PrefillItem::last);

  py::class_<SwapItem>(m, "SwapItem")
      .def_readonly("seq_id", &SwapItem::seq_id)
      .def_readonly("pages", &SwapItem::pages)
      .def_readonly("num_tokens", &SwapItem::num_tokens);

  py::class_<StepPlan>(m, "StepPlan")
      .def_readonly("num_decode", &StepPlan::num_decode)
      .def_readonly("prefill", &StepPlan::prefill)
      .def_readonly("max_blocks", &StepPlan::max_blocks)
      .def_readonly("preempted", &StepPlan::preempted)
      .def_readonly("swap_out", &StepPlan::swap_out)
      .def_readonly("swap_in", &StepPlan::swap_in)
      .def_property_readonly("idle", &StepPlan::idle)
      .def_property_readonly("num_prefill_tokens", [](const StepPlan& p) { return p.pf_tokens.size(); })
      .def_property_readonly("num_prefill_seqs", [](const StepPlan& p) { return p.prefill.size(); })
      .def_property_readonly("num_sampled_prefill",
                             [](const StepPlan& p) {
                               int n = 0;
                               for (auto& it : p.prefill) n += it.last ? 1 : 0;
                               return n;
                             })
      .def_property_readonly("dec_tokens", [](const StepPlan& p) { return to_array(p.dec_tokens); })
      .def_property_readonly("dec_positions", [](const StepPlan& p) { return to_array(p.dec_positions); })
      .def_property_readonly("dec_slot_mapping", [](const StepPlan& p) { return to_array(p.dec_slot_mapping); })
      .def_property_readonly("dec_ctx_lens", [](const StepPlan& p) { return to_array(p.dec_ctx_lens); })
      .def_property_readonly("dec_seq_ids", [](const StepPlan& p) { return to_array(p.dec_seq_ids); })
      .def_property_readonly("pf_tokens", [](const StepPlan& p) { return to_array(p.pf_tokens); })
      .def_property_readonly("pf_positions", [](const StepPlan& p) { return to_array(p.pf_positions); })
      .def_property_readonly("pf_slot_mapping", [](const StepPlan& p) { return to_array(p.pf_slot_mapping); })
      .def_property_readonly("pf_q_start", [](const StepPlan& p) { return to_array(p.pf_q_start); })
      .def_property_readonly("pf_q_len", [](const StepPlan& p) { return to_array(p.pf_q_len); })
      .def_property_readonly("pf_ctx_lens", [](const StepPlan& p) { return to_array(p.pf_ctx_lens); })
      .def_property_readonly("pf_slots", [](const StepPlan& p) { return to_array(p.pf_slots); })
      .def_property_readonly("pf_block_tables",
                             [](const StepPlan& p) { return to_array_2d(p.pf_block_tables, p.max_blocks); })
      // packs every decode-side array into one caller-provided int32 buffer laid out as
      // [tokens | positions | slot_mapping | ctx_lens] x max_slots: one host->device copy per step
      .def("pack_decode_into",
           [](const StepPlan& p, py::array_t<int32_t, py::array::c_style> dst) {
             const size_t n = p.dec_tokens.size();
             if (static_cast<size_t>(dst.size()) < 4 * n) throw std::invalid_argument("buffer too small");
             int32_t* d = dst.mutable_data();
             std::memcpy(d, p.dec_tokens.data(), n * 4);
             std::memcpy(d + n, p.dec_positions.data(), n * 4);
             std::memcpy(d + 2 * n, p.dec_slot_mapping.data(), n * 4);
             std::memcpy(d + 3 * n, p.dec_ctx_lens.data(), n * 4);
           })
      // packs the prefill side into caller-provided (pinned) buffers, no allocation:
      //   pack = [tokens T | positions T | slot_mapping T | q_start S | q_len S | ctx_lens S | last_rows L | last_slots L]
      //   bt   = [S, max_blocks]
      // and returns (T, S, L, max_q_len); L = chunks that reach the end of their prompt (they sample a token)
      .def("pack_prefill_into",
           [](const StepPlan& p, py::array_t<int32_t, py::array::c_style> pack, py::array_t<int32_t, py::array::c_style> bt) {
             const size_t T = p.pf_tokens.size(), S = p.prefill.size();
             size_t L = 0;
             for (auto& it : p.prefill) L += it.last ? 1 : 0;
             if (static_cast<size_t>(pack.size()) < 3 * T + 3 * S + 2 * L ||
                 static_cast<size_t>(bt.size()) < p.pf_block_tables.size())
               throw std::invalid_argument("prefill staging buffers too small");
             int32_t* d = pack.mutable_data();
             std::memcpy(d, p.pf_tokens.data(), T * 4);
             std::memcpy(d + T, p.pf_positions.data(), T * 4);
             std::memcpy(d + 2 * T, p.pf_slot_mapping.data(), T * 4);
             std::memcpy(d + 3 * T, p.pf_q_start.data(), S * 4);
             std::memcpy(d + 3 * T + S, p.pf_q_len.data(), S * 4);
             std::memcpy(d + 3 * T + 2 * S, p.pf_ctx_lens.data(), S * 4);
             int32_t* rows = d + 3 * T + 3 * S;
             int32_t* slots = rows + L;
             size_t k = 0;
             int max_q = 0;
             for (size_t i = 0; i < S; ++i) {
               max_q = std::max(max_q, p.pf_q_len[i]);
               if (p.prefill[i].last) {
                 rows[k] = p.pf_q_start[i] + p.prefill[i].len - 1;
                 slots[k] = p.prefill[i].slot;
                 ++k;
               }
             }
             std::memcpy(bt.mutable_data(), p.pf_block_tables.data(), p.pf_block_tables.size() * 4);
             return py::make_tuple(T, S, L, max_q);
           });

  py::class_<FinishedSeq>(m, "FinishedSeq")
      .def_readonly("id", &FinishedSeq::id)
      .def_property_readonly("tokens", [](const FinishedSeq& f) { return to_array(f.tokens); })
      .def_readonly("prompt_len", &FinishedSeq::prompt_len)
      .def_readonly("finish", &FinishedSeq::finish)
      .def_readonly("cached_prefix", &FinishedSeq::cached_prefix)
      .def_readonly("preemptions", &FinishedSeq::preemptions);

  py::class_<ContinuousBatcher>(m, "ContinuousBatcher")
      .def(py::init<int, int, int, int, PolicyConfig>(), py::arg("num_pages"), py::arg("page_size"),
           py::arg("max_slots"), py::arg("max_blocks_per_seq"), py::arg("config") = PolicyConfig())
      .def("add_request", &ContinuousBatcher::add_request, py::arg("id"), py::arg("prompt"), py::arg("params"),
           py::arg("session") = std::string())
      .def("abort", &ContinuousBatcher::abort)
      .def("schedule", &ContinuousBatcher::schedule)
      .def("commit",
           [](ContinuousBatcher& self, const StepPlan& plan,
              py::array_t<int32_t, py::array::c_style | py::array::forcecast> dec,
              py::array_t<int32_t, py::array::c_style | py::array::forcecast> pf) {
             if (plan.num_decode > 0 && dec.size() < self.max_slots())
               throw std::invalid_argument("decode token array shorter than max_slots");
             int need = 0;
             for (auto& it : plan.prefill) need += it.last ? 1 : 0;
             if (pf.size() < need) throw std::invalid_argument("prefill token array too short");
             self.commit(plan, dec.data(), pf.data());
           })
      .def("pop_finished", &ContinuousBatcher::pop_finished)
      .def("rollback", &ContinuousBatcher::rollback)
      .def("append_tokens", &ContinuousBatcher::append_tokens)
      .def("block_table_of", &ContinuousBatcher::block_table_of)
      .def("slot_block_tables",
           [](const ContinuousBatcher& self) { return to_array_2d(self.slot_block_tables(), self.max_blocks()); })
      .def("copy_slot_block_tables_into",
           [](const ContinuousBatcher& self, py::array_t<int32_t, py::array::c_style> dst) {
             const auto& t = self.slot_block_tables();
             if (static_cast<size_t>(dst.size()) < t.size()) throw std::invalid_argument("buffer too small");
             std::memcpy(dst.mutable_data(), t.data(), t.size() * 4);
           })
      .def("state_of",
           [](const ContinuousBatcher& self, int64_t id) -> py::object {
             const Sequence* s = self.find(id);
             if (!s) return py::none();
             py::dict d;
             d["state"] = static_cast<int>(s->state);
             d["num_computed"] = s->num_computed;
             d["num_tokens"] = s->tokens.size();
             d["prompt_len"] = s->prompt_len;
             d["slot"] = s->slot;
             d["cached_prefix"] = s->num_cached_prefix;
             d["pages"] = s->block_table.size();
             d["preemptions"] = s->preemptions;
             d["num_generated"] = s->num_generated();
             d["max_new_tokens"] = s->sp.max_new_tokens;
             return d;
           })
      .def("tokens_of",
           [](const ContinuousBatcher& self, int64_t id) {
             const Sequence* s = self.find(id);
             return s ? to_array(s->tokens) : py::array_t<int32_t>(0);
           })
      .def("set_system_state", &ContinuousBatcher::set_system_state)
      .def("session_cached_tokens", &ContinuousBatcher::session_cached_tokens)
      .def("session_ids", &ContinuousBatcher::session_ids)
      .def("session_tokens", &ContinuousBatcher::session_tokens)
      .def("lookup_prefix_pages", &ContinuousBatcher::lookup_prefix_pages)
      .def("import_prefix", &ContinuousBatcher::import_prefix)
      .def_property_readonly("num_waiting", &ContinuousBatcher::num_waiting)
      .def_property_readonly("num_swapped", &ContinuousBatcher::num_swapped)
      .def("set_victim_order", &ContinuousBatcher::set_victim_order)
      .def("reserve_tokens", &ContinuousBatcher::reserve_tokens)
      .def("commit_tokens", &ContinuousBatcher::commit_tokens)
      .def_property_readonly("num_running", &ContinuousBatcher::num_running)
      .def_property_readonly("num_free_pages", &ContinuousBatcher::num_free_pages)
      .def_property_readonly("num_total_pages", &ContinuousBatcher::num_total_pages)
      .def_property_readonly("cached_pages", &ContinuousBatcher::cached_pages)
      .def_property_readonly("prefix_hits", &ContinuousBatcher::prefix_hits)
      .def_property_readonly("prefix_lookups", &ContinuousBatcher::prefix_lookups)
      .def_property_readonly("memory_pressure", &ContinuousBatcher::memory_pressure)
      .def_property_readonly("fragmentation", &ContinuousBatcher::fragmentation)
      .def_property_readonly("max_slots", &ContinuousBatcher::max_slots)
      .def_property_readonly("max_blocks", &ContinuousBatcher::max_blocks)
      .def_property_readonly("page_size", &ContinuousBatcher::page_size)
      .def_property_readonly("config", &ContinuousBatcher::config, py::return_value_policy::reference_internal);
}
