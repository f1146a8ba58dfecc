// Python bindings of the CPU core (module name: kvcm_core).  The engine, the replay tool and
// the tests all drive the same C++ objects; Python never re-implements their logic.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "batch.h"
#include "block_allocator.h"
#include "hash.h"
#include "kv_manager.h"
#include "native_engine.h"
#include "paged_manager.h"
#include "prefix_cache.h"
#include "safetensors.h"
#include "scheduler.h"
#include "sequence.h"

namespace py = pybind11;
using namespace kvcm;

namespace {

std::vector<BatchEntry> entries_from_plan(const std::vector<ScheduledSeq>& plan) {
  std::vector<BatchEntry> entries;
  entries.reserve(plan.size());
  for (const ScheduledSeq& p : plan) {
    BatchEntry e;
    e.seq = p.seq.get();
    e.start = p.start;
    e.num_tokens = p.num_tokens;
    if (p.wants_logits) e.want.push_back(p.num_tokens - 1);
    entries.push_back(std::move(e));
  }
  return entries;
}

}  // namespace

PYBIND11_MODULE(kvcm_core, m) {
  m.doc() = "CPU core: page allocator, prefix cache, cache managers, state slots, scheduler, batch builder";

  m.def("xxh64", [](py::bytes data, uint64_t seed) {
    const std::string s = data;
    return XXH64::digest(s.data(), s.size(), seed);
  }, py::arg("data"), py::arg("seed") = 0);
  m.def("page_hash", [](uint64_t parent, const std::vector<int32_t>& tokens) {
    return page_hash(parent, tokens.data(), static_cast<int>(tokens.size()));
  });

  // One memory-mapped .safetensors file.  Faults of the file raise RuntimeError with the message.
  py::class_<SafetensorsReader>(m, "SafetensorsReader")
      .def(py::init<const std::string&>())
      .def_property_readonly("path", &SafetensorsReader::path)
      .def("names", &SafetensorsReader::names)
      .def("has", &SafetensorsReader::has)
      .def("metadata", [](const SafetensorsReader& r) {
        py::dict d;
        for (const auto& kv : r.metadata()) d[py::str(kv.first)] = py::str(kv.second);
        return d;
      })
      .def("info", [](const SafetensorsReader& r, const std::string& name) {
        const SafetensorsEntry& e = r.entry(name);
        return py::make_tuple(e.dtype, e.shape, e.end - e.begin);
      }, "(dtype name, shape, bytes) of a tensor")
      .def("address", &SafetensorsReader::address, "address of the tensor's bytes inside the map")
      .def("data_bytes", &SafetensorsReader::data_bytes);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("seed", &SamplingParams::seed);

  py::class_<Sequence, std::shared_ptr<Sequence>>(m, "Sequence")
      .def(py::init<>())
      .def_readwrite("id", &Sequence::id)
      .def_readwrite("tokens", &Sequence::tokens)
      .def_readwrite("prompt_len", &Sequence::prompt_len)
      .def_readwrite("max_new_tokens", &Sequence::max_new_tokens)
      .def_readwrite("num_computed", &Sequence::num_computed)
      .def_readwrite("tables", &Sequence::tables)
      .def_readonly("window_freed", &Sequence::window_freed)
      .def_readonly("page_hashes", &Sequence::page_hashes)
      .def_readwrite("cached_tokens", &Sequence::cached_tokens)
      .def_readwrite("state_slot", &Sequence::state_slot)
      .def_readwrite("sampling", &Sequence::sampling)
      .def_readwrite("arrival", &Sequence::arrival)
      .def_readwrite("admitted", &Sequence::admitted)
      .def_readwrite("first_token", &Sequence::first_token)
      .def_readwrite("finished", &Sequence::finished)
      .def_readwrite("rejected", &Sequence::rejected)
      .def_readwrite("num_preemptions", &Sequence::num_preemptions)
      .def_readwrite("prefill_tokens_computed", &Sequence::prefill_tokens_computed)
      .def_readwrite("prefill_tokens_saved", &Sequence::prefill_tokens_saved)
      .def("length", &Sequence::length)
      .def("num_generated", &Sequence::num_generated)
      .def("append_token", [](Sequence& s, int32_t t) { s.tokens.push_back(t); })
      .def("extend_tokens", [](Sequence& s, const std::vector<int32_t>& t) {
        s.tokens.insert(s.tokens.end(), t.begin(), t.end());
      })
      .def("token_at", [](const Sequence& s, int i) { return s.tokens.at(i); })
      .def("generated", [](const Sequence& s) {
        return std::vector<int32_t>(s.tokens.begin() + s.prompt_len, s.tokens.end());
      })
      .def("table", [](const Sequence& s, int g) { return s.tables.at(g); });

  py::class_<BlockAllocator>(m, "BlockAllocator")
      .def(py::init<int>())
      .def("allocate", &BlockAllocator::allocate)
      .def("free", &BlockAllocator::free)
      .def("incref", &BlockAllocator::incref)
      .def("decref", &BlockAllocator::decref)
      .def("push_free", &BlockAllocator::push_free)
      .def("revive", &BlockAllocator::revive)
      .def("refcount", &BlockAllocator::refcount)
      .def("is_free", &BlockAllocator::is_free)
      .def("num_free", &BlockAllocator::num_free)
      .def("num_blocks", &BlockAllocator::num_blocks);

  py::class_<PrefixCacheStats>(m, "PrefixCacheStats")
      .def_readonly("queried_blocks", &PrefixCacheStats::queried_blocks)
      .def_readonly("hit_blocks", &PrefixCacheStats::hit_blocks)
      .def_readonly("inserted_blocks", &PrefixCacheStats::inserted_blocks)
      .def_readonly("evictions", &PrefixCacheStats::evictions)
      .def_readonly("duplicate_inserts", &PrefixCacheStats::duplicate_inserts);

  py::class_<PrefixCache>(m, "PrefixCache")
      .def(py::init<BlockAllocator&, int, bool>(), py::keep_alive<1, 2>())
      .def("enabled", &PrefixCache::enabled)
      .def("allocate", &PrefixCache::allocate)
      .def("release", &PrefixCache::release)
      .def("match_and_acquire", [](PrefixCache& c, const std::vector<int32_t>& tokens, int num_blocks) {
        std::vector<int32_t> pages;
        std::vector<uint64_t> hashes;
        c.match_and_acquire(tokens.data(), num_blocks, pages, hashes);
        return py::make_tuple(pages, hashes);
      })
      .def("count_match", [](const PrefixCache& c, const std::vector<int32_t>& tokens, int num_blocks) {
        int parked = 0;
        const int hits = c.count_match(tokens.data(), num_blocks, &parked);
        return py::make_tuple(hits, parked);
      })
      .def("insert", [](PrefixCache& c, int page, uint64_t parent, uint64_t hash,
                        const std::vector<int32_t>& tokens) {
        return c.insert(page, parent, hash, tokens.data());
      })
      .def("num_available", &PrefixCache::num_available)
      .def("num_cached_free", &PrefixCache::num_cached_free)
      .def("num_hashed", &PrefixCache::num_hashed)
      .def("is_hashed", &PrefixCache::is_hashed)
      .def("stats", &PrefixCache::stats)
      .def("lru_order", &PrefixCache::lru_order);

  py::class_<LayerGroupSpec>(m, "LayerGroupSpec")
      .def(py::init([](int window) { LayerGroupSpec g; g.window = window; return g; }),
           py::arg("window") = 0)
      .def_readwrite("window", &LayerGroupSpec::window);

  py::class_<KVStats>(m, "KVStats")
      .def_readonly("num_blocks", &KVStats::num_blocks)
      .def_readonly("block_size", &KVStats::block_size)
      .def_readonly("blocks_in_use", &KVStats::blocks_in_use)
      .def_readonly("blocks_cached_free", &KVStats::blocks_cached_free)
      .def_readonly("allocated_slots", &KVStats::allocated_slots)
      .def_readonly("used_slots", &KVStats::used_slots)
      .def_readonly("tail_waste_slots", &KVStats::tail_waste_slots)
      .def_readonly("reserved_unused_slots", &KVStats::reserved_unused_slots)
      .def_readonly("block_table_entries", &KVStats::block_table_entries)
      .def_readonly("num_seqs", &KVStats::num_seqs)
      .def_readonly("prefix", &KVStats::prefix)
      .def("fragmentation", &KVStats::fragmentation);

  py::class_<KVManagerConfig>(m, "KVManagerConfig")
      .def(py::init<>())
      .def_readwrite("policy", &KVManagerConfig::policy)
      .def_readwrite("num_blocks", &KVManagerConfig::num_blocks)
      .def_readwrite("block_size", &KVManagerConfig::block_size)
      .def_readwrite("max_seq_len", &KVManagerConfig::max_seq_len)
      .def_readwrite("prefix_caching", &KVManagerConfig::prefix_caching)
      .def_readwrite("watermark_blocks", &KVManagerConfig::watermark_blocks)
      .def_readwrite("watermark_frac", &KVManagerConfig::watermark_frac)
      .def_readwrite("groups", &KVManagerConfig::groups);

  py::class_<KVManager>(m, "KVManager")
      .def("name", &KVManager::name)
      .def("block_size", &KVManager::block_size)
      .def("num_blocks", &KVManager::num_blocks)
      .def("max_seq_len", &KVManager::max_seq_len)
      .def("num_groups", &KVManager::num_groups)
      .def("group_window", [](const KVManager& k, int g) { return k.group(g).window; })
      .def("can_admit", &KVManager::can_admit)
      .def("admit", &KVManager::admit)
      .def("ensure", &KVManager::ensure)
      .def("commit", &KVManager::commit)
      .def("release", &KVManager::release)
      .def("blocks_in_use", &KVManager::blocks_in_use, py::arg("group") = 0)
      .def("blocks_cached_free", &KVManager::blocks_cached_free)
      .def("prefix_stats", &KVManager::prefix_stats)
      .def("stats", [](const KVManager& k, const std::vector<std::shared_ptr<Sequence>>& live) {
        std::vector<const Sequence*> raw;
        for (const auto& q : live) raw.push_back(q.get());
        return k.stats(raw);
      });

  py::class_<PagedManager, KVManager>(m, "PagedManager")
      .def(py::init<int, int, int, bool, int, std::vector<LayerGroupSpec>>(), py::arg("num_blocks"),
           py::arg("block_size"), py::arg("max_seq_len"), py::arg("prefix_caching") = false,
           py::arg("watermark_blocks") = 0,
           py::arg("groups") = std::vector<LayerGroupSpec>{LayerGroupSpec{}})
      .def("refcount", [](const PagedManager& p, int id, int g) { return p.allocator(g).refcount(id); },
           py::arg("id"), py::arg("group") = 0)
      .def("num_free", [](const PagedManager& p, int g) { return p.allocator(g).num_free(); },
           py::arg("group") = 0)
      .def("num_available", [](const PagedManager& p, int g) { return p.cache(g).num_available(); },
           py::arg("group") = 0)
      .def("lru_order", [](const PagedManager& p) { return p.cache(0).lru_order(); })
      .def("num_hashed", [](const PagedManager& p) { return p.cache(0).num_hashed(); });

  py::class_<ContiguousManager, KVManager>(m, "ContiguousManager")
      .def(py::init<int, int, int, std::vector<LayerGroupSpec>>(), py::arg("num_blocks"),
           py::arg("block_size"), py::arg("max_seq_len"),
           py::arg("groups") = std::vector<LayerGroupSpec>{LayerGroupSpec{}})
      .def("reserve_blocks", &ContiguousManager::reserve_blocks)
      .def("num_free_extents", &ContiguousManager::num_free_extents);

  m.def("make_kv_manager", &make_kv_manager);

  py::class_<StateSlots>(m, "StateSlots")
      .def(py::init<int>())
      .def("take", &StateSlots::take)
      .def("give_back", &StateSlots::give_back)
      .def("num_slots", &StateSlots::num_slots)
      .def("num_taken", &StateSlots::num_taken)
      .def("is_taken", &StateSlots::is_taken);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_batched_tokens", &SchedulerConfig::max_batched_tokens)
      .def_readwrite("prefill_chunk", &SchedulerConfig::prefill_chunk)
      .def_readwrite("chunked_prefill", &SchedulerConfig::chunked_prefill)
      .def_readwrite("eos_token_id", &SchedulerConfig::eos_token_id);

  py::class_<ScheduledSeq>(m, "ScheduledSeq")
      .def_property_readonly("seq", [](const ScheduledSeq& p) { return p.seq; })
      .def_readonly("start", &ScheduledSeq::start)
      .def_readonly("num_tokens", &ScheduledSeq::num_tokens)
      .def_readonly("is_prefill", &ScheduledSeq::is_prefill)
      .def_readonly("wants_logits", &ScheduledSeq::wants_logits);

  py::class_<SchedulerCounters>(m, "SchedulerCounters")
      .def_readonly("steps", &SchedulerCounters::steps)
      .def_readonly("preemptions", &SchedulerCounters::preemptions)
      .def_readonly("admissions", &SchedulerCounters::admissions)
      .def_readonly("admission_blocked_steps", &SchedulerCounters::admission_blocked_steps)
      .def_readonly("rejected", &SchedulerCounters::rejected)
      .def_readonly("prefill_tokens", &SchedulerCounters::prefill_tokens)
      .def_readonly("decode_tokens", &SchedulerCounters::decode_tokens)
      .def_readonly("prefill_tokens_saved", &SchedulerCounters::prefill_tokens_saved)
      .def_readonly("batch_size_sum", &SchedulerCounters::batch_size_sum)
      .def_readonly("max_running", &SchedulerCounters::max_running);

  py::class_<BatchLayout>(m, "BatchLayout")
      .def_readonly("rows", &BatchLayout::rows)
      .def_readonly("seqs", &BatchLayout::seqs)
      .def_readonly("logit_rows", &BatchLayout::logit_rows)
      .def_readonly("groups", &BatchLayout::groups)
      .def_readonly("max_blocks", &BatchLayout::max_blocks)
      .def_readonly("real_rows", &BatchLayout::real_rows)
      .def_readonly("real_seqs", &BatchLayout::real_seqs)
      .def_readonly("decode_seqs", &BatchLayout::decode_seqs)
      .def_readonly("prefill_rows", &BatchLayout::prefill_rows)
      .def_readonly("prefill_tiles", &BatchLayout::prefill_tiles)
      .def_readonly("tile_rows", &BatchLayout::tile_rows)
      .def_readonly("max_ctx", &BatchLayout::max_ctx)
      .def_readonly("max_decode_ctx", &BatchLayout::max_decode_ctx)
      .def_readonly("max_q_len", &BatchLayout::max_q_len)
      .def_readonly("off_tokens", &BatchLayout::off_tokens)
      .def_readonly("off_positions", &BatchLayout::off_positions)
      .def_readonly("off_row_seq", &BatchLayout::off_row_seq)
      .def_readonly("off_slot_mapping", &BatchLayout::off_slot_mapping)
      .def_readonly("off_seq_q_start", &BatchLayout::off_seq_q_start)
      .def_readonly("off_seq_q_len", &BatchLayout::off_seq_q_len)
      .def_readonly("off_seq_ctx_len", &BatchLayout::off_seq_ctx_len)
      .def_readonly("off_seq_state_slot", &BatchLayout::off_seq_state_slot)
      .def_readonly("off_logit_rows", &BatchLayout::off_logit_rows)
      .def_readonly("off_tile_seq", &BatchLayout::off_tile_seq)
      .def_readonly("off_tile_q0", &BatchLayout::off_tile_q0)
      .def_readonly("off_block_tables", &BatchLayout::off_block_tables)
      .def_readonly("total_ints", &BatchLayout::total_ints)
      .def_readonly("entry_order", &BatchLayout::entry_order);

  py::class_<BatchBuilder>(m, "BatchBuilder")
      .def(py::init<int, int, int, int>(), py::arg("block_size"), py::arg("max_blocks_per_seq"),
           py::arg("num_groups"), py::arg("tile_rows"))
      .def("capacity_for", &BatchBuilder::capacity_for)
      // entries: list of (Sequence, start, num_tokens, [wanted places]); `address` is the host
      // address of an int32 buffer of `capacity` elements (e.g. a pinned torch tensor).
      .def("build", [](const BatchBuilder& b, const std::vector<std::tuple<const Sequence*, int, int, std::vector<int32_t>>>& items,
                       uintptr_t address, int64_t capacity, int pad_rows, int pad_seqs,
                       int pad_logit_rows) {
        std::vector<BatchEntry> entries;
        entries.reserve(items.size());
        for (const auto& it : items) {
          BatchEntry e;
          e.seq = std::get<0>(it);
          e.start = std::get<1>(it);
          e.num_tokens = std::get<2>(it);
          e.want = std::get<3>(it);
          entries.push_back(std::move(e));
        }
        return b.build(entries, reinterpret_cast<int32_t*>(address), capacity, pad_rows, pad_seqs,
                       pad_logit_rows);
      }, py::arg("entries"), py::arg("address"), py::arg("capacity"), py::arg("pad_rows") = 0,
         py::arg("pad_seqs") = 0, py::arg("pad_logit_rows") = 0);

  py::class_<Scheduler>(m, "Scheduler")
      .def(py::init<KVManager&, SchedulerConfig>(), py::keep_alive<1, 2>())
      .def("add_request", [](Scheduler& s, int64_t id, const std::vector<int32_t>& tokens,
                             int max_new_tokens, float temperature, uint64_t seed, double arrival) {
        auto q = std::make_shared<Sequence>();
        q->id = id;
        q->tokens = tokens;
        q->prompt_len = static_cast<int>(tokens.size());
        q->max_new_tokens = max_new_tokens;
        q->sampling.temperature = temperature;
        q->sampling.seed = seed;
        q->arrival = arrival;
        s.add(std::move(q));
      }, py::arg("id"), py::arg("tokens"), py::arg("max_new_tokens"), py::arg("temperature") = 0.f,
         py::arg("seed") = 0, py::arg("arrival") = 0.0)
      .def("schedule", [](Scheduler& s, double now) { return s.schedule(now); },
           py::return_value_policy::reference_internal)
      .def("plan", &Scheduler::plan, py::return_value_policy::reference_internal)
      // (rows, entries, entries that sample, prompt tokens, single-row entries) of the current plan
      .def("plan_summary", [](const Scheduler& s) {
        int rows = 0, wants = 0, prefill = 0, singles = 0, tempered = 0;
        for (const auto& p : s.plan()) {
          rows += p.num_tokens;
          wants += p.wants_logits;
          if (p.is_prefill) prefill += p.num_tokens;
          singles += p.num_tokens == 1;
          tempered += p.wants_logits && p.seq->sampling.temperature > 0.f;
        }
        // rows, entries, entries that sample, prompt tokens, single-row entries, entries that sample
        // with a temperature (0 = the whole step is greedy)
        return py::make_tuple(rows, static_cast<int>(s.plan().size()), wants, prefill, singles, tempered);
      })
      // Per plan entry that samples: (request id, position of the drawn token, temperature, seed)
      .def("plan_sampling", [](const Scheduler& s) {
        std::vector<int64_t> ids; std::vector<int32_t> pos; std::vector<float> temp; std::vector<uint64_t> seed;
        for (const auto& p : s.plan()) {
          if (!p.wants_logits) continue;
          ids.push_back(p.seq->id);
          pos.push_back(p.start + p.num_tokens);
          temp.push_back(p.seq->sampling.temperature);
          seed.push_back(p.seq->sampling.seed);
        }
        return py::make_tuple(ids, pos, temp, seed);
      })
      .def("build_batch", [](const Scheduler& s, const BatchBuilder& b, uintptr_t address,
                             int64_t capacity, int pad_rows, int pad_seqs, int pad_logit_rows) {
        return b.build(entries_from_plan(s.plan()), reinterpret_cast<int32_t*>(address), capacity,
                       pad_rows, pad_seqs, pad_logit_rows);
      }, py::arg("builder"), py::arg("address"), py::arg("capacity"), py::arg("pad_rows") = 0,
         py::arg("pad_seqs") = 0, py::arg("pad_logit_rows") = 0)
      .def("update", &Scheduler::update)
      .def("take_finished", [](Scheduler& s) {
        return s.take_finished();
      })
      .def("idle", &Scheduler::idle)
      .def("num_waiting", &Scheduler::num_waiting)
      .def("num_running", &Scheduler::num_running)
      .def("live", [](const Scheduler& s) {
        return std::vector<std::shared_ptr<Sequence>>(s.running().begin(), s.running().end());
      })
      // sum over running requests of the tokens whose keys and values are in the cache
      .def("cached_tokens_total", [](const Scheduler& s) {
        int64_t n = 0;
        for (const auto& q : s.running()) n += q->num_computed;
        return n;
      })
      .def("counters", &Scheduler::counters)
      .def("reset_counters", &Scheduler::reset_counters)
      .def("slots_taken", [](const Scheduler& s) { return s.slots().num_taken(); })
      .def("kv_stats", [](Scheduler& s) { return s.kv().stats(s.live()); });

  // ---- the request loop in C++ (native_engine.h)
  py::class_<NativeStepInfo>(m, "NativeStepInfo")
      .def_readonly("rows", &NativeStepInfo::rows)
      .def_readonly("seqs", &NativeStepInfo::seqs)
      .def_readonly("prefill_tokens", &NativeStepInfo::prefill_tokens)
      .def_readonly("decode_seqs", &NativeStepInfo::decode_seqs)
      .def_readonly("sampled", &NativeStepInfo::sampled)
      .def_readonly("launches", &NativeStepInfo::launches)
      .def_readonly("h2d_bytes", &NativeStepInfo::h2d_bytes)
      .def_readonly("d2h_bytes", &NativeStepInfo::d2h_bytes)
      .def_readonly("graph", &NativeStepInfo::graph)
      .def_readonly("ms", &NativeStepInfo::ms)
      .def_readonly("device_ms", &NativeStepInfo::device_ms);

  m.def("device_backend_bytes", []() { return sizeof(KvcmDeviceBackend); });
  m.def("forward_args_bytes", []() { return py::make_tuple(sizeof(KvcmForwardArgs), sizeof(KvcmForwardLayer)); });
  m.def("fake_next_token", &fake_next_token);
  m.def("fake_backend_forward_calls", &fake_backend_forward_calls);

  py::class_<NativeEngine>(m, "NativeEngine")
      // model: dict with the sizes, the device addresses of embed / final_norm / lm_head / inv_freq and
      // `layers`: a list of dicts (addresses w_qkv, w_o, w_gate_up, w_down, norm1, norm2, k_cache, v_cache;
      // eps1, eps2, group, window, writes, num_pages).  config: dict of NativeEngineConfig fields.
      // backend_address: address of a KvcmDeviceBackend filled by the kernel library, 0 = the stand-in
      // device that runs on the CPU (tests).
      .def(py::init([](KVManager& kv, Scheduler& sched, const py::dict& model, const py::dict& config,
                       uintptr_t backend_address) {
             NativeModel mm;
             auto geti = [](const py::dict& d, const char* k) { return d[k].cast<long long>(); };
             auto getf = [](const py::dict& d, const char* k) { return d[k].cast<double>(); };
             mm.embed = geti(model, "embed"); mm.final_norm = geti(model, "final_norm");
             mm.lm_head = geti(model, "lm_head"); mm.inv_freq = geti(model, "inv_freq");
             mm.f32 = int(geti(model, "f32")); mm.H = int(geti(model, "H")); mm.I = int(geti(model, "I"));
             mm.nh = int(geti(model, "nh")); mm.nkv = int(geti(model, "nkv")); mm.hd = int(geti(model, "hd"));
             mm.V = int(geti(model, "V")); mm.sm_count = int(geti(model, "sm_count"));
             mm.final_eps = float(getf(model, "final_eps")); mm.scale = float(getf(model, "scale"));
             for (const py::handle& item : model["layers"].cast<py::list>()) {
               const py::dict d = item.cast<py::dict>();
               KvcmForwardLayer L{};
               L.w_qkv = reinterpret_cast<const void*>(geti(d, "w_qkv")); L.w_o = reinterpret_cast<const void*>(geti(d, "w_o"));
               L.w_gate_up = reinterpret_cast<const void*>(geti(d, "w_gate_up"));
               L.w_down = reinterpret_cast<const void*>(geti(d, "w_down"));
               L.norm1 = reinterpret_cast<const void*>(geti(d, "norm1")); L.norm2 = reinterpret_cast<const void*>(geti(d, "norm2"));
               L.k_cache = reinterpret_cast<void*>(geti(d, "k_cache")); L.v_cache = reinterpret_cast<void*>(geti(d, "v_cache"));
               L.eps1 = float(getf(d, "eps1")); L.eps2 = float(getf(d, "eps2"));
               L.group = int(geti(d, "group")); L.window = int(geti(d, "window")); L.writes = int(geti(d, "writes"));
               L.num_pages = int(geti(d, "num_pages"));
               mm.layers.push_back(L);
             }
             NativeEngineConfig c;
             c.block_size = int(geti(config, "block_size")); c.max_seq_len = int(geti(config, "max_seq_len"));
             c.num_groups = int(geti(config, "num_groups")); c.max_rows = int(geti(config, "max_rows"));
             c.max_seqs = int(geti(config, "max_seqs")); c.graphs = config["graphs"].cast<bool>();
             if (config.contains("tile_rows")) c.tile_rows = int(geti(config, "tile_rows"));
             if (config.contains("lookahead")) c.lookahead = config["lookahead"].cast<bool>();
             if (config.contains("fuse_norms")) c.fuse_norms = config["fuse_norms"].cast<bool>();
             if (config.contains("attn_scratch_floats")) c.attn_scratch_floats = geti(config, "attn_scratch_floats");
             if (config.contains("lib_workspace_bytes")) c.lib_workspace_bytes = geti(config, "lib_workspace_bytes");
             const KvcmDeviceBackend backend = backend_address
                 ? *reinterpret_cast<const KvcmDeviceBackend*>(backend_address) : make_fake_backend();
             return std::make_unique<NativeEngine>(kv, sched, std::move(mm), c, backend);
           }), py::keep_alive<1, 2>(), py::keep_alive<1, 3>(), py::arg("kv"), py::arg("scheduler"), py::arg("model"),
           py::arg("config"), py::arg("backend_address") = 0)
      // (the step waits for the device: other Python threads may run meanwhile)
      .def("step", &NativeEngine::step, py::call_guard<py::gil_scoped_release>())
      .def("drain", &NativeEngine::drain, py::call_guard<py::gil_scoped_release>())
      .def("in_flight", &NativeEngine::in_flight)
      .def("lookahead_steps", &NativeEngine::lookahead_steps)
      .def("now", &NativeEngine::now)
      .def("reset_clock", &NativeEngine::reset_clock)
      .def("set_timing", &NativeEngine::set_timing)
      .def("device_ms_total", &NativeEngine::device_ms_total)
      .def("reset_device_ms", &NativeEngine::reset_device_ms)
      .def("graphs_captured", &NativeEngine::graphs_captured)
      .def("graph_replays", &NativeEngine::graph_replays)
      .def("graph_shapes", &NativeEngine::graph_shapes)
      .def("stream", [](const NativeEngine& e) { return reinterpret_cast<uintptr_t>(e.stream()); })
      // host microseconds per step, by phase, averaged over the steps since the last reset
      .def("host_times_us", [](const NativeEngine& e) {
        const auto& t = e.host_times();
        const double n = t.steps ? double(t.steps) : 1.0;
        py::dict d;
        d["schedule"] = 1e6 * t.schedule / n; d["build"] = 1e6 * t.build / n; d["enqueue"] = 1e6 * t.enqueue / n;
        d["wait"] = 1e6 * t.wait / n; d["update"] = 1e6 * t.update / n; d["steps"] = t.steps;
        return d;
      })
      .def("reset_host_times", &NativeEngine::reset_host_times)
      .def_static("batch_bucket", &NativeEngine::batch_bucket)
      .def_static("ctx_bucket", &NativeEngine::ctx_bucket);
}
