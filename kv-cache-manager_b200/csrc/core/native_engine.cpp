#include "native_engine.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <stdexcept>

namespace kvcm {

namespace {
constexpr int kBatchBuckets[] = {1, 2, 4, 8, 16, 32, 64, 128, 256, 512};
constexpr int kMinCtxBucket = 256;
const char* const kFamilies[] = {"gemm_stream", "gemm_tcgen05", "gemm_tcgen05_pair", "gemm_tcgen05_splitk",
                                 "attention_tcgen05"};
}  // namespace

int NativeEngine::batch_bucket(int n) {
  for (int b : kBatchBuckets)
    if (n <= b) return b;
  return (n + 255) / 256 * 256;
}

int NativeEngine::ctx_bucket(int n) {
  int b = kMinCtxBucket;
  while (b < n) b *= 2;
  return b;
}

void NativeEngine::check(int rc, const char* what) const {
  if (rc != 0) throw std::runtime_error(std::string("engine: ") + what + " failed with code " + std::to_string(rc));
}

NativeEngine::NativeEngine(KVManager& kv, Scheduler& sched, NativeModel model, NativeEngineConfig cfg,
                           const KvcmDeviceBackend& backend)
    : kv_(kv), sched_(sched), model_(std::move(model)), cfg_(cfg), dev_(backend),
      builder_(cfg.block_size, (cfg.max_seq_len + cfg.block_size - 1) / cfg.block_size, cfg.num_groups, cfg.tile_rows) {
  if (model_.layers.empty() || model_.H <= 0 || model_.V <= 0 || model_.nkv <= 0 || model_.nh % model_.nkv)
    throw std::invalid_argument("NativeEngine: the model's sizes are incomplete");
  if (cfg_.num_groups < 1 || cfg_.num_groups > KVCM_FORWARD_MAX_GROUPS)
    throw std::invalid_argument("NativeEngine: between 1 and " + std::to_string(KVCM_FORWARD_MAX_GROUPS) + " layer groups");
  if (cfg_.max_rows < cfg_.max_seqs) cfg_.max_rows = cfg_.max_seqs;
  max_logits_ = std::max(cfg_.max_seqs, batch_bucket(cfg_.max_seqs));
  const int pad_rows = std::max(cfg_.max_rows, max_logits_);
  capacity_ = builder_.capacity_for(pad_rows, max_logits_, max_logits_);
  check(dev_.stream_create(&stream_), "creating the stream");
  for (int i = 0; i < 2; ++i) {
    check(dev_.event_create(&ev0_[i]), "creating an event");
    check(dev_.event_create(&ev1_[i]), "creating an event");
    check(dev_.event_create(&done_[i]), "creating an event");
  }

  auto device = [&](size_t bytes) {
    void* p = nullptr;
    check(dev_.device_alloc(&p, bytes), "device allocation");
    device_allocs_.push_back(p);
    return p;
  };
  auto host = [&](size_t bytes) {
    void* p = nullptr;
    check(dev_.host_alloc(&p, bytes), "pinned host allocation");
    return p;
  };
  const size_t esz = model_.f32 ? 4 : 2;
  const size_t T = size_t(pad_rows), H = size_t(model_.H), I = size_t(model_.I);
  const size_t QK = size_t(model_.nh) * model_.hd, QKV = size_t(model_.nh + 2 * model_.nkv) * model_.hd;
  for (int i = 0; i < 2; ++i) {
    h_ints_[i] = static_cast<int32_t*>(host(size_t(capacity_) * 4));
    h_packed_[i] = static_cast<int32_t*>(host(size_t(2 + max_logits_) * 4));
  }
  d_ints_ = static_cast<int32_t*>(device(size_t(capacity_) * 4));
  d_packed_ = static_cast<int32_t*>(device(size_t(2 + max_logits_) * 4));
  sampling_bytes_ = size_t(max_logits_) * (4 + 4 + 8 + 8);
  h_sampling_ = static_cast<unsigned char*>(host(sampling_bytes_));
  d_sampling_ = static_cast<unsigned char*>(device(sampling_bytes_));
  x_ = device(T * H * 4);
  h_ = device(T * H * esz);
  proj_ = device(T * H * esz);
  qkv_ = device(T * QKV * esz);
  attn_ = device(T * QK * esz);
  gate_up_ = device(T * 2 * I * esz);
  act_ = device(T * I * esz);
  h_last_ = device(size_t(max_logits_) * H * esz);
  logits_ = device(size_t(max_logits_) * model_.V * 4);
  if (cfg_.attn_scratch_floats > 0) attn_scratch_ = device(size_t(cfg_.attn_scratch_floats) * 4);
  if (cfg_.fuse_norms && !model_.f32) norm_partials_ = device(size_t((model_.H + 15) / 16 * 16) * 4);
  if (!model_.f32) rope_table_ = device(size_t(cfg_.max_rows) * model_.hd * 4);
  if (!model_.f32 && cfg_.lib_workspace_bytes > 0) lib_ws_ = device(size_t(cfg_.lib_workspace_bytes));
}

NativeEngine::~NativeEngine() {
  if (stream_) dev_.stream_sync(stream_);
  for (auto& g : graphs_) {
    if (g.second.exec) dev_.graph_destroy(g.second.exec);
    for (void* x : g.second.exec_chained) if (x) dev_.graph_destroy(x);
    if (g.second.ints) dev_.device_free(g.second.ints);
  }
  for (void* p : device_allocs_) dev_.device_free(p);
  for (int i = 0; i < 2; ++i) {
    if (h_ints_[i]) dev_.host_free(h_ints_[i]);
    if (h_packed_[i]) dev_.host_free(h_packed_[i]);
    if (ev0_[i]) dev_.event_destroy(ev0_[i]);
    if (ev1_[i]) dev_.event_destroy(ev1_[i]);
    if (done_[i]) dev_.event_destroy(done_[i]);
  }
  if (h_sampling_) dev_.host_free(h_sampling_);
  if (stream_) dev_.stream_destroy(stream_);
}

std::vector<std::tuple<int, int, int>> NativeEngine::graph_shapes() const {
  std::vector<std::tuple<int, int, int>> v;
  for (const auto& g : graphs_) v.push_back(g.first);
  return v;
}

void NativeEngine::fill_args(KvcmForwardArgs& a, const BatchLayout& L, const int32_t* base, int max_decode_ctx) const {
  std::memset(&a, 0, sizeof a);
  a.layers = model_.layers.data();
  a.embed = reinterpret_cast<const void*>(model_.embed);
  a.final_norm = reinterpret_cast<const void*>(model_.final_norm);
  a.lm_head = reinterpret_cast<const void*>(model_.lm_head);
  a.inv_freq = reinterpret_cast<const float*>(model_.inv_freq);
  a.tokens = base + L.off_tokens;
  a.positions = base + L.off_positions;
  a.row_seq = base + L.off_row_seq;
  a.seq_q_start = base + L.off_seq_q_start;
  a.seq_q_len = base + L.off_seq_q_len;
  a.seq_ctx_len = base + L.off_seq_ctx_len;
  a.tile_seq = base + L.off_tile_seq;
  a.tile_q0 = base + L.off_tile_q0;
  a.logit_rows = base + L.off_logit_rows;
  for (int g = 0; g < L.groups; ++g) {
    a.group_tables[g] = base + L.off_block_tables + int64_t(g) * L.seqs * L.max_blocks;
    a.group_slots[g] = base + L.off_slot_mapping + int64_t(g) * L.rows;
  }
  a.x = static_cast<float*>(x_);
  a.h = h_; a.qkv = qkv_; a.attn = attn_; a.proj = proj_; a.gate_up = gate_up_; a.act = act_; a.h_last = h_last_;
  a.logits = static_cast<float*>(logits_);
  a.attn_scratch = static_cast<float*>(attn_scratch_);
  a.attn_scratch_floats = attn_scratch_ ? cfg_.attn_scratch_floats : 0;
  a.rope_table = static_cast<float*>(rope_table_);
  a.rope_table_floats = rope_table_ ? (long long)cfg_.max_rows * model_.hd : 0;
  a.norm_partials = static_cast<float*>(norm_partials_);
  a.norm_partials_floats = norm_partials_ ? (model_.H + 15) / 16 * 16 : 0;
  a.lib_workspace = lib_ws_;
  a.lib_workspace_bytes = lib_ws_ ? cfg_.lib_workspace_bytes : 0;
  a.num_layers = static_cast<int>(model_.layers.size());
  a.f32 = model_.f32;
  a.H = model_.H; a.I = model_.I; a.nh = model_.nh; a.nkv = model_.nkv; a.hd = model_.hd; a.V = model_.V;
  a.block_size = cfg_.block_size;
  a.max_blocks = L.max_blocks;
  a.sm_count = model_.sm_count;
  a.rows = L.rows;
  a.seqs = L.seqs;
  a.decode_seqs = L.decode_seqs + (L.seqs - L.real_seqs);      // padding entries are single rows too
  a.prefill_tiles = L.prefill_tiles;
  a.tile_rows = L.tile_rows;
  a.max_decode_ctx = max_decode_ctx;
  a.num_logits = L.logit_rows;
  a.final_eps = model_.final_eps;
  a.scale = model_.scale;
}

// Per-row sampling parameters of the plan's entries that sample, rows beyond them greedy.
void NativeEngine::stage_sampling(const std::vector<ScheduledSeq>& plan, int rows) {
  const size_t R = size_t(max_logits_);
  float* temps = reinterpret_cast<float*>(h_sampling_);
  int32_t* pos = reinterpret_cast<int32_t*>(h_sampling_ + 4 * R);
  uint64_t* seeds = reinterpret_cast<uint64_t*>(h_sampling_ + 8 * R);
  int64_t* ids = reinterpret_cast<int64_t*>(h_sampling_ + 16 * R);
  int n = 0;
  for (const ScheduledSeq& p : plan) {
    if (!p.wants_logits) continue;
    temps[n] = p.seq->sampling.temperature;
    pos[n] = p.start + p.num_tokens;
    seeds[n] = p.seq->sampling.seed;
    ids[n] = p.seq->id;
    ++n;
  }
  for (; n < rows; ++n) { temps[n] = 0.f; pos[n] = 0; seeds[n] = 0; ids[n] = 0; }
  check(dev_.copy_to_device(d_sampling_, h_sampling_, sampling_bytes_, stream_), "copying the sampling parameters");
}

int NativeEngine::run_device(const KvcmForwardArgs& a, int logit_rows, bool tempered, const int32_t* fetch_from,
                             int32_t* fetch_to, long long fetch_ints, int32_t* mirror) {
  int launches = 0, extra = 0;
  if (fetch_from != nullptr) {
    check(dev_.fetch_ints(fetch_from, fetch_to, fetch_ints, stream_), "fetching the batch");
    extra = 1;
  }
  check(dev_.forward(&a, &launches, stream_), "the forward pass");
  launches += extra;
  if (logit_rows > 0) {
    const size_t R = size_t(max_logits_);
    if (tempered)
      check(dev_.sample(static_cast<const float*>(logits_), reinterpret_cast<const float*>(d_sampling_),
                        reinterpret_cast<const unsigned long long*>(d_sampling_ + 8 * R),
                        reinterpret_cast<const long long*>(d_sampling_ + 16 * R),
                        reinterpret_cast<const int*>(d_sampling_ + 4 * R), d_packed_ + 2, logit_rows, model_.V, d_packed_,
                        stream_),
            "the sampling kernel");
    else
      check(dev_.argmax(static_cast<const float*>(logits_), d_packed_ + 2, logit_rows, model_.V, d_packed_, mirror,
                        stream_),
            "the argmax kernel");
    ++launches;
  }
  return launches;
}

void NativeEngine::raise_status(int first, int word) {
  dev_.clear_errors();
  const int n = int(sizeof(kFamilies) / sizeof(kFamilies[0]));
  const std::string name = (first >= 1 && first <= n) ? kFamilies[first - 1] : "family " + std::to_string(first);
  throw std::runtime_error(name + ": a bounded wait ran out on the device (code " + std::to_string((word >> 16) & 0xffff) +
                           ", block " + std::to_string(word & 0xffff) + "); the outputs of this step are not valid");
}

NativeEngine::Planned NativeEngine::summarise() {
  Planned p;
  entries_.clear();
  for (const ScheduledSeq& q : sched_.plan()) {
    p.rows += q.num_tokens;
    p.wants += q.wants_logits;
    if (q.is_prefill) p.prefill += q.num_tokens;
    p.singles += q.num_tokens == 1;
    p.tempered += q.wants_logits && q.seq->sampling.temperature > 0.f;
    BatchEntry e;
    e.seq = q.seq.get();
    e.start = q.start;
    e.num_tokens = q.num_tokens;
    if (q.wants_logits) e.want.push_back(q.num_tokens - 1);
    entries_.push_back(std::move(e));
  }
  p.n = static_cast<int>(sched_.plan().size());
  if (p.rows > cfg_.max_rows || p.n > cfg_.max_seqs)
    throw std::runtime_error("engine: a step of " + std::to_string(p.rows) + " rows / " + std::to_string(p.n) +
                             " requests exceeds the limits " + std::to_string(cfg_.max_rows) + " / " +
                             std::to_string(cfg_.max_seqs));
  return p;
}

// Records the forms of a decode shape: token ids from the batch arrays and copies by command (the
// first step of a run of decode steps), and the chained form of the lookahead, once per pair of
// pinned buffers: token ids from the sampled tokens of the step before, the batch arrays fetched by a
// kernel, the tokens written to pinned memory by the sampling kernel.
void NativeEngine::record_shape(Captured& c, const KvcmForwardArgs& args, int b, bool tempered) {
  for (int form = 0; form < 3; ++form) {
    KvcmForwardArgs a = args;
    if (form > 0) a.tokens = d_packed_ + 2;
    void** exec = form == 0 ? &c.exec : &c.exec_chained[form - 1];
    int rc = dev_.graph_begin(stream_);
    if (rc == 0) {
      try {
        if (form == 0) run_device(a, b, tempered);
        else run_device(a, b, tempered, h_ints_[form - 1], c.ints, (c.total_ints + 3) / 4 * 4, h_packed_[form - 1]);
      } catch (...) {
        void* dead = nullptr;
        dev_.graph_end(stream_, &dead);
        if (dead) dev_.graph_destroy(dead);
        throw;
      }
      rc = dev_.graph_end(stream_, exec);
    }
    check(rc, "recording a CUDA graph");
    if (tempered || !cfg_.lookahead) break;               // the chained forms serve greedy steps only
  }
}

// The plan as schedule() made it, run to its end before this returns.
NativeStepInfo NativeEngine::run_planned(const Planned& p, double t_start) {
  NativeStepInfo info;
  const std::vector<ScheduledSeq>& plan = sched_.plan();
  const int par = int(step_no_++ & 1);
  const double t_scheduled = now();
  double t_built = t_scheduled, t_enqueued = t_scheduled;
  const int n = p.n, wants = p.wants;
  const bool decode_only = cfg_.graphs && p.singles == n && wants == n;
  KvcmForwardArgs args;
  if (decode_only) {
    const int b = std::min(batch_bucket(n), std::max(max_logits_, n));
    const BatchLayout L = builder_.build(entries_, h_ints_[par], capacity_, b, b, b);
    t_built = now();
    const auto key = std::make_tuple(b, ctx_bucket(L.max_decode_ctx), p.tempered > 0 ? 1 : 0);
    if (p.tempered > 0) stage_sampling(plan, b);
    auto it = graphs_.find(key);
    if (it == graphs_.end()) {
      // Record this shape.  The step at hand runs eagerly first (lazy set-up of kernels and of the
      // library must not fall into a recording, and a recording runs nothing): it is the real run.
      Captured c;
      void* ints = nullptr;
      check(dev_.device_alloc(&ints, size_t((L.total_ints + 3) / 4 * 4) * 4), "device allocation for a graph");
      c.ints = static_cast<int32_t*>(ints);
      c.total_ints = L.total_ints;
      try {
        check(dev_.copy_to_device(c.ints, h_ints_[par], size_t(L.total_ints) * 4, stream_), "copying the batch");
        fill_args(args, L, c.ints, std::get<1>(key));
        if (timing_) check(dev_.event_record(ev0_[par], stream_), "recording an event");
        c.launches = run_device(args, b, p.tempered > 0);
        if (timing_) check(dev_.event_record(ev1_[par], stream_), "recording an event");
        check(dev_.copy_to_host(h_packed_[par], d_packed_, size_t(2 + n) * 4, stream_), "reading the tokens back");
        check(dev_.stream_sync(stream_), "waiting for the step");
        record_shape(c, args, b, p.tempered > 0);
      } catch (...) {
        if (c.exec) dev_.graph_destroy(c.exec);
        for (void* x : c.exec_chained) if (x) dev_.graph_destroy(x);
        dev_.device_free(c.ints);
        throw;
      }
      graphs_[key] = c;
      info.launches = c.launches;
    } else {
      Captured& c = it->second;
      if (c.total_ints != L.total_ints) throw std::runtime_error("engine: batch layout changed for a recorded shape");
      check(dev_.copy_to_device(c.ints, h_ints_[par], size_t(L.total_ints) * 4, stream_), "copying the batch");
      if (timing_) check(dev_.event_record(ev0_[par], stream_), "recording an event");
      check(dev_.graph_launch(c.exec, stream_), "launching a CUDA graph");
      if (timing_) check(dev_.event_record(ev1_[par], stream_), "recording an event");
      check(dev_.copy_to_host(h_packed_[par], d_packed_, size_t(2 + n) * 4, stream_), "reading the tokens back");
      t_enqueued = now();
      check(dev_.stream_sync(stream_), "waiting for the step");
      ++replays_;
      info.launches = c.launches;
      info.graph = true;
    }
    info.h2d_bytes = L.total_ints * 4 + (p.tempered > 0 ? static_cast<long long>(sampling_bytes_) : 0);
  } else {
    const BatchLayout L = builder_.build(entries_, h_ints_[par], capacity_);
    t_built = now();
    check(dev_.copy_to_device(d_ints_, h_ints_[par], size_t(L.total_ints) * 4, stream_), "copying the batch");
    if (wants > 0 && p.tempered > 0) stage_sampling(plan, wants);
    fill_args(args, L, d_ints_, L.max_decode_ctx);
    if (timing_) check(dev_.event_record(ev0_[par], stream_), "recording an event");
    info.launches = run_device(args, wants, p.tempered > 0);
    if (timing_) check(dev_.event_record(ev1_[par], stream_), "recording an event");
    if (wants > 0)
      check(dev_.copy_to_host(h_packed_[par], d_packed_, size_t(2 + wants) * 4, stream_), "reading the tokens back");
    t_enqueued = now();
    check(dev_.stream_sync(stream_), "waiting for the step");
    info.h2d_bytes = L.total_ints * 4 + (wants > 0 && p.tempered > 0 ? static_cast<long long>(sampling_bytes_) : 0);
  }
  if (timing_) {
    float ms = 0.f;
    check(dev_.event_elapsed_ms(ev0_[par], ev1_[par], &ms), "reading the events");
    info.device_ms = ms;
    device_ms_total_ += ms;
  }
  const double t_waited = now();
  sampled_.clear();
  if (wants > 0) {
    const int32_t* packed = h_packed_[par];
    if (packed[0] != 0) raise_status(packed[0], packed[1]);
    sampled_.assign(packed + 2, packed + 2 + wants);
    info.d2h_bytes = 4ll * (2 + wants);
  }
  const double t_end = now();
  sched_.update(sampled_, t_end);
  if (t_enqueued > t_built) {                                   // (the recording step is left out)
    host_.schedule += t_scheduled - t_start;
    host_.build += t_built - t_scheduled;
    host_.enqueue += t_enqueued - t_built;
    host_.wait += t_waited - t_enqueued;
    host_.update += now() - t_waited;
    ++host_.steps;
  }
  info.rows = p.rows;
  info.seqs = n;
  info.prefill_tokens = p.prefill;
  info.decode_seqs = p.singles;
  info.sampled = wants;
  info.ms = (t_end - t_start) * 1e3;
  return info;
}

// A greedy decode step of a recorded shape, enqueued and not waited for.  `chained`: the token ids
// are the tokens that the step before it samples (it is still on the device).  False: this step
// cannot go that way (its shape is not recorded yet, or not in both forms).
bool NativeEngine::enqueue_decode(const Planned& p, bool chained, double t_start) {
  const int n = p.n;
  const int b = std::min(batch_bucket(n), std::max(max_logits_, n));
  const int par = int(step_no_ & 1);
  const BatchLayout L = builder_.build(entries_, h_ints_[par], capacity_, b, b, b);
  auto it = graphs_.find(std::make_tuple(b, ctx_bucket(L.max_decode_ctx), 0));
  if (it == graphs_.end() || it->second.exec_chained[par] == nullptr || it->second.total_ints != L.total_ints) return false;
  ++step_no_;
  Captured& c = it->second;
  if (chained) {
    // no copy commands: the recording fetches h_ints_[par] itself and writes its tokens into
    // h_packed_[par], which holds -1 until then
    for (int i = 0; i < 2 + b; ++i) h_packed_[par][i] = -1;
    std::atomic_thread_fence(std::memory_order_seq_cst);
    if (timing_) check(dev_.event_record(ev0_[par], stream_), "recording an event");
    check(dev_.graph_launch(c.exec_chained[par], stream_), "launching a CUDA graph");
    if (timing_) check(dev_.event_record(ev1_[par], stream_), "recording an event");
  } else {
    check(dev_.copy_to_device(c.ints, h_ints_[par], size_t(L.total_ints) * 4, stream_), "copying the batch");
    if (timing_) check(dev_.event_record(ev0_[par], stream_), "recording an event");
    check(dev_.graph_launch(c.exec, stream_), "launching a CUDA graph");
    if (timing_) check(dev_.event_record(ev1_[par], stream_), "recording an event");
    check(dev_.copy_to_host(h_packed_[par], d_packed_, size_t(2 + n) * 4, stream_), "reading the tokens back");
    check(dev_.event_record(done_[par], stream_), "recording an event");
  }
  ++replays_;
  flight_ = InFlight{};
  flight_.active = true;
  flight_.parity = par;
  flight_.mirrored = chained;
  flight_.timed = timing_;
  flight_.n = n;
  flight_.t_start = t_start;
  flight_.info.rows = p.rows;
  flight_.info.seqs = n;
  flight_.info.decode_seqs = p.singles;
  flight_.info.sampled = p.wants;
  flight_.info.launches = c.launches;
  flight_.info.graph = true;
  flight_.info.h2d_bytes = L.total_ints * 4;
  flight_.info.d2h_bytes = 4ll * (2 + n);
  for (const ScheduledSeq& q : sched_.plan()) {
    flight_.seqs.push_back(q.seq);
    flight_.places.push_back(q.start + q.num_tokens);          // the sampled token follows the portion
  }
  return true;
}

// The device writes a chained step's status pair and tokens straight into pinned memory: the host
// watches the words turn from -1.  Bounded: a device that never answers raises after half a minute.
void NativeEngine::wait_for_mirror(const InFlight& f) {
  const volatile int32_t* m = h_packed_[f.parity];
  const double t0 = now();
  for (int i = 0; i < 2 + f.n; ++i) {
    unsigned spins = 0;
    while (m[i] == -1) {
      if ((++spins & 0xfffff) == 0 && now() - t0 > 30.0)
        throw std::runtime_error("engine: the tokens of a decode step did not arrive within 30 s");
    }
  }
  std::atomic_thread_fence(std::memory_order_seq_cst);
}

// Waits for the tokens of a step in flight and puts them where the placeholders stand.
NativeStepInfo NativeEngine::finish(InFlight& f) {
  const double t0 = now();
  if (f.mirrored) {
    wait_for_mirror(f);
    if (f.timed) check(dev_.event_sync(ev1_[f.parity]), "waiting for the step");
  } else {
    check(dev_.event_sync(done_[f.parity]), "waiting for the step");
  }
  const double t1 = now();
  const int32_t* packed = h_packed_[f.parity];
  if (packed[0] != 0) raise_status(packed[0], packed[1]);
  if (!f.updated) {                                            // nothing was enqueued behind it
    sampled_.assign(packed + 2, packed + 2 + f.n);
    sched_.update(sampled_, t1);
  } else {
    for (int i = 0; i < f.n; ++i) f.seqs[i]->tokens[size_t(f.places[i])] = packed[2 + i];
  }
  if (f.timed) {                                               // (timing may have been switched on since it was enqueued)
    float ms = 0.f;
    check(dev_.event_elapsed_ms(ev0_[f.parity], ev1_[f.parity], &ms), "reading the events");
    f.info.device_ms = ms;
    device_ms_total_ += ms;
  }
  host_.wait += t1 - t0;
  host_.update += now() - t1;
  ++host_.steps;
  f.info.ms = (now() - f.t_start) * 1e3;
  f.active = false;
  return f.info;
}

void NativeEngine::drain() {
  if (flight_.active) ready_.push_back(finish(flight_));
}

NativeStepInfo NativeEngine::step() {
  if (!ready_.empty()) {
    NativeStepInfo info = ready_.front();
    ready_.erase(ready_.begin());
    return info;
  }
  if (!flight_.active) {
    // Nothing on the device.  Plan a step (unless the lookahead of the call before already did).
    const double t_start = planned_ ? planned_at_ : now();
    if (!planned_) sched_.schedule(t_start);
    planned_ = false;
    if (sched_.plan().empty()) return NativeStepInfo{};
    const Planned p = summarise();
    const bool greedy_decode = cfg_.graphs && cfg_.lookahead && p.singles == p.n && p.wants == p.n && p.tempered == 0;
    if (!greedy_decode || !enqueue_decode(p, false, t_start)) return run_planned(p, t_start);
    host_.schedule += now() - t_start;
  }
  // A greedy decode step is on the device.  Put placeholders where its tokens will go, so that the
  // scheduler can plan the step after it, and enqueue that one behind it if the batch stays as it is.
  InFlight cur = std::move(flight_);
  flight_ = InFlight{};
  const long long evictions = sched_.counters().preemptions;
  sampled_.assign(size_t(cur.n), 0);
  sched_.update(sampled_, now());
  cur.updated = true;
  bool same = sched_.num_waiting() == 0 && static_cast<int>(sched_.num_running()) == cur.n;
  if (same) {
    const double t_next = now();
    sched_.schedule(t_next);
    planned_ = true;
    planned_at_ = t_next;
    const std::vector<ScheduledSeq>& plan = sched_.plan();
    same = static_cast<int>(plan.size()) == cur.n && sched_.counters().preemptions == evictions;
    for (int i = 0; same && i < cur.n; ++i)
      same = plan[i].seq.get() == cur.seqs[i].get() && plan[i].num_tokens == 1 && plan[i].wants_logits &&
             plan[i].seq->sampling.temperature <= 0.f;
    if (same) {
      const Planned p = summarise();
      const double t_built = now();
      if (enqueue_decode(p, true, t_next)) {
        planned_ = false;
        ++lookahead_steps_;
        host_.schedule += t_built - t_next;
        host_.enqueue += now() - t_built;
      }
    }
  }
  return finish(cur);
}

// ------------------------------------------------------------------------ the stand-in device
namespace {

struct FakeGraph {
  std::vector<std::function<void()>> calls;
};
struct FakeState {
  bool recording = false;
  FakeGraph* open = nullptr;
  long long forward_calls = 0;
};
FakeState g_fake;

void fake_forward_now(KvcmForwardArgs a) {
  ++g_fake.forward_calls;
  // logits[r][v] = 1 at v = next_token(token, position) of the wanted row, 0 elsewhere
  for (int r = 0; r < a.num_logits; ++r) {
    const int row = a.logit_rows[r];
    float* out = a.logits + size_t(r) * a.V;
    std::fill(out, out + a.V, 0.f);
    const int pos = a.positions[row];
    if (pos >= 0) out[fake_next_token(a.tokens[row], pos, a.V)] = 1.f;
  }
}
int fake_forward(const KvcmForwardArgs* a, int* launches, void*) {
  if (launches) *launches = 1;
  if (g_fake.recording) g_fake.open->calls.push_back([args = *a] { fake_forward_now(args); });
  else fake_forward_now(*a);
  return 0;
}
void fake_argmax_now(const float* logits, int* out, int rows, int vocab, int* status, int* mirror) {
  for (int r = 0; r < rows; ++r) {
    const float* l = logits + size_t(r) * vocab;
    out[r] = static_cast<int>(std::max_element(l, l + vocab) - l);
    if (mirror) mirror[2 + r] = out[r];
  }
  if (status) status[0] = status[1] = 0;
  if (mirror) mirror[0] = mirror[1] = 0;
}
int fake_argmax(const float* logits, int* out, int rows, int vocab, int* status, int* mirror, void*) {
  if (g_fake.recording) g_fake.open->calls.push_back([=] { fake_argmax_now(logits, out, rows, vocab, status, mirror); });
  else fake_argmax_now(logits, out, rows, vocab, status, mirror);
  return 0;
}
int fake_fetch_ints(const int* src, int* dst, long long ints, void*) {
  if (g_fake.recording) g_fake.open->calls.push_back([=] { std::memcpy(dst, src, size_t(ints) * 4); });
  else std::memcpy(dst, src, size_t(ints) * 4);
  return 0;
}
int fake_sample(const float* logits, const float*, const unsigned long long*, const long long*, const int*, int* out,
                int rows, int vocab, int* status, void* s) {
  return fake_argmax(logits, out, rows, vocab, status, nullptr, s);
}
int fake_copy(void* dst, const void* src, size_t bytes, void*) { std::memcpy(dst, src, bytes); return 0; }
int fake_stream_create(void** s) { *s = reinterpret_cast<void*>(0x1); return 0; }
int fake_ok_ptr(void*) { return 0; }
int fake_alloc(void** p, size_t bytes) { *p = std::calloc(bytes ? bytes : 1, 1); return *p ? 0 : 2; }
int fake_free(void* p) { std::free(p); return 0; }
int fake_event_create(void** e) { *e = reinterpret_cast<void*>(0x2); return 0; }
int fake_event_record(void*, void*) { return 0; }
int fake_event_elapsed(void*, void*, float* ms) { *ms = 0.f; return 0; }
int fake_event_sync(void*) { return 0; }
int fake_graph_begin(void*) {
  g_fake.recording = true;
  g_fake.open = new FakeGraph();
  return 0;
}
int fake_graph_end(void*, void** exec) {
  g_fake.recording = false;
  *exec = g_fake.open;
  g_fake.open = nullptr;
  return 0;
}
int fake_graph_launch(void* exec, void*) {
  for (auto& f : static_cast<FakeGraph*>(exec)->calls) f();
  return 0;
}
int fake_graph_destroy(void* exec) { delete static_cast<FakeGraph*>(exec); return 0; }
int fake_clear() { return 0; }

}  // namespace

int32_t fake_next_token(int32_t token, int32_t position, int vocab) {
  return static_cast<int32_t>((int64_t(token) * 31 + int64_t(position) * 7 + 1) % vocab);
}
long long fake_backend_forward_calls() { return g_fake.forward_calls; }

KvcmDeviceBackend make_fake_backend() {
  KvcmDeviceBackend b{};
  b.forward = fake_forward;
  b.argmax = fake_argmax;
  b.fetch_ints = fake_fetch_ints;
  b.sample = fake_sample;
  b.copy_to_device = fake_copy;
  b.copy_to_host = fake_copy;
  b.stream_create = fake_stream_create;
  b.stream_destroy = fake_ok_ptr;
  b.stream_sync = fake_ok_ptr;
  b.device_alloc = fake_alloc;
  b.device_free = fake_free;
  b.host_alloc = fake_alloc;
  b.host_free = fake_free;
  b.event_create = fake_event_create;
  b.event_destroy = fake_ok_ptr;
  b.event_record = fake_event_record;
  b.event_elapsed_ms = fake_event_elapsed;
  b.event_sync = fake_event_sync;
  b.graph_begin = fake_graph_begin;
  b.graph_end = fake_graph_end;
  b.graph_launch = fake_graph_launch;
  b.graph_destroy = fake_graph_destroy;
  b.clear_errors = fake_clear;
  return b;
}

}  // namespace kvcm
