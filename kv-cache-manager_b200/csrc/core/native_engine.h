// The request loop in C++: one object above the scheduler, the cache manager and the batch builder
// that runs a step from "which requests, which portions" to "these tokens were sampled" without an
// interpreter in between.  API after the reference's Engine (src/engine/engine.h:29-52): add a
// request, step(), take what finished.  One step (src/engine/engine.cpp:73-90): schedule; pack the
// batch's integer arrays into one pinned buffer; one host-to-device copy; the model's forward pass
// (csrc/cuda/step_forward.cu); sampling on the device; one device-to-host copy of the sampled tokens
// with the kernels' status pair in front; one synchronisation; update the scheduler.
//
// Steps in which every request brings exactly one token are recorded once per shape (batch bucket,
// context bucket, greedy or with temperatures) as a CUDA graph and replayed: the batch is padded to
// the bucket with rows that read and write nothing; the step at hand runs eagerly while its shape is
// recorded, so no step ever runs twice.
//
// One step of lookahead: while the device runs decode step k, the host already schedules, packs and
// enqueues step k+1, whose token ids are step k's sampled tokens and therefore already lie on the
// device (a second recording of each shape reads its tokens from there).  Everything else a decode
// step needs (positions, page slots, context lengths, page tables) follows from the lengths alone.
// The host then waits for step k's tokens only, puts them into the requests, and returns step k.
// So the device never waits for the host between decode steps.  This holds only while the batch
// stays what it was: all requests decode greedily, none ends, none arrives, no page runs out; the
// moment one of these fails the loop waits for the tokens first, as before.  It is switched off where
// a token's value decides what happens next (an end-of-sequence token) or enters host state at once
// (page hashes of the prefix cache).
//
// The device is reached through a table of C functions (csrc/include/device_backend.h): the kernel
// library fills it on a GPU, a test fills it with stand-ins that run on the CPU.  This file knows
// nothing of CUDA.
#pragma once
#include <chrono>
#include <cstdint>
#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "../include/device_backend.h"
#include "../include/forward_args.h"
#include "batch.h"
#include "kv_manager.h"
#include "scheduler.h"

namespace kvcm {

// The model as the forward pass needs it: sizes and device addresses (owned by the caller).
struct NativeModel {
  std::vector<KvcmForwardLayer> layers;
  uintptr_t embed = 0, final_norm = 0, lm_head = 0, inv_freq = 0;
  int f32 = 0, H = 0, I = 0, nh = 0, nkv = 0, hd = 0, V = 0, sm_count = 0;
  float final_eps = 1e-5f, scale = 1.f;
};

struct NativeEngineConfig {
  int block_size = 16, max_seq_len = 2048, num_groups = 1;
  int max_rows = 4096, max_seqs = 256;
  int tile_rows = 64;
  bool graphs = true;
  bool fuse_norms = true;          // steps of at most 8 rows: residual add and norms inside the streaming products
  bool lookahead = true;           // enqueue the next decode step before the tokens of this one are read
  long long attn_scratch_floats = 0, lib_workspace_bytes = 32ll << 20;
};

struct NativeStepInfo {
  int rows = 0, seqs = 0, prefill_tokens = 0, decode_seqs = 0, sampled = 0, launches = 0;
  long long h2d_bytes = 0, d2h_bytes = 0;
  bool graph = false;
  double ms = 0, device_ms = 0;
};

class NativeEngine {
 public:
  NativeEngine(KVManager& kv, Scheduler& sched, NativeModel model, NativeEngineConfig cfg,
               const KvcmDeviceBackend& backend);
  ~NativeEngine();
  NativeEngine(const NativeEngine&) = delete;
  NativeEngine& operator=(const NativeEngine&) = delete;

  NativeStepInfo step();
  // Finishes a step that is still on the device (its result is handed out by the next step()).
  void drain();
  bool in_flight() const { return flight_.active; }
  long long lookahead_steps() const { return lookahead_steps_; }
  double now() const { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0_).count(); }
  void reset_clock() { t0_ = std::chrono::steady_clock::now(); }
  void set_timing(bool on) { timing_ = on; }                  // events around the device work of every step
  double device_ms_total() const { return device_ms_total_; }
  void reset_device_ms() { device_ms_total_ = 0; }
  int graphs_captured() const { return static_cast<int>(graphs_.size()); }
  long long graph_replays() const { return replays_; }
  std::vector<std::tuple<int, int, int>> graph_shapes() const;
  void* stream() const { return stream_; }
  // Host seconds spent, summed over the steps so far: scheduling, packing the batch, enqueueing the
  // step (copies and launches), waiting for the device, updating the scheduler.
  struct HostTimes { double schedule = 0, build = 0, enqueue = 0, wait = 0, update = 0; long long steps = 0; };
  const HostTimes& host_times() const { return host_; }
  void reset_host_times() { host_ = {}; }

  static int batch_bucket(int n);
  static int ctx_bucket(int n);

 private:
  struct Captured {
    void* exec = nullptr;
    // The same step with its token ids read from the sampled tokens, its batch arrays fetched from
    // pinned memory by a kernel and its tokens written to pinned memory by the sampling kernel: one per
    // pair of pinned buffers (their addresses are part of the recording).
    void* exec_chained[2] = {nullptr, nullptr};
    int32_t* ints = nullptr;                                  // the graph's own copy of the batch arrays (device)
    long long total_ints = 0;
    int launches = 0;
  };
  struct Planned {                                            // what schedule() decided, summarised
    int rows = 0, wants = 0, prefill = 0, singles = 0, tempered = 0, n = 0;
  };
  struct InFlight {                                           // a decode step enqueued and not yet read
    bool active = false, updated = false, timed = false, mirrored = false;
    int parity = 0, n = 0;
    NativeStepInfo info;
    std::vector<std::shared_ptr<Sequence>> seqs;              // the plan's requests, in order
    std::vector<int> places;                                  // where each one's sampled token goes
    double t_start = 0;
  };
  Planned summarise();
  NativeStepInfo run_planned(const Planned& p, double t_start);          // the plan made, not pipelined
  bool enqueue_decode(const Planned& p, bool chained, double t_start);   // replay of a recorded shape, not waited for
  NativeStepInfo finish(InFlight& f);                                    // wait, check, put the tokens in
  void record_shape(Captured& c, const KvcmForwardArgs& args, int b, bool tempered);
  void wait_for_mirror(const InFlight& f);
  void check(int rc, const char* what) const;
  void fill_args(KvcmForwardArgs& a, const BatchLayout& L, const int32_t* base, int max_decode_ctx) const;
  // forward + sampling; launches made.  `fetch_from` / `mirror`: the chained form (pinned buffers of one parity).
  int run_device(const KvcmForwardArgs& a, int logit_rows, bool tempered, const int32_t* fetch_from = nullptr,
                 int32_t* fetch_to = nullptr, long long fetch_ints = 0, int32_t* mirror = nullptr);
  void stage_sampling(const std::vector<ScheduledSeq>& plan, int rows);
  [[noreturn]] void raise_status(int first, int word);

  KVManager& kv_;
  Scheduler& sched_;
  NativeModel model_;
  NativeEngineConfig cfg_;
  KvcmDeviceBackend dev_;
  BatchBuilder builder_;
  void* stream_ = nullptr;
  void *ev0_[2] = {nullptr, nullptr}, *ev1_[2] = {nullptr, nullptr}, *done_[2] = {nullptr, nullptr};
  bool timing_ = false;
  double device_ms_total_ = 0;
  long long replays_ = 0;
  std::chrono::steady_clock::time_point t0_ = std::chrono::steady_clock::now();

  // host (pinned) and device buffers
  long long capacity_ = 0;
  int max_logits_ = 0;
  int32_t* h_ints_[2] = {nullptr, nullptr};                   // two of each: a step may be packed while the one
  int32_t* d_ints_ = nullptr;                                 // before it is still being copied
  int32_t* h_packed_[2] = {nullptr, nullptr};                 // [status pair | tokens]
  int32_t* d_packed_ = nullptr;
  unsigned char* h_sampling_ = nullptr;                       // temps | positions | seeds | ids
  unsigned char* d_sampling_ = nullptr;
  size_t sampling_bytes_ = 0;
  void *x_ = nullptr, *h_ = nullptr, *qkv_ = nullptr, *attn_ = nullptr, *proj_ = nullptr, *gate_up_ = nullptr,
       *act_ = nullptr, *h_last_ = nullptr, *logits_ = nullptr, *attn_scratch_ = nullptr, *lib_ws_ = nullptr,
       *norm_partials_ = nullptr, *rope_table_ = nullptr;
  std::vector<void*> device_allocs_;
  std::map<std::tuple<int, int, int>, Captured> graphs_;
  std::vector<BatchEntry> entries_;
  std::vector<int32_t> sampled_;
  HostTimes host_;
  InFlight flight_;
  bool planned_ = false;                                      // schedule() has been called for the next step already
  double planned_at_ = 0;
  long long step_no_ = 0, lookahead_steps_ = 0;
  std::vector<NativeStepInfo> ready_;                         // results of steps finished by drain()
};

// A stand-in device that runs on the CPU, for tests of the loop above: "device" memory is host
// memory, the forward pass writes logits whose maximum is a fixed function of (token, position),
// and a recorded graph replays the calls made while it was recorded (which, as on a GPU, do not run
// while they are recorded).
KvcmDeviceBackend make_fake_backend();
long long fake_backend_forward_calls();
int32_t fake_next_token(int32_t token, int32_t position, int vocab);

}  // namespace kvcm
