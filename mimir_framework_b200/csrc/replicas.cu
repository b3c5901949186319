// replicas.cu — one process driving several GPUs: a full model replica per device, the batch cut into contiguous
// per-device slices, one host thread per device, every slice's result copied straight into its place in the
// caller's (pinned) output buffer, then a host join.  There is no exchange step between the devices: samples are
// independent, so nothing but the join synchronises them.
//
// The reference is one process with one Model and a singleton Lua context (LuaScripting.cpp:625-683) whose
// forward loops over samples on the host; this is the entry point such a process calls instead of eight processes.
#include "common.h"

#include <algorithm>
#include <functional>
#include <memory>
#include <string>
#include <thread>
#include <vector>

struct MimirB200Replicas {
  std::vector<int> devices;
  std::vector<MimirB200ModelHandle> models;
  std::vector<long long> begin, end;  // batch slice of every rank in the last plan
  long long planned_total = 0;
  int pipeline = 1;
  int fail_rank = -1;                 // host-injected failure (test hook)
};

namespace mb {
namespace {

// Runs job(rank) on one host thread per rank and joins.  A failing rank does not stop the others (each works on its own
// device); the first failing rank's status is returned and the message names every rank that failed.
int fan_out(int n, const std::function<int(int)>& job, const std::function<std::string(int)>& who) {
  std::vector<int> status(static_cast<size_t>(n), MIMIR_B200_OK);
  std::vector<std::string> msg(static_cast<size_t>(n));
  std::vector<std::thread> threads;
  threads.reserve(static_cast<size_t>(n));
  for (int r = 0; r < n; ++r) {
    threads.emplace_back([&, r] {
      status[static_cast<size_t>(r)] = job(r);
      if (status[static_cast<size_t>(r)] != MIMIR_B200_OK) msg[static_cast<size_t>(r)] = last_error();  // this thread's message
    });
  }
  for (auto& t : threads) t.join();
  int first = MIMIR_B200_OK;
  std::string all;
  for (int r = 0; r < n; ++r) {
    if (status[static_cast<size_t>(r)] == MIMIR_B200_OK) continue;
    if (first == MIMIR_B200_OK) first = status[static_cast<size_t>(r)];
    if (!all.empty()) all += "; ";
    all += who(r) + ": " + msg[static_cast<size_t>(r)];
  }
  if (first != MIMIR_B200_OK) return fail(first, "%s", all.c_str());
  return MIMIR_B200_OK;
}

std::string who_of(const MimirB200Replicas* h, int r) {
  return "replica " + std::to_string(r) + " (device " + std::to_string(h->devices[static_cast<size_t>(r)]) + ")";
}

}  // namespace
}  // namespace mb

using namespace mb;

extern "C" {

int mimir_b200_shard_range(long long total, int world, int rank, long long* begin, long long* end) {
  if (total < 0 || world <= 0 || rank < 0 || rank >= world || !begin || !end) return fail(MIMIR_B200_E_INVALID, "shard_range: bad arguments");
  const long long base = total / world, extra = total % world;
  *begin = rank * base + std::min<long long>(rank, extra);
  *end = *begin + base + (rank < extra ? 1 : 0);
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_create(const int* devices, int n_devices, size_t hbm_budget_bytes, const MimirLayerDesc* layers, int n_layers,
                               int precision, MimirB200ReplicasHandle* out) {
  if (!devices || n_devices <= 0 || n_devices > MAX_DEVICES || !out) return fail(MIMIR_B200_E_INVALID, "replicas_create: bad device list");
  for (int i = 0; i < n_devices; ++i)
    for (int j = 0; j < i; ++j)
      if (devices[i] == devices[j]) return fail(MIMIR_B200_E_INVALID, "replicas_create: device %d listed twice", devices[i]);
  auto h = std::make_unique<MimirB200Replicas>();
  h->devices.assign(devices, devices + n_devices);
  h->models.assign(static_cast<size_t>(n_devices), nullptr);
  MimirB200Replicas* raw = h.get();
  const int s = fan_out(
      n_devices,
      [&](int r) -> int {
        MB_TRY(mimir_b200_init(raw->devices[static_cast<size_t>(r)], hbm_budget_bytes));  // makes the device current on this thread
        MB_TRY(mimir_b200_model_create(layers, n_layers, &raw->models[static_cast<size_t>(r)]));
        return mimir_b200_model_set_precision(raw->models[static_cast<size_t>(r)], precision);
      },
      [&](int r) { return who_of(raw, r); });
  if (s != MIMIR_B200_OK) {
    const std::string keep = last_error();
    for (auto m : raw->models)
      if (m) mimir_b200_model_destroy(m);
    return fail(s, "%s", keep.c_str());
  }
  *out = h.release();
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_destroy(MimirB200ReplicasHandle h) {
  if (!h) return MIMIR_B200_OK;
  for (auto m : h->models)
    if (m) mimir_b200_model_destroy(m);
  delete h;
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_count(MimirB200ReplicasHandle h, int* n) {
  if (!h || !n) return fail(MIMIR_B200_E_INVALID, "replicas_count: null argument");
  *n = static_cast<int>(h->devices.size());
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_upload_weights(MimirB200ReplicasHandle h, int layer_index, const float* host, uint64_t n) {
  if (!h) return fail(MIMIR_B200_E_INVALID, "replicas: null handle");
  return fan_out(
      static_cast<int>(h->devices.size()), [&](int r) { return mimir_b200_model_upload_weights(h->models[static_cast<size_t>(r)], layer_index, host, n); },
      [&](int r) { return who_of(h, r); });
}

int mimir_b200_replicas_set_pipeline(MimirB200ReplicasHandle h, int micro_batches) {
  if (!h || micro_batches < 1) return fail(MIMIR_B200_E_INVALID, "replicas_set_pipeline: bad arguments");
  h->pipeline = micro_batches;
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_plan(MimirB200ReplicasHandle h, const MimirNamedInput* inputs, int n_inputs, int batch_total, uint64_t* arena_peak_bytes) {
  if (!h || batch_total <= 0) return fail(MIMIR_B200_E_INVALID, "replicas_plan: bad arguments");
  const int n = static_cast<int>(h->devices.size());
  h->begin.assign(static_cast<size_t>(n), 0);
  h->end.assign(static_cast<size_t>(n), 0);
  for (int r = 0; r < n; ++r) MB_TRY(mimir_b200_shard_range(batch_total, n, r, &h->begin[static_cast<size_t>(r)], &h->end[static_cast<size_t>(r)]));
  std::vector<uint64_t> peak(static_cast<size_t>(n), 0);
  MB_TRY(fan_out(
      n,
      [&](int r) -> int {
        const int mine = static_cast<int>(h->end[static_cast<size_t>(r)] - h->begin[static_cast<size_t>(r)]);
        if (mine == 0) return MIMIR_B200_OK;  // more devices than samples
        // micro-batches must divide the slice: fall back to the largest divisor not above the request
        int micro = std::min(h->pipeline, mine);
        while (mine % micro != 0) --micro;
        MB_TRY(mimir_b200_model_set_pipeline(h->models[static_cast<size_t>(r)], micro));
        return mimir_b200_model_plan(h->models[static_cast<size_t>(r)], inputs, n_inputs, mine, &peak[static_cast<size_t>(r)]);
      },
      [&](int r) { return who_of(h, r); }));
  h->planned_total = batch_total;
  if (arena_peak_bytes) *arena_peak_bytes = *std::max_element(peak.begin(), peak.end());
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_inject_failure(MimirB200ReplicasHandle h, int rank) {
  if (!h || rank >= static_cast<int>(h->devices.size())) return fail(MIMIR_B200_E_INVALID, "replicas_inject_failure: bad rank");
  h->fail_rank = rank;
  return MIMIR_B200_OK;
}

int mimir_b200_replicas_forward(MimirB200ReplicasHandle h, const MimirNamedInput* inputs, int n_inputs, int batch_total, float* out_host,
                                uint64_t out_capacity, uint64_t* out_len) {
  if (!h || !inputs || n_inputs <= 0 || !out_host) return fail(MIMIR_B200_E_INVALID, "replicas_forward: bad arguments");
  if (batch_total != h->planned_total) return fail(MIMIR_B200_E_INVALID, "replicas_forward: batch %d differs from the planned %lld", batch_total, h->planned_total);
  const int n = static_cast<int>(h->devices.size());
  std::vector<uint64_t> len(static_cast<size_t>(n), 0);
  // the per-sample output length is known from the plan, so every rank gets its slice of the output buffer up front
  uint64_t per = 0;
  int first = 0;
  while (first < n && h->end[static_cast<size_t>(first)] == h->begin[static_cast<size_t>(first)]) ++first;
  if (first == n) return fail(MIMIR_B200_E_INVALID, "replicas_forward: nothing planned");
  MB_TRY(mimir_b200_model_output_len(h->models[static_cast<size_t>(first)], &per));
  if (out_len) *out_len = per;
  if (out_capacity < per * static_cast<uint64_t>(batch_total)) return fail(MIMIR_B200_E_INVALID, "replicas_forward: output capacity too small");
  const int fail_rank = h->fail_rank;
  h->fail_rank = -1;
  return fan_out(
      n,
      [&](int r) -> int {
        const long long b = h->begin[static_cast<size_t>(r)], e = h->end[static_cast<size_t>(r)];
        if (r == fail_rank) return fail(MIMIR_B200_E_INVALID, "injected failure (host side, nothing was launched)");
        if (e == b) return MIMIR_B200_OK;
        std::vector<MimirNamedInput> mine(inputs, inputs + n_inputs);
        for (auto& in : mine)
          if (!in.broadcast) in.data = in.data + static_cast<size_t>(b) * in.per_sample;
        return mimir_b200_model_forward(h->models[static_cast<size_t>(r)], mine.data(), n_inputs, static_cast<int>(e - b),
                                        out_host + static_cast<size_t>(b) * per, per * static_cast<uint64_t>(e - b), &len[static_cast<size_t>(r)]);
      },
      [&](int r) { return who_of(h, r); });
}

/* The fan-out / join of the calls above with a stand-in job that touches no device: rank `fail_rank` (if >= 0) fails on
 * the host.  Lets the reporting of a failed rank be checked on a machine without GPUs. */
int mimir_b200_replicas_selftest_join(int n_ranks, int fail_rank) {
  if (n_ranks <= 0 || n_ranks > MAX_DEVICES) return fail(MIMIR_B200_E_INVALID, "selftest_join: bad rank count");
  std::vector<int> visited(static_cast<size_t>(n_ranks), 0);
  const int s = fan_out(
      n_ranks,
      [&](int r) -> int {
        visited[static_cast<size_t>(r)] = 1;
        if (r == fail_rank) return fail(MIMIR_B200_E_INVALID, "injected failure (host side, nothing was launched)");
        return MIMIR_B200_OK;
      },
      [&](int r) { return "replica " + std::to_string(r) + " (device " + std::to_string(r) + ")"; });
  for (int v : visited)
    if (!v) return fail(MIMIR_B200_E_INVALID, "selftest_join: a rank did not run");
  return s;
}

}  // extern "C"
