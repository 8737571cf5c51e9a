// Process-group bookkeeping that the reference keeps in its native distributed backend
// (cc/src/tyr_distributed.cpp): argument validation BEFORE any rendezvous (:71-90) and the table of
// pending asynchronous work handles with erase-before-wait semantics (:618-661) so a handle is
// released exactly once even when waiting on it throws.  The transport itself (NCCL / Gloo
// communicators, TCPStore) is torch's c10d, reached through three callbacks the binding supplies (rendezvous, wait on one
// handle, shut down); the ORDER of operations is decided here: validate -> rendezvous -> mark initialised (:154-217),
// erase -> wait (:618-661), and on destroy: drain every pending handle, shut the transport down, reset the state, then
// report the first error that was seen (:260-285).
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#define TYR_HOST_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
std::mutex g_mu;
std::map<uint64_t, int> g_pending;   // handle id -> state (0 pending, 1 completed, 2 failed)
uint64_t g_next_id = 1;
bool g_initialized = false;
int g_rank = 0, g_world = 1;
std::string g_first_error;           // first failure recorded during the running lifecycle operation
}  // namespace

// Callbacks of the transport binding.  Each returns 0 on success; on failure it first calls tyr_pg_record_error.
typedef int (*tyr_pg_rendezvous_fn)(void* ctx);
typedef int (*tyr_pg_wait_fn)(void* ctx, uint64_t handle);
typedef int (*tyr_pg_shutdown_fn)(void* ctx);

TYR_HOST_EXPORT void tyr_pg_record_error(const char* message) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_first_error.empty()) g_first_error = (message && message[0]) ? message : "unknown error";
}
// Copies the first recorded error (NUL-terminated, truncated to cap) and returns its full length; 0 = none.
TYR_HOST_EXPORT long long tyr_pg_first_error(char* out, long long cap) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (out != nullptr && cap > 0) {
    const size_t n = g_first_error.size() < static_cast<size_t>(cap - 1) ? g_first_error.size() : static_cast<size_t>(cap - 1);
    memcpy(out, g_first_error.data(), n);
    out[n] = '\0';
  }
  return static_cast<long long>(g_first_error.size());
}

// 0 ok; 1 bad backend; 2 bad port; 3 bad world size; 4 bad rank; 5 empty address; 6 already initialised
TYR_HOST_EXPORT int tyr_pg_validate_init(const char* backend, const char* addr, long long port, long long rank,
                                         long long world) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_initialized) return 6;
  if (backend == nullptr || (strcmp(backend, "nccl") != 0 && strcmp(backend, "gloo") != 0)) return 1;
  if (addr == nullptr || addr[0] == '\0') return 5;
  if (port <= 0 || port > 65535) return 2;
  if (world <= 0 || world > (1 << 20)) return 3;
  if (rank < 0 || rank >= world) return 4;
  return 0;
}
TYR_HOST_EXPORT void tyr_pg_mark_initialized(long long rank, long long world) {
  std::lock_guard<std::mutex> lock(g_mu);
  g_initialized = true;
  g_rank = static_cast<int>(rank);
  g_world = static_cast<int>(world);
}
TYR_HOST_EXPORT int tyr_pg_is_initialized() {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_initialized ? 1 : 0;
}
TYR_HOST_EXPORT int tyr_pg_rank() { std::lock_guard<std::mutex> lock(g_mu); return g_rank; }
TYR_HOST_EXPORT int tyr_pg_world() { std::lock_guard<std::mutex> lock(g_mu); return g_world; }

TYR_HOST_EXPORT uint64_t tyr_pg_register_work() {
  std::lock_guard<std::mutex> lock(g_mu);
  uint64_t id = g_next_id++;
  g_pending[id] = 0;
  return id;
}
// Removes the handle from the table BEFORE the caller waits on it; returns 1 if it was pending.
TYR_HOST_EXPORT int tyr_pg_take_work(uint64_t id) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_pending.find(id);
  if (it == g_pending.end()) return 0;
  g_pending.erase(it);
  return 1;
}
TYR_HOST_EXPORT int tyr_pg_has_work(uint64_t id) {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_pending.count(id) ? 1 : 0;
}
TYR_HOST_EXPORT long long tyr_pg_pending_count() {
  std::lock_guard<std::mutex> lock(g_mu);
  return static_cast<long long>(g_pending.size());
}
// Fills `out` with up to `cap` pending ids (drain on destroy); returns the total count.
TYR_HOST_EXPORT long long tyr_pg_pending_ids(uint64_t* out, long long cap) {
  std::lock_guard<std::mutex> lock(g_mu);
  long long k = 0;
  for (auto& kv : g_pending) {
    if (k < cap) out[k] = kv.first;
    ++k;
  }
  return k;
}
// init: validate (nothing is contacted when the arguments are bad), rendezvous through the binding, then mark the group
// initialised.  Returns the validation code (1..6), 100 when the rendezvous failed (state stays uninitialised), 0 on success.
TYR_HOST_EXPORT int tyr_pg_validate_init(const char*, const char*, long long, long long, long long);
TYR_HOST_EXPORT void tyr_pg_mark_initialized(long long, long long);
TYR_HOST_EXPORT int tyr_pg_init(const char* backend, const char* addr, long long port, long long rank, long long world,
                                tyr_pg_rendezvous_fn rendezvous, void* ctx) {
  const int rc = tyr_pg_validate_init(backend, addr, port, rank, world);
  if (rc != 0) return rc;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_first_error.clear();
  }
  if (rendezvous != nullptr && rendezvous(ctx) != 0) {
    tyr_pg_record_error("rendezvous failed");
    return 100;
  }
  tyr_pg_mark_initialized(rank, world);
  return 0;
}

// wait: the handle leaves the table BEFORE the transport is asked to wait, so it is released exactly once even when the
// wait fails.  Returns 0 ok, 1 unknown / already consumed handle, 2 the wait failed (message in the error record).
TYR_HOST_EXPORT int tyr_pg_wait(uint64_t id, tyr_pg_wait_fn wait, void* ctx) {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_pending.find(id);
    if (it == g_pending.end()) return 1;
    g_pending.erase(it);
    g_first_error.clear();
  }
  if (wait != nullptr && wait(ctx, id) != 0) {
    tyr_pg_record_error("wait failed");
    return 2;
  }
  return 0;
}

// destroy: drain all pending handles (every one is waited on, failures do not stop the drain), shut the transport down,
// reset the state, and only then report: 0 clean, 2 something failed (the FIRST failure is in the error record).
TYR_HOST_EXPORT int tyr_pg_destroy(tyr_pg_wait_fn wait, tyr_pg_shutdown_fn shutdown, void* ctx) {
  std::map<uint64_t, int> pending;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    pending.swap(g_pending);
    g_first_error.clear();
  }
  bool failed = false;
  for (auto& kv : pending)
    if (wait != nullptr && wait(ctx, kv.first) != 0) {
      tyr_pg_record_error("pending work failed");
      failed = true;
    }
  if (shutdown != nullptr && shutdown(ctx) != 0) {
    tyr_pg_record_error("shutdown failed");
    failed = true;
  }
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_pending.clear();
    g_initialized = false;
    g_rank = 0;
    g_world = 1;
  }
  return failed ? 2 : 0;
}
