// Process-group bookkeeping that the reference keeps in its native distributed backend
// (cc/src/tyr_distributed.cpp): argument validation BEFORE any rendezvous (:71-90) and the table of
// pending asynchronous work handles with erase-before-wait semantics (:618-661) so a handle is
// released exactly once even when waiting on it throws.  The transport itself (NCCL / Gloo
// communicators, TCPStore) is torch's c10d; this library only owns ids and lifecycle state.
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
}  // namespace

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
TYR_HOST_EXPORT void tyr_pg_reset() {
  std::lock_guard<std::mutex> lock(g_mu);
  g_pending.clear();
  g_initialized = false;
  g_rank = 0;
  g_world = 1;
}
