// Library-wide bits: version, status text, last CUDA error per thread.
#include <stdio.h>

#include <atomic>

#include "common.cuh"

namespace b200moe {
static thread_local char g_last_error[256] = "";
static std::atomic<long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_last_error(const char* what, cudaError_t err) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(err));
}
}  // namespace b200moe

extern "C" const char* b200moe_version(void) { return "b200moe 0.1 (sm_100a)"; }

extern "C" const char* b200moe_last_error(void) { return b200moe::g_last_error; }

extern "C" long long b200moe_launch_count(void) {
  return b200moe::g_launches.load(std::memory_order_relaxed);
}

extern "C" const char* b200moe_status_string(int status) {
  switch (status) {
    case B200MOE_OK: return "ok";
    case B200MOE_INVALID_ARG: return "invalid argument";
    case B200MOE_UNSUPPORTED: return "unsupported configuration";
    case B200MOE_WORKSPACE_TOO_SMALL: return "workspace too small";
    case B200MOE_CUDA_ERROR: return "CUDA error";
    case B200MOE_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}
