// Host-side helpers shared by the C-ABI entry points: error text, device checks,
// tensor-map construction, workspace layout.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/b200attn.h"

namespace b2a {

// Thread-local error text behind b2a_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define B2A_CUDA_OK(expr)                                                             \
    do {                                                                              \
        cudaError_t err__ = (expr);                                                   \
        if (err__ != cudaSuccess) {                                                   \
            return ::b2a::fail(B2A_ERR_CUDA, "%s failed: %s", #expr,                  \
                               cudaGetErrorString(err__));                            \
        }                                                                             \
    } while (0)

#define B2A_REQUIRE(cond, ...)                                         \
    do {                                                               \
        if (!(cond)) {                                                 \
            return ::b2a::fail(B2A_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
        }                                                              \
    } while (0)

struct DeviceInfo {
    int device;
    int sm_count;
    int cc_major;
    int cc_minor;
    int max_smem_optin;
};

// Cached per-device properties of the current device (requires compute capability 10.x).
int current_device_info(DeviceInfo* info);

// 3-D tiled tensor map over a flat bf16 [tokens, heads, 128] tensor with a
// (64 columns, 1 head, box_rows tokens) box and 128-byte swizzle.
int make_token_map(CUtensorMap* map, const void* base, uint64_t tokens, uint64_t heads,
                   uint32_t box_rows);

// Header words at the start of every workspace.
struct WorkspaceHeader {
    int sched_counter;        // dynamic tile scheduler ticket
    int num_entries;          // varlen: number of planned work-list entries
    unsigned int status;      // device status word (0 = ok)
    int reserved;
};
static_assert(sizeof(WorkspaceHeader) == 16, "workspace header is 16 bytes");

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Upper bound on work-list entries when documents are cut into `rows`-token pieces.
inline size_t max_entries(int batch, int total_tokens, int rows) {
    return static_cast<size_t>(total_tokens) / rows + static_cast<size_t>(batch) + 1;
}

constexpr uint32_t kDefaultTimeoutNs = 2000000000u;   // bounded device waits: 2 s
constexpr uint32_t kMaxTimeoutNs = 4000000000u;       // the waits compare 32-bit nanosecond timers

// Limit of every bounded device-side wait of launches made from now on (b2a_set_wait_timeout_ns).
uint32_t wait_timeout_ns();
// Limit of the cross-rank completion wait that ends the context-parallel backward: ten times
// the limit above, because it covers the other ranks' whole backward launch and their launch skew.
unsigned long long completion_timeout_ns();

// Device address of the scratch array built into the library for b2a_fwd_noalloc (looked up
// once per device with cudaGetSymbolAddress; defined beside the array in b2a_fwd.cu).
int noalloc_scratch_ptr(void** out);

// Runs `fn` once per (device, slot) under a lock; used for cudaFuncSetAttribute calls.
// Returns fn's code the first time and B2A_OK afterwards.
int once_per_device(int device, int slot, int (*fn)());

// Raises the dynamic shared-memory limit of the forward kernel once per device (b2a_fwd.cu).
int configure_fwd_kernel(const DeviceInfo& dev, bool merge);

// Planner launch (b2a_plan.cu).  kind 0: forward items (256 query rows of a
// document, cost = visible key blocks).  kind 1: backward items (128 key rows
// of a document, cost = query tiles that see them).
int launch_varlen_plan(int kind, const int* cu_seqlens_q, const int* cu_seqlens_k, int batch,
                       int causal, int2* work_list, int* num_entries, int max_entries_cap,
                       cudaStream_t stream);

// Optional per-thread kernel timing (b2a_profile_enable / b2a_profile_read).  The launchers
// call profile_mark(kind, false, stream) right before and profile_mark(kind, true, stream)
// right after the main kernel launch; both are no-ops unless profiling is enabled.
void profile_mark(int kernel, bool after, cudaStream_t stream);

}  // namespace b2a
