// Host-side helpers: error text, device properties, tensor-map encoding, status read-back.
#include "b2a_host.cuh"

#include <atomic>
#include <cstring>
#include <mutex>

namespace b2a {

char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

int current_device_info(DeviceInfo* info) {
    static std::mutex mu;
    static DeviceInfo cache[64];
    static bool valid[64] = {false};
    int dev = 0;
    B2A_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        return fail(B2A_ERR_CUDA, "device index %d out of range", dev);
    }
    // The tensor-map encoder is a driver entry point and needs the device's primary context to
    // be current on the calling thread.  A thread that has only ever used cached state (for
    // example an autograd worker thread whose allocations all came from a caching allocator)
    // may not have it bound yet; cudaSetDevice binds it.  Once per thread and device.
    static thread_local bool bound[64] = {false};
    if (!bound[dev]) {
        B2A_CUDA_OK(cudaSetDevice(dev));
        bound[dev] = true;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!valid[dev]) {
        DeviceInfo d{};
        d.device = dev;
        B2A_CUDA_OK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        B2A_CUDA_OK(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        B2A_CUDA_OK(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev));
        B2A_CUDA_OK(
            cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        cache[dev] = d;
        valid[dev] = true;
    }
    *info = cache[dev];
    if (info->cc_major != 10) {
        return fail(B2A_ERR_UNSUPPORTED_DEVICE,
                    "b200attn only supports Blackwell SM100. Current device capability is %d.%d",
                    info->cc_major, info->cc_minor);
    }
    return B2A_OK;
}

namespace {
std::atomic<uint32_t> g_wait_timeout_ns{kDefaultTimeoutNs};
}  // namespace

uint32_t wait_timeout_ns() { return g_wait_timeout_ns.load(std::memory_order_relaxed); }

unsigned long long completion_timeout_ns() { return 10ull * wait_timeout_ns(); }

int once_per_device(int device, int slot, int (*fn)()) {
    static std::mutex mu;
    static bool done[64][8] = {};
    if (device < 0 || device >= 64 || slot < 0 || slot >= 8) {
        return fail(B2A_ERR_CUDA, "device index %d out of range", device);
    }
    std::lock_guard<std::mutex> lock(mu);
    if (done[device][slot]) return B2A_OK;
    const int rc = fn();
    if (rc == B2A_OK) done[device][slot] = true;
    return rc;
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t err =
            cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
        if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

}  // namespace

int make_token_map(CUtensorMap* map, const void* base, uint64_t tokens, uint64_t heads,
                   uint32_t box_rows) {
    EncodeTiledFn encode = get_encode_fn();
    if (encode == nullptr) {
        return fail(B2A_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    }
    if ((reinterpret_cast<uintptr_t>(base) & 0xF) != 0) {
        return fail(B2A_ERR_INVALID_ARGUMENT, "tensor base address must be 16-byte aligned");
    }
    if (tokens == 0 || heads == 0) {
        return fail(B2A_ERR_INVALID_ARGUMENT, "tensor map needs tokens > 0 and heads > 0");
    }
    cuuint64_t dims[3] = {128, heads, tokens};
    cuuint64_t strides[2] = {256, heads * 256};
    cuuint32_t box[3] = {64, 1, box_rows};
    cuuint32_t elem_strides[3] = {1, 1, 1};
    CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                          strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) {
        return fail(B2A_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
                    static_cast<int>(res));
    }
    return B2A_OK;
}

namespace {

constexpr int kProfileSlots = 256;

struct ProfileState {
    bool enabled = false;
    int count[2] = {0, 0};
    cudaEvent_t start[2][kProfileSlots] = {};
    cudaEvent_t stop[2][kProfileSlots] = {};
};

ProfileState& profile_state() {
    static thread_local ProfileState st;
    return st;
}

}  // namespace

void profile_mark(int kernel, bool after, cudaStream_t stream) {
    ProfileState& st = profile_state();
    if (!st.enabled || kernel < 0 || kernel > 1) return;
    int idx = st.count[kernel];
    if (idx >= kProfileSlots) return;
    cudaEvent_t* ev = after ? &st.stop[kernel][idx] : &st.start[kernel][idx];
    if (*ev == nullptr && cudaEventCreate(ev) != cudaSuccess) return;
    cudaEventRecord(*ev, stream);
    if (after) st.count[kernel] = idx + 1;
}

}  // namespace b2a

extern "C" {

int b2a_profile_enable(int enable) {
    b2a::ProfileState& st = b2a::profile_state();
    st.enabled = enable != 0;
    st.count[0] = st.count[1] = 0;
    return B2A_OK;
}

int b2a_profile_read(int kernel, float* ms, int capacity) {
    using namespace b2a;
    B2A_REQUIRE(kernel == 0 || kernel == 1, "kernel must be B2A_KERNEL_FWD or B2A_KERNEL_BWD");
    B2A_REQUIRE(ms != nullptr && capacity >= 0, "ms must not be NULL");
    ProfileState& st = profile_state();
    int n = st.count[kernel] < capacity ? st.count[kernel] : capacity;
    for (int i = 0; i < n; ++i) {
        B2A_CUDA_OK(cudaEventSynchronize(st.stop[kernel][i]));
        B2A_CUDA_OK(cudaEventElapsedTime(&ms[i], st.start[kernel][i], st.stop[kernel][i]));
    }
    return n;
}

int b2a_abi_version(void) { return 2; }

const char* b2a_last_error(void) { return b2a::error_buffer(); }

int b2a_set_wait_timeout_ns(uint64_t nanoseconds) {
    using namespace b2a;
    if (nanoseconds == 0) nanoseconds = kDefaultTimeoutNs;
    B2A_REQUIRE(nanoseconds >= 1000 && nanoseconds <= kMaxTimeoutNs,
                "wait timeout must be between 1000 ns and %u ns (0 restores the default), got %llu",
                kMaxTimeoutNs, static_cast<unsigned long long>(nanoseconds));
    g_wait_timeout_ns.store(static_cast<uint32_t>(nanoseconds), std::memory_order_relaxed);
    return B2A_OK;
}

int b2a_check_status(const void* workspace, void* cuda_stream) {
    using namespace b2a;
    if (workspace == nullptr) {
        // The scratch of b2a_fwd_noalloc lives inside the library; its header is read the same way.
        void* scratch = nullptr;
        const int rc = noalloc_scratch_ptr(&scratch);
        if (rc != B2A_OK) return rc;
        workspace = scratch;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    WorkspaceHeader hdr{};
    B2A_CUDA_OK(cudaMemcpyAsync(&hdr, workspace, sizeof(hdr), cudaMemcpyDeviceToHost, stream));
    B2A_CUDA_OK(cudaStreamSynchronize(stream));
    if (hdr.status != 0) {
        unsigned code = hdr.status >> 24;
        unsigned detail = hdr.status & 0xFFFFFFu;
        return fail(B2A_ERR_DEVICE_STATUS,
                    "device status 0x%08x: %s (wait site %u, CTA %u)", hdr.status,
                    code == 1 ? "bounded wait timed out" : "device-side check failed",
                    detail >> 12, detail & 0xFFFu);
    }
    return B2A_OK;
}

}  // extern "C"
