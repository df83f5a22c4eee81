// Peer memory over NVLink: CUDA-IPC export / import of device buffers and a peer -> local
// bulk copy kernel.  A buffer is always exported as (handle of its allocation base, byte
// offset inside the allocation), so views into a larger allocation map correctly on the
// importing side.  No multicast is used anywhere.
#include "b2a_host.cuh"
#include "b2a_ptx.cuh"

#include <cstring>

namespace b2a {
namespace {

using GetAddressRangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

GetAddressRangeFn get_address_range_fn() {
    static GetAddressRangeFn fn = []() -> GetAddressRangeFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t err = cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &qres);
        if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<GetAddressRangeFn>(ptr);
    }();
    return fn;
}

constexpr int kCopyThreads = 128;
constexpr uint32_t kCopySlotBytes = 32 * 1024;
constexpr int kCopySlots = 6;

// One CTA streams slots of 32 KiB: bulk load peer -> shared, bulk store shared -> local.
// Thread 0 drives the loads, thread 32 the stores; both waits are bounded.
__global__ void __launch_bounds__(kCopyThreads)
peer_copy_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, size_t bytes,
                 unsigned int* status, uint32_t timeout_ns) {
    extern __shared__ __align__(128) uint8_t copy_smem[];
    __shared__ uint64_t full[kCopySlots];
    __shared__ uint64_t empty[kCopySlots];
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        for (int i = 0; i < kCopySlots; ++i) {
            mbar_init(smem_u32(&full[i]), 1);
            mbar_init(smem_u32(&empty[i]), 1);
        }
        abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    __syncthreads();
    WaitCtx wctx{smem_u32(&abort_flag), status, timeout_ns};
    const size_t num_chunks = (bytes + kCopySlotBytes - 1) / kCopySlotBytes;
    const uint32_t smem_base = smem_u32(copy_smem);

    if (threadIdx.x == 0) {
        uint32_t it = 0;
        for (size_t c = blockIdx.x; c < num_chunks; c += gridDim.x, ++it) {
            const uint32_t slot = it % kCopySlots;
            if (!mbar_wait(wctx, smem_u32(&empty[slot]), ((it / kCopySlots) & 1u) ^ 1u, 1)) break;
            const size_t off = c * kCopySlotBytes;
            const uint32_t n = static_cast<uint32_t>(min(static_cast<size_t>(kCopySlotBytes), bytes - off));
            mbar_arrive_expect_tx(smem_u32(&full[slot]), n);
            bulk_load_1d(smem_base + slot * kCopySlotBytes, src + off, n, smem_u32(&full[slot]));
        }
    } else if (threadIdx.x == 32) {
        uint32_t it = 0;
        for (size_t c = blockIdx.x; c < num_chunks; c += gridDim.x, ++it) {
            const uint32_t slot = it % kCopySlots;
            if (!mbar_wait(wctx, smem_u32(&full[slot]), (it / kCopySlots) & 1u, 2)) break;
            const size_t off = c * kCopySlotBytes;
            const uint32_t n = static_cast<uint32_t>(min(static_cast<size_t>(kCopySlotBytes), bytes - off));
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(reinterpret_cast<uint64_t>(dst + off)),
                           "r"(smem_base + slot * kCopySlotBytes), "r"(n)
                         : "memory");
            bulk_commit_group();
            // The slot may be refilled once the store has finished reading shared memory.
            bulk_wait_group_read<0>();
            mbar_arrive(smem_u32(&empty[slot]));
        }
        bulk_wait_group<0>();
    }
}

}  // namespace
}  // namespace b2a

extern "C" {

int b2a_ipc_export(const void* ptr, unsigned char* handle, uint64_t* offset) {
    using namespace b2a;
    B2A_REQUIRE(ptr != nullptr && handle != nullptr && offset != nullptr, "arguments must not be NULL");
    GetAddressRangeFn range = get_address_range_fn();
    if (range == nullptr) return fail(B2A_ERR_CUDA, "cuMemGetAddressRange is not available from the driver");
    CUdeviceptr base = 0;
    size_t size = 0;
    CUresult res = range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
    if (res != CUDA_SUCCESS) return fail(B2A_ERR_CUDA, "cuMemGetAddressRange failed with CUresult %d", (int)res);
    cudaIpcMemHandle_t h;
    B2A_CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
    memcpy(handle, &h, 64);
    *offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
    return B2A_OK;
}

int b2a_ipc_import(const unsigned char* handle, uint64_t offset, void** out_ptr) {
    using namespace b2a;
    B2A_REQUIRE(handle != nullptr && out_ptr != nullptr, "arguments must not be NULL");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void* base = nullptr;
    B2A_CUDA_OK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *out_ptr = static_cast<uint8_t*>(base) + offset;
    return B2A_OK;
}

int b2a_ipc_close(void* ptr, uint64_t offset) {
    using namespace b2a;
    B2A_REQUIRE(ptr != nullptr, "ptr must not be NULL");
    B2A_CUDA_OK(cudaIpcCloseMemHandle(static_cast<uint8_t*>(ptr) - offset));
    return B2A_OK;
}

int b2a_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                size_t rows, int32_t kind, void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(dst != nullptr && src != nullptr, "dst and src must not be NULL");
    B2A_REQUIRE(row_bytes > 0 && rows > 0, "row_bytes and rows must be positive");
    B2A_REQUIRE(dst_pitch >= row_bytes && src_pitch >= row_bytes, "pitches must be at least row_bytes");
    B2A_REQUIRE(kind >= 1 && kind <= 3, "kind must be 1 (host->device), 2 (device->host) or 3 (device->device)");
    const cudaMemcpyKind k = kind == 1 ? cudaMemcpyHostToDevice
                             : kind == 2 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    B2A_CUDA_OK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, k,
                                  static_cast<cudaStream_t>(cuda_stream)));
    return B2A_OK;
}

int b2a_peer_copy(void* dst, const void* src, size_t bytes, int32_t num_blocks, unsigned int* status,
                  void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(dst != nullptr && src != nullptr, "dst and src must not be NULL");
    B2A_REQUIRE(bytes > 0 && bytes % 16 == 0, "bytes must be a positive multiple of 16, got %zu", bytes);
    B2A_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 0xF) == 0 && (reinterpret_cast<uintptr_t>(src) & 0xF) == 0,
                "dst and src must be 16-byte aligned");
    B2A_REQUIRE(num_blocks > 0, "num_blocks must be > 0, got %d", num_blocks);
    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != B2A_OK) return rc;
    const int smem = kCopySlots * kCopySlotBytes;
    rc = once_per_device(dev.device, 3, [] {
        B2A_CUDA_OK(cudaFuncSetAttribute(peer_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kCopySlots * kCopySlotBytes));
        return static_cast<int>(B2A_OK);
    });
    if (rc != B2A_OK) return rc;
    const size_t chunks = (bytes + kCopySlotBytes - 1) / kCopySlotBytes;
    int grid = num_blocks;
    if (static_cast<size_t>(grid) > chunks) grid = static_cast<int>(chunks);
    peer_copy_kernel<<<grid, kCopyThreads, smem, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), bytes, status, wait_timeout_ns());
    B2A_CUDA_OK(cudaGetLastError());
    return B2A_OK;
}

}  // extern "C"
