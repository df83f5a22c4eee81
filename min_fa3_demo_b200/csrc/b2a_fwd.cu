// C-ABI entry point and launcher of the forward attention kernel.
#include "b2a_fwd.cuh"
#include "b2a_host.cuh"

#include <cmath>
#include <mutex>

namespace b2a {

namespace {

constexpr size_t kFwdSmemBytes = sizeof(FwdShared) + 1024;   // + slack for 1 KiB alignment

template <bool kMerge>
int set_fwd_smem_attribute() {
    B2A_CUDA_OK(cudaFuncSetAttribute(fwd_kernel<kMerge>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kFwdSmemBytes)));
    return B2A_OK;
}

}  // namespace

int configure_fwd_kernel(const DeviceInfo& dev, bool merge) {
    if (static_cast<size_t>(dev.max_smem_optin) < kFwdSmemBytes) {
        return fail(B2A_ERR_UNSUPPORTED_DEVICE, "device offers %d bytes of shared memory, need %zu",
                    dev.max_smem_optin, kFwdSmemBytes);
    }
    return merge ? once_per_device(dev.device, 1, set_fwd_smem_attribute<true>)
                 : once_per_device(dev.device, 0, set_fwd_smem_attribute<false>);
}

}  // namespace b2a

extern "C" {

size_t b2a_fwd_workspace_bytes(int32_t batch, int32_t total_q, int32_t is_varlen) {
    size_t bytes = sizeof(b2a::WorkspaceHeader);
    if (is_varlen) {
        bytes += b2a::max_entries(batch, total_q, b2a::kFwdRowsPerWork) * sizeof(int2);
    }
    return b2a::align_up(bytes, 256);
}

int b2a_fwd(const b2a_fwd_args* a, void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(a != nullptr, "args must not be NULL");
    B2A_REQUIRE(a->q && a->k && a->v && a->out && a->lse, "q, k, v, out and lse must not be NULL");
    B2A_REQUIRE(a->head_dim == kHeadDim, "head_dim must be 128, got %d", a->head_dim);
    B2A_REQUIRE(a->batch >= 1, "batch must be >= 1, got %d", a->batch);
    B2A_REQUIRE(a->heads_q >= 1 && a->heads_k >= 1 && a->heads_q % a->heads_k == 0,
                "heads_q %% heads_k must be 0, got heads_q=%d heads_k=%d", a->heads_q, a->heads_k);
    B2A_REQUIRE(a->total_q >= 1 && a->total_k >= 1, "total_q and total_k must be positive");
    B2A_REQUIRE((a->cu_seqlens_q == nullptr) == (a->cu_seqlens_k == nullptr),
                "cu_seqlens_q and cu_seqlens_k must both be given or both be NULL");
    const bool varlen = a->cu_seqlens_q != nullptr;
    if (!varlen) {
        B2A_REQUIRE(a->seqlen_q >= 1 && a->seqlen_k >= 1, "seqlen_q and seqlen_k must be positive");
        B2A_REQUIRE(static_cast<long long>(a->batch) * a->seqlen_q == a->total_q &&
                        static_cast<long long>(a->batch) * a->seqlen_k == a->total_k,
                    "BSHD sizes must satisfy total = batch * seqlen");
    }
    B2A_REQUIRE(a->grid_blocks >= 0, "grid_blocks must be >= 0, got %d", a->grid_blocks);
    const bool prefetch = a->prefetch_bytes != 0;
    if (prefetch) {
        B2A_REQUIRE(a->prefetch_src_k && a->prefetch_src_v && a->prefetch_dst_k && a->prefetch_dst_v,
                    "prefetch source and destination pointers must not be NULL when prefetch_bytes > 0");
        B2A_REQUIRE(a->prefetch_bytes % 16 == 0, "prefetch_bytes must be a multiple of 16, got %zu", a->prefetch_bytes);
        B2A_REQUIRE(a->prefetch_blocks > 0, "prefetch_blocks must be positive when prefetch_bytes > 0, got %d",
                    a->prefetch_blocks);
        const uintptr_t align = reinterpret_cast<uintptr_t>(a->prefetch_src_k) | reinterpret_cast<uintptr_t>(a->prefetch_src_v) |
                                reinterpret_cast<uintptr_t>(a->prefetch_dst_k) | reinterpret_cast<uintptr_t>(a->prefetch_dst_v);
        B2A_REQUIRE((align & 0xF) == 0, "prefetch buffers must be 16-byte aligned");
    }
    B2A_REQUIRE(a->workspace != nullptr && (reinterpret_cast<uintptr_t>(a->workspace) & 0xF) == 0,
                "workspace must be a 16-byte aligned device pointer");
    const size_t need = b2a_fwd_workspace_bytes(a->batch, a->total_q, varlen ? 1 : 0);
    if (a->workspace_bytes < need) {
        return fail(B2A_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, need %zu",
                    a->workspace_bytes, need);
    }

    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != B2A_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    CUtensorMap map_q, map_k, map_v;
    rc = make_token_map(&map_q, a->q, a->total_q, a->heads_q, kTileM);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_k, a->k, a->total_k, a->heads_k, kTileN);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_v, a->v, a->total_k, a->heads_k, kTileN);
    if (rc != B2A_OK) return rc;

    auto* hdr = static_cast<WorkspaceHeader*>(a->workspace);
    int2* work_list = reinterpret_cast<int2*>(hdr + 1);
    B2A_CUDA_OK(cudaMemsetAsync(hdr, 0, sizeof(WorkspaceHeader), stream));

    FwdParams p{};
    p.o = static_cast<__nv_bfloat16*>(a->out);
    p.lse = a->lse;
    p.cu_seqlens_q = a->cu_seqlens_q;
    p.cu_seqlens_k = a->cu_seqlens_k;
    p.work_list = varlen ? work_list : nullptr;
    p.num_entries_dev = &hdr->num_entries;
    p.sched_counter = &hdr->sched_counter;
    p.status = &hdr->status;
    p.batch = a->batch;
    p.seqlen_q = a->seqlen_q;
    p.seqlen_k = a->seqlen_k;
    p.total_q = a->total_q;
    p.total_k = a->total_k;
    p.heads_q = a->heads_q;
    p.heads_k = a->heads_k;
    p.causal = a->is_causal ? 1 : 0;
    p.scale = a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / std::sqrt(static_cast<float>(kHeadDim));
    p.scale_log2 = p.scale * kLog2e;
    p.merge = a->merge_running ? 1 : 0;
    p.timeout_ns = wait_timeout_ns();

    long long work_items;
    if (varlen) {
        const int cap = static_cast<int>(max_entries(a->batch, a->total_q, kFwdRowsPerWork));
        rc = launch_varlen_plan(0, a->cu_seqlens_q, a->cu_seqlens_k, a->batch, p.causal, work_list,
                                &hdr->num_entries, cap, stream);
        if (rc != B2A_OK) return rc;
        p.num_entries_host = cap;
        p.lse_head_stride = a->total_q;
        p.lse_batch_stride = 0;
        work_items = static_cast<long long>(cap) * a->heads_q;
    } else {
        const int nmb = (a->seqlen_q + kFwdRowsPerWork - 1) / kFwdRowsPerWork;
        p.num_entries_host = a->batch * nmb;
        p.lse_head_stride = a->seqlen_q;
        p.lse_batch_stride = static_cast<long long>(a->heads_q) * a->seqlen_q;
        work_items = static_cast<long long>(p.num_entries_host) * a->heads_q;
    }

    int grid = a->grid_blocks > 0 ? a->grid_blocks : dev.sm_count;
    if (work_items < grid) grid = static_cast<int>(work_items);
    if (grid < 1) grid = 1;
    p.num_comp = grid;
    if (prefetch) {
        // Copy CTAs ride in the same launch behind the compute CTAs; neither kind waits for the other.
        p.prefetch_src[0] = static_cast<const uint8_t*>(a->prefetch_src_k);
        p.prefetch_src[1] = static_cast<const uint8_t*>(a->prefetch_src_v);
        p.prefetch_dst[0] = static_cast<uint8_t*>(a->prefetch_dst_k);
        p.prefetch_dst[1] = static_cast<uint8_t*>(a->prefetch_dst_v);
        p.prefetch_bytes = a->prefetch_bytes;
        grid += a->prefetch_blocks;
    }

    if (p.merge) {
        rc = configure_fwd_kernel(dev, true);
        if (rc != B2A_OK) return rc;
        profile_mark(B2A_KERNEL_FWD, false, stream);
        fwd_kernel<true><<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(map_q, map_k, map_v, p);
    } else {
        rc = configure_fwd_kernel(dev, false);
        if (rc != B2A_OK) return rc;
        profile_mark(B2A_KERNEL_FWD, false, stream);
        fwd_kernel<false><<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(map_q, map_k, map_v, p);
    }
    profile_mark(B2A_KERNEL_FWD, true, stream);
    B2A_CUDA_OK(cudaGetLastError());
    return B2A_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Forward for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------
namespace b2a {
namespace {

// Scratch of b2a_fwd_noalloc: the 16-byte workspace header plus the varlen work list.
// 64 KiB holds 8190 work pieces (a piece is 256 query rows of one document), i.e. packed
// batches with total_q / 256 + batch + 1 <= 8190.  Every GPU that loads the library keeps
// this array resident until the process exits.
constexpr size_t kNoAllocScratchBytes = 64 * 1024;
static __device__ __align__(256) unsigned char g_fwd_noalloc_scratch[kNoAllocScratchBytes];

}  // namespace

// Device address of the array on each device.  The array's name is only a host-side handle
// in host code; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device while that device is current.
int noalloc_scratch_ptr(void** out) {
    static std::mutex mu;
    static void* ptrs[64] = {};
    int dev = 0;
    B2A_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) {
        return fail(B2A_ERR_CUDA, "device index %d out of range", dev);
    }
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&p, g_fwd_noalloc_scratch);
        if (err != cudaSuccess || p == nullptr) {
            return fail(B2A_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev,
                        cudaGetErrorString(err));
        }
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return B2A_OK;
}

}  // namespace b2a

extern "C" {

size_t b2a_fwd_noalloc_scratch_limit(void) { return b2a::kNoAllocScratchBytes; }

int b2a_fwd_noalloc(const b2a_fwd_args* a, void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(a != nullptr, "args must not be NULL");
    B2A_REQUIRE(a->batch >= 1 && a->total_q >= 1, "batch and total_q must be positive");
    const bool varlen = a->cu_seqlens_q != nullptr;
    const size_t need = b2a_fwd_workspace_bytes(a->batch, a->total_q, varlen ? 1 : 0);
    if (need > kNoAllocScratchBytes) {
        return fail(B2A_ERR_WORKSPACE_TOO_SMALL,
                    "b2a_fwd_noalloc: this problem needs %zu bytes of scratch but the built-in scratch "
                    "holds %zu (packed batches up to total_q / 256 + batch + 1 <= 8190); "
                    "use b2a_fwd with a caller-provided workspace",
                    need, kNoAllocScratchBytes);
    }
    void* scratch = nullptr;
    int rc = noalloc_scratch_ptr(&scratch);
    if (rc != B2A_OK) return rc;
    b2a_fwd_args local = *a;
    local.workspace = scratch;
    local.workspace_bytes = kNoAllocScratchBytes;
    return b2a_fwd(&local, cuda_stream);
}

}  // extern "C"
