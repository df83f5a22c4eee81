// C-ABI entry point and launcher of the backward pass (preprocess, main kernel, postprocess).
#include "b2a_bwd.cuh"
#include "b2a_host.cuh"

#include <cmath>

namespace b2a {

namespace {

constexpr size_t kBwdSmemBytes = sizeof(BwdShared);

struct BwdLayout {
    size_t work_list_off;
    size_t lse2_off;
    size_t dpsum_off;
    size_t dq_accum_off;
    size_t total;
    int padded_q;
    int entries_cap;
};

BwdLayout bwd_layout(int batch, int seqlen_q, int total_q, int total_k, int heads_q, bool varlen) {
    BwdLayout l{};
    size_t off = sizeof(WorkspaceHeader);
    l.work_list_off = off;
    l.entries_cap = 0;
    if (varlen) {
        l.entries_cap = static_cast<int>(max_entries(batch, total_k, kTileN));
        off += static_cast<size_t>(l.entries_cap) * sizeof(int2);
        l.padded_q = static_cast<int>(align_up(static_cast<size_t>(total_q) + 256ull * batch + 256, 128));
    } else {
        l.padded_q = batch * static_cast<int>(align_up(seqlen_q, 128));
    }
    off = align_up(off, 256);
    const size_t vec_bytes = static_cast<size_t>(heads_q) * l.padded_q * sizeof(float);
    l.lse2_off = off;
    off += align_up(vec_bytes, 256);
    l.dpsum_off = off;
    off += align_up(vec_bytes, 256);
    l.dq_accum_off = off;
    off += vec_bytes * kHeadDim;
    l.total = align_up(off, 256);
    return l;
}

int configure_bwd_kernel(const DeviceInfo& dev) {
    static bool done[64] = {};
    if (!done[dev.device]) {
        if (static_cast<size_t>(dev.max_smem_optin) < kBwdSmemBytes) {
            return fail(B2A_ERR_UNSUPPORTED_DEVICE, "device offers %d bytes of shared memory, need %zu",
                        dev.max_smem_optin, kBwdSmemBytes);
        }
        B2A_CUDA_OK(cudaFuncSetAttribute(bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kBwdSmemBytes)));
        done[dev.device] = true;
    }
    return B2A_OK;
}

}  // namespace

}  // namespace b2a

extern "C" {

size_t b2a_bwd_workspace_bytes(int32_t batch, int32_t total_q, int32_t total_k, int32_t heads_q,
                               int32_t heads_k, int32_t is_varlen) {
    (void)heads_k;
    // For BSHD the padded length is derived from seqlen_q = total_q / batch.
    const int seqlen_q = batch > 0 ? total_q / batch : total_q;
    return b2a::bwd_layout(batch, seqlen_q, total_q, total_k, heads_q, is_varlen != 0).total;
}

int b2a_bwd(const b2a_bwd_args* a, void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(a != nullptr, "args must not be NULL");
    B2A_REQUIRE(a->dout && a->q && a->k && a->v && a->out && a->lse,
                "dout, q, k, v, out and lse must not be NULL");
    B2A_REQUIRE(a->dq && a->dk && a->dv, "dq, dk and dv must not be NULL");
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
    B2A_REQUIRE(a->workspace != nullptr && (reinterpret_cast<uintptr_t>(a->workspace) & 0xFF) == 0,
                "workspace must be a 256-byte aligned device pointer");
    const BwdLayout lay = bwd_layout(a->batch, a->seqlen_q, a->total_q, a->total_k, a->heads_q, varlen);
    if (a->workspace_bytes < lay.total) {
        return fail(B2A_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, need %zu",
                    a->workspace_bytes, lay.total);
    }

    DeviceInfo dev{};
    int rc = current_device_info(&dev);
    if (rc != B2A_OK) return rc;
    rc = configure_bwd_kernel(dev);
    if (rc != B2A_OK) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    CUtensorMap map_q, map_k, map_v, map_do;
    rc = make_token_map(&map_q, a->q, a->total_q, a->heads_q, kTileM);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_k, a->k, a->total_k, a->heads_k, kTileN);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_v, a->v, a->total_k, a->heads_k, kTileN);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_do, a->dout, a->total_q, a->heads_q, kTileM);
    if (rc != B2A_OK) return rc;

    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    auto* hdr = reinterpret_cast<WorkspaceHeader*>(ws);
    int2* work_list = reinterpret_cast<int2*>(ws + lay.work_list_off);
    float* lse2 = reinterpret_cast<float*>(ws + lay.lse2_off);
    float* dpsum = reinterpret_cast<float*>(ws + lay.dpsum_off);
    float* dq_accum = reinterpret_cast<float*>(ws + lay.dq_accum_off);

    const float scale =
        a->softmax_scale > 0.f ? a->softmax_scale : 1.0f / std::sqrt(static_cast<float>(kHeadDim));
    const int causal = a->is_causal ? 1 : 0;

    B2A_CUDA_OK(cudaMemsetAsync(hdr, 0, sizeof(WorkspaceHeader), stream));
    B2A_CUDA_OK(cudaMemsetAsync(dq_accum, 0,
                                static_cast<size_t>(a->heads_q) * lay.padded_q * kHeadDim * sizeof(float),
                                stream));

    // Preprocess.
    BwdPreParams pre{};
    pre.o = static_cast<const __nv_bfloat16*>(a->out);
    pre.dout = static_cast<const __nv_bfloat16*>(a->dout);
    pre.lse = a->lse;
    pre.lse2 = lse2;
    pre.dpsum = dpsum;
    pre.cu_seqlens_q = a->cu_seqlens_q;
    pre.batch = a->batch;
    pre.seqlen_q = a->seqlen_q;
    pre.heads_q = a->heads_q;
    pre.padded_q = lay.padded_q;
    if (varlen) {
        pre.lse_head_stride = a->total_q;
        pre.lse_batch_stride = 0;
    } else {
        pre.lse_head_stride = a->seqlen_q;
        pre.lse_batch_stride = static_cast<long long>(a->heads_q) * a->seqlen_q;
    }
    {
        dim3 grid((lay.padded_q + 7) / 8, a->heads_q);
        bwd_preprocess_kernel<<<grid, 256, 0, stream>>>(pre);
        B2A_CUDA_OK(cudaGetLastError());
    }

    // Main kernel.
    BwdParams p{};
    p.dk = static_cast<__nv_bfloat16*>(a->dk);
    p.dv = static_cast<__nv_bfloat16*>(a->dv);
    p.dq_accum = dq_accum;
    p.lse2 = lse2;
    p.dpsum = dpsum;
    p.cu_seqlens_q = a->cu_seqlens_q;
    p.cu_seqlens_k = a->cu_seqlens_k;
    p.work_list = varlen ? work_list : nullptr;
    p.num_entries_dev = &hdr->num_entries;
    p.sched_counter = &hdr->sched_counter;
    p.status = &hdr->status;
    p.batch = a->batch;
    p.seqlen_q = a->seqlen_q;
    p.seqlen_k = a->seqlen_k;
    p.heads_q = a->heads_q;
    p.heads_k = a->heads_k;
    p.causal = causal;
    p.padded_q = lay.padded_q;
    p.scale = scale;
    p.scale_log2 = scale * kLog2e;
    p.timeout_ns = kDefaultTimeoutNs;

    long long work_items;
    if (varlen) {
        rc = launch_varlen_plan(1, a->cu_seqlens_q, a->cu_seqlens_k, a->batch, causal, work_list,
                                &hdr->num_entries, lay.entries_cap, stream);
        if (rc != B2A_OK) return rc;
        p.num_entries_host = lay.entries_cap;
        work_items = static_cast<long long>(lay.entries_cap) * a->heads_k;
    } else {
        const int nnb = (a->seqlen_k + kTileN - 1) / kTileN;
        p.num_entries_host = a->batch * nnb;
        work_items = static_cast<long long>(p.num_entries_host) * a->heads_k;
    }
    int grid = a->grid_blocks > 0 ? a->grid_blocks : dev.sm_count;
    if (work_items < grid) grid = static_cast<int>(work_items);
    if (grid < 1) grid = 1;
    profile_mark(B2A_KERNEL_BWD, false, stream);
    bwd_kernel<<<grid, kBwdThreads, kBwdSmemBytes, stream>>>(map_q, map_k, map_v, map_do, p);
    profile_mark(B2A_KERNEL_BWD, true, stream);
    B2A_CUDA_OK(cudaGetLastError());

    // Postprocess.
    BwdPostParams post{};
    post.dq_accum = dq_accum;
    post.dq = static_cast<__nv_bfloat16*>(a->dq);
    post.cu_seqlens_q = a->cu_seqlens_q;
    post.batch = a->batch;
    post.seqlen_q = a->seqlen_q;
    post.heads_q = a->heads_q;
    post.padded_q = lay.padded_q;
    post.scale = scale;
    {
        dim3 pgrid(lay.padded_q / kTileM, a->heads_q);
        bwd_postprocess_kernel<<<pgrid, 128, 0, stream>>>(post);
        B2A_CUDA_OK(cudaGetLastError());
    }
    return B2A_OK;
}

}  // extern "C"
