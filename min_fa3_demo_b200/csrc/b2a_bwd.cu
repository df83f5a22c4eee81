// C-ABI entry point and launcher of the backward pass (preprocess, main kernel, postprocess).
#include "b2a_bwd.cuh"
#include "b2a_host.cuh"
#include "b2a_ring_host.cuh"

#include <cmath>
#include <cstring>

namespace b2a {

namespace {

constexpr size_t kBwdSmemBytes = sizeof(BwdShared);

// Key/value heads scheduled together ("supergroup"): as many as keep the fp32 dQ accumulator
// rows that the concurrently running CTAs add into (query heads of the group x query rows x
// 512 bytes) within about the size of L2.  Measured on B200 (QH=32, KVH=8): at S=8192 all 8 heads
// together are best (B=2: 1.9 GB of DRAM traffic per launch against 5.3 GB with 3 heads and 3.8 GB
// with 1; 2.33 / 2.52 / 2.42 ms); on one 131,072-token sequence 1 or 2 heads are best (329 / 331 ms
// against 350 ms with all 8).
int pick_sg_heads(int heads_q, int heads_k, long long q_rows) {
    const long long per_head = static_cast<long long>(heads_q / heads_k) * (q_rows > 0 ? q_rows : 1) * 512;
    const long long budget = 160ll << 20;
    long long n = budget / per_head;
    if (n < 1) n = 1;
    return n < heads_k ? static_cast<int>(n) : heads_k;
}

struct BwdLayout {
    size_t work_list_off;
    size_t lse2_off;
    size_t dpsum_off;
    size_t dq_accum_off;
    size_t dq_sem_off;     // int per (query head, 128-row query tile): deterministic dQ order
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
    l.dq_sem_off = off;
    off += align_up(static_cast<size_t>(heads_q) * (l.padded_q / kTileM) * sizeof(int), 256);
    l.total = align_up(off, 256);
    return l;
}

int set_bwd_smem_attribute() {
    B2A_CUDA_OK(cudaFuncSetAttribute(bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kBwdSmemBytes)));
    return B2A_OK;
}

int configure_bwd_kernel(const DeviceInfo& dev) {
    if (static_cast<size_t>(dev.max_smem_optin) < kBwdSmemBytes) {
        return fail(B2A_ERR_UNSUPPORTED_DEVICE, "device offers %d bytes of shared memory, need %zu",
                    dev.max_smem_optin, kBwdSmemBytes);
    }
    return once_per_device(dev.device, 2, set_bwd_smem_attribute);
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
    int* dq_sem = nullptr;
    if (a->deterministic) {
        dq_sem = reinterpret_cast<int*>(ws + lay.dq_sem_off);
        B2A_CUDA_OK(cudaMemsetAsync(dq_sem, 0, static_cast<size_t>(a->heads_q) * (lay.padded_q / kTileM) * sizeof(int),
                                    stream));
    }

    // Preprocess.
    BwdPreParams pre{};
    pre.o = static_cast<const __nv_bfloat16*>(a->out);
    pre.dout = static_cast<const __nv_bfloat16*>(a->dout);
    pre.lse = a->lse;
    pre.lse2 = lse2;
    pre.dpsum = dpsum;
    pre.dq_accum = dq_accum;     // cleared by the preprocess: no separate memset pass
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
        dim3 grid((lay.padded_q + kPreRows - 1) / kPreRows);
        bwd_preprocess_kernel<<<grid, 256, 0, stream>>>(pre);
        B2A_CUDA_OK(cudaGetLastError());
    }

    // Main kernel.
    BwdParams p{};
    p.dk = static_cast<__nv_bfloat16*>(a->dk);
    p.dv = static_cast<__nv_bfloat16*>(a->dv);
    p.dq_accum = dq_accum;
    p.dq_sem = dq_sem;
    // Batch-minor hand-out only in deterministic mode: for the default mode it was measured slower
    // (B=4, S=8192: 5.5 ms vs 5.2 ms) because the dQ accumulators of all batch elements are live at once.
    p.batch_minor = dq_sem != nullptr ? 1 : 0;
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
    p.timeout_ns = wait_timeout_ns();

    p.sg_heads = pick_sg_heads(a->heads_q, a->heads_k, varlen ? a->total_q : a->seqlen_q);
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

// ---------------------------------------------------------------------------------------
// Context-parallel backward
// ---------------------------------------------------------------------------------------

namespace b2a {
namespace {

constexpr size_t kRingBwdSmemBytes = sizeof(BwdShared);

struct RingBwdLayout {
    size_t docs_off, work_off, tasks_off, flags_off, lse2_off, dpsum_off, dq_accum_off, total;
    size_t work_cap, task_cap, flag_count;
};

RingBwdLayout ring_bwd_layout(int batch, int world, int cap, int total_q, int heads_q) {
    RingBwdLayout l{};
    l.flag_count = static_cast<size_t>(world) * cap / kTileN;
    l.work_cap = l.flag_count;     // one entry per visible 128-row key block of the arena
    l.task_cap = l.flag_count;
    size_t off = sizeof(WorkspaceHeader);
    l.docs_off = off;
    off = align_up(off + static_cast<size_t>(batch) * sizeof(RingDoc), 16);
    l.work_off = off;
    off = align_up(off + l.work_cap * sizeof(int4), 16);
    l.tasks_off = off;
    off = align_up(off + l.task_cap * sizeof(int2), 16);
    l.flags_off = off;
    off = align_up(off + l.flag_count * sizeof(int), 256);
    const size_t vec_bytes = static_cast<size_t>(heads_q) * total_q * sizeof(float);
    l.lse2_off = off;
    off += align_up(vec_bytes, 256);
    l.dpsum_off = off;
    off += align_up(vec_bytes, 256);
    l.dq_accum_off = off;
    off += vec_bytes * kHeadDim;
    l.total = align_up(off, 256);
    return l;
}

}  // namespace
}  // namespace b2a

extern "C" {

size_t b2a_ring_bwd_workspace_bytes(int32_t batch, int32_t world_size, int32_t rank_kv_capacity,
                                    int32_t total_q, int32_t heads_q) {
    return b2a::ring_bwd_layout(batch, world_size, rank_kv_capacity, total_q, heads_q).total;
}

int b2a_ring_bwd(const b2a_ring_bwd_args* a, void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(a != nullptr, "args must not be NULL");
    B2A_REQUIRE(a->head_dim == kHeadDim, "head_dim must be 128, got %d", a->head_dim);
    B2A_REQUIRE(a->heads_q >= 1 && a->heads_k >= 1 && a->heads_q % a->heads_k == 0,
                "heads_q %% heads_k must be 0, got heads_q=%d heads_k=%d", a->heads_q, a->heads_k);
    B2A_REQUIRE(a->cu_seqlens_q_host && a->global_seqlens_host && a->ring_sizes_host && a->ring_starts_host,
                "host metadata arrays must not be NULL");
    B2A_REQUIRE(a->num_comp_sm > 0, "num_comp_sm must be positive. Got %d", a->num_comp_sm);
    B2A_REQUIRE(a->num_comm_sm >= 0, "num_comm_sm must be non-negative. Got %d", a->num_comm_sm);
    B2A_REQUIRE(a->total_q >= 0 && a->total_q % 128 == 0, "total_q must be a non-negative multiple of 128");
    const int causal = a->is_causal ? 1 : 0;
    const int world = a->world_size, rank = a->rank, cap = a->rank_kv_capacity;

    RingPlan plan;
    int rc = build_ring_plan(&plan, a->batch, world, rank, cap, causal, a->cu_seqlens_q_host,
                             a->global_seqlens_host, a->ring_sizes_host, a->ring_starts_host);
    if (rc != B2A_OK) return rc;
    B2A_REQUIRE(a->cu_seqlens_q_host[a->batch] == a->total_q, "cu_seqlens_q_host[-1] must equal total_q");
    B2A_REQUIRE(a->local_total_k == a->total_q, "local_total_k must equal total_q for context-parallel backward");
    // kv_resident: the forward left every remote block this rank needs in the arena; no copy
    // tasks, no block flags, and the CTAs past num_comp_sm compute from the start.
    const bool pull = !plan.comm_tasks.empty() && a->kv_resident == 0;
    B2A_REQUIRE(!pull || a->num_comm_sm > 0,
                "num_comm_sm must be positive when documents are sharded over more than one rank");
    for (int r = 0; r < world; ++r) {
        B2A_REQUIRE(a->dk_accum_peer[r] && a->dv_accum_peer[r] && a->completion_peer[r],
                    "accumulator / completion pointers of rank %d must not be NULL", r);
    }
    DeviceInfo dev{};
    rc = current_device_info(&dev);
    if (rc != B2A_OK) return rc;
    B2A_REQUIRE(a->num_comp_sm + a->num_comm_sm <= dev.sm_count,
                "num_comp_sm + num_comm_sm = %d exceeds the %d SMs of the device",
                a->num_comp_sm + a->num_comm_sm, dev.sm_count);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const RingBwdLayout lay = ring_bwd_layout(a->batch, world, cap, a->total_q, a->heads_q);
    B2A_REQUIRE(a->workspace != nullptr && (reinterpret_cast<uintptr_t>(a->workspace) & 0xFF) == 0,
                "workspace must be a 256-byte aligned device pointer");
    if (a->workspace_bytes < lay.total) {
        return fail(B2A_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, need %zu", a->workspace_bytes, lay.total);
    }

    // Work list: every 128-row key block (of any ring member) that a local query half sees.
    struct Entry { int4 e; int cost; };
    std::vector<Entry> entries;
    for (int d : plan.doc_order) {
        const RingDoc& doc = plan.docs[d];
        const int g = doc.ring_size, r = doc.ring_rank, hb = doc.half_len / kTileN;
        const int halves = ring_halves(causal, g);
        for (int s = 0; s < g; ++s) {
            for (int hf = 0; hf < halves; ++hf) {
                const int ck = g == 1 ? 0 : (hf == 0 ? s : 2 * g - 1 - s);
                for (int blk = 0; blk < hb; ++blk) {
                    int cost = 0;
                    for (int h = 0; h < halves; ++h) {
                        if (!causal) { cost += hb; continue; }
                        const int cq = g == 1 ? 0 : (h == 0 ? r : 2 * g - 1 - r);
                        if (ck < cq) cost += hb;
                        else if (ck == cq) cost += hb - blk;
                    }
                    if (cost > 0) entries.push_back({make_int4(d, s, hf, blk), cost});
                }
            }
        }
    }
    std::stable_sort(entries.begin(), entries.end(), [](const Entry& x, const Entry& y) { return x.cost > y.cost; });
    B2A_REQUIRE(entries.size() <= lay.work_cap && plan.comm_tasks.size() <= lay.task_cap,
                "internal: ring work list exceeds its workspace bound");

    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    auto* hdr = reinterpret_cast<WorkspaceHeader*>(ws);
    float* lse2 = reinterpret_cast<float*>(ws + lay.lse2_off);
    float* dpsum = reinterpret_cast<float*>(ws + lay.dpsum_off);
    float* dq_accum = reinterpret_cast<float*>(ws + lay.dq_accum_off);
    B2A_CUDA_OK(cudaMemsetAsync(hdr, 0, sizeof(WorkspaceHeader), stream));
    B2A_CUDA_OK(cudaMemsetAsync(ws + lay.flags_off, 0, lay.flag_count * sizeof(int), stream));

    const float scale = 1.0f / std::sqrt(static_cast<float>(kHeadDim));
    if (a->total_q > 0) {
        std::vector<uint8_t> host(lay.flags_off - lay.docs_off, 0);
        memcpy(host.data(), plan.docs.data(), plan.docs.size() * sizeof(RingDoc));
        int4* w = reinterpret_cast<int4*>(host.data() + (lay.work_off - lay.docs_off));
        for (size_t i = 0; i < entries.size(); ++i) w[i] = entries[i].e;
        if (pull) {
            memcpy(host.data() + (lay.tasks_off - lay.docs_off), plan.comm_tasks.data(),
                   plan.comm_tasks.size() * sizeof(int2));
        }
        B2A_CUDA_OK(cudaMemcpyAsync(ws + lay.docs_off, host.data(), host.size(), cudaMemcpyHostToDevice, stream));

        // Preprocess over the packed local tokens (every local length is a multiple of 128, so the
        // padded layout is the identity: one "document" of total_q rows).
        BwdPreParams pre{};
        pre.o = static_cast<const __nv_bfloat16*>(a->out);
        pre.dout = static_cast<const __nv_bfloat16*>(a->dout);
        pre.lse = a->lse;
        pre.lse2 = lse2;
        pre.dpsum = dpsum;
        pre.dq_accum = dq_accum;
        pre.batch = 1;
        pre.seqlen_q = a->total_q;
        pre.heads_q = a->heads_q;
        pre.padded_q = a->total_q;
        pre.lse_head_stride = a->total_q;
        pre.lse_batch_stride = 0;
        dim3 pgrid((a->total_q + kPreRows - 1) / kPreRows);
        bwd_preprocess_kernel<<<pgrid, 256, 0, stream>>>(pre);
        B2A_CUDA_OK(cudaGetLastError());

        const int arena_rows = world * cap;
        CUtensorMap map_q, map_k, map_v, map_do;
        rc = make_token_map(&map_q, a->q, a->total_q, a->heads_q, kTileM);
        if (rc != B2A_OK) return rc;
        rc = make_token_map(&map_k, a->arena_k, arena_rows, a->heads_k, kTileN);
        if (rc != B2A_OK) return rc;
        rc = make_token_map(&map_v, a->arena_v, arena_rows, a->heads_k, kTileN);
        if (rc != B2A_OK) return rc;
        rc = make_token_map(&map_do, a->dout, a->total_q, a->heads_q, kTileM);
        if (rc != B2A_OK) return rc;

        BwdParams p{};
        p.dq_accum = dq_accum;
        p.lse2 = lse2;
        p.dpsum = dpsum;
        p.num_entries_dev = &hdr->num_entries;
        p.sched_counter = &hdr->sched_counter;
        p.status = &hdr->status;
        p.batch = a->batch;
        p.heads_q = a->heads_q;
        p.heads_k = a->heads_k;
        p.causal = causal;
        p.num_entries_host = static_cast<int>(entries.size());
        p.sg_heads = pick_sg_heads(a->heads_q, a->heads_k, a->total_q);
        p.padded_q = a->total_q;
        p.scale = scale;
        p.scale_log2 = scale * kLog2e;
        p.timeout_ns = wait_timeout_ns();
        p.ring_docs = reinterpret_cast<const RingDoc*>(ws + lay.docs_off);
        p.ring_work = reinterpret_cast<const int4*>(ws + lay.work_off);
        p.comm_tasks = reinterpret_cast<const int2*>(ws + lay.tasks_off);
        p.comm_task_count = pull ? static_cast<int>(plan.comm_tasks.size()) : 0;
        p.num_comp = a->num_comp_sm;
        p.my_rank = rank;
        p.kv_row_bytes = a->heads_k * kHeadDim * 2;
        p.cap = cap;
        for (int r = 0; r < 8; ++r) {
            const bool in = r < world;
            p.peer_k[r] = in ? static_cast<const uint8_t*>(a->peer_k[r]) : nullptr;
            p.peer_v[r] = in ? static_cast<const uint8_t*>(a->peer_v[r]) : nullptr;
            p.dk_accum_peer[r] = in ? a->dk_accum_peer[r] : nullptr;
            p.dv_accum_peer[r] = in ? a->dv_accum_peer[r] : nullptr;
            p.completion_peer[r] = in ? a->completion_peer[r] : nullptr;
        }
        p.arena_k = static_cast<uint8_t*>(a->arena_k);
        p.arena_v = static_cast<uint8_t*>(a->arena_v);
        p.kv_flags = reinterpret_cast<int*>(ws + lay.flags_off);
        p.done_ctas = &hdr->reserved;
        p.world = world;

        rc = configure_bwd_kernel(dev);
        if (rc != B2A_OK) return rc;
        // Without copies the extra CTAs are attention CTAs like the others (sharded documents
        // only: a launch that never had copy tasks keeps its grid).
        const int comm = plan.comm_tasks.empty() ? 0 : a->num_comm_sm;
        const int grid = a->num_comp_sm + comm;
        profile_mark(B2A_KERNEL_BWD, false, stream);
        bwd_kernel<<<grid, kBwdThreads, kRingBwdSmemBytes, stream>>>(map_q, map_k, map_v, map_do, p);
        profile_mark(B2A_KERNEL_BWD, true, stream);
        B2A_CUDA_OK(cudaGetLastError());

        BwdPostParams post{};
        post.dq_accum = dq_accum;
        post.dq = static_cast<__nv_bfloat16*>(a->dq);
        post.batch = 1;
        post.seqlen_q = a->total_q;
        post.heads_q = a->heads_q;
        post.padded_q = a->total_q;
        post.scale = scale;
        dim3 qgrid(a->total_q / kTileM, a->heads_q);
        bwd_postprocess_kernel<<<qgrid, 128, 0, stream>>>(post);
        B2A_CUDA_OK(cudaGetLastError());
    } else {
        // A rank without tokens contributes nothing but must still report completion.
        ring_signal_kernel<<<1, 1, 0, stream>>>(a->completion_peer[0], a->completion_peer[1], a->completion_peer[2],
                                                a->completion_peer[3], a->completion_peer[4], a->completion_peer[5],
                                                a->completion_peer[6], a->completion_peer[7], world);
        B2A_CUDA_OK(cudaGetLastError());
    }

    // Every rank has added its contributions once this rank's counter reaches the world size.
    ring_wait_kernel<<<1, 1, 0, stream>>>(a->completion_peer[rank], world, &hdr->status, completion_timeout_ns());
    B2A_CUDA_OK(cudaGetLastError());
    if (a->local_total_k > 0) {
        for (int which = 0; which < 2; ++which) {
            BwdPostParams cast{};
            cast.dq_accum = which == 0 ? a->dk_accum_peer[rank] : a->dv_accum_peer[rank];
            cast.dq = static_cast<__nv_bfloat16*>(which == 0 ? a->dk : a->dv);
            cast.batch = 1;
            cast.seqlen_q = a->local_total_k;
            cast.heads_q = a->heads_k;
            cast.padded_q = a->local_total_k;
            cast.scale = 1.0f;
            cast.tile_head_stride = 1;
            cast.tile_row_stride = a->heads_k;
            dim3 cgrid(a->local_total_k / kTileN, a->heads_k);
            bwd_postprocess_kernel<<<cgrid, 128, 0, stream>>>(cast);
            B2A_CUDA_OK(cudaGetLastError());
        }
    }
    return B2A_OK;
}

}  // extern "C"
