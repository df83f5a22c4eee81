// C-ABI entry point of the context-parallel ("mega ring") forward: one persistent launch per
// rank that pulls the other ranks' K/V blocks into the local arena with a few copy CTAs while
// the remaining CTAs run attention over blocks as they become ready.
#include "b2a_ring_host.cuh"

#include <cmath>
#include <cstring>

namespace b2a {
namespace {

constexpr size_t kRingFwdSmemBytes = sizeof(FwdShared) + 1024;

struct RingFwdLayout {
    size_t docs_off, work_off, tasks_off, flags_off, total;
    size_t work_cap, task_cap, flag_count;
};

RingFwdLayout ring_fwd_layout(int batch, int world, int cap, int total_q) {
    RingFwdLayout l{};
    l.work_cap = static_cast<size_t>(total_q) / kFwdRowsPerWork + 2 * static_cast<size_t>(batch) + 1;
    l.flag_count = static_cast<size_t>(world) * cap / kTileN;
    l.task_cap = l.flag_count;
    size_t off = sizeof(WorkspaceHeader);
    l.docs_off = off;
    off = align_up(off + static_cast<size_t>(batch) * sizeof(RingDoc), 16);
    l.work_off = off;
    off = align_up(off + l.work_cap * sizeof(int4), 16);
    l.tasks_off = off;
    off = align_up(off + l.task_cap * sizeof(int2), 16);
    l.flags_off = off;
    off += l.flag_count * sizeof(int);
    l.total = align_up(off, 256);
    return l;
}

}  // namespace
}  // namespace b2a

extern "C" {

size_t b2a_ring_fwd_workspace_bytes(int32_t batch, int32_t world_size, int32_t rank_kv_capacity,
                                    int32_t total_q) {
    return b2a::ring_fwd_layout(batch, world_size, rank_kv_capacity, total_q).total;
}

int b2a_ring_fwd(const b2a_ring_fwd_args* a, void* cuda_stream) {
    using namespace b2a;
    B2A_REQUIRE(a != nullptr, "args must not be NULL");
    B2A_REQUIRE(a->head_dim == kHeadDim, "head_dim must be 128, got %d", a->head_dim);
    B2A_REQUIRE(a->heads_q >= 1 && a->heads_k >= 1 && a->heads_q % a->heads_k == 0,
                "heads_q %% heads_k must be 0, got heads_q=%d heads_k=%d", a->heads_q, a->heads_k);
    B2A_REQUIRE(a->cu_seqlens_q_host && a->global_seqlens_host && a->ring_sizes_host && a->ring_starts_host,
                "host metadata arrays must not be NULL");
    B2A_REQUIRE(a->arena_k && a->arena_v, "arena_k and arena_v must not be NULL");
    B2A_REQUIRE(a->num_comp_sm > 0, "num_comp_sm must be positive. Got %d", a->num_comp_sm);
    B2A_REQUIRE(a->num_comm_sm >= 0, "num_comm_sm must be non-negative. Got %d", a->num_comm_sm);
    B2A_REQUIRE(a->total_q >= 0, "total_q must be non-negative");
    const int causal = a->is_causal ? 1 : 0;

    RingPlan plan;
    int rc = build_ring_plan(&plan, a->batch, a->world_size, a->rank, a->rank_kv_capacity, causal,
                             a->cu_seqlens_q_host, a->global_seqlens_host, a->ring_sizes_host,
                             a->ring_starts_host);
    if (rc != B2A_OK) return rc;
    B2A_REQUIRE(a->cu_seqlens_q_host[a->batch] == a->total_q, "cu_seqlens_q_host[-1] must equal total_q");
    B2A_REQUIRE(plan.comm_tasks.empty() || a->num_comm_sm > 0,
                "num_comm_sm must be positive when documents are sharded over more than one rank");
    for (int r = 0; r < a->world_size; ++r) {
        B2A_REQUIRE(r == a->rank || plan.comm_tasks.empty() || (a->peer_k[r] && a->peer_v[r]),
                    "peer_k / peer_v of rank %d must not be NULL", r);
    }

    DeviceInfo dev{};
    rc = current_device_info(&dev);
    if (rc != B2A_OK) return rc;
    B2A_REQUIRE(a->num_comp_sm + a->num_comm_sm <= dev.sm_count,
                "num_comp_sm + num_comm_sm = %d exceeds the %d SMs of the device (all CTAs must be co-resident)",
                a->num_comp_sm + a->num_comm_sm, dev.sm_count);
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

    const RingFwdLayout lay = ring_fwd_layout(a->batch, a->world_size, a->rank_kv_capacity, a->total_q);
    B2A_REQUIRE(a->workspace != nullptr && (reinterpret_cast<uintptr_t>(a->workspace) & 0xF) == 0,
                "workspace must be a 16-byte aligned device pointer");
    if (a->workspace_bytes < lay.total) {
        return fail(B2A_ERR_WORKSPACE_TOO_SMALL, "workspace has %zu bytes, need %zu", a->workspace_bytes, lay.total);
    }

    // Work list: (document, half, 256-row piece), most expensive first.
    struct Entry { int4 e; int cost; };
    std::vector<Entry> entries;
    for (int d : plan.doc_order) {
        const RingDoc& doc = plan.docs[d];
        const int hb = doc.half_len / kTileN;
        const int halves = ring_halves(causal, doc.ring_size);
        for (int h = 0; h < halves; ++h) {
            const int n_full = ring_full_chunks(causal, doc.ring_size, doc.ring_rank, h) * hb;
            for (int pair = 0; pair * 2 < hb; ++pair) {
                const int t_last = std::min(hb - 1, pair * 2 + 1);
                entries.push_back({make_int4(d, h, pair, 0), n_full + (causal ? t_last + 1 : 0)});
            }
        }
    }
    std::stable_sort(entries.begin(), entries.end(), [](const Entry& x, const Entry& y) { return x.cost > y.cost; });
    B2A_REQUIRE(entries.size() <= lay.work_cap && plan.comm_tasks.size() <= lay.task_cap,
                "internal: ring work list exceeds its workspace bound");

    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    auto* hdr = reinterpret_cast<WorkspaceHeader*>(ws);
    B2A_CUDA_OK(cudaMemsetAsync(hdr, 0, sizeof(WorkspaceHeader), stream));
    B2A_CUDA_OK(cudaMemsetAsync(ws + lay.flags_off, 0, lay.flag_count * sizeof(int), stream));
    if (a->stats != nullptr) {
        B2A_CUDA_OK(cudaMemsetAsync(a->stats, 0, 2 * sizeof(long long), stream));   // the kernel counts
    }
    if (entries.empty()) return B2A_OK;   // this rank holds no tokens

    // One staged upload of [documents | work list | copy tasks].
    std::vector<uint8_t> host(lay.flags_off - lay.docs_off, 0);
    memcpy(host.data(), plan.docs.data(), plan.docs.size() * sizeof(RingDoc));
    {
        int4* w = reinterpret_cast<int4*>(host.data() + (lay.work_off - lay.docs_off));
        for (size_t i = 0; i < entries.size(); ++i) w[i] = entries[i].e;
        if (!plan.comm_tasks.empty()) {
            memcpy(host.data() + (lay.tasks_off - lay.docs_off), plan.comm_tasks.data(),
                   plan.comm_tasks.size() * sizeof(int2));
        }
    }
    B2A_CUDA_OK(cudaMemcpyAsync(ws + lay.docs_off, host.data(), host.size(), cudaMemcpyHostToDevice, stream));

    const int arena_rows = a->world_size * a->rank_kv_capacity;
    CUtensorMap map_q, map_k, map_v;
    rc = make_token_map(&map_q, a->q, a->total_q, a->heads_q, kTileM);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_k, a->arena_k, arena_rows, a->heads_k, kTileN);
    if (rc != B2A_OK) return rc;
    rc = make_token_map(&map_v, a->arena_v, arena_rows, a->heads_k, kTileN);
    if (rc != B2A_OK) return rc;

    FwdParams p{};
    p.o = static_cast<__nv_bfloat16*>(a->out);
    p.lse = a->lse;
    p.sched_counter = &hdr->sched_counter;
    p.num_entries_dev = &hdr->num_entries;
    p.status = &hdr->status;
    p.batch = a->batch;
    p.total_q = a->total_q;
    p.total_k = arena_rows;
    p.heads_q = a->heads_q;
    p.heads_k = a->heads_k;
    p.causal = causal;
    p.num_entries_host = static_cast<int>(entries.size());
    p.scale = 1.0f / std::sqrt(static_cast<float>(kHeadDim));
    p.scale_log2 = p.scale * kLog2e;
    p.lse_head_stride = a->total_q;
    p.timeout_ns = wait_timeout_ns();
    p.ring_docs = reinterpret_cast<const RingDoc*>(ws + lay.docs_off);
    p.ring_work = reinterpret_cast<const int4*>(ws + lay.work_off);
    p.comm_tasks = reinterpret_cast<const int2*>(ws + lay.tasks_off);
    p.comm_task_count = static_cast<int>(plan.comm_tasks.size());
    p.my_rank = a->rank;
    p.kv_row_bytes = a->heads_k * kHeadDim * 2;
    for (int r = 0; r < 8; ++r) {
        p.peer_k[r] = r < a->world_size ? static_cast<const uint8_t*>(a->peer_k[r]) : nullptr;
        p.peer_v[r] = r < a->world_size ? static_cast<const uint8_t*>(a->peer_v[r]) : nullptr;
    }
    p.arena_k = static_cast<uint8_t*>(a->arena_k);
    p.arena_v = static_cast<uint8_t*>(a->arena_v);
    p.kv_flags = reinterpret_cast<int*>(ws + lay.flags_off);
    p.copy_done = &hdr->reserved;
    p.stats = reinterpret_cast<unsigned long long*>(a->stats);

    const int comm = p.comm_task_count > 0 ? a->num_comm_sm : 0;
    int grid = a->num_comp_sm + comm;
    p.num_comp = a->num_comp_sm;

    rc = configure_fwd_kernel(dev, false);
    if (rc != B2A_OK) return rc;
    profile_mark(B2A_KERNEL_FWD, false, stream);
    fwd_kernel<false><<<grid, kFwdThreads, kRingFwdSmemBytes, stream>>>(map_q, map_k, map_v, p);
    profile_mark(B2A_KERNEL_FWD, true, stream);
    B2A_CUDA_OK(cudaGetLastError());
    return B2A_OK;
}

}  // extern "C"
