// Host-side planning shared by the context-parallel forward and backward entry points:
// turns the ring metadata (global lengths, ring sizes, ring starts) into the per-document
// placement table, the copy-task list and the per-rank slice offsets.
#pragma once

#include <algorithm>
#include <cstdint>
#include <vector>

#include "b2a_fwd.cuh"
#include "b2a_host.cuh"

namespace b2a {

struct RingPlan {
    int batch = 0;
    int world = 0;
    int rank = 0;
    int cap = 0;                         // arena rows per rank
    std::vector<RingDoc> docs;           // one per document (non-members have half_len 0)
    std::vector<int> local_len;          // this rank's local length per document
    std::vector<int2> comm_tasks;        // (source rank, arena 128-row block)
    std::vector<int> doc_order;          // member documents, longest first
};

// Validates the metadata the way the reference bindings do
// (csrc/mega_ring_min_fa3_varlen_ring_bindings.cu:423-468) and fills the plan.
inline int build_ring_plan(RingPlan* plan, int batch, int world, int rank, int cap, int causal,
                           const int32_t* cu_seqlens_q_host, const int32_t* global_seqlens,
                           const int32_t* ring_sizes, const int32_t* ring_starts) {
    B2A_REQUIRE(batch >= 1, "batch must be >= 1");
    B2A_REQUIRE(world == 1 || world == 2 || world == 4 || world == 8, "world size must be 1, 2, 4 or 8, got %d", world);
    B2A_REQUIRE(rank >= 0 && rank < world, "rank %d out of range for world size %d", rank, world);
    B2A_REQUIRE(cap > 0 && cap % 128 == 0, "rank_kv_capacity must be a positive multiple of 128, got %d", cap);
    plan->batch = batch;
    plan->world = world;
    plan->rank = rank;
    plan->cap = cap;
    plan->docs.assign(batch, RingDoc{});
    plan->local_len.assign(batch, 0);
    std::vector<int> off(world, 0);   // running slice offset of every rank
    int prev_size = 1 << 30;
    for (int d = 0; d < batch; ++d) {
        const int g = ring_sizes[d], start = ring_starts[d], glen = global_seqlens[d];
        B2A_REQUIRE(g == 1 || g == 2 || g == 4 || g == 8, "ring size must be 1, 2, 4 or 8, got %d", g);
        B2A_REQUIRE(g <= world, "ring size %d exceeds world size %d", g, world);
        B2A_REQUIRE(g <= prev_size, "batch must be ordered by non-increasing ring size");
        prev_size = g;
        B2A_REQUIRE(start >= 0 && start % g == 0 && start + g <= world,
                    "ring start %d must be aligned to ring size %d and fit the world", start, g);
        B2A_REQUIRE(glen > 0 && glen % g == 0, "global length %d must be a positive multiple of ring size %d", glen, g);
        const int llen = glen / g;
        B2A_REQUIRE(llen % 128 == 0, "local length %d must be a multiple of 128", llen);
        if (causal && g > 1) {
            B2A_REQUIRE((llen / 2) % 128 == 0, "causal ring halves must be multiples of 128, got local length %d", llen);
        }
        const bool member = rank >= start && rank < start + g;
        const int mine = cu_seqlens_q_host[d + 1] - cu_seqlens_q_host[d];
        B2A_REQUIRE(mine == (member ? llen : 0),
                    "local length of document %d is %d but the ring metadata implies %d", d, mine, member ? llen : 0);
        RingDoc& doc = plan->docs[d];
        doc.q_begin = cu_seqlens_q_host[d];
        doc.ring_size = g;
        doc.ring_rank = member ? rank - start : 0;
        doc.half_len = member ? llen / ring_halves(causal, g) : 0;
        for (int j = 0; j < 8; ++j) doc.member_row[j] = 0;
        for (int j = 0; j < g; ++j) {
            doc.member_row[j] = (start + j) * cap + off[start + j];
            off[start + j] += llen;
            B2A_REQUIRE(off[start + j] <= cap, "rank %d holds more than rank_kv_capacity=%d key rows", start + j, cap);
        }
        if (member) {
            plan->local_len[d] = llen;
            plan->doc_order.push_back(d);
        }
    }
    std::stable_sort(plan->doc_order.begin(), plan->doc_order.end(),
                     [&](int a, int b) { return global_seqlens[a] > global_seqlens[b]; });
    // Copy tasks in the order the attention loops consume remote chunks: for every document,
    // sources r-1, r-2, ... around its ring.  Causal: the front half always, the back half only
    // for sources after r (a local query half can see it).  Without a mask a shard is one chunk.
    for (int d : plan->doc_order) {
        const RingDoc& doc = plan->docs[d];
        const int g = doc.ring_size, r = doc.ring_rank, start = ring_starts[d];
        const int hb = doc.half_len / 128;
        for (int i = 1; i < g; ++i) {
            const int s = (r - i + g) % g;
            const int row0 = doc.member_row[s];
            for (int w = 0; w < hb; ++w) plan->comm_tasks.push_back(make_int2(start + s, row0 / 128 + w));
            if (causal && s > r) {
                for (int w = 0; w < hb; ++w) {
                    plan->comm_tasks.push_back(make_int2(start + s, (row0 + doc.half_len) / 128 + w));
                }
            }
        }
    }
    return B2A_OK;
}

}  // namespace b2a
