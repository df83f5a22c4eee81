// Forward attention for sm_100a: O = softmax(scale * Q K^T [+ causal mask]) V, LSE.
//
// One persistent CTA per SM.  A work item is 256 query rows of one document and
// one query head, processed as two 128-row tiles (A, B) that ping-pong on the
// tensor core.  Where a document (or its last piece) has at most 128 rows left there is
// no second row tile; the item then covers TWO query heads of the same K/V head for those
// rows (tile A = head h, tile B = head h + 1, same K/V stream), so that the ping-pong --
// and with it the overlap of softmax and tensor core -- is kept for short documents and tails.
//
//   warp  0-3   softmax warpgroup of tile A (one thread per query row)
//   warp  4-7   softmax warpgroup of tile B
//   warp  8     tcgen05.mma issue
//   warp  9     TMA loads and work fetch
//   warp 10-11  idle (they only donate their registers)
//
// Tensor memory (512 columns): S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512).
// P (bf16) overwrites the first 64 columns of its S tile and is consumed by the
// P*V MMA straight from tensor memory.  K and V tiles travel through one shared
// ring of 32 KiB stages in the order K(j0) V(j0) K(j0-1) V(j0-1) ...
//
// BSHD and varlen inputs share the code path: both are addressed as a flat
// [tokens, heads, 128] tensor plus per-document (begin, length) pairs.
#pragma once

#include "b2a_ptx.cuh"

namespace b2a {

// Which of the 16 four-element groups of a 64-column half row take two of their exponentials
// from the FMA-pipe polynomial instead of the special-function unit (bit g: group g).
// Measured in SM clocks per 128x128 block: none 1830, every second group (25 % of the
// exponentials) 1797, all groups (50 %) 1866.
#ifndef B2A_FWD_EXP_POLY_MASK
#define B2A_FWD_EXP_POLY_MASK 0x5555u
#endif
constexpr uint32_t kFwdExpPolyMask = B2A_FWD_EXP_POLY_MASK;

constexpr int kHeadDim = 128;
constexpr int kTileM = 128;          // query rows per tile
constexpr int kTileN = 128;          // key rows per K/V block
constexpr int kFwdTilesPerCta = 2;   // tiles per work item
constexpr int kFwdRowsPerWork = kTileM * kFwdTilesPerCta;
constexpr int kFwdStages = 4;        // K/V ring stages
constexpr int kFwdThreads = 384;
constexpr uint32_t kTileBytes = kTileM * kHeadDim * 2;   // 32 KiB bf16 tile
constexpr uint32_t kHalfTileBytes = kTileBytes / 2;      // one 64-column half
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units; lazy O rescale

struct FwdParams {
    __nv_bfloat16* o;            // [tokens_q, heads_q, 128]
    float* lse;                  // see lse_head_stride / lse_batch_stride
    const int* cu_seqlens_q;     // [batch + 1] or null for BSHD
    const int* cu_seqlens_k;
    const int2* work_list;       // varlen: (doc, m_block) in LPT order; null for BSHD
    const int* num_entries_dev;  // varlen: number of work_list entries (device word)
    int* sched_counter;          // zeroed before launch
    unsigned int* status;
    int batch;
    int seqlen_q;                // BSHD: S_q.  varlen: unused
    int seqlen_k;
    int total_q;
    int total_k;
    int heads_q;
    int heads_k;
    int causal;
    int num_entries_host;        // BSHD: batch * m_blocks.  varlen: upper bound (unused)
    float scale;                 // softmax scale
    float scale_log2;            // scale * log2(e)
    long long lse_head_stride;   // elements between heads
    long long lse_batch_stride;  // BSHD: elements between batches (heads_q * S_q)
    // Running-merge mode (context-parallel steps): O/LSE already hold a partial
    // result that this call's contribution is merged into.
    int merge;
    // Offset added to key positions for the causal rule: a key at local index c
    // is visible to local query row r when c + k_pos_offset <= r + q_pos_offset + (k_len - q_len)
    // (both 0 for plain attention).
    uint32_t timeout_ns;
    // ---- context-parallel ("mega ring") mode: all of this is null / 0 otherwise -------
    const struct RingDoc* ring_docs;   // per document ring placement (device)
    const int4* ring_work;             // (doc, half, row-pair index, 0) in LPT order
    const int2* comm_tasks;            // (source rank, arena 128-row block) in fetch order
    int comm_task_count;
    int num_comp;                      // CTAs [num_comp, gridDim.x) start as copy CTAs
    int my_rank;
    int kv_row_bytes;                  // heads_k * 256
    const uint8_t* peer_k[8];          // arena base of every rank as mapped on this device
    const uint8_t* peer_v[8];
    uint8_t* arena_k;                  // this rank's arena (the tensor maps of K/V cover it)
    uint8_t* arena_v;
    int* kv_flags;                     // per 128-row arena block: 1 once K and V have landed
    int* copy_done;                    // number of copy CTAs that have finished all their tasks
    unsigned long long* stats;         // optional [2]: query tiles visited, K/V tile reads (counted by the kernel)
    // ---- ring step mode: CTAs [num_comp, gridDim.x) first copy two flat buffers (another rank's
    // K and V) into local prefetch buffers, then join the attention work queue.  0 otherwise.
    const uint8_t* prefetch_src[2];
    uint8_t* prefetch_dst[2];
    unsigned long long prefetch_bytes; // per buffer, a multiple of 16
};

// Placement of one document on its ring.  Lengths are in tokens, multiples of 128.
struct RingDoc {
    int q_begin;        // first local token of the document on this rank
    int half_len;       // local length / 2 on a causal ring (zigzag halves), else the local length
    int ring_size;      // G
    int ring_rank;      // this rank's position in the ring (global rank - ring_start)
    int member_row[8];  // arena row of the document's slice on ring member s
};

struct FwdWork {
    int q_begin;   // first token of the document in the flat Q tensor
    int q_len;
    int k_begin;
    int k_len;
    int m0;        // first query row (document-local) of the work item
    int head;
    int head_k;
    long long lse_base;   // element offset of document row 0 for this head
    int n_full;    // ring mode: unmasked K/V blocks of other chunks that precede the own chunk
    int doc;       // ring mode: document index
    int half;      // ring mode: 0 = front half, 1 = back half of the local zigzag shard
    int pair;      // 1: at most 128 rows left -> tiles A / B are heads `head`, `head + 1` of the same rows
                   // (only the even head of each pair carries the work; the odd one's item is empty)
};

// First row (document-local) and query head of tile x of a work item.
__device__ __forceinline__ int fwd_tile_row0(const FwdWork& wk, int x) {
    return wk.m0 + (wk.pair ? 0 : x * kTileM);
}
__device__ __forceinline__ int fwd_tile_head(const FwdWork& wk, int x) {
    return wk.head + (wk.pair ? x : 0);
}

// Whether a piece that starts at row m0 of a q_len-row document runs as a pair of heads.
__device__ __forceinline__ int fwd_pair_mode(const FwdParams& p, int q_len, int m0) {
    return (q_len - m0 <= kTileM && ((p.heads_q / p.heads_k) & 1) == 0) ? 1 : 0;
}

struct __align__(1024) FwdShared {
    uint8_t q[kFwdTilesPerCta][kTileBytes];
    uint8_t kv[kFwdStages][kTileBytes];
    uint64_t q_full[kFwdTilesPerCta];
    uint64_t q_empty[kFwdTilesPerCta];
    uint64_t kv_full[kFwdStages];
    uint64_t kv_empty[kFwdStages];
    uint64_t s_full[kFwdTilesPerCta];
    uint64_t p_full[kFwdTilesPerCta];
    uint64_t o_full[kFwdTilesPerCta];
    uint64_t sched_full[2];
    uint64_t sched_empty[2];
    uint64_t comm_full[6];
    uint64_t comm_empty[6];
    int sched_w[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// Pieces a member's shard is cut into: two zigzag halves on a causal ring, otherwise one.
__host__ __device__ __forceinline__ int ring_halves(int causal, int ring_size) {
    return (causal && ring_size > 1) ? 2 : 1;
}

// Number of whole (unmasked) chunks a query piece sees before its own chunk.  A chunk is
// half_len tokens.  Causal: zigzag rank r of a ring of G holds global chunks r (front) and
// 2G-1-r (back), and a query chunk sees every chunk with a smaller global index.  Without a
// mask every member's shard is one chunk and all G of them are visible.
__host__ __device__ __forceinline__ int ring_full_chunks(int causal, int ring_size, int ring_rank, int half) {
    if (causal) {
        if (ring_size == 1) return 0;
        return half == 0 ? ring_rank : 2 * ring_size - 1 - ring_rank;
    }
    return ring_size;
}

__device__ __forceinline__ FwdWork fwd_decode_work(const FwdParams& p, int w) {
    FwdWork wk;
    int entry = w / p.heads_q;
    wk.head = w - entry * p.heads_q;
    wk.head_k = wk.head / (p.heads_q / p.heads_k);
    wk.n_full = 0;
    wk.doc = 0;
    wk.half = 0;
    if (p.ring_docs != nullptr) {
        const int4 e = p.ring_work[entry];
        const RingDoc& d = p.ring_docs[e.x];
        wk.doc = e.x;
        wk.half = e.y;
        wk.q_begin = d.q_begin + e.y * d.half_len;
        wk.q_len = d.half_len;
        wk.k_begin = 0;
        wk.k_len = p.causal ? d.half_len : 0;   // own-chunk keys (none when everything is unmasked)
        wk.m0 = e.z * kFwdRowsPerWork;
        wk.n_full = ring_full_chunks(p.causal, d.ring_size, d.ring_rank, e.y) * (d.half_len / kTileN);
        wk.lse_base = static_cast<long long>(wk.head) * p.lse_head_stride + wk.q_begin;
        wk.pair = fwd_pair_mode(p, wk.q_len, wk.m0);
        return wk;
    }
    if (p.cu_seqlens_q == nullptr) {
        int nmb = (p.seqlen_q + kFwdRowsPerWork - 1) / kFwdRowsPerWork;
        int b = entry / nmb;
        int mi = entry - b * nmb;
        int mblk = p.causal ? (nmb - 1 - mi) : mi;
        wk.q_begin = b * p.seqlen_q;
        wk.q_len = p.seqlen_q;
        wk.k_begin = b * p.seqlen_k;
        wk.k_len = p.seqlen_k;
        wk.m0 = mblk * kFwdRowsPerWork;
        wk.lse_base = static_cast<long long>(b) * p.lse_batch_stride +
                      static_cast<long long>(wk.head) * p.lse_head_stride;
    } else {
        int2 e = p.work_list[entry];
        int doc = e.x;
        wk.q_begin = p.cu_seqlens_q[doc];
        wk.q_len = p.cu_seqlens_q[doc + 1] - wk.q_begin;
        wk.k_begin = p.cu_seqlens_k[doc];
        wk.k_len = p.cu_seqlens_k[doc + 1] - wk.k_begin;
        wk.m0 = e.y * kFwdRowsPerWork;
        wk.lse_base = static_cast<long long>(wk.head) * p.lse_head_stride + wk.q_begin;
    }
    wk.pair = fwd_pair_mode(p, wk.q_len, wk.m0);
    return wk;
}

// Number of K/V blocks tile `x` of the work item needs (0 when the tile has no
// query row, or no visible key).
__device__ __forceinline__ int fwd_num_kv_blocks(const FwdParams& p, const FwdWork& wk, int x) {
    if (wk.pair && (wk.head & 1)) {
        return 0;   // the even head of the pair carries both
    }
    int row0 = fwd_tile_row0(wk, x);
    if (row0 >= wk.q_len) {
        return 0;
    }
    int limit = wk.k_len;
    if (p.causal) {
        int row_last = min(row0 + kTileM, wk.q_len) - 1;
        limit = min(limit, row_last + 1 + wk.k_len - wk.q_len);
    }
    const int own = limit <= 0 ? 0 : (limit + kTileN - 1) / kTileN;
    return wk.n_full + own;
}

// Ring mode: arena row of virtual K/V block j of a work item, and whether it comes from
// another rank (then its arena block must be flagged ready before it is read).  Blocks
// j >= n_full are the own (diagonal) chunk; below that the chunks are visited in the order
// the copy CTAs fetch them: the other local half, then sources r-1, r-2, ... around the ring.
__device__ __forceinline__ int ring_kv_row(const FwdParams& p, const FwdWork& wk, int j, bool* remote) {
    const RingDoc& d = p.ring_docs[wk.doc];
    const int hb = d.half_len / kTileN;
    const int g = d.ring_size;
    const int r = d.ring_rank;
    int s, hf, blk;
    if (j >= wk.n_full) {
        s = r;
        hf = wk.half;
        blk = j - wk.n_full;
    } else {
        const int idx = wk.n_full - 1 - j;
        const int slot = idx / hb;
        blk = idx - slot * hb;
        if (p.causal) {
            if (wk.half == 0) {
                s = r - 1 - slot;
                hf = 0;
            } else if (slot <= r) {
                s = r - slot;
                hf = 0;
            } else {
                const int k = slot - r - 1;
                s = g - 1 - (k >> 1);
                hf = k & 1;
            }
        } else {
            // no mask: the own shard first, then sources r-1, r-2, ... around the ring
            s = (r - slot + g) % g;
            hf = 0;
        }
    }
    *remote = (s != r);
    return d.member_row[s] + hf * d.half_len + blk * kTileN;
}

// Bounded wait until a device-scope flag word becomes non-zero (acquire).
__device__ __forceinline__ bool flag_wait(const WaitCtx& ctx, const int* flag, uint32_t tag) {
    const uint32_t start = global_timer_lo();
    uint32_t polls = 0;
#pragma unroll 1
    while (true) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v != 0) return true;
        if ((++polls & 0xFu) == 0u) {
            if (ld_shared_volatile_u32(ctx.abort_smem) != 0u) return false;
            if (global_timer_lo() - start > ctx.timeout_ns) {
                st_shared_volatile_u32(ctx.abort_smem, 1u);
                set_status(ctx.status, kStatusTimeout, (tag << 12) | (blockIdx.x & 0xFFFu));
                return false;
            }
            __nanosleep(100);
        }
    }
}

// Copy role of a ring-mode CTA: tasks are 128-row arena blocks owned by other ranks.  One
// thread streams 32 KiB bulk loads peer -> shared (6 slots over the Q and K/V tile buffers),
// another streams bulk stores shared -> local arena and publishes the block's flag once its
// K and V have both landed.  No multicast; every wait is bounded.
__device__ __forceinline__ void ring_copy_role(const FwdParams& p, FwdShared& sh, const WaitCtx& wctx,
                                               int warp, int lane) {
    constexpr uint32_t kSlotBytes = kTileBytes;   // 32 KiB
    const uint32_t block_bytes = static_cast<uint32_t>(kTileN) * p.kv_row_bytes;
    const uint32_t chunks = block_bytes / kSlotBytes;
    const uint32_t slot_base = smem_u32(&sh.q[0][0]);
    const int first = static_cast<int>(blockIdx.x) - p.num_comp;
    const int stride = static_cast<int>(gridDim.x) - p.num_comp;
    if (warp == 9 && lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int t = first; t < p.comm_task_count && ok; t += stride) {
            const int2 task = p.comm_tasks[t];
            const size_t off = static_cast<size_t>(task.y) * block_bytes;
            for (int kv = 0; kv < 2 && ok; ++kv) {
                const uint8_t* src = (kv == 0 ? p.peer_k[task.x] : p.peer_v[task.x]) + off;
                for (uint32_t c = 0; c < chunks; ++c, ++it) {
                    const uint32_t slot = it % 6u;
                    ok = mbar_wait(wctx, smem_u32(&sh.comm_empty[slot]), ((it / 6u) & 1u) ^ 1u, 14);
                    if (!ok) break;
                    mbar_arrive_expect_tx(smem_u32(&sh.comm_full[slot]), kSlotBytes);
                    bulk_load_1d(slot_base + slot * kSlotBytes, src + static_cast<size_t>(c) * kSlotBytes,
                                 kSlotBytes, smem_u32(&sh.comm_full[slot]));
                }
            }
        }
    } else if (warp == 10 && lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int t = first; t < p.comm_task_count && ok; t += stride) {
            const int2 task = p.comm_tasks[t];
            const size_t off = static_cast<size_t>(task.y) * block_bytes;
            for (int kv = 0; kv < 2 && ok; ++kv) {
                uint8_t* dst = (kv == 0 ? p.arena_k : p.arena_v) + off;
                for (uint32_t c = 0; c < chunks; ++c, ++it) {
                    const uint32_t slot = it % 6u;
                    ok = mbar_wait(wctx, smem_u32(&sh.comm_full[slot]), (it / 6u) & 1u, 15);
                    if (!ok) break;
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                 ::"l"(reinterpret_cast<uint64_t>(dst + static_cast<size_t>(c) * kSlotBytes)),
                                   "r"(slot_base + slot * kSlotBytes), "r"(kSlotBytes)
                                 : "memory");
                    bulk_commit_group();
                    bulk_wait_group_read<0>();
                    mbar_arrive(smem_u32(&sh.comm_empty[slot]));
                }
            }
            if (ok) {
                bulk_wait_group<0>();        // the block's K and V are in the arena
                fence_proxy_async_all();
                asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.kv_flags + task.y), "r"(1)
                             : "memory");
            }
        }
        bulk_wait_group<0>();
        // Once every copy CTA has reported here, all remote blocks are in place and the load
        // warps stop looking at per-block flags.
        fence_proxy_async_all();
        asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p.copy_done), "r"(ok ? 1 : 0) : "memory");
    }
}

// Copy role of a ring-step CTA: two flat buffers (K, then V) are cut into 32 KiB pieces that
// the copy CTAs take round-robin and move peer -> shared -> local with the same two-thread,
// six-slot pipeline as above.  The last piece of a buffer may be shorter (still a multiple of 16).
__device__ __forceinline__ void prefetch_copy_role(const FwdParams& p, FwdShared& sh, const WaitCtx& wctx,
                                                   int warp, int lane) {
    constexpr unsigned long long kSlotBytes = kTileBytes;
    const uint32_t slot_base = smem_u32(&sh.q[0][0]);
    const long long per_buf = static_cast<long long>((p.prefetch_bytes + kSlotBytes - 1) / kSlotBytes);
    const long long first = static_cast<long long>(blockIdx.x) - p.num_comp;
    const long long stride = static_cast<long long>(gridDim.x) - p.num_comp;
    if ((warp != 9 && warp != 10) || lane != 0) return;
    uint32_t it = 0;
    bool ok = true;
    for (long long t = first; t < 2 * per_buf && ok; t += stride, ++it) {
        const int kv = t >= per_buf ? 1 : 0;
        const unsigned long long off = static_cast<unsigned long long>(t - kv * per_buf) * kSlotBytes;
        const unsigned long long left = p.prefetch_bytes - off;
        const uint32_t bytes = static_cast<uint32_t>(left < kSlotBytes ? left : kSlotBytes);
        const uint32_t slot = it % 6u;
        if (warp == 9) {
            ok = mbar_wait(wctx, smem_u32(&sh.comm_empty[slot]), ((it / 6u) & 1u) ^ 1u, 27);
            if (!ok) break;
            mbar_arrive_expect_tx(smem_u32(&sh.comm_full[slot]), bytes);
            bulk_load_1d(slot_base + slot * static_cast<uint32_t>(kSlotBytes), p.prefetch_src[kv] + off, bytes,
                         smem_u32(&sh.comm_full[slot]));
        } else {
            ok = mbar_wait(wctx, smem_u32(&sh.comm_full[slot]), (it / 6u) & 1u, 28);
            if (!ok) break;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(reinterpret_cast<uint64_t>(p.prefetch_dst[kv] + off)),
                           "r"(slot_base + slot * static_cast<uint32_t>(kSlotBytes)), "r"(bytes)
                         : "memory");
            bulk_commit_group();
            bulk_wait_group_read<0>();
            mbar_arrive(smem_u32(&sh.comm_empty[slot]));
        }
    }
    if (warp == 10) bulk_wait_group<0>();
}

template <bool kMerge>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const FwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    FwdShared& sh = *reinterpret_cast<FwdShared*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kFwdTilesPerCta; ++i) {
            mbar_init(smem_u32(&sh.q_full[i]), 1);
            mbar_init(smem_u32(&sh.q_empty[i]), 1);
            mbar_init(smem_u32(&sh.s_full[i]), 1);
            mbar_init(smem_u32(&sh.p_full[i]), kTileM);
            mbar_init(smem_u32(&sh.o_full[i]), 1);
        }
        for (int i = 0; i < kFwdStages; ++i) {
            mbar_init(smem_u32(&sh.kv_full[i]), 1);
            mbar_init(smem_u32(&sh.kv_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sh.sched_full[i]), 1);
            mbar_init(smem_u32(&sh.sched_empty[i]), 1 + 2 * 4);  // MMA warp + 8 softmax warps
        }
        for (int i = 0; i < 6; ++i) {
            mbar_init(smem_u32(&sh.comm_full[i]), 1);
            mbar_init(smem_u32(&sh.comm_empty[i]), 1);
        }
        sh.abort_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh.tmem_base);

    WaitCtx wctx{smem_u32(&sh.abort_flag), p.status, p.timeout_ns};

    const int total_work =
        (p.cu_seqlens_q == nullptr ? p.num_entries_host : *p.num_entries_dev) * p.heads_q;

    // Copy CTAs (ring mode): pull the other ranks' K/V blocks into the local arena first, then
    // join the attention work queue like every other CTA.
    if (p.ring_docs != nullptr && static_cast<int>(blockIdx.x) >= p.num_comp && p.comm_task_count > 0) {
        ring_copy_role(p, sh, wctx, warp, lane);
        __syncthreads();
    }
    if (p.prefetch_bytes != 0ull && static_cast<int>(blockIdx.x) >= p.num_comp) {
        prefetch_copy_role(p, sh, wctx, warp, lane);
        __syncthreads();
    }

    if (warp >= 8) {
        reg_dealloc<72>();
        if (warp == 9) {
            // ------------------------------------------------------------ load warp
            if (lane == 0) {
                tma_prefetch_desc(&map_q);
                tma_prefetch_desc(&map_k);
                tma_prefetch_desc(&map_v);
            }
            uint32_t kv_it = 0;
            uint32_t q_cnt[2] = {0, 0};
            bool ok = true;
            // Ring mode: true once all copy CTAs are done, i.e. every remote block has landed.
            bool all_landed = p.ring_docs == nullptr || p.comm_task_count == 0;
            const int copy_ctas = static_cast<int>(gridDim.x) - p.num_comp;
            for (uint32_t it = 0; ok; ++it) {
                const uint32_t slot = it & 1u;
                ok = mbar_wait(wctx, smem_u32(&sh.sched_empty[slot]), ((it >> 1) & 1u) ^ 1u, 1);
                if (!ok) break;
                int w = 0;
                if (lane == 0) {
                    w = atomicAdd(p.sched_counter, 1);
                    if (w >= total_work) w = -1;
                    sh.sched_w[slot] = w;
                }
                w = __shfl_sync(0xFFFFFFFFu, w, 0);
                if (lane == 0) {
                    mbar_arrive(smem_u32(&sh.sched_full[slot]));
                }
                if (w < 0) break;
                const FwdWork wk = fwd_decode_work(p, w);
                int nblk[2] = {fwd_num_kv_blocks(p, wk, 0), fwd_num_kv_blocks(p, wk, 1)};
                const int n_max = max(nblk[0], nblk[1]);
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (nblk[x] > 0) {
                        ok = mbar_wait(wctx, smem_u32(&sh.q_empty[x]), (q_cnt[x] & 1u) ^ 1u, 2);
                        if (!ok) break;
                        ++q_cnt[x];
                        if (lane == 0) {
                            const uint32_t bar = smem_u32(&sh.q_full[x]);
                            const uint32_t dst = smem_u32(&sh.q[x][0]);
                            const int row = wk.q_begin + fwd_tile_row0(wk, x);
                            mbar_arrive_expect_tx(bar, kTileBytes);
                            tma_load_3d(dst, &map_q, bar, 0, fwd_tile_head(wk, x), row);
                            tma_load_3d(dst + kHalfTileBytes, &map_q, bar, 64, fwd_tile_head(wk, x), row);
                        }
                    }
                }
                for (int j = n_max - 1; j >= 0 && ok; --j) {
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {
                        const uint32_t stage = kv_it % kFwdStages;
                        ok = mbar_wait(wctx, smem_u32(&sh.kv_empty[stage]),
                                       ((kv_it / kFwdStages) & 1u) ^ 1u, 3);
                        if (!ok) break;
                        ++kv_it;
                        int row = wk.k_begin + j * kTileN;
                        if (p.ring_docs != nullptr) {
                            bool remote = false;
                            row = ring_kv_row(p, wk, j, &remote);
                            if (remote && kv == 0 && !all_landed) {
                                int landed;
                                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(landed) : "l"(p.copy_done)
                                             : "memory");
                                if (landed >= copy_ctas) {
                                    all_landed = true;
                                } else {
                                    ok = flag_wait(wctx, p.kv_flags + row / kTileN, 13);
                                    if (!ok) break;
                                }
                                fence_proxy_async_all();
                            }
                        }
                        if (lane == 0) {
                            const uint32_t bar = smem_u32(&sh.kv_full[stage]);
                            const uint32_t dst = smem_u32(&sh.kv[stage][0]);
                            const CUtensorMap* map = kv == 0 ? &map_k : &map_v;
                            mbar_arrive_expect_tx(bar, kTileBytes);
                            tma_load_3d(dst, map, bar, 0, wk.head_k, row);
                            tma_load_3d(dst + kHalfTileBytes, map, bar, 64, wk.head_k, row);
                        }
                    }
                }
            }
        } else if (warp == 8) {
            // ------------------------------------------------------------ MMA warp
            constexpr uint32_t idesc_qk = make_idesc_bf16(kTileM, kTileN, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_bf16(kTileM, kHeadDim, 0, 1);
            uint32_t kv_it = 0;
            uint32_t q_cnt[2] = {0, 0};
            uint32_t p_cnt[2] = {0, 0};
            bool ok = true;
            unsigned long long tile_visits = 0, kv_tile_reads = 0;   // CTA-local totals for p.stats
            PH_DECL(8)   // 0 other, 1 wait p_full, 2 issue PV, 3 wait K, 4 issue S
            const uint32_t s_tmem[2] = {tmem_base + 0u, tmem_base + 128u};
            const uint32_t o_tmem[2] = {tmem_base + 256u, tmem_base + 384u};

            // Descriptor low words of the Q tiles and of K/V stage 0 (a stage is 32 KiB further).
            const uint32_t q_lo[2] = {desc_lo_kmajor(smem_u32(&sh.q[0][0])), desc_lo_kmajor(smem_u32(&sh.q[1][0]))};
            const uint32_t k_lo0 = desc_lo_kmajor(smem_u32(&sh.kv[0][0]));
            const uint32_t v_lo0 = desc_lo_mnmajor(smem_u32(&sh.kv[0][0]));
            constexpr uint32_t kStageStep = kTileBytes >> 4;

            // S_x = Q_x * K^T for the K tile in `stage` (8 k-steps of 16 over head_dim).
            auto issue_qk = [&](int x, uint32_t stage) {
                umma_ss_kk_x8_w(s_tmem[x], q_lo[x], k_lo0 + stage * kStageStep, idesc_qk, 0u);
            };
            // O_x (+)= P_x * V for the V tile in `stage` (8 k-steps of 16 over keys).
            auto issue_pv = [&](int x, uint32_t stage, uint32_t accumulate) {
                umma_ts_x8_w(o_tmem[x], s_tmem[x], v_lo0 + stage * kStageStep, idesc_pv, accumulate);
            };

            for (uint32_t it = 0; ok; ++it) {
                const uint32_t slot = it & 1u;
                ok = mbar_wait(wctx, smem_u32(&sh.sched_full[slot]), (it >> 1) & 1u, 4);
                if (!ok) break;
                // Broadcast from lane 0 so that everything derived from the work index (block counts,
                // ring stages, operand descriptors) is provably warp-uniform for the compiler.
                const int w = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<volatile int*>(&sh.sched_w[slot]), 0);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(&sh.sched_empty[slot]));
                }
                if (w < 0) break;
                const FwdWork wk = fwd_decode_work(p, w);
                int nblk[2] = {fwd_num_kv_blocks(p, wk, 0), fwd_num_kv_blocks(p, wk, 1)};
                const int n_max = max(nblk[0], nblk[1]);
                if (n_max == 0) continue;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (nblk[x] > 0) {
                        ok = ok && mbar_wait(wctx, smem_u32(&sh.q_full[x]), q_cnt[x] & 1u, 5);
                        ++q_cnt[x];
                        tile_visits += 1;
                        kv_tile_reads += static_cast<unsigned long long>(nblk[x]);
                    }
                }
                if (!ok) break;
                // Prologue: S(j0) for every tile that owns block j0.
                {
                    const int j0 = n_max - 1;
                    const uint32_t stage = kv_it % kFwdStages;
                    ok = mbar_wait(wctx, smem_u32(&sh.kv_full[stage]), (kv_it / kFwdStages) & 1u, 6);
                    if (!ok) break;
                    ++kv_it;
                    tc_fence_after_sync();
                    {
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            if (j0 < nblk[x]) {
                                issue_qk(x, stage);
                                tc_commit_w(smem_u32(&sh.s_full[x]));
                                if (j0 == 0) tc_commit_w(smem_u32(&sh.q_empty[x]));
                            }
                        }
                        tc_commit_w(smem_u32(&sh.kv_empty[stage]));
                    }
                    __syncwarp();
                }
                for (int j = n_max - 1; j >= 0 && ok; --j) {
                    const uint32_t stage_v = kv_it % kFwdStages;
                    ok = mbar_wait(wctx, smem_u32(&sh.kv_full[stage_v]),
                                   (kv_it / kFwdStages) & 1u, 7);
                    if (!ok) break;
                    ++kv_it;
                    uint32_t stage_k = 0;
                    if (j > 0) {
                        stage_k = kv_it % kFwdStages;
                    }
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        if (j < nblk[x]) {
                            PH_MARK(0);
                            ok = mbar_wait(wctx, smem_u32(&sh.p_full[x]), p_cnt[x] & 1u, 8);
                            if (!ok) break;
                            ++p_cnt[x];
                            tc_fence_after_sync();
                            PH_MARK(1);
                            {
                                issue_pv(x, stage_v, j != nblk[x] - 1 ? 1u : 0u);
                                if (j == 0) tc_commit_w(smem_u32(&sh.o_full[x]));
                            }
                            __syncwarp();
                            PH_MARK(2);
#ifdef B2A_PHASES
                            ph_[9] += 1;
#endif
                        }
                        if (x == 1) {
                            tc_commit_w(smem_u32(&sh.kv_empty[stage_v]));
                        }
                        if (j > 0) {
                            if (x == 0) {
                                ok = mbar_wait(wctx, smem_u32(&sh.kv_full[stage_k]),
                                               (kv_it / kFwdStages) & 1u, 9);
                                if (!ok) break;
                                tc_fence_after_sync();
                            }
                            PH_MARK(3);
                            if (j - 1 < nblk[x]) {
                                issue_qk(x, stage_k);
                                tc_commit_w(smem_u32(&sh.s_full[x]));
                                if (j - 1 == 0) tc_commit_w(smem_u32(&sh.q_empty[x]));
                            }
                            if (x == 1) {
                                tc_commit_w(smem_u32(&sh.kv_empty[stage_k]));
                            }
                            __syncwarp();
                            PH_MARK(4);
                        }
                    }
                    if (j > 0) ++kv_it;
                }
            }
            // Each CTA submits its two totals once (reference: include/min_fa3_kernel.h:618-625).
            if (p.stats != nullptr && lane == 0 && tile_visits != 0) {
                atomicAdd(p.stats, tile_visits);
                atomicAdd(p.stats + 1, kv_tile_reads);
            }
            PH_PRINT("fwd mma", 5);
        }
    } else {
        // ---------------------------------------------------------------- softmax warpgroups
        reg_alloc<216>();
        const int x = warp >> 2;                        // tile index
        const int r = (warp & 3) * 32 + lane;           // row within the tile
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem_base + lane_base + static_cast<uint32_t>(x) * 128u;
        const uint32_t o_tmem = tmem_base + lane_base + 256u + static_cast<uint32_t>(x) * 128u;
        uint32_t s_cnt = 0;
        uint32_t o_cnt = 0;
        bool ok = true;
        const float sl2 = p.scale_log2;
        PH_DECL(8)   // 0 other, 1 wait s_full, 2 tmem load, 3 max/rescale, 4 exp + store, 5 st wait + arrive

        for (uint32_t it = 0; ok; ++it) {
            const uint32_t slot = it & 1u;
            ok = mbar_wait(wctx, smem_u32(&sh.sched_full[slot]), (it >> 1) & 1u, 10);
            if (!ok) break;
            const int w = *reinterpret_cast<volatile int*>(&sh.sched_w[slot]);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(smem_u32(&sh.sched_empty[slot]));
            }
            if (w < 0) break;
            const FwdWork wk = fwd_decode_work(p, w);
            const int tile_row0 = fwd_tile_row0(wk, x);
            if (tile_row0 >= wk.q_len || (wk.pair && (wk.head & 1))) continue;
            const int nblk = fwd_num_kv_blocks(p, wk, x);
            const int row = tile_row0 + r;
            const bool row_valid = row < wk.q_len;
            const long long tok = static_cast<long long>(wk.q_begin) + row;
            const int tile_head = fwd_tile_head(wk, x);
            __nv_bfloat16* o_row = p.o + (tok * p.heads_q + tile_head) * kHeadDim;
            float* lse_ptr = p.lse + wk.lse_base + static_cast<long long>(tile_head - wk.head) * p.lse_head_stride + row;

            // Key columns [0, col_limit) are visible to this row.
            int col_limit = wk.k_len;
            if (p.causal) {
                col_limit = min(col_limit, row + 1 + wk.k_len - wk.q_len);
            }
            // Smallest limit in the tile (its first row) decides whether a block needs masking.
            int tile_min_limit = wk.k_len;
            if (p.causal) {
                tile_min_limit = min(tile_min_limit, tile_row0 + 1 + wk.k_len - wk.q_len);
            }

            float m_used = -INFINITY;   // running reference max (raw score units)
            float l = 0.f;              // running row sum relative to m_used

            for (int j = nblk - 1; j >= 0; --j) {
                PH_MARK(0);
                ok = mbar_wait(wctx, smem_u32(&sh.s_full[x]), s_cnt & 1u, 11);
                if (!ok) break;
                ++s_cnt;
                tc_fence_after_sync();
                PH_MARK(1);

                float s[kTileN];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t t[32];
                    tmem_ld_x32(s_tmem + c * 32, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(t[i]);
                }
                tmem_wait_ld();
                PH_MARK(2);

                const int n0 = (j - wk.n_full) * kTileN;   // own-chunk column of the block
                if (j >= wk.n_full && n0 + kTileN > tile_min_limit) {
                    const int lim = col_limit - n0;
#pragma unroll
                    for (int i = 0; i < kTileN; ++i) {
                        if (i >= lim) s[i] = -INFINITY;
                    }
                }

                // Row maximum with four independent chains of 3-input maxima (a single chain of
                // 127 dependent operations would be pure latency for the one warp per scheduler).
                float bm;
                {
                    float m0 = s[0], m1 = s[1], m2 = s[2], m3 = s[3];
#pragma unroll
                    for (int i = 4; i + 7 < kTileN; i += 8) {
                        m0 = max3(m0, s[i], s[i + 1]);
                        m1 = max3(m1, s[i + 2], s[i + 3]);
                        m2 = max3(m2, s[i + 4], s[i + 5]);
                        m3 = max3(m3, s[i + 6], s[i + 7]);
                    }
                    // 4 + 15 * 8 = 124 consumed; four left
                    m0 = max3(m0, s[124], s[125]);
                    m1 = max3(m1, s[126], s[127]);
                    bm = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                }

                const bool first = (j == nblk - 1);
                const float m_new = fmaxf(m_used, bm);
                if (first) {
                    m_used = m_new;
                } else {
                    const bool want = (m_new - m_used) * sl2 > kRescaleThreshold;
                    if (__any_sync(0xFFFFFFFFu, want)) {
                        const float factor =
                            (m_new == -INFINITY) ? 1.f : fast_exp2((m_used - m_new) * sl2);
                        l *= factor;
                        m_used = m_new;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t t[32];
                            tmem_ld_x32(o_tmem + c * 32, t);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                t[i] = __float_as_uint(__uint_as_float(t[i]) * factor);
                            }
                            tmem_st_x32(o_tmem + c * 32, t);
                        }
                    }
                }

                PH_MARK(3);
                const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used * sl2;
                const float2 sl2v = make_float2(sl2, sl2);
                const float2 negv = make_float2(neg_m, neg_m);
                float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t t[32];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 x0 = fma2(make_float2(s[c * 64 + 2 * i], s[c * 64 + 2 * i + 1]), sl2v, negv);
                        const float2 x1 = fma2(make_float2(s[c * 64 + 2 * i + 2], s[c * 64 + 2 * i + 3]), sl2v, negv);
                        // Half of the exponentials run on the special-function unit, half as a
                        // polynomial on the FMA pipe, so the two units work side by side.
                        const float2 p0 = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
                        const float2 p1 = ((kFwdExpPolyMask >> (i / 2)) & 1u)
                                              ? exp2_poly2(x1)
                                              : make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
                        acc0 = add2(acc0, p0);
                        acc1 = add2(acc1, p1);
                        t[i] = pack_bf16x2(p0.x, p0.y);
                        t[i + 1] = pack_bf16x2(p1.x, p1.y);
                    }
                    tmem_st_x32(s_tmem + c * 32, t);
                }
                l += (acc0.x + acc0.y) + (acc1.x + acc1.y);
                PH_MARK(4);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&sh.p_full[x]));
                PH_MARK(5);
            }
            if (!ok) break;

            float inv = 0.f;
            float lse_val = -INFINITY;
            if (nblk > 0) {
                ok = mbar_wait(wctx, smem_u32(&sh.o_full[x]), o_cnt & 1u, 12);
                if (!ok) break;
                ++o_cnt;
                tc_fence_after_sync();
                // A row that never saw a key keeps m_used = -inf (its polynomial exponentials are
                // 2^-126 rather than exactly 0, so the row sum alone does not tell).
                if (l > 0.f && m_used != -INFINITY) {
                    inv = 1.f / l;
                    lse_val = (m_used * sl2 + fast_log2(l)) * kLn2;
                }
            }

            if constexpr (kMerge) {
                // Merge this call's (O_b, L_b) into the running (O_p, L_p):
                //   L = logaddexp(L_p, L_b);  O = O_p * e^(L_p - L) + O_b * e^(L_b - L)
                float lse_prev = row_valid ? *lse_ptr : -INFINITY;
                float lse_new = lse_prev;
                float w_prev = 1.f;
                float w_blk = 0.f;
                if (lse_val != -INFINITY) {
                    const float mx = fmaxf(lse_prev, lse_val);
                    const float e_prev = (lse_prev == -INFINITY) ? 0.f : __expf(lse_prev - mx);
                    const float e_blk = __expf(lse_val - mx);
                    const float den = e_prev + e_blk;
                    lse_new = mx + __logf(den);
                    w_prev = e_prev / den;
                    w_blk = e_blk / den;
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t t[32];
                    if (nblk > 0) {
                        tmem_ld_x32(o_tmem + c * 32, t);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) t[i] = 0u;
                    }
                    if (row_valid) {
                        uint4* dst = reinterpret_cast<uint4*>(o_row + c * 32);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint4 prev = dst[v];
                            uint32_t pw[4] = {prev.x, prev.y, prev.z, prev.w};
                            uint32_t out[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float a0 = __uint_as_float(pw[e] << 16);
                                const float a1 = __uint_as_float(pw[e] & 0xFFFF0000u);
                                const float b0 = __uint_as_float(t[v * 8 + 2 * e]) * inv;
                                const float b1 = __uint_as_float(t[v * 8 + 2 * e + 1]) * inv;
                                out[e] = pack_bf16x2(a0 * w_prev + b0 * w_blk,
                                                     a1 * w_prev + b1 * w_blk);
                            }
                            dst[v] = make_uint4(out[0], out[1], out[2], out[3]);
                        }
                    }
                }
                if (row_valid) *lse_ptr = lse_new;
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t t[32];
                    if (nblk > 0) {
                        tmem_ld_x32(o_tmem + c * 32, t);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) t[i] = 0u;
                    }
                    if (row_valid) {
                        uint4* dst = reinterpret_cast<uint4*>(o_row + c * 32);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint32_t out[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                out[e] = pack_bf16x2(__uint_as_float(t[v * 8 + 2 * e]) * inv,
                                                     __uint_as_float(t[v * 8 + 2 * e + 1]) * inv);
                            }
                            dst[v] = make_uint4(out[0], out[1], out[2], out[3]);
                        }
                    }
                }
                if (row_valid) *lse_ptr = lse_val;
            }
            tc_fence_before_sync();
        }
        PH_PRINT("fwd softmax", 6);
    }

    // Common exit: every role arrives here (normally or after an abort).
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace b2a
