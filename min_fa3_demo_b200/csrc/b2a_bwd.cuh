// Backward attention for sm_100a.
//
// Three kernels on one stream:
//   bwd_preprocess_kernel  D = rowsum(dO * O), LSE2 = LSE * log2(e) (padded per document)
//   bwd_kernel             dK, dV (bf16, written directly) and fp32 dQ partial sums
//   bwd_postprocess_kernel dQ = bf16(scale * dq_accum)
//
// bwd_kernel keeps one 128-row K/V block of one KV head stationary per work item and
// loops over every (query head of the group, 128-row query tile) that sees it, so dK and
// dV accumulate in tensor memory across the whole loop (GQA included) and need no fp32
// global accumulators.  Everything is computed transposed (FA-style "S^T = K Q^T"): a
// compute thread owns one key row, P^T goes back to tensor memory as the A operand of
// dV += P^T dO, and dS^T is written once to shared memory where it is both the K-major A
// operand of dK += dS^T Q and the MN-major A operand of dQ = dS K.
//
//   warp  0-3   compute warpgroup 0: query columns 0-63 of the S^T / dP^T tiles
//   warp  4-7   compute warpgroup 1: query columns 64-127
//   warp  8-11  dQ warpgroup: drains dQ tiles from tensor memory, red.add into dq_accum
//   warp 12     tcgen05.mma issue
//   warp 13     TMA loads and work fetch
//   warp 14     deterministic mode only: "scout" that watches the per-tile order counters ahead of
//               the dQ warpgroup (otherwise idle)
//   warp 15     idle
//
// Tensor memory (512 columns): S^T/P^T [0,128)  dP^T/dQ [128,256)  dV [256,384)  dK [384,512).
#pragma once

#include "b2a_fwd.cuh"

namespace b2a {

constexpr int kBwdThreads = 512;
// Which of the 16 four-element groups of a thread's 64 probabilities take two of their
// exponentials from the FMA-pipe polynomial instead of the special-function unit.  Off by
// default: measured in SM clocks per step, 0 / 25 % / 50 % polynomial gave 3990 / 4090 / 4280
// (the compute warps of this kernel are short of issue slots, not of special-function rate).
#ifndef B2A_BWD_EXP_POLY_MASK
#define B2A_BWD_EXP_POLY_MASK 0x0000u
#endif
constexpr uint32_t kBwdExpPolyMask = B2A_BWD_EXP_POLY_MASK;
constexpr int kBwdStages = 2;          // Q ring stages (with their LSE2 / D vectors)
constexpr int kDoStages = 1;           // dO is single-buffered: it lives only from dP(t) to dV(t)
constexpr uint32_t kDqBarrier = 1;          // named barrier of the dQ warpgroup
constexpr uint32_t kDqChunkBytes = 16384;   // 32 dQ columns x 128 rows fp32: one bulk reduction
constexpr uint32_t kRowVecBytes = kTileM * 4;   // 128 fp32 (LSE2 or D of one query tile)

// dq_accum layout: [head][padded 128-row tile][32 column chunks][128 rows][4 floats], so a
// warp-wide 16-byte red.add touches 512 contiguous bytes.
constexpr int kDqTileFloats = kTileM * kHeadDim;

struct BwdParams {
    __nv_bfloat16* dk;             // [tokens_k, heads_k, 128]
    __nv_bfloat16* dv;
    float* dq_accum;               // see layout above
    int* dq_sem;                   // deterministic mode: per (query head, query tile) count of key blocks
                                   // already added, zeroed before launch; null otherwise
    const float* lse2;             // [heads_q, padded_q]  -(LSE * log2 e); -inf = row contributes nothing
    const float* dpsum;            // [heads_q, padded_q]  -rowsum(dO * O)
                                   // (both negated by the preprocess so that the main loop adds them)
    const int* cu_seqlens_q;
    const int* cu_seqlens_k;
    const int2* work_list;         // varlen: (doc, n_block) in LPT order
    const int* num_entries_dev;
    int* sched_counter;
    unsigned int* status;
    int batch;
    int seqlen_q;
    int seqlen_k;
    int heads_q;
    int heads_k;
    int causal;
    int num_entries_host;
    int sg_heads;      // key/value heads per scheduling supergroup (1..heads_k)
    int batch_minor;   // BSHD: hand out work key block major, batch element minor (deterministic mode)
    int padded_q;                  // padded query rows per head (multiple of 128)
    float scale;
    float scale_log2;
    uint32_t timeout_ns;
    // ---- context-parallel mode: null / 0 otherwise ------------------------------------
    const RingDoc* ring_docs;
    const int4* ring_work;             // (doc, source ring member, key half, 128-row block)
    const int2* comm_tasks;            // (source rank, arena block) for the copy CTAs
    int comm_task_count;
    int num_comp;
    int my_rank;
    int ring_start_unused;
    int kv_row_bytes;
    int cap;                           // arena rows per rank
    const uint8_t* peer_k[8];
    const uint8_t* peer_v[8];
    uint8_t* arena_k;
    uint8_t* arena_v;
    int* kv_flags;
    float* dk_accum_peer[8];           // fp32 dK / dV accumulators of every rank (owner-directed adds)
    float* dv_accum_peer[8];
    int* completion_peer[8];           // completion counter of every rank
    int* done_ctas;                    // local counter of finished CTAs
    int world;
};

struct BwdWork {
    int q_begin;
    int q_len;
    int k_begin;
    int k_len;
    int q_pad_begin;   // first padded row of the document (multiple of 128)
    int n0;            // first key row (document-local) of the block
    int head_k;
    // Query tiles that see the block: count0 tiles starting at first0 in the first segment
    // (the whole document, or the front half of a zigzag shard) followed by count1 tiles
    // starting at first1 in the second segment (the back half).
    int first0;
    int count0;
    int first1;
    int count1;
    int seg_len;       // rows between the two segments (half length); 0 outside ring mode
    int k_row;         // first row of the K/V block in the tensor the K/V maps cover
    int diag_seg;      // ring mode: segment whose tile `diag_tile` is the masked diagonal (-1: none)
    int diag_tile;
    int owner;         // ring mode: rank that owns the K/V block
    int owner_block;   // ring mode: 128-row block index inside the owner's slice
};

// Query tile of step t (within one head): document-local first row and whether it is the
// masked diagonal of a ring work item.
__device__ __forceinline__ int bwd_step_row(const BwdWork& wk, int t, bool* diag) {
    int seg = 0, tile = wk.first0 + t;
    if (t >= wk.count0) {
        seg = 1;
        tile = wk.first1 + (t - wk.count0);
    }
    *diag = (seg == wk.diag_seg && tile == wk.diag_tile);
    return seg * wk.seg_len + tile * kTileM;
}

// Padded row offset of a document: every document starts on a 128-row boundary and owns
// at least round_up(len, 128) rows.
__host__ __device__ __forceinline__ int bwd_padded_begin(int cu_begin, int doc) {
    return ((cu_begin + 127) / 128) * 128 + 256 * doc;
}

__device__ __forceinline__ BwdWork bwd_decode_work(const BwdParams& p, int w) {
    BwdWork wk;
    // Work order: key/value heads are taken `sg_heads` at a time ("supergroup", sized by the host
    // so that the dQ accumulator rows being added to stay within L2); inside a supergroup the
    // entries run in list order (most expensive first) with the head minor.  BSHD applies this
    // per batch element.
    const int entries = p.cu_seqlens_q == nullptr ? p.num_entries_host : *p.num_entries_dev;
    int per_batch = entries, b_idx = 0;
    const bool bshd = p.cu_seqlens_q == nullptr && p.ring_docs == nullptr;
    if (bshd && p.batch_minor != 0) {
        // Deterministic mode: key block major, then batch element, then head.  A block waits for
        // the previous block of the same (batch element, head); spreading the running CTAs over
        // the batch keeps those chains short.
        const int nnb = (p.seqlen_k + kTileN - 1) / kTileN;
        const int per_n = p.batch * p.heads_k;
        const int ni = w / per_n;
        const int r = w - ni * per_n;
        const int b = r / p.heads_k;
        w = (b * nnb + ni) * p.heads_k + (r - b * p.heads_k);   // index in the default order
    }
    if (bshd) {
        per_batch = (p.seqlen_k + kTileN - 1) / kTileN;
        b_idx = w / (per_batch * p.heads_k);
        w -= b_idx * per_batch * p.heads_k;
    }
    // The last batch element is scheduled as one group over all heads: its most expensive items
    // then start while plenty of work is left, which keeps the tail of the launch short.
    const int sg_heads = (bshd && b_idx == p.batch - 1) ? p.heads_k : p.sg_heads;
    const int per_sg = per_batch * sg_heads;
    const int sg = w / per_sg;
    const int sg_base = sg * sg_heads;
    const int sg_cnt = min(sg_heads, p.heads_k - sg_base);
    const int sg_r = w - sg * per_sg;
    int entry = sg_r / sg_cnt;
    wk.head_k = sg_base + (sg_r - entry * sg_cnt);
    entry += b_idx * per_batch;
    wk.first1 = 0;
    wk.count1 = 0;
    wk.seg_len = 0;
    wk.diag_seg = -1;
    wk.diag_tile = 0;
    wk.owner = 0;
    wk.owner_block = 0;
    if (p.ring_docs != nullptr) {
        const int4 e = p.ring_work[entry];
        const RingDoc& d = p.ring_docs[e.x];
        const int g = d.ring_size, r = d.ring_rank, s = e.y, hf = e.z, blk = e.w;
        const int hb = d.half_len / kTileM;
        wk.q_begin = d.q_begin;
        wk.q_len = d.half_len;
        wk.k_begin = 0;
        wk.k_len = d.half_len;
        wk.q_pad_begin = d.q_begin;
        wk.n0 = blk * kTileN;                       // chunk-local key row
        wk.seg_len = d.half_len;
        wk.k_row = d.member_row[s] + hf * d.half_len + blk * kTileN;
        wk.owner = wk.k_row / p.cap;
        wk.owner_block = (wk.k_row - wk.owner * p.cap) / kTileN;
        // Global chunk indices: key chunk ck, query chunks cq of the two local halves.
        const int ck = g == 1 ? 0 : (hf == 0 ? s : 2 * g - 1 - s);
        int first[2] = {0, 0}, count[2] = {0, 0};
        const int halves = ring_halves(p.causal, g);
        for (int h = 0; h < halves; ++h) {
            if (!p.causal) {
                count[h] = hb;
            } else {
                const int cq = g == 1 ? 0 : (h == 0 ? r : 2 * g - 1 - r);
                if (ck < cq) {
                    count[h] = hb;
                } else if (ck == cq) {
                    first[h] = blk;
                    count[h] = hb - blk;
                    wk.diag_seg = h;
                    wk.diag_tile = blk;
                }
            }
        }
        wk.first0 = first[0];
        wk.count0 = count[0];
        wk.first1 = first[1];
        wk.count1 = count[1];
        return wk;
    }
    int nblk;
    if (p.cu_seqlens_q == nullptr) {
        int nnb = (p.seqlen_k + kTileN - 1) / kTileN;
        int b = entry / nnb;
        int ni = entry - b * nnb;
        // Causal: early key blocks are seen by the most query tiles -> run them first.
        nblk = ni;
        wk.q_begin = b * p.seqlen_q;
        wk.q_len = p.seqlen_q;
        wk.k_begin = b * p.seqlen_k;
        wk.k_len = p.seqlen_k;
        wk.q_pad_begin = b * (((p.seqlen_q + 127) / 128) * 128);
    } else {
        int2 e = p.work_list[entry];
        int doc = e.x;
        nblk = e.y;
        wk.q_begin = p.cu_seqlens_q[doc];
        wk.q_len = p.cu_seqlens_q[doc + 1] - wk.q_begin;
        wk.k_begin = p.cu_seqlens_k[doc];
        wk.k_len = p.cu_seqlens_k[doc + 1] - wk.k_begin;
        wk.q_pad_begin = bwd_padded_begin(wk.q_begin, doc);
    }
    wk.n0 = nblk * kTileN;
    int m_tiles = (wk.q_len + kTileM - 1) / kTileM;
    int first = 0;
    if (p.causal) {
        int first_row = max(0, wk.n0 + wk.q_len - wk.k_len);
        first = min(m_tiles, first_row / kTileM);
    }
    wk.first0 = first;
    wk.count0 = m_tiles - first;
    wk.k_row = wk.k_begin + wk.n0;
    return wk;
}

struct __align__(1024) BwdShared {
    uint8_t k[kTileBytes];
    uint8_t v[kTileBytes];
    uint8_t q[kBwdStages][kTileBytes];
    uint8_t dout[kDoStages][kTileBytes];
    uint8_t dq_stage[2][kDqChunkBytes];   // dQ chunks on their way to the bulk reduce-add
    uint8_t ds[kTileBytes];
    float lse2[kBwdStages][kTileM];
    float dpsum[kBwdStages][kTileM];
    uint64_t kv_full;
    uint64_t kv_empty;
    uint64_t q_full[kBwdStages];
    uint64_t q_empty[kBwdStages];
    uint64_t do_full[kDoStages];
    uint64_t do_empty[kDoStages];
    uint64_t s_full;
    uint64_t dp_full;
    uint64_t p_ready;
    uint64_t ds_ready;
    uint64_t ds_empty;
    uint64_t dq_full;
    uint64_t dq_drained;
    uint64_t dkv_full;
    uint64_t dkv_empty;
    uint64_t sched_full[2];
    uint64_t sched_empty[2];
    uint64_t comm_full[6];
    uint64_t comm_empty[6];
    int sched_w[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t order_step;     // deterministic mode: dQ tiles (CTA-wide running count) cleared for adding
};
static_assert(sizeof(BwdShared) <= 232448, "backward shared storage exceeds the 227 KiB opt-in limit");

// Bounded wait until a global counter reaches `value` (acquire at GPU scope).
__device__ __forceinline__ bool value_wait(const WaitCtx& ctx, const int* counter, int value, uint32_t tag) {
    const uint32_t start = global_timer_lo();
    uint32_t polls = 0;
    while (true) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= value) return true;
        if ((++polls & 0xFu) == 0u) {
            if (ld_shared_volatile_u32(ctx.abort_smem) != 0u) return false;
            if (global_timer_lo() - start > ctx.timeout_ns) {
                st_shared_volatile_u32(ctx.abort_smem, 1u);
                set_status(ctx.status, kStatusTimeout, (tag << 12) | (blockIdx.x & 0xFFFu));
                return false;
            }
        }
        __nanosleep(64);
    }
}

// Copy role of a ring-mode backward CTA (same protocol as the forward's): six 32 KiB slots laid
// over the K ... dO tile buffers and the dQ staging area, one loading thread, one storing thread, per-block ready flags.
__device__ __forceinline__ void bwd_ring_copy_role(const BwdParams& p, BwdShared& sh, const WaitCtx& wctx,
                                                   int warp, int lane) {
    constexpr uint32_t kSlotBytes = kTileBytes;
    const uint32_t block_bytes = static_cast<uint32_t>(kTileN) * p.kv_row_bytes;
    const uint32_t chunks = block_bytes / kSlotBytes;
    const uint32_t slot_base = smem_u32(&sh.k[0]);
    const int first = static_cast<int>(blockIdx.x) - p.num_comp;
    const int stride = static_cast<int>(gridDim.x) - p.num_comp;
    if (warp == 13 && lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int t = first; t < p.comm_task_count && ok; t += stride) {
            const int2 task = p.comm_tasks[t];
            const size_t off = static_cast<size_t>(task.y) * block_bytes;
            for (int kv = 0; kv < 2 && ok; ++kv) {
                const uint8_t* src = (kv == 0 ? p.peer_k[task.x] : p.peer_v[task.x]) + off;
                for (uint32_t c = 0; c < chunks; ++c, ++it) {
                    const uint32_t slot = it % 6u;
                    ok = mbar_wait(wctx, smem_u32(&sh.comm_empty[slot]), ((it / 6u) & 1u) ^ 1u, 24);
                    if (!ok) break;
                    mbar_arrive_expect_tx(smem_u32(&sh.comm_full[slot]), kSlotBytes);
                    bulk_load_1d(slot_base + slot * kSlotBytes, src + static_cast<size_t>(c) * kSlotBytes,
                                 kSlotBytes, smem_u32(&sh.comm_full[slot]));
                }
            }
        }
    } else if (warp == 14 && lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int t = first; t < p.comm_task_count && ok; t += stride) {
            const int2 task = p.comm_tasks[t];
            const size_t off = static_cast<size_t>(task.y) * block_bytes;
            for (int kv = 0; kv < 2 && ok; ++kv) {
                uint8_t* dst = (kv == 0 ? p.arena_k : p.arena_v) + off;
                for (uint32_t c = 0; c < chunks; ++c, ++it) {
                    const uint32_t slot = it % 6u;
                    ok = mbar_wait(wctx, smem_u32(&sh.comm_full[slot]), (it / 6u) & 1u, 25);
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
                bulk_wait_group<0>();
                fence_proxy_async_all();
                asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.kv_flags + task.y), "r"(1)
                             : "memory");
            }
        }
        bulk_wait_group<0>();
    }
}

__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
           const BwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    BwdShared& sh = *reinterpret_cast<BwdShared*>(smem_raw);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if ((smem_u32(smem_raw) & 1023u) != 0u) {
        // The swizzled tiles need a 1 KiB aligned base; report instead of computing garbage.
        if (threadIdx.x == 0) set_status(p.status, kStatusBadArg, 1);
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&sh.kv_full), 1);
        mbar_init(smem_u32(&sh.kv_empty), 1);
        for (int i = 0; i < kBwdStages; ++i) {
            mbar_init(smem_u32(&sh.q_full[i]), 1);
            mbar_init(smem_u32(&sh.q_empty[i]), 1);
        }
        for (int i = 0; i < kDoStages; ++i) {
            mbar_init(smem_u32(&sh.do_full[i]), 1);
            mbar_init(smem_u32(&sh.do_empty[i]), 1);
        }
        mbar_init(smem_u32(&sh.s_full), 1);
        mbar_init(smem_u32(&sh.dp_full), 1);
        mbar_init(smem_u32(&sh.p_ready), 256);
        mbar_init(smem_u32(&sh.ds_ready), 256);
        mbar_init(smem_u32(&sh.ds_empty), 1);
        mbar_init(smem_u32(&sh.dq_full), 1);
        mbar_init(smem_u32(&sh.dq_drained), 128);
        mbar_init(smem_u32(&sh.dkv_full), 1);
        mbar_init(smem_u32(&sh.dkv_empty), 256);
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sh.sched_full[i]), 1);
            mbar_init(smem_u32(&sh.sched_empty[i]), 2 + 12);   // MMA warp, scout warp + 12 consumer warps
        }
        for (int i = 0; i < 6; ++i) {
            mbar_init(smem_u32(&sh.comm_full[i]), 1);
            mbar_init(smem_u32(&sh.comm_empty[i]), 1);
        }
        sh.abort_flag = 0;
        sh.order_step = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 12) {
        tmem_alloc(smem_u32(&sh.tmem_base), 512);
        tmem_relinquish();
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&sh.tmem_base);
    constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;

    WaitCtx wctx{smem_u32(&sh.abort_flag), p.status, p.timeout_ns};
    const int total_work =
        (p.cu_seqlens_q == nullptr ? p.num_entries_host : *p.num_entries_dev) * p.heads_k;
    const int group = p.heads_q / p.heads_k;

    // Copy CTAs (ring mode) first pull the other ranks' K/V blocks into the local arena.
    if (p.ring_docs != nullptr && static_cast<int>(blockIdx.x) >= p.num_comp && p.comm_task_count > 0) {
        bwd_ring_copy_role(p, sh, wctx, warp, lane);
        __syncthreads();
    }

    if (warp >= 12) {
        reg_dealloc<80>();
        if (warp == 13) {
            // ------------------------------------------------------------ load warp
            if (lane == 0) {
                tma_prefetch_desc(&map_q);
                tma_prefetch_desc(&map_k);
                tma_prefetch_desc(&map_v);
                tma_prefetch_desc(&map_do);
            }
            uint32_t item_cnt = 0;   // work items that loaded K/V
            uint32_t step_it = 0;    // global (h, m) step counter -> Q/dO ring position
            bool ok = true;
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
                if (lane == 0) mbar_arrive(smem_u32(&sh.sched_full[slot]));
                if (w < 0) break;
                const BwdWork wk = bwd_decode_work(p, w);
                const int per_head = wk.count0 + wk.count1;
                const int steps = per_head * group;
                if (steps == 0) continue;
                ok = mbar_wait(wctx, smem_u32(&sh.kv_empty), (item_cnt & 1u) ^ 1u, 2);
                if (!ok) break;
                ++item_cnt;
                if (p.ring_docs != nullptr && wk.owner != p.my_rank && p.comm_task_count > 0) {
                    ok = flag_wait(wctx, p.kv_flags + wk.k_row / kTileN, 23);
                    if (!ok) break;
                    fence_proxy_async_all();
                }
                if (lane == 0) {
                    const uint32_t bar = smem_u32(&sh.kv_full);
                    const int row = wk.k_row;
                    mbar_arrive_expect_tx(bar, 2 * kTileBytes);
                    tma_load_3d(smem_u32(&sh.k[0]), &map_k, bar, 0, wk.head_k, row);
                    tma_load_3d(smem_u32(&sh.k[0]) + kHalfTileBytes, &map_k, bar, 64, wk.head_k, row);
                    tma_load_3d(smem_u32(&sh.v[0]), &map_v, bar, 0, wk.head_k, row);
                    tma_load_3d(smem_u32(&sh.v[0]) + kHalfTileBytes, &map_v, bar, 64, wk.head_k, row);
                }
                for (int t = 0; t < steps && ok; ++t) {
                    const int hq = wk.head_k * group + t / per_head;
                    bool diag;
                    const int q_local = bwd_step_row(wk, t % per_head, &diag);
                    const uint32_t stage = step_it % kBwdStages;
                    const uint32_t par = ((step_it / kBwdStages) & 1u) ^ 1u;
                    const uint32_t do_stage = step_it % kDoStages;
                    const uint32_t do_par = ((step_it / kDoStages) & 1u) ^ 1u;
                    ++step_it;
                    ok = mbar_wait(wctx, smem_u32(&sh.q_empty[stage]), par, 3);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&sh.q_full[stage]);
                        const uint32_t dst = smem_u32(&sh.q[stage][0]);
                        const int row = wk.q_begin + q_local;
                        const long long vec =
                            static_cast<long long>(hq) * p.padded_q + wk.q_pad_begin + q_local;
                        mbar_arrive_expect_tx(bar, kTileBytes + 2 * kRowVecBytes);
                        tma_load_3d(dst, &map_q, bar, 0, hq, row);
                        tma_load_3d(dst + kHalfTileBytes, &map_q, bar, 64, hq, row);
                        bulk_load_1d(smem_u32(&sh.lse2[stage][0]), p.lse2 + vec, kRowVecBytes, bar);
                        bulk_load_1d(smem_u32(&sh.dpsum[stage][0]), p.dpsum + vec, kRowVecBytes, bar);
                    }
                    ok = mbar_wait(wctx, smem_u32(&sh.do_empty[do_stage]), do_par, 4);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&sh.do_full[do_stage]);
                        const uint32_t dst = smem_u32(&sh.dout[do_stage][0]);
                        const int row = wk.q_begin + q_local;
                        mbar_arrive_expect_tx(bar, kTileBytes);
                        tma_load_3d(dst, &map_do, bar, 0, hq, row);
                        tma_load_3d(dst + kHalfTileBytes, &map_do, bar, 64, hq, row);
                    }
                }
            }
        } else if (warp == 12) {
            // ------------------------------------------------------------ MMA warp
            constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);   // K-major A, K-major B
            constexpr uint32_t idesc_kn = make_idesc_bf16(128, 128, 0, 1);   // K-major A, MN-major B
            constexpr uint32_t idesc_nn = make_idesc_bf16(128, 128, 1, 1);   // MN-major A, MN-major B
            // Descriptor low words (see desc_lo_kmajor): K, V, dS^T tiles and stage 0 of Q / dO.
            const uint32_t k_lo_k = desc_lo_kmajor(smem_u32(&sh.k[0]));
            const uint32_t k_lo_n = desc_lo_mnmajor(smem_u32(&sh.k[0]));
            const uint32_t v_lo_k = desc_lo_kmajor(smem_u32(&sh.v[0]));
            const uint32_t ds_lo_k = desc_lo_kmajor(smem_u32(&sh.ds[0]));
            const uint32_t ds_lo_n = desc_lo_mnmajor(smem_u32(&sh.ds[0]));
            const uint32_t q_lo_k0 = desc_lo_kmajor(smem_u32(&sh.q[0][0]));
            const uint32_t q_lo_n0 = desc_lo_mnmajor(smem_u32(&sh.q[0][0]));
            const uint32_t do_lo_k0 = desc_lo_kmajor(smem_u32(&sh.dout[0][0]));
            const uint32_t do_lo_n0 = desc_lo_mnmajor(smem_u32(&sh.dout[0][0]));
            constexpr uint32_t kStageStep = kTileBytes >> 4;

            // D[128 x 128] = A * B^T with both operands K-major [rows][128] tiles.
            auto issue_kmajor = [&](uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
                umma_ss_kk_x8_w(d_tmem, a_lo, b_lo, idesc_kk, 0u);
            };

            uint32_t item_cnt = 0;
            uint32_t step_it = 0;
            uint32_t p_cnt = 0, ds_cnt = 0, drain_cnt = 0;
            bool ok = true;
            PH_DECL(8)   // 0 other, 1 wait p_ready, 2 issue dV/S, 3 wait ds_ready, 4 issue dQ/dK, 5 wait drained, 6 wait dO + issue dP
            for (uint32_t it = 0; ok; ++it) {
                const uint32_t slot = it & 1u;
                ok = mbar_wait(wctx, smem_u32(&sh.sched_full[slot]), (it >> 1) & 1u, 5);
                if (!ok) break;
                const int w = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<volatile int*>(&sh.sched_w[slot]), 0);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh.sched_empty[slot]));
                if (w < 0) break;
                const BwdWork wk = bwd_decode_work(p, w);
                const int steps = (wk.count0 + wk.count1) * group;
                if (steps == 0) continue;
                ok = mbar_wait(wctx, smem_u32(&sh.kv_full), item_cnt & 1u, 6);
                if (!ok) break;
                const uint32_t dkv_parity = (item_cnt & 1u) ^ 1u;
                ++item_cnt;

                // Prologue: S^T(0) and dP^T(0).
                {
                    const uint32_t stage = step_it % kBwdStages;
                    const uint32_t par = (step_it / kBwdStages) & 1u;
                    ok = mbar_wait(wctx, smem_u32(&sh.q_full[stage]), par, 8);
                    if (!ok) break;
                    tc_fence_after_sync();
                    {
                        issue_kmajor(tmem_base + kColS, k_lo_k, q_lo_k0 + stage * kStageStep);
                        tc_commit_w(smem_u32(&sh.s_full));
                    }
                    __syncwarp();
                    const uint32_t do_stage = step_it % kDoStages;
                    ok = mbar_wait(wctx, smem_u32(&sh.do_full[do_stage]), (step_it / kDoStages) & 1u, 9);
                    if (!ok) break;
                    tc_fence_after_sync();
                    {
                        issue_kmajor(tmem_base + kColDP, v_lo_k, do_lo_k0 + do_stage * kStageStep);
                        tc_commit_w(smem_u32(&sh.dp_full));
                    }
                    __syncwarp();
                }
                for (int t = 0; t < steps && ok; ++t) {
                    const uint32_t stage = step_it % kBwdStages;
                    const uint32_t nstage = (step_it + 1) % kBwdStages;
                    const uint32_t npar = ((step_it + 1) / kBwdStages) & 1u;
                    const uint32_t do_stage = step_it % kDoStages;
                    const uint32_t do_nstage = (step_it + 1) % kDoStages;
                    const uint32_t do_npar = ((step_it + 1) / kDoStages) & 1u;
                    ++step_it;
                    const uint32_t q_lo_n = q_lo_n0 + stage * kStageStep;
                    const uint32_t do_lo_n = do_lo_n0 + do_stage * kStageStep;
                    const bool has_next = t + 1 < steps;

                    // dV += P^T dO   (A = P^T from tensor memory, B = dO as MN-major)
                    PH_MARK(0);
                    ok = mbar_wait(wctx, smem_u32(&sh.p_ready), p_cnt & 1u, 10);
                    if (!ok) break;
                    ++p_cnt;
                    PH_MARK(1);
                    if (t == 0) {
                        // dK/dV accumulators must have been read out by the previous item's
                        // epilogue before they are overwritten.
                        ok = mbar_wait(wctx, smem_u32(&sh.dkv_empty), dkv_parity, 7);
                        if (!ok) break;
                    }
                    tc_fence_after_sync();
                    {
                        // P^T sits in two runs of 32 packed columns (one per compute warpgroup).
                        umma_ts_x4_w(tmem_base + kColDV, tmem_base + kColS, do_lo_n, idesc_kn, t > 0 ? 1u : 0u);
                        umma_ts_x4_w(tmem_base + kColDV, tmem_base + kColS + 64, do_lo_n + kstep_mnmajor(4), idesc_kn, 1u);
                        tc_commit_w(smem_u32(&sh.do_empty[do_stage]));
                    }
                    __syncwarp();
                    PH_MARK(7);
#ifdef B2A_PHASES
                    ph_[9] += 1;
#endif
                    // S^T(t+1) = K Q(t+1)^T
                    if (has_next) {
                        ok = mbar_wait(wctx, smem_u32(&sh.q_full[nstage]), npar, 11);
                        if (!ok) break;
                        PH_MARK(8);
                        tc_fence_after_sync();
                        {
                            issue_kmajor(tmem_base + kColS, k_lo_k, q_lo_k0 + nstage * kStageStep);
                            tc_commit_w(smem_u32(&sh.s_full));
                        }
                        __syncwarp();
                    }
                    // dQ(t) = dS K  (A = dS^T tile read MN-major, B = K as MN-major), then
                    // dK += dS^T Q  (A = dS^T tile read K-major, B = Q as MN-major)
                    PH_MARK(2);
                    ok = mbar_wait(wctx, smem_u32(&sh.ds_ready), ds_cnt & 1u, 12);
                    if (!ok) break;
                    ++ds_cnt;
                    PH_MARK(3);
                    tc_fence_after_sync();
                    {
                        umma_ss_nn_x8_w(tmem_base + kColDP, ds_lo_n, k_lo_n, idesc_nn, 0u);
                        tc_commit_w(smem_u32(&sh.dq_full));
                        umma_ss_kn_x8_w(tmem_base + kColDK, ds_lo_k, q_lo_n, idesc_kn, t > 0 ? 1u : 0u);
                        tc_commit_w(smem_u32(&sh.q_empty[stage]));
                        tc_commit_w(smem_u32(&sh.ds_empty));
                        if (!has_next) {
                            tc_commit_w(smem_u32(&sh.dkv_full));
                            tc_commit_w(smem_u32(&sh.kv_empty));
                        }
                    }
                    __syncwarp();
                    // dP^T(t+1) = V dO(t+1)^T, once dQ(t) has left tensor memory.
                    PH_MARK(4);
                    ok = mbar_wait(wctx, smem_u32(&sh.dq_drained), drain_cnt & 1u, 13);
                    if (!ok) break;
                    ++drain_cnt;
                    PH_MARK(5);
                    if (has_next) {
                        ok = mbar_wait(wctx, smem_u32(&sh.do_full[do_nstage]), do_npar, 14);
                        if (!ok) break;
                        tc_fence_after_sync();
                        {
                            issue_kmajor(tmem_base + kColDP, v_lo_k, do_lo_k0 + do_nstage * kStageStep);
                            tc_commit_w(smem_u32(&sh.dp_full));
                        }
                        __syncwarp();
                    }
                    PH_MARK(6);
                }
            }
            PH_PRINT("mma", 7);
        } else if (warp == 14) {
            // ------------------------------------------------------------ order scout (deterministic mode)
            // Additions into a dQ tile happen in ascending key-block order.  This warp walks the CTA's
            // tile sequence ahead of the dQ warpgroup, waits (in global memory, with L2 latency) until
            // a tile's counter says that the blocks below this one have been added, and then raises a
            // step count in shared memory, which is all the dQ warpgroup looks at.
            bool ok = true;
            uint32_t cleared = 0;
            const int pad_tiles = p.padded_q / kTileM;
            for (uint32_t it = 0; ok; ++it) {
                const uint32_t slot = it & 1u;
                ok = mbar_wait(wctx, smem_u32(&sh.sched_full[slot]), (it >> 1) & 1u, 32);
                if (!ok) break;
                const int w = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<volatile int*>(&sh.sched_w[slot]), 0);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh.sched_empty[slot]));
                if (w < 0) break;
                if (p.dq_sem == nullptr) continue;
                const BwdWork wk = bwd_decode_work(p, w);
                const int per_head = wk.count0 + wk.count1;
                const int steps = per_head * group;
                const int blk_index = wk.n0 / kTileN;
                if (lane == 0) {
                    for (int t = 0; t < steps && ok; ++t) {
                        const int hq = wk.head_k * group + t / per_head;
                        bool diag;
                        const int q_local = bwd_step_row(wk, t % per_head, &diag);
                        const int* sem = p.dq_sem + static_cast<long long>(hq) * pad_tiles +
                                         (wk.q_pad_begin + q_local) / kTileM;
                        // Work items are handed out in ascending block order per (document, head), so
                        // the blocks waited for are running already; the wait is bounded all the same.
                        ok = value_wait(wctx, sem, blk_index, 26);
                        if (!ok) break;
                        ++cleared;
                        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&sh.order_step)), "r"(cleared)
                                     : "memory");
                    }
                }
                ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            }
        }
    } else if (warp >= 8) {
        // -------------------------------------------------------------------- dQ warpgroup
        reg_alloc<144>();
        const int r = (warp & 3) * 32 + lane;   // query row within the tile
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t dq_tmem = tmem_base + lane_base + kColDP;
        uint32_t dq_cnt = 0;
        // Deterministic mode, thread 256: the two most recent tiles whose counters are still to be
        // published (oldest first).  A tile is published once its four reductions have been performed.
        int* pend_sem[2] = {nullptr, nullptr};
        int pend_val[2] = {0, 0};
        uint32_t tiles_seen = 0;   // dQ tiles of this CTA so far (matches the scout's count)
        bool ok = true;
        PH_DECL(4)   // 0 other, 1 wait dq_full, 2 load + arrive, 3 reductions
        for (uint32_t it = 0; ok; ++it) {
            const uint32_t slot = it & 1u;
            ok = mbar_wait(wctx, smem_u32(&sh.sched_full[slot]), (it >> 1) & 1u, 15);
            if (!ok) break;
            const int w = *reinterpret_cast<volatile int*>(&sh.sched_w[slot]);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.sched_empty[slot]));
            if (w < 0) break;
            const BwdWork wk = bwd_decode_work(p, w);
            const int per_head = wk.count0 + wk.count1;
            const int steps = per_head * group;
            const int pad_tiles = p.padded_q / kTileM;
            for (int t = 0; t < steps && ok; ++t) {
                const int hq = wk.head_k * group + t / per_head;
                bool diag;
                const int q_local = bwd_step_row(wk, t % per_head, &diag);
                float* tile = p.dq_accum +
                              (static_cast<long long>(hq) * pad_tiles + (wk.q_pad_begin + q_local) / kTileM) *
                                  kDqTileFloats;
                PH_MARK(0);
                ok = mbar_wait(wctx, smem_u32(&sh.dq_full), dq_cnt & 1u, 16);
                if (!ok) break;
                ++dq_cnt;
                tc_fence_after_sync();
                PH_MARK(1);
                // Pull the whole dQ tile into registers first so that tensor memory is handed back
                // before the reductions are issued.
                uint32_t v[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld_x32(dq_tmem + c * 32, v[c]);
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&sh.dq_drained));
                PH_MARK(2);
                // Deterministic mode: the scout warp has checked that the key blocks below this one have
                // been added to the tile; wait for its step count (shared memory, a few clocks when it
                // is ahead, and bounded).
                int* sem = nullptr;
                const int blk_index = wk.n0 / kTileN;
                if (p.dq_sem != nullptr) {
                    sem = p.dq_sem + static_cast<long long>(hq) * pad_tiles + (wk.q_pad_begin + q_local) / kTileM;
                    ++tiles_seen;
                    if (threadIdx.x == 256) {
                        const uint32_t start = global_timer_lo();
                        uint32_t polls = 0;
                        while (true) {
                            uint32_t cleared;
                            asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(cleared)
                                         : "r"(smem_u32(&sh.order_step)) : "memory");
                            if (cleared >= tiles_seen) break;
                            if ((++polls & 0x3Fu) == 0u) {
                                // A wait that runs out raises the CTA's abort flag and status word; the
                                // warpgroup still goes through this step's barriers together and stops
                                // at its next wait.
                                if (ld_shared_volatile_u32(wctx.abort_smem) != 0u) break;
                                if (global_timer_lo() - start > wctx.timeout_ns) {
                                    st_shared_volatile_u32(wctx.abort_smem, 1u);
                                    set_status(wctx.status, kStatusTimeout, (34u << 12) | (blockIdx.x & 0xFFFu));
                                    break;
                                }
                            }
                        }
                    }
                }
                // Four chunks of 32 columns go through two 16 KiB staging buffers whose layout
                // equals the accumulator's ([8 column quads][128 rows][4 floats]); one thread hands
                // each to the bulk-copy engine as an fp32 reduce-add into global memory, so the
                // additions run asynchronously and do not occupy this SM's load/store path.
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t buf = smem_u32(&sh.dq_stage[c & 1][0]);
                    if (threadIdx.x == 256) bulk_wait_group_read<1>();   // the buffer's previous reduction has read it
                    named_barrier_sync(kDqBarrier, 128);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(buf + static_cast<uint32_t>((i * kTileM + r) * 16)),
                                       "r"(v[c][4 * i]), "r"(v[c][4 * i + 1]), "r"(v[c][4 * i + 2]),
                                       "r"(v[c][4 * i + 3])
                                     : "memory");
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(kDqBarrier, 128);
                    if (threadIdx.x == 256) {
                        bulk_reduce_add_f32(tile + c * (kDqChunkBytes / 4), buf, kDqChunkBytes);
                        bulk_commit_group();
                    }
                }
                if (sem != nullptr && threadIdx.x == 256) {
                    // Publish the tile of two steps ago once its four reductions are performed (the
                    // eight of the last two tiles may still be in flight).  The reductions are complete
                    // -- performed in L2 -- before the counter is stored, so a block that reads the new
                    // value can only add after them; a plain (relaxed) store is enough and, unlike a
                    // release store, does not wait for this thread's other traffic.
                    if (pend_sem[0] != nullptr) {
                        bulk_wait_group<8>();
                        asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(pend_sem[0]), "r"(pend_val[0]) : "memory");
                    }
                    pend_sem[0] = pend_sem[1];
                    pend_val[0] = pend_val[1];
                    pend_sem[1] = sem;
                    pend_val[1] = blk_index + 1;
                }
                PH_MARK(3);
            }
            if (pend_sem[1] != nullptr) {
                // End of the work item: publish its last tiles (only thread 256 holds any).
                bulk_wait_group<0>();
                fence_proxy_async_all();
                if (pend_sem[0] != nullptr) {
                    asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(pend_sem[0]), "r"(pend_val[0]) : "memory");
                }
                asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(pend_sem[1]), "r"(pend_val[1]) : "memory");
                pend_sem[0] = pend_sem[1] = nullptr;
            }
        }
        if (threadIdx.x == 256) bulk_wait_group<0>();   // all reductions performed before the CTA ends
        PH_PRINT("dq", 4);
    } else {
        // -------------------------------------------------------------------- compute warpgroups
        reg_alloc<144>();
        const int wg = warp >> 2;                      // 0: query columns 0-63, 1: 64-127
        const int i_row = (warp & 3) * 32 + lane;      // key row within the block
        const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t s_tmem = tmem_base + lane_base + kColS + wg * 64;
        const uint32_t dp_tmem = tmem_base + lane_base + kColDP + wg * 64;
        const uint32_t pt_tmem = tmem_base + lane_base + kColS + wg * 64;   // P^T: 32 packed columns
        const uint32_t ds_row = smem_u32(&sh.ds[0]) + wg * kHalfTileBytes + i_row * 128;
        const float sl2 = p.scale_log2;
        uint32_t step_it = 0;
        uint32_t s_cnt = 0, dp_cnt = 0, dse_cnt = 0, epi_cnt = 0;
        bool ok = true;
        PH_DECL(8)   // 0 other, 1 wait q_full+s_full, 2 P phase, 3 wait dp_full, 4 dP load, 5 wait ds_empty, 6 dS phase

        for (uint32_t it = 0; ok; ++it) {
            const uint32_t slot = it & 1u;
            ok = mbar_wait(wctx, smem_u32(&sh.sched_full[slot]), (it >> 1) & 1u, 17);
            if (!ok) break;
            const int w = *reinterpret_cast<volatile int*>(&sh.sched_w[slot]);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.sched_empty[slot]));
            if (w < 0) break;
            const BwdWork wk = bwd_decode_work(p, w);
            const int per_head = wk.count0 + wk.count1;
            const int steps = per_head * group;
            const bool ring = p.ring_docs != nullptr;
            const int kv_row = wk.n0 + i_row;
            const bool kv_valid = kv_row < wk.k_len;
            const int shift = wk.k_len - wk.q_len;     // key c visible to query r iff c <= r + shift

            for (int t = 0; t < steps && ok; ++t) {
                bool diag;
                const int q_local = bwd_step_row(wk, t % per_head, &diag);
                const uint32_t stage = step_it % kBwdStages;
                const uint32_t par = (step_it / kBwdStages) & 1u;
                ++step_it;
                // Query row of column 0, in the coordinates of the key rows (document-local, or
                // chunk-local for the diagonal tile of a ring work item).
                const int q0 = (ring ? q_local - (q_local >= wk.seg_len ? wk.seg_len : 0) : q_local) + wg * 64;
                // Columns c < c_min are hidden from this key row by the causal rule.
                const int c_min = (ring ? diag : p.causal != 0) ? (kv_row - shift - q0) : 0;
                const bool need_mask = !kv_valid || c_min > 0;

                // LSE2 / D of this tile arrive with Q.
                PH_MARK(0);
                ok = mbar_wait(wctx, smem_u32(&sh.q_full[stage]), par, 18);
                if (!ok) break;
                ok = mbar_wait(wctx, smem_u32(&sh.s_full), s_cnt & 1u, 19);
                if (!ok) break;
                ++s_cnt;
                tc_fence_after_sync();
                PH_MARK(1);

                float pr[64];
                {
                    uint32_t a[32], b[32];
                    tmem_ld_x32(s_tmem, a);
                    tmem_ld_x32(s_tmem + 32, b);
                    tmem_wait_ld();
                    const float4* l2 = reinterpret_cast<const float4*>(&sh.lse2[stage][wg * 64]);
#pragma unroll
                    for (int g4 = 0; g4 < 16; ++g4) {
                        const float4 l = l2[g4];
                        const uint32_t* src = g4 < 8 ? a : b;
                        const int o = (g4 & 7) * 4;
                        const float2 x0 = fma2(make_float2(__uint_as_float(src[o]), __uint_as_float(src[o + 1])),
                                               make_float2(sl2, sl2), make_float2(l.x, l.y));
                        const float2 x1 = fma2(make_float2(__uint_as_float(src[o + 2]), __uint_as_float(src[o + 3])),
                                               make_float2(sl2, sl2), make_float2(l.z, l.w));
                        // Part of the exponentials runs as a polynomial on the FMA pipe (see exp2_poly2).
                        const float2 p0 = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
                        const float2 p1 = ((kBwdExpPolyMask >> g4) & 1u)
                                              ? exp2_poly2(x1)
                                              : make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
                        pr[4 * g4 + 0] = p0.x;
                        pr[4 * g4 + 1] = p0.y;
                        pr[4 * g4 + 2] = p1.x;
                        pr[4 * g4 + 3] = p1.y;
                    }
                }
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        if (!kv_valid || c < c_min) pr[c] = 0.f;
                    }
                }
                {
                    uint32_t pk[32];
#pragma unroll
                    for (int c = 0; c < 32; ++c) pk[c] = pack_bf16x2(pr[2 * c], pr[2 * c + 1]);
                    tmem_st_x32(pt_tmem, pk);
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(smem_u32(&sh.p_ready));
                }

                // dS^T = P^T * (dP^T - D)
                PH_MARK(2);
                ok = mbar_wait(wctx, smem_u32(&sh.dp_full), dp_cnt & 1u, 20);
                if (!ok) break;
                ++dp_cnt;
                tc_fence_after_sync();
                PH_MARK(3);
                // Two halves of 32 query columns each keep the live register set small.
                uint32_t a[32], b[32];
                tmem_ld_x32(dp_tmem, a);
                tmem_ld_x32(dp_tmem + 32, b);
                const float4* dsum = reinterpret_cast<const float4*>(&sh.dpsum[stage][wg * 64]);
                tmem_wait_ld();
                PH_MARK(4);
                // The previous step's dK / dQ MMAs must be done with the dS^T tile.
                ok = mbar_wait(wctx, smem_u32(&sh.ds_empty), (dse_cnt & 1u) ^ 1u, 21);
                if (!ok) break;
                ++dse_cnt;
                PH_MARK(5);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t dsp[16];
#pragma unroll
                    for (int g4 = 0; g4 < 8; ++g4) {
                        const float4 d = dsum[half * 8 + g4];
                        const uint32_t* src = half == 0 ? a : b;
                        // dS = P * (dP - D) with D stored negated: one packed add and one packed multiply
                        // per two elements.
                        const float2 y0 = mul2(make_float2(pr[half * 32 + 4 * g4 + 0], pr[half * 32 + 4 * g4 + 1]),
                                               add2(make_float2(__uint_as_float(src[4 * g4 + 0]),
                                                                __uint_as_float(src[4 * g4 + 1])),
                                                    make_float2(d.x, d.y)));
                        const float2 y1 = mul2(make_float2(pr[half * 32 + 4 * g4 + 2], pr[half * 32 + 4 * g4 + 3]),
                                               add2(make_float2(__uint_as_float(src[4 * g4 + 2]),
                                                                __uint_as_float(src[4 * g4 + 3])),
                                                    make_float2(d.z, d.w)));
                        dsp[2 * g4] = pack_bf16x2(y0.x, y0.y);
                        dsp[2 * g4 + 1] = pack_bf16x2(y1.x, y1.y);
                    }
                    PH_MARK(6);
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const uint32_t addr = ds_row + (((half * 4 + ch) ^ (i_row & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(addr), "r"(dsp[4 * ch]), "r"(dsp[4 * ch + 1]),
                                       "r"(dsp[4 * ch + 2]), "r"(dsp[4 * ch + 3])
                                     : "memory");
                    }
                    PH_MARK(7);
                }
                fence_proxy_async_smem();
                PH_MARK(8);
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&sh.ds_ready));
                PH_MARK(9);
            }
            if (!ok) break;

            // Epilogue: warpgroup 0 writes dV, warpgroup 1 writes dK * scale.
            __nv_bfloat16* dst_base = (wg == 0 ? p.dv : p.dk) +
                                      ((static_cast<long long>(wk.k_begin) + kv_row) * p.heads_k +
                                       wk.head_k) * kHeadDim;
            const float mul = wg == 0 ? 1.f : p.scale;
            if (steps > 0) {
                ok = mbar_wait(wctx, smem_u32(&sh.dkv_full), epi_cnt & 1u, 22);
                if (!ok) break;
                ++epi_cnt;
                tc_fence_after_sync();
            }
            const uint32_t acc_tmem = tmem_base + lane_base + (wg == 0 ? kColDV : kColDK);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                if (steps > 0) {
                    tmem_ld_x32(acc_tmem + c * 32, v);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0u;
                }
                if (ring) {
                    // Owner-directed accumulation: add this rank's partial dK / dV tile into the
                    // fp32 accumulator of the rank that owns the key block (possibly over NVLink).
                    float* acc = (wg == 0 ? p.dv_accum_peer[wk.owner] : p.dk_accum_peer[wk.owner]) +
                                 (static_cast<long long>(wk.owner_block) * p.heads_k + wk.head_k) * kDqTileFloats;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float* dst = acc + ((c * 8 + i) * kTileM + i_row) * 4;
                        asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                     ::"l"(dst), "f"(__uint_as_float(v[4 * i]) * mul),
                                       "f"(__uint_as_float(v[4 * i + 1]) * mul),
                                       "f"(__uint_as_float(v[4 * i + 2]) * mul),
                                       "f"(__uint_as_float(v[4 * i + 3]) * mul)
                                     : "memory");
                    }
                } else if (kv_valid) {
                    uint4* dst = reinterpret_cast<uint4*>(dst_base + c * 32);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            o[e] = pack_bf16x2(__uint_as_float(v[q4 * 8 + 2 * e]) * mul,
                                               __uint_as_float(v[q4 * 8 + 2 * e + 1]) * mul);
                        }
                        dst[q4] = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
            }
            if (steps > 0) {
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&sh.dkv_empty));
            }
        }
        PH_PRINT("compute", 7);
    }

    if (p.ring_docs != nullptr) {
        __threadfence_system();   // this thread's peer adds are performed before the CTA reports
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 12) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
    if (p.ring_docs != nullptr && threadIdx.x == 0) {
        // The last CTA of this rank tells every rank (itself included) that all of this rank's
        // dK / dV contributions have been added.
        const int done = atomicAdd(p.done_ctas, 1);
        if (done == static_cast<int>(gridDim.x) - 1) {
            __threadfence_system();
            for (int r = 0; r < p.world; ++r) {
                asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p.completion_peer[r]), "r"(1)
                             : "memory");
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Preprocess: one warp per query row.  Writes -D = -sum_d dO * O and -LSE2 = -LSE * log2(e),
// with -inf LSE and padding rows mapped to -inf (their P = exp2(s - inf) becomes exactly 0).
// Both are stored negated because the main loop only ever subtracts them.  The same pass
// clears the fp32 dQ accumulator.
// ---------------------------------------------------------------------------------------
struct BwdPreParams {
    const __nv_bfloat16* o;
    const __nv_bfloat16* dout;
    const float* lse;
    float* lse2;
    float* dpsum;
    float* dq_accum;     // zeroed here (each CTA clears the 16 KiB slab matching its 32 rows); may be null
    const int* cu_seqlens_q;
    int batch;
    int seqlen_q;
    int heads_q;
    int padded_q;
    long long lse_head_stride;
    long long lse_batch_stride;
};

// Padded rows per CTA (all heads of them: one contiguous stretch of O / dO).  Two rows measured
// best on a packed 65,536-token batch (447 us; 455 with 8 rows, 468 with 1; 528 for one head x 32
// rows per CTA) and keep enough CTAs in flight for small problems.
constexpr int kPreRows = 2;
constexpr int kPreItemsPerWarp = 4;  // (row, head) items a warp loads together

__global__ void __launch_bounds__(256)
bwd_preprocess_kernel(const BwdPreParams p) {
    // grid: padded_q / kPreRows CTAs of 8 warps.  A CTA owns kPreRows consecutive padded rows and
    // every head of them, so (for consecutive tokens) it streams one contiguous stretch of
    // kPreRows * heads_q * 256 bytes of O and of dO: consecutive warps read consecutive 256-byte
    // (row, head) items, kPreItemsPerWarp of them in flight per warp.
    __shared__ long long s_tok[kPreRows];   // packed token index of the padded row, -1 for padding rows
    __shared__ long long s_lse[kPreRows];   // LSE index of the row without the head term
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int prow_base = blockIdx.x * kPreRows;

    if (threadIdx.x < kPreRows) {
        const int prow = prow_base + threadIdx.x;
        long long tok = -1, lse_base = 0;
        if (prow < p.padded_q) {
            // Locate the document that owns this padded row.
            int doc, q_begin, q_len, pad_begin;
            if (p.cu_seqlens_q == nullptr) {
                const int per = ((p.seqlen_q + 127) / 128) * 128;
                doc = prow / per;
                pad_begin = doc * per;
                q_begin = doc * p.seqlen_q;
                q_len = p.seqlen_q;
                if (doc >= p.batch) doc = -1;
            } else {
                // Binary search over padded begins (monotone in doc).
                int lo = 0, hi = p.batch - 1;
                while (lo < hi) {
                    int mid = (lo + hi + 1) >> 1;
                    if (bwd_padded_begin(p.cu_seqlens_q[mid], mid) <= prow) lo = mid; else hi = mid - 1;
                }
                doc = lo;
                q_begin = p.cu_seqlens_q[doc];
                q_len = p.cu_seqlens_q[doc + 1] - q_begin;
                pad_begin = bwd_padded_begin(q_begin, doc);
                if (prow < pad_begin) doc = -1;
            }
            const int r = prow - pad_begin;
            if (doc >= 0 && r < q_len) {
                tok = static_cast<long long>(q_begin) + r;
                lse_base = p.cu_seqlens_q == nullptr ? static_cast<long long>(doc) * p.lse_batch_stride + r : tok;
            }
        }
        s_tok[threadIdx.x] = tok;
        s_lse[threadIdx.x] = lse_base;
    }

    // The fp32 dQ accumulator is heads_q * padded_q rows of 512 bytes: this CTA clears the
    // contiguous slab of kPreRows * heads_q rows with its index (which rows of which head they
    // are does not matter for zeroing; the slabs of all CTAs tile the accumulator).
    if (p.dq_accum != nullptr) {
        const long long slab_f4 = static_cast<long long>(kPreRows) * p.heads_q * 32;   // float4 per slab
        const long long total_f4 = static_cast<long long>(p.heads_q) * p.padded_q * 32;
        float4* base = reinterpret_cast<float4*>(p.dq_accum) + blockIdx.x * slab_f4;
        const long long room = total_f4 - blockIdx.x * slab_f4;
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        for (long long idx = threadIdx.x; idx < slab_f4 && idx < room; idx += 256) base[idx] = zero;
    }
    __syncthreads();

    const int items = kPreRows * p.heads_q;
    for (int i0 = warp * kPreItemsPerWarp; i0 < items; i0 += 8 * kPreItemsPerWarp) {
        uint2 ov[kPreItemsPerWarp], gv[kPreItemsPerWarp];
        float lv[kPreItemsPerWarp];
#pragma unroll
        for (int j = 0; j < kPreItemsPerWarp; ++j) {
            const int it = i0 + j;
            ov[j] = make_uint2(0u, 0u);
            gv[j] = make_uint2(0u, 0u);
            lv[j] = -INFINITY;
            if (it >= items) continue;
            const int row = it / p.heads_q, h = it - row * p.heads_q;
            const long long tok = s_tok[row];
            if (tok < 0) continue;
            const long long base = (tok * p.heads_q + h) * kHeadDim + lane * 4;
            ov[j] = __ldcs(reinterpret_cast<const uint2*>(p.o + base));
            gv[j] = __ldcs(reinterpret_cast<const uint2*>(p.dout + base));
            if (lane == 0) lv[j] = p.lse[s_lse[row] + static_cast<long long>(h) * p.lse_head_stride];
        }
#pragma unroll
        for (int j = 0; j < kPreItemsPerWarp; ++j) {
            const int it = i0 + j;
            if (it >= items) continue;
            const int row = it / p.heads_q, h = it - row * p.heads_q;
            const int prow = prow_base + row;
            if (prow >= p.padded_q) continue;
            const float o0 = __uint_as_float(ov[j].x << 16), o1 = __uint_as_float(ov[j].x & 0xFFFF0000u);
            const float o2 = __uint_as_float(ov[j].y << 16), o3 = __uint_as_float(ov[j].y & 0xFFFF0000u);
            const float g0 = __uint_as_float(gv[j].x << 16), g1 = __uint_as_float(gv[j].x & 0xFFFF0000u);
            const float g2 = __uint_as_float(gv[j].y << 16), g3 = __uint_as_float(gv[j].y & 0xFFFF0000u);
            float d = o0 * g0 + o1 * g1 + o2 * g2 + o3 * g3;   // 0 for padding rows
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, off);
            if (lane == 0) {
                const float l = lv[j];
                const long long out_idx = static_cast<long long>(h) * p.padded_q + prow;
                p.lse2[out_idx] = (l == -INFINITY) ? -INFINITY : -l * kLog2e;
                p.dpsum[out_idx] = -d;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Postprocess: dQ = bf16(scale * dq_accum), un-tiling the accumulator layout.
// One CTA of 128 threads per (head, padded query tile).
// ---------------------------------------------------------------------------------------
struct BwdPostParams {
    const float* dq_accum;
    __nv_bfloat16* dq;
    const int* cu_seqlens_q;
    int batch;
    int seqlen_q;
    int heads_q;
    int padded_q;
    float scale;
    // Accumulator tile of (head h, padded 128-row tile t) = h * tile_head_stride + t * tile_row_stride
    // (0, 0 selects the dq_accum layout: h * padded_q / 128 + t).
    int tile_head_stride;
    int tile_row_stride;
};

__global__ void __launch_bounds__(128)
bwd_postprocess_kernel(const BwdPostParams p) {
    // bf16 staging of the whole 128 x 128 tile; a pitch of 66 words keeps the 8-byte column-chunk
    // stores of 16 consecutive rows on distinct banks.
    constexpr int kPitch = kHeadDim + 4;
    __shared__ __align__(8) __nv_bfloat16 tile[kTileM * kPitch];
    const int pad_tile = blockIdx.x;
    const int h = blockIdx.y;
    const int pad_tiles = p.padded_q / kTileM;
    const int prow0 = pad_tile * kTileM;

    int doc = -1, q_begin = 0, q_len = 0, pad_begin = 0;
    if (p.cu_seqlens_q == nullptr) {
        const int per = ((p.seqlen_q + 127) / 128) * 128;
        doc = prow0 / per;
        pad_begin = doc * per;
        q_begin = doc * p.seqlen_q;
        q_len = p.seqlen_q;
        if (doc >= p.batch) return;
    } else {
        int lo = 0, hi = p.batch - 1;
        while (lo < hi) {
            int mid = (lo + hi + 1) >> 1;
            if (bwd_padded_begin(p.cu_seqlens_q[mid], mid) <= prow0) lo = mid; else hi = mid - 1;
        }
        doc = lo;
        q_begin = p.cu_seqlens_q[doc];
        q_len = p.cu_seqlens_q[doc + 1] - q_begin;
        pad_begin = bwd_padded_begin(q_begin, doc);
        if (prow0 < pad_begin) return;
    }
    const int r0 = prow0 - pad_begin;
    if (r0 >= q_len) return;

    const long long tile_index = p.tile_row_stride == 0
        ? static_cast<long long>(h) * pad_tiles + pad_tile
        : static_cast<long long>(h) * p.tile_head_stride + static_cast<long long>(pad_tile) * p.tile_row_stride;
    const float4* src = reinterpret_cast<const float4*>(p.dq_accum + tile_index * kDqTileFloats);
    // src[chunk * 128 + row] holds columns 4*chunk .. 4*chunk+3 of `row`: thread = row reads its 32
    // chunks (each warp instruction a contiguous 512 bytes), scales, rounds and stages them.
#pragma unroll 8
    for (int chunk = 0; chunk < 32; ++chunk) {
        const float4 v = __ldcs(src + chunk * kTileM + threadIdx.x);
        uint2 o;
        o.x = pack_bf16x2(v.x * p.scale, v.y * p.scale);
        o.y = pack_bf16x2(v.z * p.scale, v.w * p.scale);
        *reinterpret_cast<uint2*>(&tile[threadIdx.x * kPitch + chunk * 4]) = o;
    }
    __syncthreads();
    // One warp writes one whole 256-byte row per instruction (32 lanes x 8 bytes).
    const int lane = threadIdx.x & 31;
    for (int rr = threadIdx.x >> 5; rr < kTileM; rr += 4) {
        if (r0 + rr < q_len) {
            const uint2 o = *reinterpret_cast<const uint2*>(&tile[rr * kPitch + lane * 4]);
            const long long tok = static_cast<long long>(q_begin) + r0 + rr;
            *reinterpret_cast<uint2*>(p.dq + (tok * p.heads_q + h) * kHeadDim + lane * 4) = o;
        }
    }
}

// Waits (bounded) until a system-scope counter reaches `expected`: every rank adds one to every
// rank's counter when all of its dK / dV contributions have been added.
__global__ void ring_wait_kernel(const int* counter, int expected, unsigned int* status,
                                 unsigned long long timeout_ns) {
    const uint64_t start = global_timer_ns();
    while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= expected) return;
        if (global_timer_ns() - start > timeout_ns) {
            set_status(status, kStatusTimeout, (26u << 12));
            return;
        }
        __nanosleep(500);
    }
}

// Completion report of a rank that launched no attention work.
__global__ void ring_signal_kernel(int* c0, int* c1, int* c2, int* c3, int* c4, int* c5, int* c6, int* c7,
                                   int world) {
    int* c[8] = {c0, c1, c2, c3, c4, c5, c6, c7};
    for (int r = 0; r < world; ++r) {
        asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(c[r]), "r"(1) : "memory");
    }
}

}  // namespace b2a
