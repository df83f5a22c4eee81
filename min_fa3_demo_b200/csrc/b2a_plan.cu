// Varlen work planner: cuts every document into fixed-size pieces and emits a flat
// (document, piece) work list sorted longest-first, so the persistent attention
// kernels can hand out tiles with a single atomic ticket and no per-tile search.
//
//   kind 0 (forward):  a piece is 256 query rows; cost = key blocks (128) it reads.
//   kind 1 (backward): a piece is 128 key rows;  cost = query tiles (128) that see it.
//
// One CTA plans the whole batch (a packed batch has at most a few thousand pieces).
#include "b2a_host.cuh"

namespace b2a {

namespace {

constexpr int kPlanThreads = 1024;
constexpr int kCostBuckets = 2048;

__device__ __forceinline__ int plan_pieces(int kind, int q_len, int k_len) {
    return kind == 0 ? (q_len + 255) / 256 : (k_len + 127) / 128;
}

__device__ __forceinline__ int plan_cost(int kind, int causal, int q_len, int k_len, int piece) {
    int cost;
    if (kind == 0) {
        int limit = k_len;
        if (causal) {
            int row_last = min((piece + 1) * 256, q_len) - 1;
            limit = min(limit, row_last + 1 + k_len - q_len);
        }
        cost = limit <= 0 ? 0 : (limit + 127) / 128;
    } else {
        int m_tiles = (q_len + 127) / 128;
        int first = 0;
        if (causal) {
            // Query row r sees key c when c <= r + k_len - q_len.
            int first_row = max(0, piece * 128 + q_len - k_len);
            first = min(m_tiles, first_row / 128);
        }
        cost = m_tiles - first;
    }
    return min(max(cost, 0), kCostBuckets - 1);
}

__global__ void __launch_bounds__(kPlanThreads)
varlen_plan_kernel(int kind, const int* __restrict__ cu_q, const int* __restrict__ cu_k, int batch,
                   int causal, int2* __restrict__ work_list, int* __restrict__ num_entries,
                   int max_entries_cap) {
    __shared__ int bucket[kCostBuckets];
    __shared__ int warp_sum[32];
    __shared__ int total;
    static_assert(kCostBuckets == 2 * kPlanThreads, "the scan gives every thread two buckets");
    for (int i = threadIdx.x; i < kCostBuckets; i += kPlanThreads) bucket[i] = 0;
    if (threadIdx.x == 0) total = 0;
    __syncthreads();

    // Histogram of piece costs.
    for (int doc = threadIdx.x; doc < batch; doc += kPlanThreads) {
        int q_len = cu_q[doc + 1] - cu_q[doc];
        int k_len = cu_k[doc + 1] - cu_k[doc];
        int pieces = plan_pieces(kind, q_len, k_len);
        for (int pc = 0; pc < pieces; ++pc) {
            atomicAdd(&bucket[plan_cost(kind, causal, q_len, k_len, pc)], 1);
        }
        atomicAdd(&total, pieces);
    }
    __syncthreads();

    // Exclusive scan over the buckets from the most expensive down: thread t owns the two
    // buckets at descending positions 2t and 2t+1; warp scan, then a scan of the 32 warp sums.
    {
        const int t = threadIdx.x, lane = t & 31, wid = t >> 5;
        const int c_hi = kCostBuckets - 1 - 2 * t, c_lo = c_hi - 1;
        const int n_hi = bucket[c_hi], n_lo = bucket[c_lo];
        const int mine = n_hi + n_lo;
        int incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) warp_sum[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            const int ws = warp_sum[lane];
            int wincl = ws;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xFFFFFFFFu, wincl, d);
                if (lane >= d) wincl += up;
            }
            warp_sum[lane] = wincl - ws;
        }
        __syncthreads();
        const int excl = warp_sum[wid] + incl - mine;
        bucket[c_hi] = excl;
        bucket[c_lo] = excl + n_hi;
        if (t == 0) *num_entries = min(total, max_entries_cap);
    }
    __syncthreads();

    // Scatter.  Pieces of equal cost land in arbitrary order, which is harmless:
    // work items are independent.
    for (int doc = threadIdx.x; doc < batch; doc += kPlanThreads) {
        int q_len = cu_q[doc + 1] - cu_q[doc];
        int k_len = cu_k[doc + 1] - cu_k[doc];
        int pieces = plan_pieces(kind, q_len, k_len);
        for (int pc = 0; pc < pieces; ++pc) {
            int pos = atomicAdd(&bucket[plan_cost(kind, causal, q_len, k_len, pc)], 1);
            if (pos < max_entries_cap) {
                work_list[pos] = make_int2(doc, pc);
            }
        }
    }
}

}  // namespace

int launch_varlen_plan(int kind, const int* cu_seqlens_q, const int* cu_seqlens_k, int batch,
                       int causal, int2* work_list, int* num_entries, int max_entries_cap,
                       cudaStream_t stream) {
    varlen_plan_kernel<<<1, kPlanThreads, 0, stream>>>(kind, cu_seqlens_q, cu_seqlens_k, batch, causal,
                                                      work_list, num_entries, max_entries_cap);
    B2A_CUDA_OK(cudaGetLastError());
    return B2A_OK;
}

}  // namespace b2a
