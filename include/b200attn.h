/*
 * b200attn — C ABI of the B200 (sm_100a) attention engine.
 *
 * This is the drop-in boundary for the attention path of min_fa3_demo: every
 * entry point takes plain device pointers, sizes and a CUDA stream handle, and
 * replaces one host binding of the reference (cited per function, paths relative
 * to the reference project).  The library allocates no device memory: outputs
 * and scratch ("workspace") are owned by the caller; b2a_*_workspace_bytes()
 * says how much scratch a call needs.  All functions return 0 on success and a
 * negative B2A_ERR_* code on failure; b2a_last_error() returns a thread-local
 * description of the last failure.  Nothing here throws or exits.
 *
 * Tensors are bf16, head_dim = 128, laid out as a flat [tokens, heads, 128]
 * array.  A fixed-length BSHD batch is the special case tokens = batch * seqlen
 * with cu_seqlens == NULL.  Launches are asynchronous on the given stream.
 */
#ifndef B200ATTN_H_
#define B200ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2A_OK 0
#define B2A_ERR_INVALID_ARGUMENT (-1)
#define B2A_ERR_CUDA (-2)
#define B2A_ERR_WORKSPACE_TOO_SMALL (-3)
#define B2A_ERR_UNSUPPORTED_DEVICE (-4)
#define B2A_ERR_DEVICE_STATUS (-5)

/* Version of this ABI (bumped when a struct layout changes). */
int b2a_abi_version(void);

/* Thread-local text of the last error returned on this thread ("" if none). */
const char* b2a_last_error(void);

/* ------------------------------------------------------------------------- */
/* Forward                                                                    */
/* ------------------------------------------------------------------------- */

typedef struct b2a_fwd_args {
    const void* q;              /* bf16 [total_q, heads_q, 128] */
    const void* k;              /* bf16 [total_k, heads_k, 128] */
    const void* v;              /* bf16 [total_k, heads_k, 128] */
    void* out;                  /* bf16 [total_q, heads_q, 128] */
    float* lse;                 /* BSHD: [batch, heads_q, seqlen_q]; varlen: [heads_q, total_q] */
    const int32_t* cu_seqlens_q; /* device int32 [batch + 1], NULL for BSHD */
    const int32_t* cu_seqlens_k; /* device int32 [batch + 1], NULL for BSHD */
    int32_t batch;
    int32_t seqlen_q;           /* BSHD: S_q.  varlen: max_seqlen_q */
    int32_t seqlen_k;           /* BSHD: S_k.  varlen: max_seqlen_k */
    int32_t total_q;            /* tokens in q (batch * seqlen_q for BSHD) */
    int32_t total_k;
    int32_t heads_q;
    int32_t heads_k;
    int32_t head_dim;           /* must be 128 */
    int32_t is_causal;          /* bottom-right aligned causal mask */
    int32_t merge_running;      /* 1: merge into the partial result already in out/lse */
    int32_t grid_blocks;        /* 0 = one CTA per SM; >0 overrides the CTA count */
    float softmax_scale;        /* 0 = 1/sqrt(head_dim) */
    void* workspace;            /* device scratch, 16-byte aligned */
    size_t workspace_bytes;
    /* Ring step (all NULL / 0 otherwise): prefetch_blocks extra CTAs of the same launch first copy
     * prefetch_bytes (a multiple of 16) from prefetch_src_k / _v -- normally another rank's K / V
     * reached through a peer mapping -- to prefetch_dst_k / _v, then join the attention work. */
    const void* prefetch_src_k;
    const void* prefetch_src_v;
    void* prefetch_dst_k;
    void* prefetch_dst_v;
    size_t prefetch_bytes;
    int32_t prefetch_blocks;
} b2a_fwd_args;

/* Scratch needed by b2a_fwd for these sizes. */
size_t b2a_fwd_workspace_bytes(int32_t batch, int32_t total_q, int32_t is_varlen);

/*
 * Attention forward: out = softmax(scale * q k^T [+causal]) v, lse = logsumexp.
 * Replaces `forward` (bindings.cpp:240) and `forward_varlen` (bindings.cpp:280)
 * of the reference, including its varlen scheduler-metadata kernel
 * (csrc/min_fa3_varlen_prepare_scheduler.cu:214); with merge_running = 1 it is
 * `forward_varlen_ring` (csrc/min_fa3_varlen_ring_bindings.cu:231): attention merged into
 * the running out/lse on CTAs [0, grid_blocks) and, with the prefetch_* fields set, the copy
 * of the next source rank's K/V on CTAs [grid_blocks, grid_blocks + prefetch_blocks) of the
 * same launch (the reference's compute + communication kernel,
 * include/min_fa3_varlen_ring_launch.h:217).
 */
int b2a_fwd(const b2a_fwd_args* args, void* cuda_stream);

/*
 * Forward for callers that must not allocate device memory.  No counterpart in the
 * reference (its bindings allocate outputs and scratch on every call, bindings.cpp:267-269).
 *
 * Who needs it: code that runs where cudaMalloc is unavailable or forbidden -- a plugin
 * inside a serving runtime that hands out one fixed memory pool at start-up, a hard
 * real-time loop that may not touch the allocator, or a call site that owns q/k/v/out/lse
 * but has no way to size and pass a workspace.  Same computation and arguments as b2a_fwd,
 * except that args->workspace / workspace_bytes are ignored: the scratch (scheduler ticket,
 * status word and the varlen work list) lives in a 64 KiB array built into the library,
 * resident on every GPU that loads it.  The call and everything under it use no cudaMalloc,
 * cudaFree or allocating library routine.
 *
 * Limit: problems whose scratch exceeds b2a_fwd_noalloc_scratch_limit() bytes -- packed
 * batches with total_q / 256 + batch + 1 > 8190; fixed-length BSHD always fits -- are
 * rejected with B2A_ERR_WORKSPACE_TOO_SMALL and a message naming both sizes.
 * Set-up: the first call on each device (with that device current) looks up the array's
 * device address; make that first call before starting any stream capture.
 * Sharing: all calls on a device use the same array.  The words that must start at zero are
 * cleared on the stream by every call; the rest keeps the previous call's contents.  Two
 * calls that may overlap on the GPU (different streams, no dependency) race on it -- order
 * them, or use b2a_fwd with separate workspaces.
 * Status: b2a_check_status(NULL, stream) reads the status word of the built-in scratch.
 */
int b2a_fwd_noalloc(const b2a_fwd_args* args, void* cuda_stream);

/* Size in bytes of the built-in scratch of b2a_fwd_noalloc. */
size_t b2a_fwd_noalloc_scratch_limit(void);

/* ------------------------------------------------------------------------- */
/* Backward                                                                   */
/* ------------------------------------------------------------------------- */

typedef struct b2a_bwd_args {
    const void* dout;           /* bf16 [total_q, heads_q, 128] */
    const void* q;
    const void* k;
    const void* v;
    const void* out;            /* forward output */
    const float* lse;           /* forward LSE (layout as in b2a_fwd_args) */
    void* dq;                   /* bf16 [total_q, heads_q, 128] */
    void* dk;                   /* bf16 [total_k, heads_k, 128] */
    void* dv;                   /* bf16 [total_k, heads_k, 128] */
    const int32_t* cu_seqlens_q;
    const int32_t* cu_seqlens_k;
    int32_t batch;
    int32_t seqlen_q;
    int32_t seqlen_k;
    int32_t total_q;
    int32_t total_k;
    int32_t heads_q;
    int32_t heads_k;
    int32_t head_dim;
    int32_t is_causal;
    int32_t deterministic;      /* 1: bitwise repeatable dq accumulation order */
    int32_t grid_blocks;
    float softmax_scale;
    void* workspace;
    size_t workspace_bytes;
} b2a_bwd_args;

size_t b2a_bwd_workspace_bytes(int32_t batch, int32_t total_q, int32_t total_k, int32_t heads_q,
                               int32_t heads_k, int32_t is_varlen);

/*
 * Attention backward: dq, dk, dv from dout and the forward's q, k, v, out, lse.
 * Replaces `backward` (csrc/backward/min_fa3_bwd_bindings.cu:156) and
 * `backward_varlen` (csrc/backward/min_fa3_bwd_bindings.cu:255): the dO*O
 * preprocess, the dK/dV main loop that recomputes P from LSE, fp32 dQ
 * accumulation and the cast back to bf16.
 */
int b2a_bwd(const b2a_bwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------- */
/* Peer memory (single node, NVLink)                                          */
/* ------------------------------------------------------------------------- */

/*
 * Export a device buffer for other processes of the node: writes the 64-byte CUDA-IPC
 * handle of the allocation that contains `ptr` and the byte offset of `ptr` inside it.
 * Together with b2a_ipc_import this replaces the peer-pointer table of the reference's
 * TKParallelTensor (`raw_ptrs_`, csrc/backward/min_fa3_bwd_bindings.cu:711-715; created at
 * min_fa3_op.py:201-206).  Carrying the offset explicitly avoids mapping an offset view at
 * its allocation base (problem_record/tkparallel_ipc_offset_repro/README.md:15-27).
 */
int b2a_ipc_export(const void* ptr, unsigned char* handle64, uint64_t* offset);

/* Map a buffer exported by another process; *out_ptr is usable by kernels on this device. */
int b2a_ipc_import(const unsigned char* handle64, uint64_t offset, void** out_ptr);

/* Unmap a pointer returned by b2a_ipc_import (pass the same offset). */
int b2a_ipc_close(void* ptr, uint64_t offset);

/*
 * Asynchronous strided copy between pinned host memory and device memory (or device to device):
 * `rows` rows of `row_bytes` bytes, the rows `src_pitch` / `dst_pitch` bytes apart.  A thin
 * wrapper over the runtime's 2-D memcpy for callers that move a subset of heads of a
 * [tokens, heads, 128] host tensor without staging it (the host-buffer pipeline of this
 * package).  No counterpart in the reference, whose operators take device tensors only.
 * kind: 1 host->device, 2 device->host, 3 device->device.
 */
int b2a_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t row_bytes,
                size_t rows, int32_t kind, void* cuda_stream);

/*
 * Copy `bytes` (multiple of 16) from `src` (typically a peer pointer) to local `dst` with
 * `num_blocks` CTAs of bulk asynchronous copies through shared memory.  Replaces
 * RemoteLoadTileKernel / RemoteLoadVecKernel (csrc/parallel/remote_load.cu:21-128).
 * `status` may be NULL or point to a zeroed device word that receives an error code if a
 * bounded wait runs out.
 */
int b2a_peer_copy(void* dst, const void* src, size_t bytes, int32_t num_blocks,
                  unsigned int* status, void* cuda_stream);

/* ------------------------------------------------------------------------- */
/* Context-parallel forward ("mega ring")                                     */
/* ------------------------------------------------------------------------- */

typedef struct b2a_ring_fwd_args {
    const void* q;                       /* bf16 [total_q, heads_q, 128], this rank's queries */
    void* out;                           /* bf16 [total_q, heads_q, 128] */
    float* lse;                          /* fp32 [heads_q, total_q] */
    void* arena_k;                       /* bf16 [world_size * rank_kv_capacity, heads_k, 128]: rank-major */
    void* arena_v;                       /*   K/V arena of this rank; rank r's keys live in rows [r*cap, ...) */
    const void* peer_k[8];               /* arena_k base of every rank as mapped on this device */
    const void* peer_v[8];
    const int32_t* cu_seqlens_q_host;    /* HOST int32 [batch + 1]: this rank's local document offsets */
    const int32_t* global_seqlens_host;  /* HOST int32 [batch]: document length over its whole ring */
    const int32_t* ring_sizes_host;      /* HOST int32 [batch]: 1, 2, 4 or 8, non-increasing */
    const int32_t* ring_starts_host;     /* HOST int32 [batch]: first rank of the ring, multiple of its size */
    int64_t* stats;                      /* optional device int64[2]: (query-tile visits, K/V tile reads) */
    int32_t batch;
    int32_t world_size;
    int32_t rank;
    int32_t rank_kv_capacity;            /* arena rows per rank, multiple of 128 */
    int32_t total_q;
    int32_t heads_q;
    int32_t heads_k;
    int32_t head_dim;
    int32_t is_causal;                   /* zigzag causal: rank r of a ring of G holds half-chunks r and 2G-1-r */
    int32_t num_comp_sm;                 /* CTAs that only compute */
    int32_t num_comm_sm;                 /* CTAs that first copy peers' K/V into the arena, then compute */
    void* workspace;
    size_t workspace_bytes;
} b2a_ring_fwd_args;

size_t b2a_ring_fwd_workspace_bytes(int32_t batch, int32_t world_size, int32_t rank_kv_capacity,
                                    int32_t total_q);

/*
 * Context-parallel attention forward over a single node: every document is sharded over a
 * ring of 1/2/4/8 ranks (zigzag halves when causal).  One launch per rank: copy CTAs pull the
 * K/V blocks of the other ring members from their arenas over NVLink into this rank's arena
 * and flag each 128-row block; compute CTAs run attention over local blocks first and over
 * remote blocks as their flags appear, keeping the softmax state on chip across all ring
 * members (no partial O/LSE round trips).  Every rank must have written its own arena slice
 * and all ranks must have synchronised before the call.  Replaces
 * `forward_varlen_mega_ring` (csrc/mega_ring_min_fa3_varlen_ring_bindings.cu:304) including
 * the hierarchical sub-rings (include/min_fa3_mega_ring_hierarchy.h:13-33).
 *
 * Host work per call (this entry point and b2a_ring_bwd): the work list and the copy tasks are
 * built on the host from the `*_host` arrays and uploaded with one cudaMemcpyAsync from an
 * ordinary (pageable) std::vector.  The runtime stages such a copy before the call returns, so
 * the vector may be freed at once, but the copy is why these two calls may not be captured into
 * a CUDA graph and why they are not fully asynchronous to the host (the host blocks until the
 * staging copy is taken, not until the kernels end).  Callers that need capture or no host
 * work use the plain entry points (b2a_fwd_noalloc, b2a_fwd, b2a_bwd) per ring step.
 */
int b2a_ring_fwd(const b2a_ring_fwd_args* args, void* cuda_stream);

typedef struct b2a_ring_bwd_args {
    const void* dout;                    /* bf16 [total_q, heads_q, 128] */
    const void* q;
    const void* out;
    const float* lse;                    /* fp32 [heads_q, total_q] from the forward */
    void* dq;                            /* bf16 [total_q, heads_q, 128] */
    void* dk;                            /* bf16 [local_total_k, heads_k, 128] (compact, not arena shaped) */
    void* dv;
    void* arena_k;                       /* as in b2a_ring_fwd_args */
    void* arena_v;
    const void* peer_k[8];
    const void* peer_v[8];
    float* dk_accum_peer[8];             /* fp32 dK accumulator of every rank, zeroed by the caller: */
    float* dv_accum_peer[8];             /*   >= rank_kv_capacity * heads_k * 128 floats each */
    int32_t* completion_peer[8];         /* int32[1] completion counter of every rank, zeroed by the caller */
    const int32_t* cu_seqlens_q_host;
    const int32_t* global_seqlens_host;
    const int32_t* ring_sizes_host;
    const int32_t* ring_starts_host;
    int32_t batch;
    int32_t world_size;
    int32_t rank;
    int32_t rank_kv_capacity;
    int32_t total_q;
    int32_t local_total_k;
    int32_t heads_q;
    int32_t heads_k;
    int32_t head_dim;
    int32_t is_causal;
    int32_t num_comp_sm;
    int32_t num_comm_sm;
    int32_t kv_resident;                 /* non-zero: the arena still holds every remote K/V block this rank's
                                            queries see, left there by b2a_ring_fwd on the same metadata and
                                            K/V; nothing is pulled again and all CTAs compute from the start.
                                            0 (the reference's behaviour): the backward pulls them itself. */
    void* workspace;
    size_t workspace_bytes;
} b2a_ring_bwd_args;

size_t b2a_ring_bwd_workspace_bytes(int32_t batch, int32_t world_size, int32_t rank_kv_capacity,
                                    int32_t total_q, int32_t heads_q);

/*
 * Context-parallel attention backward.  Each rank runs the KV-stationary backward over every
 * key block (local or pulled from a ring member into the arena) that its queries see; dQ stays
 * local, while the dK / dV partial tiles are added in fp32 straight into the accumulator of the
 * rank that owns the key block (over NVLink for remote owners).  When a rank has added all its
 * contributions it bumps every rank's completion counter; each rank waits (bounded) for its
 * counter to reach the world size and then casts its accumulator to bf16 dk / dv.  The caller
 * zeroes the accumulators and counters and synchronises all ranks before every call.  Replaces
 * `backward_varlen_mega_ring` (csrc/backward/min_fa3_bwd_bindings.cu:375-722).
 */
int b2a_ring_bwd(const b2a_ring_bwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------- */
/* Device status                                                              */
/* ------------------------------------------------------------------------- */

/*
 * Synchronises the stream and reads the status word that kernels launched with
 * this workspace wrote.  Returns B2A_OK, or B2A_ERR_DEVICE_STATUS with the
 * decoded status in b2a_last_error() (for example a bounded wait that ran out).
 * No counterpart in the reference, whose device-side waits are unbounded
 * (include/mega_ring_semaphore.cuh:69-80).  workspace == NULL reads the status
 * word of the scratch built into the library, i.e. of the last b2a_fwd_noalloc
 * call on the current device.
 */
int b2a_check_status(const void* workspace, void* cuda_stream);

/*
 * Limit, in nanoseconds, of every bounded device-side wait (mbarriers, K/V block
 * flags, deterministic-order counters) of launches made after the call; the
 * cross-rank completion wait that ends b2a_ring_bwd gets ten times this value.
 * Default 2 s; accepted range 1 us .. 4 s; 0 restores the default.  Process-wide.
 * A wait that runs out never traps or hangs: the kernel records
 * (wait site, CTA) in the status word, drains and returns, and b2a_check_status
 * reports it.  No counterpart in the reference (include/mega_ring_semaphore.cuh:69-80
 * spins without a limit).
 */
int b2a_set_wait_timeout_ns(uint64_t nanoseconds);

/* ------------------------------------------------------------------------- */
/* Kernel timing                                                              */
/* ------------------------------------------------------------------------- */

#define B2A_KERNEL_FWD 0
#define B2A_KERNEL_BWD 1

/*
 * While enabled (per calling thread), every launch of the forward / backward main kernel
 * is bracketed by CUDA events on the launch stream; up to 256 launches per kernel are kept.
 * Enabling resets the record.  No counterpart in the reference (its scripts time whole
 * calls, ring_test/benchmark_topology_forward.py:382-411).
 */
int b2a_profile_enable(int enable);

/*
 * Synchronises the recorded events and writes the duration in milliseconds of each recorded
 * launch of `kernel` (B2A_KERNEL_*) to ms[0..]; returns the number written (<= capacity) or
 * a negative error code.
 */
int b2a_profile_read(int kernel, float* ms, int capacity);

#ifdef __cplusplus
}
#endif

#endif /* B200ATTN_H_ */
