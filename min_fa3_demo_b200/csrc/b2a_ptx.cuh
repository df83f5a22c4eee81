// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarrier (with bounded waits), TMA tiled loads, tcgen05 MMA / TMEM load-store,
// bulk reduce-add.  Every spin wait in this file is bounded: after the deadline
// the waiter records an error code and returns false, so a protocol bug shows
// up as a status word on the host instead of a hung GPU.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

// Optional phase timing (compile with -DB2A_PHASES): per-role cycle accumulators printed by
// CTA 0 at kernel exit.  Compiled out by default.
#ifdef B2A_PHASES
#include <cstdio>
#define PH_DECL(n) long long ph_[10] = {0}; long long ph_t_ = clock64();
#define PH_MARK(i) do { long long now_ = clock64(); ph_[i] += now_ - ph_t_; ph_t_ = now_; } while (0)
#define PH_PRINT(name, n) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) { \
    printf("[phases] %s warp %d: %lld %lld %lld %lld %lld %lld %lld %lld %lld %lld\n", name, (int)(threadIdx.x >> 5), \
           ph_[0], ph_[1], ph_[2], ph_[3], ph_[4], ph_[5], ph_[6], ph_[7], ph_[8], ph_[9]); } } while (0)
#else
#define PH_DECL(n)
#define PH_MARK(i)
#define PH_PRINT(name, n)
#endif

namespace b2a {

// ----------------------------------------------------------------------------
// Device status word.  0 = ok.  Non-zero values are (code << 24) | detail.
// ----------------------------------------------------------------------------
enum : uint32_t {
    kStatusOk = 0,
    kStatusTimeout = 1,   // a bounded wait ran out
    kStatusBadArg = 2,    // a device-side argument check failed
};

__device__ __forceinline__ void set_status(unsigned int* status, uint32_t code, uint32_t detail) {
    if (status != nullptr) {
        atomicCAS(status, 0u, (code << 24) | (detail & 0xFFFFFFu));
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(pred));
    return pred;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

__device__ __forceinline__ uint32_t global_timer_lo() {
    uint32_t t;
    asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_shared_volatile_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void st_shared_volatile_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.volatile.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Shared abort word: once any waiter of the CTA gives up, every later wait of
// the CTA returns immediately so that all roles drain to the common exit.
// The deadline uses the low 32 bits of the nanosecond timer, so it must stay
// below 4.29 s.
struct WaitCtx {
    uint32_t abort_smem;      // shared-memory address of the abort word
    unsigned int* status;     // in global memory (may be null)
    uint32_t timeout_ns;
};

// Bounded wait on an mbarrier phase.  `tag` identifies the wait site in the
// status word.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(const WaitCtx& ctx, uint32_t bar, uint32_t parity,
                                          uint32_t tag) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const uint32_t start = global_timer_lo();
    uint32_t polls = 0;
#pragma unroll 1
    while (true) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
        if ((++polls & 0x3Fu) == 0u) {
            if (ld_shared_volatile_u32(ctx.abort_smem) != 0u) {
                return false;
            }
            if (global_timer_lo() - start > ctx.timeout_ns) {
                st_shared_volatile_u32(ctx.abort_smem, 1u);
                set_status(ctx.status, kStatusTimeout, (tag << 12) | (blockIdx.x & 0xFFFu));
                return false;
            }
        }
    }
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, no multicast anywhere)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Untiled bulk copy global -> shared (16-byte aligned addresses and size).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
        : "memory");
}

// Bulk fp32 reduce-add shared -> global (16-byte aligned, size multiple of 16).
__device__ __forceinline__ void bulk_reduce_add_f32(void* dst_global, uint32_t src_smem,
                                                    uint32_t bytes) {
    asm volatile(
        "cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
        ::"l"(reinterpret_cast<uint64_t>(dst_global)), "r"(src_smem), "r"(bytes)
        : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: tensor memory management
// ----------------------------------------------------------------------------
// Whole-warp collective.  Writes the allocated TMEM base address to *dst_smem.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(dst_smem), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Arrive on an mbarrier once every tcgen05 operation issued so far by this
// thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar)
                 : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: descriptors
// ----------------------------------------------------------------------------
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile.
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4
//   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    desc |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format,
//   bit 15 A major (0 = K-major, 1 = MN-major), bit 16 B major,
//   bits [17,23) N >> 3, bits [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major,
                                                       int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem].  Issued by one thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem].  Issued by one thread.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Split form of the 128-byte-swizzle descriptor for the issue loops: the high word is a
// constant (stride offset 1024 B, version 1, layout 2) and the low word is
// (address >> 4) | (leading offset >> 4) << 16, so stepping through a tile is one 32-bit add
// per operand.  (A single issuing thread has little instruction-level parallelism: building
// full 64-bit descriptors per MMA costs more than the 64 cycles the MMA itself takes.)
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);

__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t smem_addr) {
    return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}

// MN-major operand made of two 64-column halves 16 KiB apart.
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t smem_addr) {
    return ((smem_addr & 0x3FFFFu) >> 4) | ((16384u >> 4) << 16);
}

// Low-word increment of k-step `ks` (16 elements) inside a [128 rows][128 columns] tile.
__host__ __device__ constexpr uint32_t kstep_kmajor(int ks) {
    return static_cast<uint32_t>((ks >> 2) * (16384 >> 4) + (ks & 3) * (32 >> 4));
}
__host__ __device__ constexpr uint32_t kstep_mnmajor(int ks) {
    return static_cast<uint32_t>(ks * (2048 >> 4));
}

__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 db;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// Warp-collective forms: every lane of a converged warp executes the call and one elected lane
// issues the instruction.  Keeping the issuing warp's control flow uniform (instead of a
// `lane == 0` branch around the issue code) matters when other warps of the SM run dense
// arithmetic: measured on B200 with eight FMA-bound warps beside the issuing warp, a
// single-thread branch sustained one 128x128x16 MMA per 183 clocks, an elected branch one per
// 93-131, and this form one per 71 (64 is the tensor pipe's own rate).
__device__ __forceinline__ void umma_ss_lo_w(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

__device__ __forceinline__ void umma_ts_lo_w(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe;\n\t"
        ".reg .b64 db;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// Whole-contraction forms: the eight (or four) k-steps of one 128 x N x 128 (or x 64) product as
// ONE instruction group with a single lane election, so that the issuing warp spends a handful
// of instructions per MMA instead of an election, a predicate and two register pairs each.
// `accumulate` applies to the first k-step; the others always accumulate.
// A and B both K-major [rows][128] tiles.
__device__ __forceinline__ void umma_ss_kk_x8_w(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe, pt;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
        "add.u32 ra, %1, 2;\n\t"
        "add.u32 rb, %2, 2;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 4;\n\t"
        "add.u32 rb, %2, 4;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 6;\n\t"
        "add.u32 rb, %2, 6;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1024;\n\t"
        "add.u32 rb, %2, 1024;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1026;\n\t"
        "add.u32 rb, %2, 1026;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1028;\n\t"
        "add.u32 rb, %2, 1028;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1030;\n\t"
        "add.u32 rb, %2, 1030;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// A and B both MN-major tiles.
__device__ __forceinline__ void umma_ss_nn_x8_w(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe, pt;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
        "add.u32 ra, %1, 128;\n\t"
        "add.u32 rb, %2, 128;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 256;\n\t"
        "add.u32 rb, %2, 256;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 384;\n\t"
        "add.u32 rb, %2, 384;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 512;\n\t"
        "add.u32 rb, %2, 512;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 640;\n\t"
        "add.u32 rb, %2, 640;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 768;\n\t"
        "add.u32 rb, %2, 768;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 896;\n\t"
        "add.u32 rb, %2, 896;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// A K-major, B MN-major.
__device__ __forceinline__ void umma_ss_kn_x8_w(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe, pt;\n\t"
        ".reg .b64 da, db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
        "add.u32 ra, %1, 2;\n\t"
        "add.u32 rb, %2, 128;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 4;\n\t"
        "add.u32 rb, %2, 256;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 6;\n\t"
        "add.u32 rb, %2, 384;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1024;\n\t"
        "add.u32 rb, %2, 512;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1026;\n\t"
        "add.u32 rb, %2, 640;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1028;\n\t"
        "add.u32 rb, %2, 768;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "add.u32 ra, %1, 1030;\n\t"
        "add.u32 rb, %2, 896;\n\t"
        "mov.b64 da, {ra, %5};\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, pt;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// A from tensor memory (8 columns per k-step), B MN-major.
__device__ __forceinline__ void umma_ts_x8_w(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe, pt;\n\t"
        ".reg .b64 db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
        "add.u32 ra, %1, 8;\n\t"
        "add.u32 rb, %2, 128;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 16;\n\t"
        "add.u32 rb, %2, 256;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 24;\n\t"
        "add.u32 rb, %2, 384;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 32;\n\t"
        "add.u32 rb, %2, 512;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 40;\n\t"
        "add.u32 rb, %2, 640;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 48;\n\t"
        "add.u32 rb, %2, 768;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 56;\n\t"
        "add.u32 rb, %2, 896;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// Four k-steps (64 contraction elements): A from tensor memory, B MN-major.
__device__ __forceinline__ void umma_ts_x4_w(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, pe, pt;\n\t"
        ".reg .b64 db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
        "add.u32 ra, %1, 8;\n\t"
        "add.u32 rb, %2, 128;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 16;\n\t"
        "add.u32 rb, %2, 256;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "add.u32 ra, %1, 24;\n\t"
        "add.u32 rb, %2, 384;\n\t"
        "mov.b64 db, {rb, %5};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, pt;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiSw128)
        : "memory");
}

// Same elected lane as the *_w MMA forms (the commit must come from the thread that issued them).
__device__ __forceinline__ void tc_commit_w(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred pe;\n\t"
        "elect.sync _|pe, 0xFFFFFFFF;\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n"
        ::"r"(bar)
        : "memory");
}

// ----------------------------------------------------------------------------
// tcgen05: TMEM <-> registers.  Shape 32x32b: thread t of the warp addresses
// TMEM lane (lane_base + t); xN moves N consecutive 32-bit columns.
// A warp may only touch the lane quarter (warp_id % 4) * 32 .. +31.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}

// ----------------------------------------------------------------------------
// Small math helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_log2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32x2 arithmetic (two lanes per instruction on sm_100): halves the issue slots of
// the scale/subtract and row-sum steps of the softmax.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}\n"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// 2^x for two values on the FMA pipe instead of the special-function unit (16 ex2 per clock
// per SM, which a 128x128 score tile keeps busy exactly as long as its two MMAs keep the tensor
// pipe busy).  x = n + f with n = round(x) taken from the low mantissa bits of x + 1.5*2^23 and
// f in [-0.5, 0.5]; 2^f by a degree-3 minimax polynomial (relative error 7.5e-5, far below the
// bf16 rounding of the probabilities it feeds); n is then added into the exponent field.
// Inputs below -126 (including -inf) give 2^-126, which rounds away in every later sum.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    constexpr float kMagic = 12582912.f;
    x.x = fmaxf(x.x, -126.f);
    x.y = fmaxf(x.y, -126.f);
    const float2 t = add2(x, make_float2(kMagic, kMagic));
    const float2 n = add2(t, make_float2(-kMagic, -kMagic));
    const float2 f = fma2(n, make_float2(-1.f, -1.f), x);
    float2 p = fma2(f, make_float2(0.0551716648042202f, 0.0551716648042202f),
                    make_float2(0.2426111400127411f, 0.2426111400127411f));
    p = fma2(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
    p = fma2(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
    float2 r;
    r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
    r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
    return r;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <uint32_t RegCount>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(RegCount));
}

template <uint32_t RegCount>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(RegCount));
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace b2a
