// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier, TMA tiled loads, tcgen05 (TMEM allocation, MMA, commit, ld) and
// the shared-memory / instruction descriptors that tcgen05.mma consumes.
//
// Everything here is device-only and header-only.  Every wait is bounded by
// wall-clock time (%globaltimer): a wait that runs out returns false so the
// caller can record a status word and leave the kernel cleanly instead of
// spinning forever on a shared GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------------------
// addresses, timers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------------------
// programmatic dependent launch
// ---------------------------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may become resident
// while the kernel before it in the stream is still running.  grid_dependency_wait() returns once
// that earlier kernel has completed and its memory is visible: nothing that it may have written
// (or may still read) is touched before this call.  Without the attribute both are no-ops.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets the next kernel of the stream (if it was launched with the attribute) start its own
// set-up; it still waits for this kernel's completion before it touches memory.
__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------
// a monotone counter in shared memory (release add / acquire load, CTA scope)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void smem_add_release(uint32_t addr, uint32_t v) {
    asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t smem_load_acquire(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

// ---------------------------------------------------------------------------
// register re-partitioning between warpgroups (four consecutive, aligned warps)
// ---------------------------------------------------------------------------
template <int kRegs>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (TMA, tcgen05.commit).
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Default budget of every device-side wait.  Far above any legitimate wait
// (a full 16384-deep mainloop is tens of milliseconds) and far below the
// watchdog of the machine.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s

// Waits for the phase with the given parity to complete.  Returns false if the
// budget ran out (nothing else is touched; the caller decides what to record).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          uint64_t budget_ns = kWaitBudgetNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (global_timer_ns() - start > budget_ns) return false;
    }
}

// ---------------------------------------------------------------------------
// thread-block clusters (CTA pairs)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Cluster-wide barrier with release/acquire ordering; every thread of every CTA calls it.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

// Arrive on a barrier that may live in another CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// try_wait that also acquires writes released by threads of the peer CTA.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Orders generic-proxy shared-memory writes (st.shared) before later reads by
// the async proxy (tcgen05.mma operand fetch, TMA stores).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA (tiled loads, never multicast)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// x is the innermost (contiguous) coordinate and must keep x * 4 bytes a
// multiple of 16.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* map,
                                            uint32_t bar, int32_t x, int32_t y, int32_t z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        :
        : "r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM allocation
// ---------------------------------------------------------------------------
// All three are warp-wide (.sync.aligned): call them from one fully converged warp.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

// The cta_group::2 forms are executed by the same warp of BOTH CTAs of a pair, with the
// same shared-memory destination offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: descriptors
// ---------------------------------------------------------------------------
// Swizzle / layout-type codes of the shared-memory matrix descriptor (bits 61..63).
constexpr uint32_t kLayoutSw128 = 2;
constexpr uint32_t kLayoutSw64 = 4;

// 64-bit shared-memory matrix descriptor.
//   bits  0..13  start address >> 4
//   bits 16..29  leading-dimension byte offset >> 4
//   bits 32..45  stride-dimension byte offset >> 4
//   bits 46..47  descriptor version (1 on sm_100)
//   bits 61..63  layout type
// For 128-byte-swizzled tiles of 32-bit elements:
//   K-major  (K contiguous): rows of 128 B (32 k), 8-row groups every `sbo` bytes,
//            `lbo` unused (encoded 16 B).
//   MN-major (M or N contiguous): one 128 B row holds 32 consecutive m (or n) of one k,
//            8 such k-rows form a 1024 B group; groups along K every `sbo` bytes,
//            the next 32 m (or n) start `lbo` bytes further.
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= static_cast<uint64_t>(layout & 7u) << 61;
    return d;
}

// 32-bit instruction descriptor for kind::tf32 with fp32 accumulation.
//   bits 4..5 D format (1 = f32); bits 7..9 / 10..12 A / B format (2 = tf32);
//   bit 15 / 16: A / B major (0 = K-major, 1 = MN-major);
//   bits 17..22 N >> 3; bits 24..28 M >> 4.
__host__ __device__ __forceinline__ uint32_t make_idesc_tf32(uint32_t m, uint32_t n,
                                                             uint32_t a_mn_major,
                                                             uint32_t b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major & 1u) << 15) |
           ((b_mn_major & 1u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// tcgen05: MMA, commit
// ---------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Pair form: one thread of the leader CTA issues an M = 256 product; each CTA of the pair
// supplies 128 rows of A and half of the columns of B from the SAME shared-memory offsets,
// and receives 128 rows of D in its own TMEM.
__device__ __forceinline__ void mma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Pair commit: arrives on the barrier at the same offset in every CTA of `cta_mask`.  (This
// is a barrier signal, not a data copy.)
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// Arrives once on `bar` when every tcgen05 operation issued so far by this
// thread has completed.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM <-> registers (32 lanes x 32 bit, warp w touches lanes 32*(w%4)..+31)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TF32 split used by the error-compensated ("3xTF32") product
// ---------------------------------------------------------------------------
// Rounds an fp32 bit pattern to the nearest TF32 value (10 explicit mantissa
// bits), ties away from zero, and clears the 13 low bits so the tensor core sees
// an exactly representable operand whatever it does with those bits.
__host__ __device__ __forceinline__ uint32_t tf32_round_bits(uint32_t x) {
    return (x + 0x1000u) & 0xFFFFE000u;
}

// x = hi + lo + r with hi, lo exactly representable in TF32 and |r| <= 2^-22 |x|.
__device__ __forceinline__ void tf32_split(float x, float& hi, float& lo) {
    hi = __uint_as_float(tf32_round_bits(__float_as_uint(x)));
    lo = __uint_as_float(tf32_round_bits(__float_as_uint(x - hi)));
}

// The tail that goes with a head the tensor core makes itself by truncation:
// x = trunc_tf32(x) + t exactly; returns t rounded to TF32 (|t| < 2^-10 |x|, error <= 2^-21 |x|).
__device__ __forceinline__ float tf32_tail_of_truncated(float x) {
    const float head = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    return __uint_as_float(tf32_round_bits(__float_as_uint(x - head)));
}

}  // namespace b200
