// Thin inline-PTX wrappers for the sm_100a features the tensor-core expert
// kernels use: mbarrier, TMA (tiled and untiled bulk copies, each to one thread block only),
// tcgen05 (TMEM allocation, block-scaled MMA, SMEM->TMEM scale copies, TMEM
// loads, commit) and the two shared-memory descriptor forms they need.
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include <cstdint>

namespace p92b::ptx {

__device__ __forceinline__ std::uint32_t smem_u32(const void* p) {
    return static_cast<std::uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    std::uint32_t pred;
    asm volatile(
        "{ .reg .pred p;\n"
        "  elect.sync _|p, 0xffffffff;\n"
        "  selp.u32 %0, 1, 0, p; }\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- programmatic dependent launch ---------------------------------------------
// No-ops unless the kernel was launched with the programmatic-stream-serialization attribute.
// pdl_wait: blocks until the preceding kernel in the stream has completed and its writes are visible.
// pdl_launch_dependents: lets the next kernel in the stream start its prologue now.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(std::uint32_t bar, std::uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(std::uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(std::uint32_t bar, std::uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(std::uint32_t bar, std::uint32_t parity) {
    std::uint32_t done;
    asm volatile(
        "{ .reg .pred p;\n"
        "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "  selp.u32 %0, 1, 0, p; }\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ std::uint64_t global_timer_ns() {
    std::uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after about one second of wall time, so a protocol error
// ends the kernel with a status word instead of a hang.
__device__ __forceinline__ bool mbar_wait(std::uint32_t bar, std::uint32_t parity) {
    for (int i = 0; i < 64; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    const std::uint64_t start = global_timer_ns();
    while (true) {
        for (int i = 0; i < 256; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (global_timer_ns() - start > 1000000000ULL) return false;
    }
}

// ---- tagged words ----------------------------------------------------------------
// Data handed from one block (or one GPU) to another without a barrier or a fence: every word is
// 8 bytes, {4 bytes of payload, the number of the launch it belongs to}, stored and loaded as ONE
// access, and the reader polls the word itself until the number is the one it waits for.  The loads
// carry no memory clobber so that a caller can request many words before looking at the first.
__device__ __forceinline__ void st_tagged(void* p, std::uint32_t payload, std::uint32_t tag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_tagged(const void* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// Two neighbouring words: (payload, tag, payload, tag).
__device__ __forceinline__ uint4 ld_tagged_pair(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Bounded polls: false after about a second of wall time.
__device__ __forceinline__ bool poll_expired(std::uint64_t start) { return global_timer_ns() - start > 1000000000ULL; }
__device__ __forceinline__ bool poll_tagged(const void* p, std::uint32_t tag, std::uint32_t* payload) {
    uint2 v = ld_tagged(p);
    if (v.y != tag) {
        const std::uint64_t start = global_timer_ns();
        do {
            if (poll_expired(start)) return false;
            v = ld_tagged(p);
        } while (v.y != tag);
    }
    *payload = v.x;
    return true;
}
__device__ __forceinline__ bool poll_tagged_pair(const void* p, std::uint32_t tag, std::uint32_t* first, std::uint32_t* second) {
    uint4 v = ld_tagged_pair(p);
    if (v.y != tag || v.w != tag) {
        const std::uint64_t start = global_timer_ns();
        do {
            if (poll_expired(start)) return false;
            v = ld_tagged_pair(p);
        } while (v.y != tag || v.w != tag);
    }
    *first = v.x;
    *second = v.z;
    return true;
}

// ---- TMA ----------------------------------------------------------------------
// The innermost coordinate x must be a multiple of 16 bytes' worth of elements;
// every call site passes multiples of 128 bytes.
__device__ __forceinline__ void tma_load_2d(std::uint32_t dst, const CUtensorMap* map, std::uint32_t bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Untiled bulk copy: both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(std::uint32_t dst, const void* src, std::uint32_t bytes, std::uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// The same with an L2 policy: weights that are read once per launch are marked "evict first", so a
// 120 MB stream does not push everything else (code, routing tables, token rows) out of the L2.
__device__ __forceinline__ std::uint64_t l2_policy_evict_first() {
    std::uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_load_hint(std::uint32_t dst, const void* src, std::uint32_t bytes, std::uint32_t bar,
                                               std::uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}


__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tcgen05 --------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(std::uint32_t smem_slot, std::uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(std::uint32_t addr, std::uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrives on the mbarrier once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(std::uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], E2M1 operands with one UE4M3 scale per 16
// elements along K (scale factors in TMEM), M=128, K=64 per instruction.
__device__ __forceinline__ void mma_nvf4(std::uint32_t d_tmem, std::uint64_t a_desc, std::uint64_t b_desc,
                                         std::uint32_t idesc, std::uint32_t sfa_tmem, std::uint32_t sfb_tmem,
                                         bool accumulate) {
    asm volatile(
        "{ .reg .pred p;\n"
        "  setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p; }\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<std::uint32_t>(accumulate)),
          "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, broadcast to the four 32-lane quarters.
__device__ __forceinline__ void tc_copy_sf(std::uint32_t tmem, std::uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem), "l"(smem_desc) : "memory");
}

// 16 consecutive 32-bit columns of this warp's 32 TMEM lanes.
__device__ __forceinline__ void tmem_load16(std::uint32_t addr, std::uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors -------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit): start address >> 4 in bits [0,14),
// leading byte offset >> 4 in [16,30), stride byte offset >> 4 in [32,46),
// descriptor version 1 in [46,48), swizzle mode in [61,64) (0 none, 2 = 128 B).

// K-major operand tile whose rows are 128 bytes, written by TMA with the 128-byte
// swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ std::uint64_t desc_k_major_sw128(std::uint32_t smem_addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((smem_addr >> 4) & 0x3fffU);
    d |= static_cast<std::uint64_t>(1U) << 16;                  // leading offset: unused with swizzle, canonical 1
    d |= static_cast<std::uint64_t>(1024U >> 4) << 32;          // stride between 8-row groups
    d |= static_cast<std::uint64_t>(1U) << 46;
    d |= static_cast<std::uint64_t>(2U) << 61;
    return d;
}

// Scale-factor atom for tcgen05.cp 32x128b: 32 rows of 16 bytes, unswizzled,
// 8-row groups 128 bytes apart.
__device__ __forceinline__ std::uint64_t desc_scale_atom(std::uint32_t smem_addr) {
    std::uint64_t d = 0;
    d |= static_cast<std::uint64_t>((smem_addr >> 4) & 0x3fffU);
    d |= static_cast<std::uint64_t>(128U >> 4) << 32;
    d |= static_cast<std::uint64_t>(1U) << 46;
    return d;
}

// Instruction descriptor for kind::mxf4nvf4.block_scale: E2M1 A and B (format 1,
// bits [7,10) and [10,13)), both K-major, N >> 3 in [17,23), UE4M3 scales (bit 23 = 0),
// M >> 4 in [24,29), scale-factor ids 0.
__host__ __device__ constexpr std::uint32_t idesc_nvf4(int m, int n) {
    return (1U << 7) | (1U << 10) | (static_cast<std::uint32_t>(n >> 3) << 17) |
           (static_cast<std::uint32_t>(m >> 4) << 24);
}

}  // namespace p92b::ptx
