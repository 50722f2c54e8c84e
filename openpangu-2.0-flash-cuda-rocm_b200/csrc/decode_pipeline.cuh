// Device-side pieces shared by the two persistent decode kernels (decode_mega.cu: one GPU; decode_ep.cu: the
// expert-parallel variant).  Both walk gate/up and down tiles of the active experts through ONE ring of weight
// stages and one tcgen05 pipeline; what is common to them lives here: the layout of a ring stage, the TMEM budget,
// the tile queue between the three roles, the device-wide counters, and the issue of one stage's products.
#pragma once

#include "p92b_common.cuh"
#include "tc_ptx.cuh"

namespace p92b {
namespace decode {

using namespace ptx;

constexpr int kTile = 128;                          // weight rows per tile (the MMA's M)
constexpr int kKB = 128;                            // bytes per operand row per K block
constexpr int kSlab = 2048;                         // one 128x4-tiled scale slab: 128 rows x 16 scales
// Every stage starts with one 36,864-byte chunk of the bank's tile stream, copied as a whole: two 16 KB weight
// boxes and their two scale slabs.  The token boxes and token scale slabs follow; their offsets depend on the
// kernel's column count and are passed in.
constexpr int kOffA0 = 0, kOffA1 = 16384, kOffSfA0 = 32768, kOffB0 = 36864;
constexpr int kStages = 4;
constexpr int kAccumStride = 32;                    // gate at +0, up at +32 inside an accumulator buffer
constexpr int kAccumCols = 64;
constexpr int kSfColsPerBuffer = 64;                // SFA0, SFA1, SFB0, SFB1 x 16 columns
constexpr int kAccumBuffers = 4;                    // the issuer may run four tiles ahead of the epilogue
constexpr int kTmemCols = 512;

// Every active slot owns one 128-row slab of the padded position space, in slot order; the shared expert
// (slot 0) takes the slab after the last routed one.
__device__ __forceinline__ int slab_of_slot(int slot, int n_active) {
    return (slot == 0 ? n_active - 1 : slot - 1) * kTile;
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// 16-byte asynchronous copy global -> shared (through the load/store unit); the kernels' prologues bring the router
// rows and the token rows in with these so that the second request does not wait for the first answer.
__device__ __forceinline__ void async_copy16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void async_copy4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void async_copies_wait() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Bounded wait (one second of wall time) until *counter has reached `target`; wrap-safe.
__device__ __forceinline__ bool wait_counter(const unsigned* counter, unsigned target) {
    const std::uint64_t start = global_timer_ns();
    while (static_cast<int>(ld_acquire_gpu(counter) - target) < 0) {
        if (global_timer_ns() - start > 1000000000ULL) return false;
    }
    return true;
}

// Tiles are handed out through one device-wide counter.  The producer lane takes the numbers (one ahead of the
// tile it is loading, so the atomic's latency is hidden) and passes each tile to the MMA lane and the epilogue
// warps through a small queue in shared memory, published by the mbarrier arrivals that already order the three
// roles.  A negative entry ends the queue.  The producer is never more than 9 tiles ahead of the epilogue.
constexpr int kTileQueue = 16;
__device__ __forceinline__ int encode_tile(int kind, int slot, int m_tile) { return (kind << 24) | (slot << 8) | m_tile; }
__device__ __forceinline__ void decode_tile(int code, int* kind, int* slot, int* m_tile) {
    *kind = code >> 24;
    *slot = (code >> 8) & 0xffff;
    *m_tile = code & 0xff;
}

// The products of one ring stage at shared-memory address `st`.  kind 0, a gate/up stage: one K block of the
// tile's gate rows and of its up rows against the token box, into the two halves of the accumulator buffer.
// kind 1, a down stage: two K blocks of the tile's rows against the two SwiGLU-row boxes, into one accumulator.
// The stage's scale slabs are copied to the TMEM columns at `sfc` first (SFA0, SFA1, SFB0 and, for a down stage,
// SFB1, 16 columns each).  `first` is true for the first stage of a tile: its first product overwrites.
__device__ __forceinline__ void issue_stage(int kind, std::uint32_t st, int off_b1, int off_sfb0, std::uint32_t sfc,
                                            std::uint32_t accum, std::uint32_t idesc, bool first) {
    const int slabs = kind == 0 ? 3 : 4;
    for (int o = 0; o < slabs; ++o) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            tc_copy_sf(sfc + o * 16 + k * 4, desc_scale_atom(st + (o < 2 ? kOffSfA0 + o * kSlab : off_sfb0 + (o - 2) * kSlab) + k * 512));
        }
    }
    const std::uint64_t a0 = desc_k_major_sw128(st + kOffA0);
    const std::uint64_t a1 = desc_k_major_sw128(st + kOffA1);
    const std::uint64_t b0 = desc_k_major_sw128(st + kOffB0);
    const std::uint64_t b1 = desc_k_major_sw128(st + off_b1);
    if (kind == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            mma_nvf4(accum, a0 + 2 * k, b0 + 2 * k, idesc, sfc + k * 4, sfc + 32 + k * 4, !first || k > 0);
            mma_nvf4(accum + kAccumStride, a1 + 2 * k, b0 + 2 * k, idesc, sfc + 16 + k * 4, sfc + 32 + k * 4, !first || k > 0);
        }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            mma_nvf4(accum, a0 + 2 * k, b0 + 2 * k, idesc, sfc + k * 4, sfc + 32 + k * 4, !first || k > 0);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            mma_nvf4(accum, a1 + 2 * k, b1 + 2 * k, idesc, sfc + 16 + k * 4, sfc + 48 + k * 4, true);
        }
    }
}

}  // namespace decode
}  // namespace p92b
