// Shared by the two-SM GEMM kernels (gemm2_sm100.cu: one GEMM per launch; gemm2_chain_sm100.cu: a chain of dependent
// GEMMs in one persistent launch): tile geometry, shared-memory plan and the cta_group::2 / cluster helpers.
#pragma once
#include <cuda.h>

#include "gemm_epilogue.cuh"
#include "tmap.h"
#include "launch.h"

namespace ittai {

constexpr int PM = 256, PN = 256, PK = 64;   // pair tile
#ifndef ITTAI_GEMM2_STAGES
#define ITTAI_GEMM2_STAGES 5
#endif
constexpr int kStages2 = ITTAI_GEMM2_STAGES;                       // 4, 5 and 6 stages measured the same: the main loop is supply-bound
constexpr int kEpiWarps = 8;                      // 2 warps per TMEM lane quarter (16 warps were slower: the epilogue is
                                                  // bound by the conversion pipe and shared memory, not by latency)
constexpr int kEpiCols = PN / (kEpiWarps / 4);    // accumulator columns per epilogue warp
constexpr int kThreads2 = 64 + 32 * kEpiWarps;
static_assert(kEpiCols == 128, "stats_out slots and the bias / column-sum slices assume 128 columns per epilogue warp");
constexpr uint32_t kHalfA = 128 * PK * 2, kHalfB = 128 * PK * 2;                // per CTA per stage
constexpr uint32_t kStageOut = 3 * 2048;                                         // per epilogue warp: three tiles of 32 rows x 64 B
constexpr uint32_t kSmem2 = kStages2 * (kHalfA + kHalfB) + kEpiWarps * kStageOut + 2 * 4096 /*bias and column-sum slices*/ + 1024 /*alignment*/ + 512 /*barriers*/;
constexpr uint32_t kSpin2 = 1u << 24;
// tile order: N fastest (M-fastest measured the same)
#define TILE_M(t) ((t) / tiles_n)
#define TILE_N(t) ((t) % tiles_n)
constexpr uint32_t kTmemCols2 = 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Address of the same shared-memory object in CTA `rank` of the cluster, in the cluster's shared window.
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
    return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load into this CTA's shared memory whose completion bytes are counted on a barrier that may live in the
// peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const void* tmap, int x, int y, uint32_t bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(void* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs once every MMA issued so far has finished.
__device__ __forceinline__ void umma_commit_pair(void* bar) {
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}

}  // namespace ittai
