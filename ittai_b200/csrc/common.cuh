// Shared device helpers: bf16 packing, streaming loads, warp/block reductions, bounded grid barrier.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ittai_b200.h"

namespace ittai {

typedef __nv_bfloat16 bf16;

constexpr int kThreads = 512;            // threads per persistent CTA
constexpr int kWarps = kThreads / 32;
constexpr unsigned kSpinLimit = 1u << 22;  // polls before a device wait gives up (about a second)

// ---- bf16 <-> fp32 -------------------------------------------------------------------------------
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
// Round to nearest-even bf16 and widen back: the rounding step the eager modules apply after every op.
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf2f(bf16 x) { return __bfloat162float(x); }

// ---- global loads --------------------------------------------------------------------------------
// Weights: read once per token, never written while a kernel runs -> non-coherent path, no L1 allocation.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// Data other CTAs wrote earlier in the same launch (activations, KV cache, partials): L2-coherent loads.
__device__ __forceinline__ uint4 ldcg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldcg32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldcgf(const float* p) { return __uint_as_float(ldcg32(p)); }
__device__ __forceinline__ float ldcg_bf16(const bf16* p) {
    unsigned short v;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return __uint_as_float(((uint32_t)v) << 16);
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Asks L2 to fetch [p, p+bytes) from HBM; bytes and p are multiples of 16.  No shared memory, no completion wait.
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- dot products of 8 bf16 weights (one 16-byte chunk) with 8 fp32 activations ---------------------
__device__ __forceinline__ float dot8(const uint4& w, const float* x, float acc) {
    acc = fmaf(bf_lo(w.x), x[0], acc);
    acc = fmaf(bf_hi(w.x), x[1], acc);
    acc = fmaf(bf_lo(w.y), x[2], acc);
    acc = fmaf(bf_hi(w.y), x[3], acc);
    acc = fmaf(bf_lo(w.z), x[4], acc);
    acc = fmaf(bf_hi(w.z), x[5], acc);
    acc = fmaf(bf_lo(w.w), x[6], acc);
    acc = fmaf(bf_hi(w.w), x[7], acc);
    return acc;
}

// ---- reductions ----------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the CTA; every thread returns the same value (fixed summation order). `red` holds kWarps floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) t += red[i];
    __syncthreads();
    return t;
}

// ---- grid-wide synchronisation with a bounded wait -------------------------------------------------
// sync[0] arrival counter (monotonic within a launch), sync[1] abort flag.  Needs all CTAs co-resident
// (cooperative launch).  Returns false when the wait ran out or another CTA aborted; the caller must then
// leave the kernel.  The same role as the reference's arrive/ready flags (src/ittai/qwen3/base.py:42-78),
// which spin without a limit.
struct GridSync {
    uint32_t* sync;
    uint32_t* status;
    uint32_t epoch;
    uint32_t ncta;
    uint32_t limit;     // polls before giving up
};

__device__ __forceinline__ void report_status(uint32_t* status, uint32_t* sync, uint32_t code, uint32_t a, uint32_t b,
                                              uint32_t c, uint32_t d) {
    if (atomicCAS(&status[0], 0u, code) == 0u) {
        status[1] = a; status[2] = b; status[3] = c; status[4] = d;
    }
    __threadfence();
    atomicExch(&sync[1], 1u);
}

__device__ __forceinline__ bool grid_barrier(GridSync& g, int tag, int* ok_smem) {
    __syncthreads();
    g.epoch += 1;
    if (threadIdx.x == 0) {
        const uint32_t target = g.epoch * g.ncta;
        __threadfence();
        red_release_add(&g.sync[0], 1u);
        int ok = 1;
        uint32_t spins = 0, seen = 0;
        while ((seen = ld_acquire(&g.sync[0])) < target) {
            ++spins;
            if ((spins & 1023u) == 0u) {
                if (ld_relaxed(&g.sync[1]) != 0u) { ok = 0; break; }
                if (spins >= g.limit) {
                    report_status(g.status, g.sync, ITTAI_ST_BARRIER_TIMEOUT, (uint32_t)tag, blockIdx.x, seen, target);
                    ok = 0;
                    break;
                }
            }
        }
        __threadfence();
        *ok_smem = ok;
    }
    __syncthreads();
    return *ok_smem != 0;
}

}  // namespace ittai
