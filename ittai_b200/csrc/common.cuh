// Shared device helpers: bf16 packing, streaming loads, warp/block reductions, bounded grid barrier.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ittai_b200.h"

namespace ittai {

typedef __nv_bfloat16 bf16;

constexpr int kThreads = 512;            // compute threads per persistent CTA
constexpr int kWarps = kThreads / 32;
constexpr int kBlock = kThreads + 32;    // plus one warp that only feeds the weight stream
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
// Packed fp32 FMAs (two multiply-adds per instruction): even and odd elements accumulate separately and meet at the end.
__device__ __forceinline__ float dot8(const uint4& w, const float* x, float acc) {
    float2 a = make_float2(acc, 0.f);
    a = __ffma2_rn(make_float2(bf_lo(w.x), bf_hi(w.x)), make_float2(x[0], x[1]), a);
    a = __ffma2_rn(make_float2(bf_lo(w.y), bf_hi(w.y)), make_float2(x[2], x[3]), a);
    a = __ffma2_rn(make_float2(bf_lo(w.z), bf_hi(w.z)), make_float2(x[4], x[5]), a);
    a = __ffma2_rn(make_float2(bf_lo(w.w), bf_hi(w.w)), make_float2(x[6], x[7]), a);
    return a.x + a.y;
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
// Barrier over the kThreads compute threads only (named barrier 1): the stream-feeding warp never joins it.
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }
// The same barrier, returning the OR of `pred` over the compute threads.
__device__ __forceinline__ bool cta_or(bool pred) {
    uint32_t r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %1, 0;\n"
        "bar.red.or.pred p, 1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r) : "r"((uint32_t)pred), "n"(kThreads) : "memory");
    return r != 0;
}
// Sum over the compute threads; every thread returns the same value (fixed summation order). `red` holds kWarps floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    cta_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) t += red[i];
    cta_sync();
    return t;
}

// ---- flagged words: payload + tag in one 64-bit word -------------------------------------------------------
// The role of the reference's arrive/ready flags (src/ittai/qwen3/base.py:42-78), which spin without a limit; here
// the flag travels with the data and every wait is bounded.
__device__ __forceinline__ uint64_t ld_flagged(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_flagged(uint64_t* p, uint32_t payload, uint32_t tag) {
    const uint64_t v = ((uint64_t)tag << 32) | payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// 128-bit flagged words: three 32-bit payloads + the tag, moved by single-copy-atomic .b128 accesses.  They carry the
// vectors whose consumers would otherwise poll several 64-bit words one after the other.
__device__ __forceinline__ void ld_flagged128(const void* p, uint64_t& lo, uint64_t& hi) {
    asm volatile("{\n.reg .b128 t;\nld.relaxed.gpu.global.b128 t, [%2];\nmov.b128 {%0, %1}, t;\n}\n" : "=l"(lo), "=l"(hi) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_flagged128(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t tag) {
    const uint64_t lo = ((uint64_t)b << 32) | a, hi = ((uint64_t)tag << 32) | c;
    asm volatile("{\n.reg .b128 t;\nmov.b128 t, {%1, %2};\nst.relaxed.gpu.global.b128 [%0], t;\n}\n" ::"l"(p), "l"(lo), "l"(hi) : "memory");
}
// Two floats -> packed bf16 pair (round to nearest even), one conversion instruction.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// The same roundings on the integer pipe, for code whose conversion pipe is the bottleneck (it shares a quarter-rate
// unit with ex2 / tanh).  bf16r_bits: fp32 bits rounded to nearest-even bf16, still as fp32 bits (finite inputs).
__device__ __forceinline__ uint32_t bf16r_bits(uint32_t u) { return (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u; }
// Two non-negative finite floats -> packed bf16 pair, round half up (differs from nearest-even only on exact ties).
__device__ __forceinline__ uint32_t pack_bf16x2_alu(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo) + 0x8000u, __float_as_uint(hi) + 0x8000u, 0x7632);
}

// Programmatic dependent launch (see launch.h): let the next kernel of the stream start launching / wait until every
// kernel this one depends on has completed and its writes are visible.  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct Waiter {
    uint32_t* sync;     // sync[1] = abort flag
    uint32_t* status;
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

// The slow side of a poll loop, entered once per 1024 polls: has another CTA aborted, has this wait run out?  Inlined on
// purpose: as a real call (arguments by value, cold path only) it cost 20 us per decoded token on a B200, the call's
// register constraints reaching into the hot loops around it.
static __device__ __forceinline__ bool keep_waiting(uint32_t* sync, uint32_t* status, uint32_t limit, uint32_t spins, int what,
                                                    uint32_t seen, uint32_t tag) {
    if (ld_relaxed(&sync[1]) != 0u) return false;
    if (spins >= limit) {
        report_status(status, sync, ITTAI_ST_FLAG_TIMEOUT, (uint32_t)what, blockIdx.x, seen, tag);
        return false;
    }
    return true;
}

// Polls one word until its tag matches; returns false when the wait ran out or another CTA aborted.
__device__ __forceinline__ bool wait_word(const Waiter& w, const uint64_t* p, uint32_t tag, uint32_t& payload, int what) {
    uint32_t spins = 0;
    for (;;) {
        const uint64_t v = ld_flagged(p);
        if ((uint32_t)(v >> 32) == tag) { payload = (uint32_t)v; return true; }
        if (((++spins) & 1023u) == 0u && !keep_waiting(w.sync, w.status, w.limit, spins, what, (uint32_t)(v >> 32), tag)) return false;
    }
}


// The same for a 128-bit word: payloads a, b, c.
__device__ __forceinline__ bool wait_word128(const Waiter& w, const void* p, uint32_t tag, uint32_t& a, uint32_t& b, uint32_t& c, int what) {
    uint32_t spins = 0;
    for (;;) {
        uint64_t lo, hi;
        ld_flagged128(p, lo, hi);
        if ((uint32_t)(hi >> 32) == tag) { a = (uint32_t)lo; b = (uint32_t)(lo >> 32); c = (uint32_t)hi; return true; }
        if (((++spins) & 1023u) == 0u && !keep_waiting(w.sync, w.status, w.limit, spins, what, (uint32_t)(hi >> 32), tag)) return false;
    }
}


// NB words, `stride` words apart, polled together: all loads of a sweep are in flight at once, so a thread that needs NB
// words pays about one L2 round trip instead of NB of them.  (At NB = 1 this is wait_word.)
template <int NB>
__device__ __forceinline__ bool wait_words(const Waiter& w, const uint64_t* p, size_t stride, uint32_t tag, uint32_t (&payload)[NB], int what) {
    if constexpr (NB == 1) {
        return wait_word(w, p, tag, payload[0], what);
    } else {
        uint32_t spins = 0;
        for (;;) {
            uint64_t v[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) v[b] = ld_flagged(p + (size_t)b * stride);
            bool all = true;
            uint32_t seen = tag;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if ((uint32_t)(v[b] >> 32) != tag) { all = false; seen = (uint32_t)(v[b] >> 32); }
                payload[b] = (uint32_t)v[b];
            }
            if (all) return true;
            if (((++spins) & 1023u) == 0u && !keep_waiting(w.sync, w.status, w.limit, spins, what, seen, tag)) return false;
        }
    }
}

// The same for 128-bit words, `stride` 16-byte words apart: payloads a[b], b2[b], c[b].
template <int NB>
__device__ __forceinline__ bool wait_words128(const Waiter& w, const uint4* p, size_t stride, uint32_t tag, uint32_t (&a)[NB], uint32_t (&b2)[NB],
                                              uint32_t (&c)[NB], int what) {
    if constexpr (NB == 1) {
        return wait_word128(w, p, tag, a[0], b2[0], c[0], what);
    } else {
        uint32_t spins = 0;
        for (;;) {
            uint64_t lo[NB], hi[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) ld_flagged128(p + (size_t)b * stride, lo[b], hi[b]);
            bool all = true;
            uint32_t seen = tag;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if ((uint32_t)(hi[b] >> 32) != tag) { all = false; seen = (uint32_t)(hi[b] >> 32); }
                a[b] = (uint32_t)lo[b]; b2[b] = (uint32_t)(lo[b] >> 32); c[b] = (uint32_t)hi[b];
            }
            if (all) return true;
            if (((++spins) & 1023u) == 0u && !keep_waiting(w.sync, w.status, w.limit, spins, what, seen, tag)) return false;
        }
    }
}

}  // namespace ittai
