// Per-CTA weight stream: a FIFO ring in shared memory that TMA bulk copies fill far ahead of the phases that read it.
//
// Weights and old cache rows do not depend on the token being computed, only the small activation vectors do.  Each
// persistent CTA therefore knows, for the whole launch, the exact sequence of contiguous global-memory slices it will
// read (its rows of Wqkv, its cache tiles, its rows of Wo, Wgu, Wd, layer after layer, token after token).  One thread
// issues those slices as `cp.async.bulk` copies (no multicast, no tensor map: the slices are contiguous) into a byte
// ring, each tracked by an mbarrier; the phases consume the entries in the same order.  While a phase waits for its
// input vector, HBM keeps streaming the next phases' weights into the ring: the reference's "prefetch the next task's
// operand tiles while the current one drains" (src/ittai/qwen3/sm80.py:151-173), taken to a whole layer's depth.
//
// A seventeenth warp does nothing but issue: it walks the static sequence, waits for ring space and launches the next
// copy, so address arithmetic and allocation never sit between two phases.  Consumers release entries at points where
// all compute threads have synchronised anyway (the end of a phase or of an attention tile) by bumping one counter in
// shared memory, which the issuing lane polls.
#pragma once
#include "common.cuh"

#ifndef ITTAI_STREAM_EVICT_FIRST
#define ITTAI_STREAM_EVICT_FIRST 1
#endif

namespace ittai {

constexpr int kStreamSlots = 16;           // entries in flight at most
constexpr uint32_t kStreamAlign = 128;     // ring offsets are multiples of this

struct StreamShared {
    unsigned long long full[kStreamSlots]; // one mbarrier per in-flight entry (count 1 + transaction bytes)
    uint32_t q_off[kStreamSlots];          // ring offset of the entry
    uint32_t q_bytes[kStreamSlots];        // its size rounded up to kStreamAlign
    uint32_t issued;                       // entries issued so far (written by the issuing lane)
    uint32_t head;                         // next free ring offset (issuing lane)
    uint32_t consumed;                     // entries released so far (compute thread 0; release / acquire accesses)
    volatile uint32_t stop;                // compute threads are leaving early: issue nothing more
    uint32_t kv_epoch;                     // 1 + index (step * layers + layer) of the last attention output this CTA's compute
                                           // threads have received whole (compute thread 0; release / acquire accesses)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// The ring's space goes back to the issuing lane through `consumed`: the compute threads' reads of an entry come before
// the release store (they all passed a CTA barrier before thread 0 stores), the issuing lane's TMA write into that space
// comes after its acquire load.
__device__ __forceinline__ void st_release_cta(uint32_t* p, uint32_t v) {
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_cta(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}

__device__ __forceinline__ void mbar_init(void* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Contiguous global -> shared copy by the TMA unit; completion is counted in bytes on `bar`.  The destination is this
// CTA's own shared memory (a shared::cta address is a valid shared::cluster address of the executing CTA).
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, void* bar) {
#if ITTAI_STREAM_EVICT_FIRST
    // every streamed byte is read once per token: mark its L2 lines first in line for eviction, so that the stream does
    // not push out what is reused (flagged words, instruction lines, the other CTAs' polled partials)
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
#else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
#endif
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Orders this thread's earlier generic-proxy writes before later async-proxy (TMA) accesses to the same memory.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// Same, restricted to this CTA's shared memory: enough before a TMA store or an MMA reads what this thread just wrote there.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// The compute threads' view: ring base and the count of entries they have released (uniform over those threads).
struct Stream {
    StreamShared* sh;
    unsigned char* ring;     // ring base in shared memory
    uint32_t ring_bytes;
    uint32_t consumed;
};

__device__ __forceinline__ void stream_init(Stream& s, int tid) {
    if (tid == 0) {
        for (int i = 0; i < kStreamSlots; ++i) mbar_init(&s.sh->full[i], 1);
        s.sh->issued = 0;
        s.sh->head = 0;
        s.sh->consumed = 0;
        s.sh->stop = 0;
        s.sh->kv_epoch = 0;
        fence_mbar_init();
    }
    __syncthreads();        // all kBlock threads: both roles see the initialised barriers
}

// Issuing lane: find room for `bytes` (no entry wraps around the end of the ring).  Returns false when the ring is full.
__device__ __forceinline__ bool stream_alloc(const Stream& s, uint32_t bytes, uint32_t& off) {
    StreamShared* sh = s.sh;
    const uint32_t consumed = ld_acquire_cta(&sh->consumed);
    if (sh->issued - consumed >= (uint32_t)kStreamSlots) return false;
    if (sh->issued == consumed) { off = 0; return bytes <= s.ring_bytes; }   // empty: restart at the base
    const uint32_t tail = sh->q_off[consumed % kStreamSlots];
    const uint32_t head = sh->head;
    if (head > tail) {
        if (bytes <= s.ring_bytes - head) { off = head; return true; }
        if (bytes < tail) { off = 0; return true; }
        return false;
    }
    if (head < tail && bytes < tail - head) { off = head; return true; }
    return false;
}

// Issuing lane: launch one entry.
__device__ __forceinline__ void stream_issue(const Stream& s, uint32_t off, const void* src, uint32_t bytes) {
    StreamShared* sh = s.sh;
    const uint32_t slot = sh->issued % kStreamSlots;
    const uint32_t padded = (bytes + kStreamAlign - 1) / kStreamAlign * kStreamAlign;
    sh->q_off[slot] = off;
    sh->q_bytes[slot] = padded;
    sh->head = off + padded;
    mbar_expect_tx(&sh->full[slot], bytes);
    bulk_g2s(s.ring + off, src, bytes, &sh->full[slot]);
    sh->issued += 1;
}

// Compute threads: wait until entry number `n` (n >= consumed) has landed; returns its address or nullptr on a timeout.
__device__ __forceinline__ const unsigned char* stream_wait(const Stream& s, uint32_t n, const Waiter& w) {
    const uint32_t slot = n % kStreamSlots, parity = (n / kStreamSlots) & 1u;
    uint32_t spins = 0;
    while (!mbar_try_wait(&s.sh->full[slot], parity)) {
        if (((++spins) & 1023u) == 0u) {
            if (ld_relaxed(&w.sync[1]) != 0u) return nullptr;
            if (spins >= w.limit) {
                report_status(w.status, w.sync, ITTAI_ST_STREAM_TIMEOUT, n, blockIdx.x, slot, parity);
                return nullptr;
            }
        }
    }
    return s.ring + s.sh->q_off[slot];
}

// Compute threads: everyone has finished reading the `n` oldest entries; hand their space back to the issuing lane.
__device__ __forceinline__ void stream_release(Stream& s, int n) {
    cta_sync();
    s.consumed += (uint32_t)n;
    if (threadIdx.x == 0) st_release_cta(&s.sh->consumed, s.consumed);
}

// Issuing lane, before it exits: let every copy it launched land (bounded), so none is in flight when the CTA retires.
__device__ __forceinline__ void stream_drain(const Stream& s, uint32_t limit) {
    const uint32_t issued = s.sh->issued;
    const uint32_t first = issued > (uint32_t)kStreamSlots ? issued - kStreamSlots : 0;
    for (uint32_t n = first; n < issued; ++n) {
        const uint32_t slot = n % kStreamSlots, parity = (n / kStreamSlots) & 1u;
        uint32_t spins = 0;
        while (!mbar_try_wait(&s.sh->full[slot], parity) && ++spins < limit) {}
    }
}

}  // namespace ittai
