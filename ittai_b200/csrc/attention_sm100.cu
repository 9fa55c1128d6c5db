// Dense attention for short sequences (SigLIP: 196 tokens, head_dim 64) on tcgen05: S = Q K^T and O = P V are
// tensor-memory MMAs, one CTA per (sequence, head, tile of 128 query rows), two CTAs resident per SM.  The reference's
// attention task (src/ittai/siglip/kernel.py:366-500) keeps Q resident and streams K/V blocks through mma.sync; with at
// most 224 keys the whole of K and V fits in shared memory, so here there is no key loop at all: one 128 x N x 64 score
// MMA, a two-pass softmax read straight from TMEM, P written back to TMEM as packed bf16 (the A operand of the second
// MMA is read from tensor memory), one 128 x 64 x N PV MMA whose B operand is V exactly as TMA loaded it (MN-major).
//
// Roles: warp 0 (one lane) issues the TMA loads and every MMA.  Warps 1-8 are the softmax: two warps per TMEM lane
// quarter, one thread per query row, each taking half of the score columns (they exchange the row maximum and the row
// sum through shared memory) and half of the output columns.
// TMEM (256 columns): S in 0..223; P for keys 0..111 in columns 0..55 and for keys 112..223 in columns 112..167, each
// written behind the reads of the warp that owns those score columns; O in columns 192..255 once S has been consumed.
// Every wait is an mbarrier wait with a bound; on expiry the abort flag routes all roles to the common exit, where
// TMEM is freed.
#include "tcgen05.cuh"
#include "tmap.h"
#include "launch.h"

namespace ittai {

constexpr int kTcKeys = 224;                 // most keys per sequence (score columns; a multiple of 16)
constexpr int kTcHalf = 112;                 // score columns per softmax warp
constexpr int kTcHD = 64;
constexpr int kTcThreads = 288;              // 1 issuing warp + 8 softmax warps
constexpr uint32_t kTcCols = 256;
constexpr uint32_t kTcOCol = 192;
constexpr uint32_t kTcSpin = 1u << 22;
// shared-memory plan (bytes, every region 1024-aligned)
constexpr uint32_t kOffQ = 0;                // [128 rows][128 B]; reused as the output staging tile
constexpr uint32_t kOffK = 16384;            // [224 rows][128 B]
constexpr uint32_t kOffV = kOffK + kTcKeys * 128;
constexpr uint32_t kOffBar = kOffV + kTcKeys * 128;
constexpr uint32_t kOffX = kOffBar + 128;    // float [2 stats][2 halves][128 rows]
constexpr uint32_t kTcSmem = kOffX + 2048 + 1024;

struct AttnTcArgs {
    const int4* seqs;
    bf16* o;
    long long o_row, o_head;
    int group;
    float scale_log2;
    uint32_t* status;
};

__device__ __forceinline__ void mbar_arrive_cta(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait_abortable(void* bar, uint32_t parity, volatile uint32_t* abort_flag) {
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kTcSpin)) { *abort_flag = 1; return false; }
    }
    return true;
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// TMEM column of the packed P chunk that holds keys c0 .. c0+15
__device__ __forceinline__ uint32_t p_col(int c0) { return c0 < kTcHalf ? (uint32_t)(c0 >> 1) : (uint32_t)(kTcHalf + ((c0 - kTcHalf) >> 1)); }

__global__ void __launch_bounds__(kTcThreads, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const AttnTcArgs a) {
    pdl_trigger();
    const int head = blockIdx.x, mt = blockIdx.y, kvh = head / a.group;
    const int4 sinfo = a.seqs[blockIdx.z];                 // written by the host long before: safe ahead of pdl_wait
    const int q_len = sinfo.y, kv_len = sinfo.w;
    if (mt * 128 >= q_len) return;                         // the whole CTA: nothing allocated yet

    extern __shared__ __align__(1024) unsigned char tc_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sm + kOffBar);
    unsigned long long* bar_load = bars;          // Q and K landed
    unsigned long long* bar_v = bars + 5;         // V landed
    unsigned long long* bar_s = bars + 1;         // S ready
    unsigned long long* bar_mx = bars + 2;        // partial row maxima posted (256 arrivals)
    unsigned long long* bar_p = bars + 3;         // P written (256 arrivals)
    unsigned long long* bar_o = bars + 4;         // O ready
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* xmax = reinterpret_cast<float*>(sm + kOffX);    // [half][row]
    float* xsum = xmax + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_keys = max(16, (kv_len + 15) & ~15);       // score columns / keys the MMAs cover

    if (threadIdx.x == 0) {
        mbar_init(bar_load, 1); mbar_init(bar_s, 1); mbar_init(bar_mx, 256); mbar_init(bar_p, 256); mbar_init(bar_o, 1);
        mbar_init(bar_v, 1);
        *abort_flag = 0;
        fence_mbar_init();
        // the loads start before TMEM is allocated; nobody else touches the barriers until the CTA-wide sync below
        pdl_wait();                                        // Q, K, V come from the kernel before this one
        mbar_expect_tx(bar_load, 128 * 128 + kTcKeys * 128);
        tma_load_2d(sm + kOffQ, &tm_q, head * kTcHD, sinfo.x + mt * 128, bar_load);
        tma_load_2d(sm + kOffK, &tm_k, kvh * kTcHD, sinfo.z, bar_load);
        mbar_expect_tx(bar_v, kTcKeys * 128);
        tma_load_2d(sm + kOffV, &tm_v, kvh * kTcHD, sinfo.z, bar_v);
    }
    if (warp == 0) { __syncwarp(); tmem_alloc(tmem_slot, kTcCols); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = mbar_wait_abortable(bar_load, 0, abort_flag);
            if (ok) {
                // ---- S = Q K^T: 4 k-steps of 16 head dims
                tc_fence_after();
                const uint32_t idesc_s = umma_idesc_bf16(128, n_keys);
                const uint64_t dq = umma_desc_sw128(sm + kOffQ), dk = umma_desc_sw128(sm + kOffK);
#pragma unroll
                for (int k = 0; k < kTcHD / 16; ++k) umma_bf16(tmem_base, dq + 2 * k, dk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(bar_s);
                ok = mbar_wait_abortable(bar_v, 0, abort_flag) && mbar_wait_abortable(bar_p, 0, abort_flag);
            }
            if (ok) {
                // ---- O = P V: P from tensor memory, V rows (keys) 16 at a time
                tc_fence_after();
                constexpr uint32_t idesc_o = umma_idesc_bf16(128, kTcHD) | umma_idesc_b_mn;
                const uint64_t dv = umma_desc_sw128(sm + kOffV);
#pragma unroll 1
                for (int ks = 0; ks < n_keys / 16; ++ks)
                    umma_bf16_tmem_a(tmem_base + kTcOCol, tmem_base + p_col(16 * ks), dv + (uint64_t)ks * (2048 >> 4), idesc_o, ks > 0 ? 1u : 0u);
                umma_commit(bar_o);
            }
        }
    } else do {
        const int hf = (warp - 1) >> 2;                      // which half of the score columns / of the output
        const int q4 = warp & 3;                             // TMEM lane quarter this warp may touch
        const int r = q4 * 32 + lane;                        // query row inside the tile
        const bool live = mt * 128 + q4 * 32 < q_len;        // a warp whose 32 rows are all padding skips the arithmetic
        bool ok = mbar_wait_abortable(bar_s, 0, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const int c_lo = hf * kTcHalf, c_hi = min(c_lo + kTcHalf, n_keys);
        // Both passes walk this warp's score columns 16 at a time with the next chunk's TMEM load in flight.
        // ---- pass 1: row maximum
        float mx = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;   // four chains: the row maximum is latency-bound
        auto take_max = [&](const uint32_t (&v)[16], int c0) {
            if (c0 + 16 <= kv_len) {
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    mx = fmaxf(mx, __uint_as_float(v[i])); mx1 = fmaxf(mx1, __uint_as_float(v[i + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(v[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(v[i + 3]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) if (c0 + i < kv_len) mx = fmaxf(mx, __uint_as_float(v[i]));
            }
        };
        if (live && c_lo < c_hi) {
            uint32_t va[16], vb[16];
            tmem_ld_32x16(t_row + c_lo, va);
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
                tmem_ld_wait16(va);
                if (c0 + 16 < c_hi) tmem_ld_32x16(t_row + c0 + 16, vb);
                take_max(va, c0);
                if (c0 + 16 >= c_hi) break;
                tmem_ld_wait16(vb);
                if (c0 + 32 < c_hi) tmem_ld_32x16(t_row + c0 + 32, va);
                take_max(vb, c0 + 16);
            }
        }
        mx = fmaxf(fmaxf(mx, mx1), fmaxf(mx2, mx3));
        xmax[hf * 128 + r] = mx;
        mbar_arrive_cta(bar_mx);
        ok = mbar_wait_abortable(bar_mx, 0, abort_flag) && mbar_wait_abortable(bar_v, 0, abort_flag);
        if (!ok) break;
        mx = fmaxf(mx, xmax[(hf ^ 1) * 128 + r]);
        // keys between the sequence's end and the MMA's K extent belong to a neighbour: zero those V rows so that
        // 0 * V stays 0 whatever they hold
        {
            const int t = threadIdx.x - 32;
            if (t < (n_keys - kv_len) * 8) *reinterpret_cast<uint4*>(sm + kOffV + (kv_len + (t >> 3)) * 128 + (t & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        const float mb = (mx == -INFINITY ? 0.f : mx) * a.scale_log2;
        // ---- pass 2: p = 2^(s * scale - max), row sum, packed bf16 P back into tensor memory
        float l0 = 0.f, l1 = 0.f;
        auto emit_p = [&](const uint32_t (&v)[16], int c0) {
            float p[16];
            uint32_t w[8];
            if (c0 + 16 <= kv_len) {
#pragma unroll
                for (int i = 0; i < 16; ++i) p[i] = ex2_fast(fmaf(__uint_as_float(v[i]), a.scale_log2, -mb));
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) p[i] = c0 + i < kv_len ? ex2_fast(fmaf(__uint_as_float(v[i]), a.scale_log2, -mb)) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 16; i += 2) { l0 += p[i]; l1 += p[i + 1]; w[i >> 1] = pack_bf16x2_alu(p[i], p[i + 1]); }
            tmem_st_32x8(t_row + p_col(c0), w);
        };
        if (live && c_lo < c_hi) {
            uint32_t va[16], vb[16];
            tmem_ld_32x16(t_row + c_lo, va);
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
                tmem_ld_wait16(va);
                if (c0 + 16 < c_hi) tmem_ld_32x16(t_row + c0 + 16, vb);
                emit_p(va, c0);
                if (c0 + 16 >= c_hi) break;
                tmem_ld_wait16(vb);
                if (c0 + 32 < c_hi) tmem_ld_32x16(t_row + c0 + 32, va);
                emit_p(vb, c0 + 16);
            }
            tmem_st_wait();
        }
        xsum[hf * 128 + r] = l0 + l1;
        fence_proxy_async();                     // the zeroed V rows were ordinary stores; the MMA reads them through the async proxy
        tc_fence_before();
        mbar_arrive_cta(bar_p);
        // ---- epilogue: this warp's 32 output columns, O / rowsum -> bf16 -> staging tile -> 64-byte row pieces
        ok = mbar_wait_abortable(bar_o, 0, abort_flag);      // O follows everyone's arrival on bar_p, which follows their sums
        if (!ok) break;
        tc_fence_after();
        const float l = (l0 + l1) + xsum[(hf ^ 1) * 128 + r];
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        if (live) {
            uint32_t v[32];
            tmem_ld_32x32(t_row + kTcOCol + 32 * hf, v);
            tmem_ld_wait();
            unsigned char* stage = sm + kOffQ + r * 128;         // Q is dead: both MMAs that read it have completed
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(stage + (((4 * hf + j) ^ (r & 7)) << 4)) =
                    make_uint4(pack_bf16x2(__uint_as_float(v[8 * j]) * inv, __uint_as_float(v[8 * j + 1]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * j + 2]) * inv, __uint_as_float(v[8 * j + 3]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * j + 4]) * inv, __uint_as_float(v[8 * j + 5]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * j + 6]) * inv, __uint_as_float(v[8 * j + 7]) * inv));
            __syncwarp();
            // 4 lanes per row, 8 rows per instruction: every store covers whole 32-byte sectors
            const int sub = lane & 3;
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int rr = q4 * 32 + it * 8 + (lane >> 2), row = mt * 128 + rr;
                const uint4 val = *reinterpret_cast<const uint4*>(sm + kOffQ + rr * 128 + (((4 * hf + sub) ^ (rr & 7)) << 4));
                if (row < q_len)
                    *reinterpret_cast<uint4*>(a.o + (long long)(sinfo.x + row) * a.o_row + (long long)head * a.o_head + 32 * hf + 8 * sub) = val;
            }
        }
    } while (false);
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (atomicCAS(&a.status[0], 0u, (uint32_t)ITTAI_ST_GEMM_TIMEOUT) == 0u) { a.status[1] = blockIdx.x; a.status[2] = blockIdx.z; }
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
        __syncthreads();
    }
    if (warp == 0) { __syncwarp(); tmem_dealloc(tmem_base, kTcCols); }
}

int cuda_fail(cudaError_t e, const char* what);

// Whether the tensor-memory kernel covers this call: dense, head_dim 64, heads contiguous in a row, all sequences in one
// packed matrix, at most 256 queries and 224 keys per sequence.
bool attn_tc_supported(const IttaiAttention* p) {
    return p->head_dim == 64 && !p->causal && p->status != nullptr && p->max_q_len > 64 && p->max_q_len <= 256 &&
           p->max_kv_len > 0 && p->max_kv_len <= kTcKeys && p->k_seq == 0 && p->v_seq == 0 && p->q_head == 64 &&
           p->k_head == 64 && p->v_head == 64 && p->q_rows_total > 0 && p->kv_rows_total > 0 &&
           ((uintptr_t)p->q & 15) == 0 && ((uintptr_t)p->k & 15) == 0 && ((uintptr_t)p->v & 15) == 0;
}

int attn_tc_launch(const IttaiAttention* p, cudaStream_t st) {
    CUtensorMap tq, tk, tv;
    const int kv_heads = p->n_heads / p->group;
    int rc = make_tmap_bf16(&tq, p->q, p->q_rows_total, (long long)p->n_heads * 64, p->q_row, 128);
    if (rc == ITTAI_OK) rc = make_tmap_bf16(&tk, p->k, p->kv_rows_total, (long long)kv_heads * 64, p->k_row, kTcKeys);
    if (rc == ITTAI_OK) rc = make_tmap_bf16(&tv, p->v, p->kv_rows_total, (long long)kv_heads * 64, p->v_row, kTcKeys);
    if (rc != ITTAI_OK) return rc;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attn_tc_kernel)");
        attr_dev = dev;
    }
    AttnTcArgs a;
    a.seqs = reinterpret_cast<const int4*>(p->seqs);
    a.o = reinterpret_cast<bf16*>(p->o);
    a.o_row = p->o_row; a.o_head = p->o_head;
    a.group = p->group;
    a.scale_log2 = 1.4426950408889634f / 8.0f;
    a.status = p->status;
    const cudaError_t e = launch_pdl(attn_tc_kernel, dim3(p->n_heads, (p->max_q_len + 127) / 128, p->n_seqs), dim3(kTcThreads), kTcSmem, st, 1, tq, tk, tv, a);
    return e == cudaSuccess ? ITTAI_OK : cuda_fail(e, "launch attn_tc_kernel");
}

}  // namespace ittai
