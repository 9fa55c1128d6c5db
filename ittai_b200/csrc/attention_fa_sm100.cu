// Flash attention with a key loop on tcgen05, head_dim 128: the Qwen3 prefill (causal, grouped-query, keys and values in
// the cache layout, optionally behind a prefix).  Replaces the mma.sync attention task of the reference
// (src/ittai/qwen3/sm80.py:274-403) with tensor-memory MMAs: per CTA one tile of 128 query rows of one (sequence, head),
// walking the visible keys 128 at a time.
//
//   warp 0, one lane: TMA loads (Q once; K and V blocks single-buffered, each refilled as soon as the MMA that read it
//     has completed) and every MMA: S = Q K^T (M128 N128, 8 k-steps over the 128 dims), then O += P V as one
//     M128 N128 series whose A operand P is read from tensor memory and whose B operand V is used as loaded (MN-major:
//     the two 64-dim swizzle atoms of the tile are one operand, 16 KB apart in the descriptor's leading-dimension field).
//   warps 1-4: one thread per query row, no cross-thread exchange at all: row maximum over the block's 128 scores
//     (all requested from tensor memory at once, the first 64 kept in registers for the second pass),
//     P = 2^(s*scale - m) packed to bf16 and written back over the consumed S columns, running row sum.  The running
//     maximum m is only raised when the block's maximum exceeds it by more than 8 (in log2 units): O in tensor memory
//     then has to be rescaled (load, multiply, store), which is rare after the first blocks; P may exceed 1 by up to
//     2^8 in between, harmless in bf16/fp32, and the final O / rowsum is exact either way.
// TMEM (256 columns, two CTAs per SM): S / P in columns 0..127, O in 128..255.  Shared memory: Q, K, V tiles of 32 KB each
// (two 128-byte-swizzled atoms of 64 dims); the Q tile doubles as the output staging area.  Every wait is a bounded
// mbarrier wait; on expiry the abort flag routes all roles to the common exit, where TMEM is freed.
#include "launch.h"
#include "tcgen05.cuh"
#include "tmap.h"

namespace ittai {

constexpr int kFaThreads = 160;
constexpr int kFaBlk = 128;                  // keys per block = query rows per tile = head_dim
constexpr uint32_t kFaCols = 256, kFaOCol = 128;
constexpr uint32_t kFaSpin = 1u << 22;
constexpr uint32_t kFaQ = 0, kFaK = 32768, kFaV = 65536, kFaBar = 98304;
constexpr uint32_t kFaSmem = kFaBar + 256 + 1024;
constexpr float kFaRescale = 8.0f;           // raise the running maximum only past this gap (log2 units)

struct AttnFaArgs {
    const int4* seqs;
    bf16* o;
    long long o_row, o_head;
    int group, causal;
    int k_seq_rows, k_head_rows;             // cache layout: strides in rows of 128 elements
    int k_head_cols;                         // packed layout (heads side by side in a row, sequences by their row offsets): 128, else 0
    float scale_log2;
    uint32_t* status;
};

__device__ __forceinline__ void fa_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool fa_wait(void* bar, uint32_t parity, volatile uint32_t* abort_flag) {
    uint32_t spins = 0;
    while (!mbar_try_wait_parked(bar, parity)) {
        if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kFaSpin)) { *abort_flag = 1; return false; }
    }
    return true;
}
__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kFaThreads, 2)
attn_fa_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const AttnFaArgs a) {
    pdl_trigger();
    // Grid (heads, sequences, query tiles) with the tiles in descending order: CTAs are handed out in index order, so the
    // causal tiles that walk the most key blocks start first and the last wave is made of the short ones.
    const int head = blockIdx.x, seq = blockIdx.y, mt = (int)gridDim.z - 1 - (int)blockIdx.z, kvh = head / a.group;
    const int4 sinfo = a.seqs[seq];                        // written by the host long before: safe ahead of pdl_wait
    const int q_len = sinfo.y, kv_len = sinfo.w, r0 = mt * kFaBlk;
    if (r0 >= q_len) return;                               // the whole CTA: nothing allocated yet
    const int offset = kv_len - q_len;                     // causal: query r sees keys <= r + offset
    const int last_key = a.causal ? min(kv_len - 1, r0 + kFaBlk - 1 + offset) : kv_len - 1;
    const int n_blk = last_key < 0 ? 0 : last_key / kFaBlk + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (n_blk == 0) {                                      // no visible key: zero rows
        pdl_wait();
        for (int i = threadIdx.x; i < kFaBlk * 16; i += kFaThreads) {
            const int row = r0 + (i >> 4);
            if (row < q_len) *reinterpret_cast<uint4*>(a.o + (long long)(sinfo.x + row) * a.o_row + (long long)head * a.o_head + (i & 15) * 8) = make_uint4(0, 0, 0, 0);
        }
        return;
    }

    extern __shared__ __align__(1024) unsigned char fa_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fa_raw) + 1023) & ~(uintptr_t)1023);
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sm + kFaBar);
    unsigned long long* bar_q = bars;             // Q landed
    unsigned long long* bar_k = bars + 1;         // K block landed (one phase per block)
    unsigned long long* bar_v = bars + 2;         // V block landed
    unsigned long long* bar_s = bars + 3;         // S of the block ready (also: K buffer free)
    unsigned long long* bar_p = bars + 4;         // P written, O rescaled (one arrival per softmax warp)
    unsigned long long* bar_o = bars + 5;         // PV of the block done (also: V buffer free)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int kv_row = seq * a.k_seq_rows + kvh * a.k_head_rows + sinfo.z;   // first key row of this (sequence, kv head)
    const int kc = kvh * a.k_head_cols;                                             // and its first column

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1); mbar_init(bar_k, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_p, 4); mbar_init(bar_o, 1);
        *abort_flag = 0;
        fence_mbar_init();
        pdl_wait();                                        // q, k, v come from the kernels before this one
        mbar_expect_tx(bar_q, 32768);
        tma_load_2d(sm + kFaQ, &tm_q, head * 128, sinfo.x + r0, bar_q);
        tma_load_2d(sm + kFaQ + 16384, &tm_q, head * 128 + 64, sinfo.x + r0, bar_q);
        mbar_expect_tx(bar_k, 32768);
        tma_load_2d(sm + kFaK, &tm_k, kc, kv_row, bar_k);
        tma_load_2d(sm + kFaK + 16384, &tm_k, kc + 64, kv_row, bar_k);
        mbar_expect_tx(bar_v, 32768);
        tma_load_2d(sm + kFaV, &tm_v, kc, kv_row, bar_v);
        tma_load_2d(sm + kFaV + 16384, &tm_v, kc + 64, kv_row, bar_v);
    }
    if (warp == 0) { __syncwarp(); tmem_alloc(tmem_slot, kFaCols); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128), idesc_o = umma_idesc_bf16(128, 128) | umma_idesc_b_mn;
            bool ok = fa_wait(bar_q, 0, abort_flag);
            for (int j = 0; j < n_blk && ok; ++j) {
                const uint32_t ph = j & 1;
                ok = fa_wait(bar_k, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                // ---- S = Q K^T over the 128 dims: atoms of 64 dims, 4 k-steps each
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_bf16(tmem_base, umma_desc_sw128(sm + kFaQ + (k >> 2) * 16384) + 2 * (k & 3),
                              umma_desc_sw128(sm + kFaK + (k >> 2) * 16384) + 2 * (k & 3), idesc_s, k > 0 ? 1u : 0u);
                umma_commit(bar_s);
                if (j > 0) {
                    // the previous PV has finished reading the V buffer: refill it
                    ok = fa_wait(bar_o, (j - 1) & 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(bar_v, 32768);
                    tma_load_2d(sm + kFaV, &tm_v, kc, kv_row + j * kFaBlk, bar_v);
                    tma_load_2d(sm + kFaV + 16384, &tm_v, kc + 64, kv_row + j * kFaBlk, bar_v);
                }
                ok = fa_wait(bar_s, ph, abort_flag);
                if (!ok) break;
                if (j + 1 < n_blk) {
                    // S is complete, so the K buffer is free: the next block's keys travel during this block's softmax
                    mbar_expect_tx(bar_k, 32768);
                    tma_load_2d(sm + kFaK, &tm_k, kc, kv_row + (j + 1) * kFaBlk, bar_k);
                    tma_load_2d(sm + kFaK + 16384, &tm_k, kc + 64, kv_row + (j + 1) * kFaBlk, bar_k);
                }
                ok = fa_wait(bar_p, ph, abort_flag) && fa_wait(bar_v, ph, abort_flag);
                if (!ok) break;
                tc_fence_after();
                // ---- O += P V: P from tensor memory (8 columns per 16 keys), V rows 16 at a time, one series per dim half
                {
                    const uint64_t dv = umma_desc_sw128_mn(sm + kFaV, 16384);      // both 64-dim atoms of the V tile: N = 128
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        umma_bf16_tmem_a(tmem_base + kFaOCol, tmem_base + 8 * ks, dv + (uint64_t)ks * (2048 >> 4), idesc_o,
                                         (j > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(bar_o);
            }
        }
    } else do {
        const int q4 = warp & 3, r = q4 * 32 + lane;         // TMEM lane quarter; query row inside the tile
        const uint32_t t_row = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const int row_limit = a.causal ? min(kv_len - 1, r0 + r + offset) : kv_len - 1;   // last key this row sees
        float m_used = -INFINITY, l0 = 0.f, l1 = 0.f;       // running maximum in scaled (log2) units, running sum
        bool ok = true;
        for (int j = 0; j < n_blk; ++j) {
            const uint32_t ph = j & 1;
            ok = fa_wait(bar_s, ph, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int lim = row_limit - j * kFaBlk;          // columns 0..lim of this block are visible to this row
            const bool full = __all_sync(0xffffffffu, lim >= kFaBlk - 1);
            // ---- pass 1: the block's row maximum.  All 128 scores are requested at once (one wait instead of four round
            //      trips to tensor memory); the first 64 stay in registers for pass 2, the others are read again there
            //      (holding all 128 would spill: two CTAs per SM leave a thread 168 registers).
            uint32_t sv[64], su[64];
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                tmem_ld_32x16(t_row + c0, *reinterpret_cast<uint32_t(*)[16]>(&sv[c0]));
                tmem_ld_32x16(t_row + 64 + c0, *reinterpret_cast<uint32_t(*)[16]>(&su[c0]));
            }
            tmem_ld_wait();
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 16) {
                tmem_ld_tie16(*reinterpret_cast<uint32_t(*)[16]>(&sv[c0]));
                tmem_ld_tie16(*reinterpret_cast<uint32_t(*)[16]>(&su[c0]));
            }
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            if (full) {
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    mx0 = fmaxf(mx0, fmaxf(__uint_as_float(sv[i]), __uint_as_float(su[i]))); mx1 = fmaxf(mx1, fmaxf(__uint_as_float(sv[i + 1]), __uint_as_float(su[i + 1])));
                    mx2 = fmaxf(mx2, fmaxf(__uint_as_float(sv[i + 2]), __uint_as_float(su[i + 2]))); mx3 = fmaxf(mx3, fmaxf(__uint_as_float(sv[i + 3]), __uint_as_float(su[i + 3])));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    if (i <= lim) mx0 = fmaxf(mx0, __uint_as_float(sv[i]));
                    if (64 + i <= lim) mx1 = fmaxf(mx1, __uint_as_float(su[i]));
                }
            }
            const float bm = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2;
            // ---- raise the running maximum (and rescale O) only when the block exceeds it by more than the gap
            if (j == 0) {
                m_used = bm;
            } else {
                const bool need = bm - m_used > kFaRescale;      // false for NaN / -inf
                if (__any_sync(0xffffffffu, need)) {
                    ok = fa_wait(bar_o, (j - 1) & 1, abort_flag);   // O must be complete before it is rewritten
                    if (!ok) break;
                    tc_fence_after();
                    const float alpha = need ? fa_ex2(m_used - bm) : 1.0f;
                    if (need) m_used = bm;
                    l0 *= alpha; l1 *= alpha;
#pragma unroll 1
                    for (int c0 = 0; c0 < 128; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld_32x32(t_row + kFaOCol + c0, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            const uint32_t w[8] = {v[i], v[i + 1], v[i + 2], v[i + 3], v[i + 4], v[i + 5], v[i + 6], v[i + 7]};
                            tmem_st_32x8(t_row + kFaOCol + c0 + i, w);
                        }
                    }
                }
            }
            const float mb = m_used == -INFINITY ? 0.f : m_used;
            // ---- pass 2: p = 2^(s * scale - m), row sum, packed bf16 P over the consumed S columns
            auto emit_p = [&](uint32_t (&v)[16], int c0) {
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    float p0 = fa_ex2(fmaf(__uint_as_float(v[i]), a.scale_log2, -mb));
                    float p1 = fa_ex2(fmaf(__uint_as_float(v[i + 1]), a.scale_log2, -mb));
                    if (!full) { p0 = c0 + i <= lim ? p0 : 0.f; p1 = c0 + i + 1 <= lim ? p1 : 0.f; }
                    l0 += p0; l1 += p1;
                    w[i >> 1] = pack_bf16x2_alu(p0, p1);
                }
                tmem_st_32x8(t_row + (c0 >> 1), w);
            };
            {
                // the second half of the scores is on its way again while the first half, still in registers, is worked on
                uint32_t va[16], vb[16];
                tmem_ld_32x16(t_row + 64, va);
                tmem_ld_32x16(t_row + 80, vb);
#pragma unroll
                for (int c0 = 0; c0 < 64; c0 += 16) emit_p(*reinterpret_cast<uint32_t(*)[16]>(&sv[c0]), c0);
                tmem_ld_wait16(va);
                tmem_ld_tie16(vb);
                emit_p(va, 64);
                tmem_ld_32x16(t_row + 96, va);
                emit_p(vb, 80);
                tmem_ld_32x16(t_row + 112, vb);
                tmem_ld_wait16(va);
                tmem_ld_tie16(vb);
                emit_p(va, 96);
                emit_p(vb, 112);
                tmem_st_wait();
            }
            if (j == n_blk - 1 && (kv_len & (kFaBlk - 1)) != 0 && kv_len < (j + 1) * kFaBlk) {
                // rows of the V tile past the sequence belong to a neighbour (or are unwritten cache): zero them, so that
                // 0 * V stays 0 whatever they hold
                ok = fa_wait(bar_v, ph, abort_flag);
                if (!ok) break;
                const int first = kv_len - j * kFaBlk;       // first row to clear
                for (int i = threadIdx.x - 32; i < (kFaBlk - first) * 16; i += 128) {
                    const int row = first + (i >> 4), piece = i & 15;
                    *reinterpret_cast<uint4*>(sm + kFaV + (piece >> 3) * 16384 + row * 128 + (piece & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async_smem();
            }
            // one arrival per warp: 32 lanes arriving on one barrier word are 32 shared-memory atomics one after the other
            tc_fence_before();
            __syncwarp();
            if (lane == 0) fa_arrive(bar_p);
        }
        if (!ok) break;
        // ---- epilogue: O / rowsum -> bf16 -> staging tile (the Q tile is dead) -> whole 256-byte rows
        ok = fa_wait(bar_o, (n_blk - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const float l = l0 + l1;
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        unsigned char* stage = sm + kFaQ;
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32(t_row + kFaOCol + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
                *reinterpret_cast<uint4*>(stage + r * 256 + ((((c0 >> 3) + jj) ^ (r & 15)) << 4)) =
                    make_uint4(pack_bf16x2(__uint_as_float(v[8 * jj]) * inv, __uint_as_float(v[8 * jj + 1]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * jj + 2]) * inv, __uint_as_float(v[8 * jj + 3]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * jj + 4]) * inv, __uint_as_float(v[8 * jj + 5]) * inv),
                               pack_bf16x2(__uint_as_float(v[8 * jj + 6]) * inv, __uint_as_float(v[8 * jj + 7]) * inv));
        }
        __syncwarp();
        const int sub = lane & 15;
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
            const int rr = q4 * 32 + it * 2 + (lane >> 4), row = r0 + rr;
            const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((sub ^ (rr & 15)) << 4));
            if (row < q_len) *reinterpret_cast<uint4*>(a.o + (long long)(sinfo.x + row) * a.o_row + (long long)head * a.o_head + 8 * sub) = val;
        }
    } while (false);
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (atomicCAS(&a.status[0], 0u, (uint32_t)ITTAI_ST_GEMM_TIMEOUT) == 0u) { a.status[1] = blockIdx.x; a.status[2] = blockIdx.y; }
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
        __syncthreads();
    }
    if (warp == 0) { __syncwarp(); tmem_dealloc(tmem_base, kFaCols); }
}

int cuda_fail(cudaError_t e, const char* what);

// Whether the key-loop kernel covers this call: head_dim 128, heads adjacent in the q rows, keys and values as dense rows
// of 128 elements (the cache layout), identical strides for k and v, more than 64 query rows in some sequence.
// Keys and values either in the cache layout (rows of 128 elements; heads and sequences whole numbers of rows apart) or
// packed like the queries (the heads of a token side by side in one row, sequences told apart by their row offsets).
static bool fa_packed_kv(const IttaiAttention* p) { return p->k_seq == 0 && p->v_seq == 0 && p->k_head == 128 && p->v_head == 128 && p->k_row == p->v_row && p->k_row > 128; }
bool attn_fa_supported(const IttaiAttention* p) {
    const bool cache = p->k_row == 128 && p->v_row == 128 && p->k_head % 128 == 0 && p->k_seq % 128 == 0;
    return p->head_dim == 128 && p->status != nullptr && p->max_q_len > 64 && p->q_head == 128 && (cache || fa_packed_kv(p)) &&
           p->v_head == p->k_head && p->v_seq == p->k_seq && p->q_rows_total > 0 &&
           p->kv_rows_total > 0 && ((uintptr_t)p->q & 15) == 0 && ((uintptr_t)p->k & 15) == 0 && ((uintptr_t)p->v & 15) == 0 &&
           ((uintptr_t)p->o & 15) == 0 && p->o_row % 8 == 0 && p->o_head % 8 == 0;
}

int attn_fa_launch(const IttaiAttention* p, cudaStream_t st) {
    CUtensorMap tq, tk, tv;
    int rc = make_tmap_bf16(&tq, p->q, p->q_rows_total, (long long)p->n_heads * 128, p->q_row, 128);
    const bool packed = fa_packed_kv(p);
    const long long kv_cols = packed ? (long long)(p->n_heads / p->group) * 128 : 128, kv_ld = packed ? p->k_row : 128;
    if (rc == ITTAI_OK) rc = make_tmap_bf16(&tk, p->k, p->kv_rows_total, kv_cols, kv_ld, 128);
    if (rc == ITTAI_OK) rc = make_tmap_bf16(&tv, p->v, p->kv_rows_total, kv_cols, kv_ld, 128);
    if (rc != ITTAI_OK) return rc;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(attn_fa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFaSmem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attn_fa_kernel)");
        attr_dev = dev;
    }
    AttnFaArgs a;
    a.seqs = reinterpret_cast<const int4*>(p->seqs);
    a.o = reinterpret_cast<bf16*>(p->o);
    a.o_row = p->o_row; a.o_head = p->o_head;
    a.group = p->group; a.causal = p->causal;
    a.k_seq_rows = packed ? 0 : (int)(p->k_seq / 128); a.k_head_rows = packed ? 0 : (int)(p->k_head / 128);
    a.k_head_cols = packed ? 128 : 0;
    a.scale_log2 = 1.4426950408889634f * 0.08838834764831845f;
    a.status = p->status;
    const cudaError_t e = launch_pdl(attn_fa_kernel, dim3(p->n_heads, p->n_seqs, (p->max_q_len + 127) / 128), dim3(kFaThreads), kFaSmem, st, 1, tq, tk, tv, a);
    return e == cudaSuccess ? ITTAI_OK : cuda_fail(e, "launch attn_fa_kernel");
}

}  // namespace ittai
