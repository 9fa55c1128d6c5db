// Dense attention for short sequences (SigLIP: 196 tokens, head_dim 64) on tcgen05: S = Q K^T and O = P V are
// tensor-memory MMAs.  The reference's attention task (src/ittai/siglip/kernel.py:366-500) keeps Q resident and streams
// K/V blocks through mma.sync; with at most 256 keys the whole of K and V fits in shared memory, so here there is no
// key loop at all.
//
// One persistent CTA per SM holds two independent groups of 9 warps.  A group walks its share of the (sequence, head)
// items; per item it loads K and V once and handles the one or two tiles of 128 query rows one after the other.  The
// next tile's Q (and after an item's last tile the next item's K) is fetched as soon as the current score MMAs have
// completed, the next item's V once the last PV MMA has, so the loads hide behind the softmax and the epilogue of the
// tile in flight; barriers and tensor memory are set up once per CTA.  The two groups share nothing but the SM: while one is in its softmax pass the other is
// usually in its MMAs or its epilogue.
//
// The keys are handled as two halves (112 + the rest up to 224 keys, 128 + the rest above), each with its own score
// MMA, its own softmax threads and its own PV MMA into its own accumulator; the halves meet only in the epilogue.  A softmax thread owns one query row of one
// half and makes ONE pass over its score columns: p = 2^(s * scale - ref), where ref is the maximum of the row's first
// chunk of 16 columns, raised only when the running row sum passes 2^60 (then the P chunks already written and the sum
// are rescaled: a rare, warp-uniform branch).  A lagging ref costs no accuracy: P is bf16 and the sums are fp32, both
// floating point.  There is no separate row-maximum pass and no exchange between the halves before the epilogue, which
// combines O_A, O_B and the two (ref, sum) pairs of the row.
//
// Roles in a group: warp 0 (one lane) issues the TMA loads and every MMA.  Warps 1-8 are the softmax: two warps per
// TMEM lane quarter (one per half of the keys), one thread per query row; in the epilogue each takes half of the output
// columns.  TMEM (256 columns per group): half A's scores from column 0, half B's from 128; P of a half as packed bf16
// over the first half of that half's score columns, each chunk written behind the reads of the thread that owns it; O_A
// in 64..127 and O_B in 192..255, written once every score column has been consumed.
// Every wait is an mbarrier wait with a bound; on expiry the abort flag routes all roles to the common exit, where
// TMEM is freed.
#include "tcgen05.cuh"
#include "tmap.h"
#include "launch.h"

namespace ittai {

constexpr int kTcKeys = 256;                 // most keys per sequence (a multiple of 16)
// keys of the first half: 112 up to 224 keys (SigLIP's 196 tokens: 112 + 96, seven and six chunks of 16 per thread), 128 above
__host__ __device__ constexpr int tc_half(int n_keys) { return n_keys > 224 ? 128 : 112; }
constexpr int kTcHD = 64;
constexpr int kTcGroup = 288;                // threads of a group: 1 issuing warp + 8 softmax warps
constexpr int kTcThreads = 2 * kTcGroup;
constexpr uint32_t kTcCols = 256;            // tensor-memory columns of a group
constexpr uint32_t kTcColB = 128;            // first score / P column of half B
constexpr uint32_t kTcOColA = 64, kTcOColB = 192;
constexpr uint32_t kTcSpin = 1u << 22;
// shared-memory plan of a group (bytes, every tile 1024-aligned): query tiles [128 rows][128 B], K and V [box rows][128 B],
// the output staging tile [128 rows][128 B].  With loads of 224 rows there is room for two query tiles (the next tile's Q
// is fetched while the current one is still being read); with 256 rows for one.
__host__ __device__ constexpr uint32_t tc_off_k(int kv_box) { return kv_box > 224 ? 16384u : 32768u; }
__host__ __device__ constexpr uint32_t tc_off_v(int kv_box) { return tc_off_k(kv_box) + (uint32_t)kv_box * 128u; }
__host__ __device__ constexpr uint32_t tc_off_stage(int kv_box) { return tc_off_v(kv_box) + (uint32_t)kv_box * 128u; }
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffBar = 32768 + 2 * 224 * 128 + 16384;
static_assert(tc_off_stage(224) + 16384 <= kOffBar && tc_off_stage(256) + 16384 <= kOffBar, "both plans end before the barriers");
constexpr uint32_t kOffX = kOffBar + 128;    // float [2 stats][2 halves][128 rows]
constexpr uint32_t kTcGroupSmem = (kOffX + 2048 + 1023) & ~1023u;
constexpr uint32_t kTcSmem = 2 * kTcGroupSmem + 1024;

struct AttnTcArgs {
    const int4* seqs;
    bf16* o;
    long long o_row, o_head;
    int group, n_heads, n_items;
    float scale_log2;
    uint32_t* status;
};

__device__ __forceinline__ void mbar_arrive_cta(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait_abortable(void* bar, uint32_t parity, volatile uint32_t* abort_flag) {
    uint32_t spins = 0;
    while (!mbar_try_wait_parked(bar, parity)) {
        if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kTcSpin)) { *abort_flag = 1; return false; }
    }
    return true;
}
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int KVBOX>           // rows of a K / V load: 224 (two query-tile buffers) or 256 (one)
__global__ void __launch_bounds__(kTcThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const AttnTcArgs a) {
    pdl_trigger();
    extern __shared__ __align__(1024) unsigned char tc_raw[];
    unsigned char* sm0 = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    const int grp = threadIdx.x >= kTcGroup ? 1 : 0;
    const int tid = threadIdx.x - grp * kTcGroup;
    unsigned char* sm = sm0 + grp * kTcGroupSmem;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sm + kOffBar);
    unsigned long long* bar_k = bars;             // K landed                                         (one phase per item)
    unsigned long long* bar_v = bars + 1;         // V landed                                         (one phase per item)
    unsigned long long* bar_q = bars + 8;         // Q tile landed                                    (one phase per query tile)
    unsigned long long* bar_s = bars + 2;         // [2]: scores of half A / half B ready             (one phase per query tile)
    unsigned long long* bar_p = bars + 4;         // [2]: P of half A / half B written, 128 arrivals  (one phase per query tile)
    unsigned long long* bar_o = bars + 6;         // O_A and O_B ready                                (one phase per query tile)
    unsigned long long* bar_free = bars + 7;      // O read back: tensor memory may be overwritten, 256 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm0 + kOffBar + 96);      // CTA-wide, in group 0's region (behind its 9 barriers)
    volatile uint32_t* abort_flag = tmem_slot + 1;
    float* xref = reinterpret_cast<float*>(sm + kOffX);    // [half][row]: the reference the row's P is scaled by
    float* xsum = xref + 256;                              // [half][row]: sum of that P

    const int warp = tid >> 5, lane = tid & 31;
    constexpr uint32_t kOffK = tc_off_k(KVBOX), kOffV = tc_off_v(KVBOX), kOffStage = tc_off_stage(KVBOX);
    constexpr uint32_t n_qbuf = KVBOX > 224 ? 1u : 2u;
    if (tid == 0) {
        mbar_init(bar_k, 1); mbar_init(bar_q, 1); mbar_init(bar_v, 1); mbar_init(bar_s, 1); mbar_init(bar_s + 1, 1);
        mbar_init(bar_p, 128); mbar_init(bar_p + 1, 128); mbar_init(bar_o, 1); mbar_init(bar_free, 256);
        if (grp == 0) *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    }
    if (threadIdx.x < 32) { __syncwarp(); tmem_alloc(tmem_slot, 2 * kTcCols); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();                                            // Q, K, V come from the kernel before this one
    const uint32_t tmem_base = *tmem_slot + grp * kTcCols;
    const int first = blockIdx.x + grp * gridDim.x, stride = gridDim.x * 2;   // the second group only works when the items outnumber the CTAs

    if (warp == 0) {
        if (lane == 0) {
            // the sequence record of an item: {first query row, queries, first key row, keys}
            auto issue_q = [&](int it, const int4& si, int mt, uint32_t tile) {      // `tile`: running tile number, picks the buffer
                mbar_expect_tx(bar_q, 128 * 128);
                tma_load_2d(sm + kOffQ + (tile % n_qbuf) * 16384, &tm_q, (it % a.n_heads) * kTcHD, si.x + mt * 128, bar_q);
            };
            auto issue_k = [&](int it, const int4& si) {
                mbar_expect_tx(bar_k, KVBOX * 128);
                tma_load_2d(sm + kOffK, &tm_k, ((it % a.n_heads) / a.group) * kTcHD, si.z, bar_k);
            };
            auto issue_v = [&](int it, const int4& si) {
                mbar_expect_tx(bar_v, KVBOX * 128);
                tma_load_2d(sm + kOffV, &tm_v, ((it % a.n_heads) / a.group) * kTcHD, si.z, bar_v);
            };
            int4 snext = make_int4(0, 0, 0, 0);
            if (first < a.n_items) { snext = a.seqs[first / a.n_heads]; issue_q(first, snext, 0, 0u); issue_k(first, snext); issue_v(first, snext); }
            const uint64_t dk = umma_desc_sw128(sm + kOffK), dv = umma_desc_sw128(sm + kOffV);
            constexpr uint32_t idesc_o = umma_idesc_bf16(128, kTcHD) | umma_idesc_b_mn;
            uint32_t tcount = 0, icount = 0;
            bool ok = true;
#pragma unroll 1
            for (int it = first; ok && it < a.n_items; it += stride, ++icount) {
                const int4 sinfo = snext;
                const bool more = it + stride < a.n_items;
                if (more) snext = a.seqs[(it + stride) / a.n_heads];     // long before it is used
                const int n_tiles = min(2, max(1, (sinfo.y + 127) >> 7));
                const int n_keys = max(16, (sinfo.w + 15) & ~15);
                const int half = tc_half(n_keys), n_a = min(n_keys, half), n_b = n_keys - n_a;
                const uint64_t dkb = dk + (uint64_t)((half * 128) >> 4);
                const uint32_t idesc_a = umma_idesc_bf16(128, n_a), idesc_b = umma_idesc_bf16(128, max(n_b, 16));
                ok = mbar_wait_abortable(bar_k, icount & 1u, abort_flag);
#pragma unroll 1
                for (int mt = 0; ok && mt < n_tiles; ++mt, ++tcount) {
                    const uint32_t ph = tcount & 1u;
                    const bool last = mt == n_tiles - 1;
                    ok = mbar_wait_abortable(bar_q, ph, abort_flag);
                    if (ok && tcount > 0) ok = mbar_wait_abortable(bar_free, ph ^ 1u, abort_flag);   // the tile before has read its O back
                    if (!ok) break;
                    // ---- S = Q K^T per half: 4 k-steps of 16 head dims each
                    tc_fence_after();
                    const uint64_t dq = umma_desc_sw128(sm + kOffQ + (tcount % n_qbuf) * 16384);
#pragma unroll
                    for (int k = 0; k < kTcHD / 16; ++k) umma_bf16(tmem_base, dq + 2 * k, dk + 2 * k, idesc_a, k > 0 ? 1u : 0u);
                    umma_commit(bar_s);
                    if (n_b > 0) {
#pragma unroll
                        for (int k = 0; k < kTcHD / 16; ++k) umma_bf16(tmem_base + kTcColB, dq + 2 * k, dkb + 2 * k, idesc_b, k > 0 ? 1u : 0u);
                    }
                    umma_commit(bar_s + 1);          // also without a second half: the barrier keeps one phase per tile
                    if (!last || more) {
                        // the next tile's Q: at once into the other buffer, or into the only one when the score MMAs have
                        // read it; the next item's K when this item's last score MMA has read K
                        const int q_it = last ? it + stride : it, q_mt = last ? 0 : mt + 1;
                        const int4& q_si = last ? snext : sinfo;
                        if (n_qbuf == 2u) issue_q(q_it, q_si, q_mt, tcount + 1);
                        if (n_qbuf == 1u || last) {
                            ok = mbar_wait_abortable(bar_s + 1, ph, abort_flag);
                            if (!ok) break;
                        }
                        if (n_qbuf == 1u) issue_q(q_it, q_si, q_mt, tcount + 1);
                        if (last) issue_k(it + stride, snext);
                    }
                    // ---- O = P V per half: P from tensor memory, V rows (keys) 16 at a time.  The two halves
                    // accumulate into different columns, so their MMAs alternate: an MMA of this shape is bound by its
                    // latency, not its arithmetic, and two independent chains overlap.  (The padding rows of V were
                    // zeroed before any arrival on these barriers.)
                    ok = mbar_wait_abortable(bar_v, icount & 1u, abort_flag) && mbar_wait_abortable(bar_p, ph, abort_flag) &&
                         mbar_wait_abortable(bar_p + 1, ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int ks = 0; ks < n_a / 16; ++ks) {
                        umma_bf16_tmem_a(tmem_base + kTcOColA, tmem_base + 8 * ks, dv + (uint64_t)ks * (2048 >> 4), idesc_o, ks > 0 ? 1u : 0u);
                        if (ks < n_b / 16)
                            umma_bf16_tmem_a(tmem_base + kTcOColB, tmem_base + kTcColB + 8 * ks, dv + (uint64_t)(half / 16 + ks) * (2048 >> 4), idesc_o, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(bar_o);
                    if (last && more) {
                        // the item's last PV MMA has read V: fetch the next item's
                        ok = mbar_wait_abortable(bar_o, ph, abort_flag);
                        if (!ok) break;
                        issue_v(it + stride, snext);
                    }
                }
            }
        }
    } else {
        const int hf = (warp - 1) >> 2;                      // which half of the keys / of the output columns
        const int q4 = (threadIdx.x >> 5) & 3;               // TMEM lane quarter this warp may touch (by its index in the CTA)
        const int r = q4 * 32 + lane;                        // query row inside the tile
        const uint32_t t_row = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const uint32_t t_half = t_row + (hf ? kTcColB : 0u); // this half's scores; its P goes over their first columns
        unsigned char* stage = sm + kOffStage;
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2);
        uint32_t tcount = 0, icount = 0;
        bool ok = true;
        int4 snext = first < a.n_items ? a.seqs[first / a.n_heads] : make_int4(0, 0, 0, 0);
#pragma unroll 1
        for (int it = first; ok && it < a.n_items; it += stride, ++icount) {
            const int4 sinfo = snext;
            if (it + stride < a.n_items) snext = a.seqs[(it + stride) / a.n_heads];   // long before it is used
            const int head = it % a.n_heads;
            const int q_len = sinfo.y, kv_len = sinfo.w;
            const int n_tiles = min(2, max(1, (q_len + 127) >> 7));
            const int n_keys = max(16, (kv_len + 15) & ~15);
            const int half = tc_half(n_keys), n_a = min(n_keys, half), n_b = n_keys - n_a;
            const int c_lo = hf * half, c_hi = c_lo + (hf ? n_b : n_a);
            const bool has = c_lo < c_hi;                    // false for half B when the sequence has at most 112 keys
#pragma unroll 1
            for (int mt = 0; mt < n_tiles; ++mt, ++tcount) {
                const uint32_t ph = tcount & 1u;
                const bool live = mt * 128 + q4 * 32 < q_len;    // a warp whose 32 rows are all padding skips the arithmetic
                if (has) {
                    ok = mbar_wait_abortable(bar_s + hf, ph, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                }
                // ---- the one pass: p = 2^(s * scale - ref), row sum, packed bf16 P back into tensor memory
                float ref = -INFINITY;
                float2 l2 = make_float2(0.f, 0.f);           // row sum, even / odd columns
                auto emit_p = [&](const uint32_t (&v)[16], int c0) {
                    // scaled maximum of the chunk's valid columns (the first chunk of a row, and the rare path below)
                    auto chunk_max = [&]() {
                        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
                        if (c0 + 16 <= kv_len) {
#pragma unroll
                            for (int i = 0; i < 16; i += 4) {
                                m0 = fmaxf(m0, __uint_as_float(v[i])); m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
                                m2 = fmaxf(m2, __uint_as_float(v[i + 2])); m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) if (c0 + i < kv_len) m0 = fmaxf(m0, __uint_as_float(v[i]));
                        }
                        return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * a.scale_log2;
                    };
                    float2 p[8], cs;
                    auto exps = [&]() {
                        const float2 nr = make_float2(-ref, -ref);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float2 t = __ffma2_rn(make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), sc2, nr);
                            p[i] = make_float2(ex2_fast(t.x), ex2_fast(t.y));
                        }
                        if (c0 + 16 > kv_len) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) { if (c0 + 2 * i >= kv_len) p[i].x = 0.f; if (c0 + 2 * i + 1 >= kv_len) p[i].y = 0.f; }
                        }
                        cs = __fadd2_rn(__fadd2_rn(__fadd2_rn(p[0], p[1]), __fadd2_rn(p[2], p[3])), __fadd2_rn(__fadd2_rn(p[4], p[5]), __fadd2_rn(p[6], p[7])));
                    };
                    if (c0 == c_lo) {                        // warp-uniform
                        const float cm = chunk_max();
                        ref = cm == -INFINITY ? 0.f : cm;
                    }
                    uint32_t w[8];
                    auto store_p = [&]() {
#pragma unroll
                        for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2_alu(p[i].x, p[i].y);
                        tmem_st_32x8(t_half + (uint32_t)((c0 - c_lo) >> 1), w);
                    };
                    exps();
                    store_p();                               // before the check below: nothing here waits for the vote
                    // The reference lags: p may grow with later chunks.  Once the row sum passes 2^60 (or is infinite)
                    // the reference is raised to this chunk's maximum, what the thread has already written is rescaled
                    // and this chunk is written again.
                    const bool raise = (l2.x + l2.y) + (cs.x + cs.y) > 1.152921504606847e18f;
                    if (__any_sync(0xffffffffu, raise)) {
                        const float nref = raise ? fmaxf(chunk_max(), ref) : ref;
                        const float f = ex2_fast(ref - nref);    // 1 for the lanes that keep their reference
                        l2.x *= f; l2.y *= f;
                        // the TMEM accesses are warp-wide: multiplying by 1 leaves a bf16 value unchanged
                        tmem_st_wait();
#pragma unroll 1
                        for (int cp = c_lo; cp < c0; cp += 16) {
                            uint32_t u[8];
                            tmem_ld_32x8(t_half + (uint32_t)((cp - c_lo) >> 1), u);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                u[i] = pack_bf16x2_alu(__uint_as_float(u[i] << 16) * f, __uint_as_float(u[i] & 0xFFFF0000u) * f);
                            tmem_st_32x8(t_half + (uint32_t)((cp - c_lo) >> 1), u);
                        }
                        ref = nref;
                        exps();
                        store_p();
                    }
                    l2 = __fadd2_rn(l2, cs);
                };
                if (live && has) {
                    // this warp's score columns 16 at a time, the next chunk's TMEM load in flight
                    uint32_t va[16], vb[16];
                    tmem_ld_32x16(t_half, va);
#pragma unroll 1
                    for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
                        tmem_ld_wait16(va);
                        if (c0 + 16 < c_hi) tmem_ld_32x16(t_half + (uint32_t)(c0 + 16 - c_lo), vb);
                        emit_p(va, c0);
                        if (c0 + 16 >= c_hi) break;
                        tmem_ld_wait16(vb);
                        if (c0 + 32 < c_hi) tmem_ld_32x16(t_half + (uint32_t)(c0 + 32 - c_lo), va);
                        emit_p(vb, c0 + 16);
                    }
                    tmem_st_wait();
                }
                if (mt == 0) {
                    // keys between the sequence's end and the MMA's K extent belong to a neighbour: zero those V rows so
                    // that 0 * V stays 0 whatever they hold (V landed long ago; the wait only orders the stores behind it)
                    ok = mbar_wait_abortable(bar_v, icount & 1u, abort_flag);
                    if (!ok) break;
                    const int t = tid - 32;
                    if (t < (n_keys - kv_len) * 8) {
                        *reinterpret_cast<uint4*>(sm + kOffV + (kv_len + (t >> 3)) * 128 + (t & 7) * 16) = make_uint4(0, 0, 0, 0);
                        fence_proxy_async();         // ordinary stores; the MMA reads them through the async proxy
                    }
                }
                xref[hf * 128 + r] = ref;
                xsum[hf * 128 + r] = l2.x + l2.y;
                tc_fence_before();
                mbar_arrive_cta(bar_p + hf);
                // ---- epilogue: this warp's 32 output columns, (O_A 2^(ref_A - m) + O_B 2^(ref_B - m)) / l -> bf16 -> staging tile
                ok = mbar_wait_abortable(bar_o, ph, abort_flag);      // O follows every arrival on bar_p, which follows the sums
                if (!ok) break;
                tc_fence_after();
                const float ra = xref[r], rb = xref[128 + r];
                const float m = fmaxf(ra, rb);
                const float fa = ra == -INFINITY ? 0.f : ex2_fast(ra - m), fb = rb == -INFINITY ? 0.f : ex2_fast(rb - m);
                const float l = xsum[r] * fa + xsum[128 + r] * fb;
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                const float ga = fa * inv, gb = fb * inv;
                if (live) {
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        uint32_t va[16], vb[16];
                        float o[16];
                        tmem_ld_32x16(t_row + kTcOColA + 32 * hf + 16 * h2, va);
                        if (n_b > 0) {
                            tmem_ld_32x16(t_row + kTcOColB + 32 * hf + 16 * h2, vb);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] = fmaf(__uint_as_float(va[i]), ga, __uint_as_float(vb[i]) * gb);
                        } else {
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] = __uint_as_float(va[i]) * ga;
                        }
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            *reinterpret_cast<uint4*>(stage + r * 128 + (((4 * hf + 2 * h2 + j) ^ (r & 7)) << 4)) =
                                make_uint4(pack_bf16x2(o[8 * j], o[8 * j + 1]), pack_bf16x2(o[8 * j + 2], o[8 * j + 3]),
                                           pack_bf16x2(o[8 * j + 4], o[8 * j + 5]), pack_bf16x2(o[8 * j + 6], o[8 * j + 7]));
                    }
                }
                tc_fence_before();
                mbar_arrive_cta(bar_free);           // this thread is done with the tile's tensor memory and its row statistics
                if (live) {
                    __syncwarp();
                    // 4 lanes per row, 8 rows per instruction: every store covers whole 32-byte sectors
                    const int sub = lane & 3;
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const int rr = q4 * 32 + i4 * 8 + (lane >> 2), row = mt * 128 + rr;
                        const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 128 + (((4 * hf + sub) ^ (rr & 7)) << 4));
                        if (row < q_len)
                            *reinterpret_cast<uint4*>(a.o + (long long)(sinfo.x + row) * a.o_row + (long long)head * a.o_head + 32 * hf + 8 * sub) = val;
                    }
                    __syncwarp();                    // the warp's part of the staging tile is free for its next tile
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (atomicCAS(&a.status[0], 0u, (uint32_t)ITTAI_ST_GEMM_TIMEOUT) == 0u) { a.status[1] = blockIdx.x; a.status[2] = 0; }
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
        __syncthreads();
    }
    if (threadIdx.x < 32) { __syncwarp(); tmem_dealloc(*tmem_slot, 2 * kTcCols); }
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
    const int kv_box = p->max_kv_len > 224 ? 256 : 224;        // the shorter box spares SigLIP's 196 keys an eighth of the traffic
    if (rc == ITTAI_OK) rc = make_tmap_bf16(&tk, p->k, p->kv_rows_total, (long long)kv_heads * 64, p->k_row, kv_box);
    if (rc == ITTAI_OK) rc = make_tmap_bf16(&tv, p->v, p->kv_rows_total, (long long)kv_heads * 64, p->v_row, kv_box);
    if (rc != ITTAI_OK) return rc;
    static thread_local int attr_dev = -1, n_sms = 1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<224>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(attn_tc_kernel)");
        cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        attr_dev = dev;
    }
    AttnTcArgs a;
    a.seqs = reinterpret_cast<const int4*>(p->seqs);
    a.o = reinterpret_cast<bf16*>(p->o);
    a.o_row = p->o_row; a.o_head = p->o_head;
    a.group = p->group;
    a.scale_log2 = 1.4426950408889634f / 8.0f;
    a.status = p->status;
    a.n_heads = p->n_heads;
    a.n_items = p->n_heads * p->n_seqs;
    // the fewest CTAs that finish in the same number of rounds: 768 items take three rounds on 296 groups and on 256 alike,
    // and the SMs left out do not draw power (the sustained rate is power-capped)
    int grid = std::max(1, std::min(n_sms, a.n_items));
    if (a.n_items > n_sms) {
        const int rounds = (a.n_items + 2 * n_sms - 1) / (2 * n_sms);
        grid = std::min(n_sms, ((a.n_items + rounds - 1) / rounds + 1) / 2);
    }
    const cudaError_t e = kv_box == 224 ? launch_pdl(attn_tc_kernel<224>, dim3(grid), dim3(kTcThreads), kTcSmem, st, 1, tq, tk, tv, a)
                                        : launch_pdl(attn_tc_kernel<256>, dim3(grid), dim3(kTcThreads), kTcSmem, st, 1, tq, tk, tv, a);
    return e == cudaSuccess ? ITTAI_OK : cuda_fail(e, "launch attn_tc_kernel");
}

}  // namespace ittai
