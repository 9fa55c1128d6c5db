// Qwen3-0.6B decode: one persistent cooperative kernel per launch runs n_steps tokens; the chosen token id is fed
// back on the device.
//
//  * Data flow instead of grid barriers: every vector one phase hands to the next travels as flagged 64- or 128-bit words
//    (payload + tag of the producing step and layer), and a consumer polls exactly the words it needs (qwen3_ws.h).
//  * Weight stream: each CTA's slices of the layer matrices and of the KV cache are pulled into a shared-memory ring by
//    TMA bulk copies issued far ahead of use (weight_stream.cuh), so HBM keeps streaming while phases wait on each other.
//  * Batch-1 decode is HBM-bound (about 1.4 flop per weight byte): each warp multiplies whole 1024-column weight
//    sub-rows with 128-bit accesses and reduces with shuffles.  With several sequences the GEMV phases use warp-level
//    tensor-core tiles with the sequences as the N dimension (gemv_tile).
//
// Rounding points follow the eager modules: every Linear output, norm output, rotary product and sum, SiLU, gate*up
// product and residual sum is rounded to bf16 exactly once.  The math per phase mirrors the fused epilogues of the
// reference's megakernel (src/ittai/qwen3/base.py:80-129 for qkv / residual / gate-up, :147-162 for the embedding row),
// re-cut for one token: the row-norm scale is applied before the GEMV instead of after the GEMM, and keys and values go
// straight into the cache instead of a staging matrix.  KV cache, split-K decode attention, lm_head and argmax have no
// counterpart in the reference.
#include "common.cuh"
#include "qwen3_ws.h"
#include "weight_stream.cuh"

namespace ittai {

constexpr int D = ITTAI_Q3_D, NKV = ITTAI_Q3_NKV, HD = ITTAI_Q3_HD, FF = ITTAI_Q3_FF;
constexpr int DQ = ITTAI_Q3_DQ, DKV = ITTAI_Q3_DKV, DQKV = ITTAI_Q3_DQKV, DGU = ITTAI_Q3_DGU;
constexpr int kHoldMaxTiles = 2;                 // longest attention split (ring tiles) that still hands its tiles back in pairs
constexpr int kTile = 128;                       // cache positions per attention tile = one ring entry of K and one of V
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kPartFloats = 12 * 16;             // at most 12 tiles (16 rows x 256 columns) per CTA and phase
constexpr int kStreamPhases = 5;                 // phases of a layer whose weights or cache rows come through the ring (as does the head's table)

// ---- shared-memory plan (dynamic): header | activations or attention scratch | weight ring -----------------
struct SmemHdr {
    StreamShared stream;
    float red[kWarps * ITTAI_MAX_BATCH];         // per-warp partial sums of the norm
    int pos0[ITTAI_MAX_BATCH];                   // cache lengths at kernel entry
    int pos_s[ITTAI_MAX_BATCH];
    int tok_s[ITTAI_MAX_BATCH];
    float bestv[kWarps];
    int besti[kWarps];
    float sub[kPartFloats * ITTAI_MAX_BATCH];    // partial dot products of the GEMV tiles: [task][16 rows][sequence]
    float candv[Q3_MAX_CTAS];                    // argmax candidates of every CTA
    int candi[Q3_MAX_CTAS];
    long long t_ready;                           // cycle counter when the current phase had its inputs (in-kernel profile)
};
struct SmemAttn {
    float qs[2][HD];                             // rotated, pre-scaled queries of the two heads of a group
    float wm[kWarps][2], wl[kWarps][2];          // per-warp running max and sum
    bf16 knew[HD];
    bf16 vnew[HD];
    uint32_t pub[HD];                            // merged output pairs of this CTA on their way into 128-bit words
    float ored[kWarps][2][HD];
};
constexpr size_t kHdrBytes = (sizeof(SmemHdr) + 255) / 256 * 256;
__host__ __device__ constexpr size_t q3_fixed_smem_bytes(int nb) {
    size_t xs = (size_t)nb * (FF / 2) * sizeof(uint32_t);      // activations as packed bf16 pairs
    size_t at = sizeof(SmemAttn);
    return kHdrBytes + ((xs > at ? xs : at) + 255) / 256 * 256;
}

struct Cta {
    const IttaiQwen3Decode& p;
    const Q3Workspace& ws;   // the kernel's own parameter (read from constant memory where a pointer is used) at batch 1 and 2,
                             // a register copy at batch 4 and 8: see ITTAI_MAKE_CTA
    SmemHdr* hdr;
    uint32_t* xs;       // [NB][FF/2] activations of the current GEMV as packed bf16 pairs (they are bf16 values: half the
                        // shared-memory traffic of fp32 and conflict-free 128-bit reads)
    SmemAttn* at;       // aliases xs
    int cta, ncta, tid, lane, warp;
    Waiter w;
    Stream st;
    int step;           // token index inside this launch
};

// Tag of the data a (step, layer) produces; layer n_layers names the stream entering the head.  Never zero.
// In-kernel profile: thread 0 notes when the current phase had its inputs (in shared memory: a stamp kept in the context
// would hold two registers across every phase, in a kernel that runs at its register limit).
__device__ __forceinline__ void mark_ready(const Cta& c) {
    if (c.p.phase_clk != nullptr && c.tid == 0) c.hdr->t_ready = clock64();
}
__device__ __forceinline__ uint32_t tag_of(const Cta& c, int step, int l) { return (uint32_t)(step * (c.p.n_layers + 1) + l + 1); }

// CTA-uniform verdict on per-thread waits.
__device__ __forceinline__ bool all_ok(bool ok) { return !cta_or(!ok); }

__host__ __device__ __forceinline__ void split_range(int n, int parts, int i, int& lo, int& hi) {
    lo = (int)(((unsigned)n * (unsigned)i) / (unsigned)parts);          // n * parts stays far below 2^32
    hi = (int)(((unsigned)n * (unsigned)(i + 1)) / (unsigned)parts);
}

__device__ __forceinline__ int attn_splits(int ncta, int batch) {
    int s = ncta / (batch * NKV);
    return s < 1 ? 1 : (s > Q3_MAX_SPLITS ? Q3_MAX_SPLITS : s);
}

// The attention work of this CTA at one step: item (b, g, s) = CTA index; its cache range [start, start + n_old) of
// rows written by earlier tokens, and whether the token being computed (row `pos`) falls into its split.
struct AttnItem {
    bool active;
    int b, g, s, pos, start, n_old;
    bool has_new;
};
__device__ __forceinline__ AttnItem attn_item(const Cta& c, int step) {
    AttnItem it;
    const int B = c.p.batch, n_splits = attn_splits(c.ncta, B);
    it.active = c.cta < B * NKV * n_splits;
    const int item = it.active ? c.cta : 0;
    it.b = item / (NKV * n_splits); it.g = (item / n_splits) % NKV; it.s = item % n_splits;
    it.pos = c.hdr->pos0[it.b] + step;
    const int n_ctx = it.pos + 1;
    const int chunk = (((n_ctx + n_splits - 1) / n_splits) + 31) & ~31;
    it.start = it.s * chunk;
    const int end = it.start + chunk < n_ctx ? it.start + chunk : n_ctx;
    it.has_new = it.active && it.pos >= it.start && it.pos < it.start + chunk;
    const int lim = end < it.pos ? end : it.pos;         // the row of the current token never comes from the cache
    it.n_old = it.active && lim > it.start ? lim - it.start : 0;
    return it;
}

// ---- the static sequence of streamed slices ---------------------------------------------------------------
// Phase index k counts (step, layer, phase) in execution order, 5 * L + 1 phases per step (the last one is the head):
// k = step * (5 L + 1) + l * 5 + ph.  Attention contributes 2 * ceil(n_old / kTile) entries (K tile, V tile, K tile,
// ...), the head ceil(rows / kHeadRows) entries on steps that run it, every other phase exactly one.
constexpr int kHeadRows = 32;                    // table rows per streamed head entry (two per warp)

__device__ __forceinline__ bool head_runs(const Cta& c, int step) { return step >= c.p.n_forced - 1; }

// The issuing lane's whole life: walk phases [k_begin, k_end) in execution order, launch every slice as soon as the
// ring has room, then wait for the last copies to land.  It stops early when the compute threads raise `stop`.
// Slice addresses are linear in the layer index, so everything but one small division per step is hoisted.
//
// Cache tiles and the row appended one step earlier: the K/V tiles of (step s, layer l) contain the row that some CTA
// appended at (step s - 1, layer l).  The appending thread stores the row and fences (gpu scope, then the proxy fence for
// the TMA unit) before its CTA publishes its split's partial, and the attention output of (s - 1, l) needs every partial;
// so the tiles are held back until this CTA's compute threads have received that whole output and said so in `kv_epoch`.
// The hold costs nothing (the condition was met a whole token ago, except with a single layer), and it replaces an
// ordering that used to rest on the ring being smaller than what a CTA streams between the two points.  The observing
// side carries no gpu-scope fence of its own: the bulk copy reads L2, where the fenced row already is when any word
// that depends on it can be seen, and a fence.acq_rel.gpu on this side was measured at 7 us per token of a 256-token
// run in a warp of its own, 10-13 us in a compute thread, 210 us in the feeding lane with its copies in flight.
__device__ void stream_feed(const Cta& c, int k_begin, int k_end) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t limit = c.w.limit;
    const int L = p.n_layers, PS = kStreamPhases * L + 1;
    int lo, hi;
    // per-phase: base of this CTA's slice in layer 0, bytes between layers, bytes of the slice (tables indexed by the
    // phase live in local memory: 12 loads per layer in this lane only; the same values as named scalars picked by a
    // chain of selects were measured 12 us per token slower)
    const char* base[kStreamPhases];
    size_t stride[kStreamPhases];
    uint32_t nbytes[kStreamPhases];
    split_range(DQKV / 4, c.ncta, c.cta, lo, hi);    // 128-bit words of the projection: two row pairs each
    lo *= 2; hi *= 2;
    base[ITTAI_PH_QKV] = reinterpret_cast<const char*>(p.wqkv) + (size_t)2 * lo * D * 2;
    stride[ITTAI_PH_QKV] = (size_t)DQKV * D * 2; nbytes[ITTAI_PH_QKV] = (uint32_t)(hi - lo) * 2 * D * 2;
    split_range(D / 2, c.ncta, c.cta, lo, hi);
    base[ITTAI_PH_OPROJ] = reinterpret_cast<const char*>(p.wo) + (size_t)2 * lo * DQ * 2;
    stride[ITTAI_PH_OPROJ] = (size_t)D * DQ * 2; nbytes[ITTAI_PH_OPROJ] = (uint32_t)(hi - lo) * 2 * DQ * 2;
    base[ITTAI_PH_DOWN] = reinterpret_cast<const char*>(p.wd) + (size_t)2 * lo * FF * 2;
    stride[ITTAI_PH_DOWN] = (size_t)D * FF * 2; nbytes[ITTAI_PH_DOWN] = (uint32_t)(hi - lo) * 2 * FF * 2;
    split_range(FF / 6, c.ncta, c.cta, lo, hi);      // 128-bit words of the SwiGLU output: three units of four rows each
    lo *= 3; hi *= 3;
    base[ITTAI_PH_GU] = reinterpret_cast<const char*>(p.wgu) + (size_t)4 * lo * D * 2;
    stride[ITTAI_PH_GU] = (size_t)DGU * D * 2; nbytes[ITTAI_PH_GU] = (uint32_t)(hi - lo) * 4 * D * 2;
    base[ITTAI_PH_ATTN] = nullptr; stride[ITTAI_PH_ATTN] = (size_t)p.batch * NKV * p.kv_cap * HD * 2; nbytes[ITTAI_PH_ATTN] = 0;
    int h_lo, h_hi;
    split_range(p.vocab, c.ncta, c.cta, h_lo, h_hi);

    const int step_begin = k_begin / PS, step_end = (k_end + PS - 1) / PS;
    for (int step = step_begin; step < step_end; ++step) {
        const AttnItem it = attn_item(c, step);
        const size_t head0 = (((size_t)it.b * NKV + it.g) * (size_t)p.kv_cap + it.start) * HD * 2;   // bytes, layer 0
        const int n_kv = 2 * ((it.n_old + kTile - 1) / kTile);
        const int n_head = head_runs(c, step) ? (h_hi - h_lo + kHeadRows - 1) / kHeadRows : 0;
        int k = step * PS;
        for (int r = 0; r < PS; ++r, ++k) {
            if (k < k_begin || k >= k_end) continue;
            const int l = r / kStreamPhases, ph = r == PS - 1 ? ITTAI_PH_HEAD : r % kStreamPhases;
            const int n = ph == ITTAI_PH_HEAD ? n_head : (ph == ITTAI_PH_ATTN ? n_kv : 1);
            if (ph == ITTAI_PH_ATTN && n > 0 && step > 0) {
                const uint32_t need = (uint32_t)((step - 1) * L + l) + 1u;
                uint32_t spins = 0;
                while (ld_acquire_cta(&c.st.sh->kv_epoch) < need) {
                    if (c.st.sh->stop != 0u || ++spins > (limit << 4)) { stream_drain(c.st, limit); return; }
                }
            }
            for (int tile = 0; tile < n; ++tile) {
                const char* src;
                uint32_t bytes, off;
                if (ph == ITTAI_PH_HEAD) {
                    const int row = h_lo + tile * kHeadRows, rows = h_hi - row < kHeadRows ? h_hi - row : kHeadRows;
                    src = reinterpret_cast<const char*>(p.embed) + (size_t)row * D * 2;
                    bytes = (uint32_t)rows * D * 2;
                } else if (ph == ITTAI_PH_ATTN) {
                    const int j = tile >> 1, rows = it.n_old - j * kTile < kTile ? it.n_old - j * kTile : kTile;
                    src = reinterpret_cast<const char*>((tile & 1) ? p.vcache : p.kcache) + (size_t)l * stride[ITTAI_PH_ATTN] +
                          head0 + (size_t)j * kTile * HD * 2;
                    bytes = (uint32_t)rows * HD * 2;
                } else {
                    src = base[ph] + (size_t)l * stride[ph];
                    bytes = nbytes[ph];
                }
                if (bytes == 0) continue;
                uint32_t spins = 0;
                while (!stream_alloc(c.st, bytes, off)) {
                    if (c.st.sh->stop != 0u) { stream_drain(c.st, limit); return; }
                    if (++spins > (limit << 4)) {       // the compute threads never handed the space back
                        report_status(c.w.status, c.w.sync, ITTAI_ST_STREAM_TIMEOUT, (uint32_t)k, blockIdx.x, bytes, 0xffffffffu);
                        stream_drain(c.st, limit);
                        return;
                    }
                }
                stream_issue(c.st, off, src, bytes);
            }
        }
    }
    stream_drain(c.st, limit);
}

// Entry number n of the stream, with a CTA-uniform verdict.
__device__ __forceinline__ const bf16* stream_acquire(Cta& c, uint32_t n, bool& ok) {
    const unsigned char* ptr = stream_wait(c.st, n, c.w);
    ok = all_ok(ptr != nullptr);
    return reinterpret_cast<const bf16*>(ptr);
}

// ---- RMSNorm of one row (already in registers, one bf16 pair per thread) into shared memory --------------
// xs[i] = bf16(bf16(x*rstd) * gain): the value the following Linear sees in the eager model.
// NB rows (one bf16 pair per thread each) -> xs[b][i] = bf16(bf16(x*rstd) * gain), the value the following Linear sees in
// the eager model.  `gw` is this thread's pair of gains, loaded by the caller BEFORE it waits for the input: a global
// load issued after the wait would put a full memory round trip on the critical path of every layer.  `ok` is this
// thread's verdict on the waits that produced `u`; the first barrier both publishes the per-warp sums of squares and
// collects the verdicts.  Returns false (uniformly) when any thread's wait failed.
// With `ring_entry` non-null the wait for this phase's weights in the ring is folded in: its verdict rides on the barrier
// that publishes xs, instead of costing a barrier of its own.
template <int NB>
__device__ __forceinline__ bool norm_pairs_to_smem(Cta& c, const uint32_t (&u)[NB], uint32_t gw, bool ok,
                                                   const bf16** ring_entry = nullptr) {
    static_assert(kThreads * 2 == D, "one bf16 pair per thread");
    static_assert(NB * kWarps <= 32 * 4, "per-warp partial sums must fit the scratch");
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const float x0 = bf_lo(u[b]), x1 = bf_hi(u[b]);
        const float v = warp_sum(x0 * x0 + x1 * x1);
        if (c.lane == 0) c.hdr->red[b * kWarps + c.warp] = v;
    }
    if (cta_or(!ok)) return false;
    mark_ready(c);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) tot += c.hdr->red[b * kWarps + i];
        const float rstd = 1.0f / sqrtf(tot * (1.0f / D) + c.p.eps);
        c.xs[b * (FF / 2) + c.tid] = pack_bf16x2(bf16r(bf_lo(u[b]) * rstd) * bf_lo(gw), bf16r(bf_hi(u[b]) * rstd) * bf_hi(gw));
    }
    if (ring_entry != nullptr) {
        const unsigned char* ptr = stream_wait(c.st, c.st.consumed, c.w);
        *ring_entry = reinterpret_cast<const bf16*>(ptr);
        return !cta_or(ptr == nullptr);
    }
    cta_sync();
    return true;
}

// Waits for NB rows of K bf16 values in 128-bit flagged words and spreads them into xs: K = 2048 (attention output) has
// four values per word, K = 3072 (SwiGLU output) six, so every thread polls exactly one word per row.
template <int NB, int K>
__device__ __forceinline__ bool wait_rows_to_smem(Cta& c, const uint64_t* src, uint32_t tag, int what, const bf16** ring_entry = nullptr) {
    constexpr int V = K / kThreads;              // values per word
    static_assert(V == 4 || V == 6, "one 128-bit word per thread");
    uint32_t u0[NB], u1[NB], u2[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) u0[b] = u1[b] = u2[b] = 0u;
    bool ok = wait_words128<NB>(c.w, reinterpret_cast<const uint4*>(src) + c.tid, kThreads, tag, u0, u1, u2, what);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        uint32_t* dst = c.xs + b * (FF / 2) + c.tid * (V / 2);
        dst[0] = u0[b]; dst[1] = u1[b];
        if constexpr (V == 6) dst[2] = u2[b];
    }
    if (ring_entry != nullptr) {
        const unsigned char* ptr = stream_wait(c.st, c.st.consumed, c.w);
        *ring_entry = reinterpret_cast<const bf16*>(ptr);
        ok = ok && ptr != nullptr;
    }
    return all_ok(ok);
}

// ---- 1024-column sub-row dot products ------------------------------------------------------------------
// Lane owns the 16-byte chunks lane, lane+32, lane+64, lane+96 of a sub-row: four independent 128-bit accesses per
// sub-row, R sub-rows at a time.  Batch 1 keeps its 32 activations in registers; larger batches read shared memory.
// GLOBAL selects streaming global loads (the head's table) over the shared-memory ring.
template <bool GLOBAL>
__device__ __forceinline__ uint4 load_w(const bf16* p) {
    if constexpr (GLOBAL) return ldg_stream(p);
    else return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ void load_xreg(const uint32_t* xs, int lane, float (&xr)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 q = *reinterpret_cast<const uint4*>(xs + (lane + 32 * i) * 4);
        xr[i * 8 + 0] = bf_lo(q.x); xr[i * 8 + 1] = bf_hi(q.x); xr[i * 8 + 2] = bf_lo(q.y); xr[i * 8 + 3] = bf_hi(q.y);
        xr[i * 8 + 4] = bf_lo(q.z); xr[i * 8 + 5] = bf_hi(q.z); xr[i * 8 + 6] = bf_lo(q.w); xr[i * 8 + 7] = bf_hi(q.w);
    }
}

template <bool GLOBAL, int R>
__device__ __forceinline__ void dot_subrows_xreg(const bf16* const (&wp)[R], const float (&xr)[32], int lane,
                                                 float (&acc)[R]) {
    uint4 w[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[r][i] = load_w<GLOBAL>(wp[r] + (lane + 32 * i) * 8);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = dot8(w[r][i], &xr[i * 8], 0.f);      // four independent chains
        acc[r] = warp_sum((a[0] + a[1]) + (a[2] + a[3]));
    }
}

// xseg points at the 1024-value segment (512 words) this sub-row multiplies, for batch row 0; batch rows are FF/2 words apart.
template <bool GLOBAL, int NB, int R>
__device__ __forceinline__ void dot_subrows_smem(const bf16* const (&wp)[R], const uint32_t* const (&xseg)[R], int lane,
                                                 float (&acc)[R][NB]) {
    uint4 w[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[r][i] = load_w<GLOBAL>(wp[r] + (lane + 32 * i) * 8);
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 q = *reinterpret_cast<const uint4*>(xseg[r] + b * (FF / 2) + (lane + 32 * i) * 4);
                const float xv[8] = {bf_lo(q.x), bf_hi(q.x), bf_lo(q.y), bf_hi(q.y), bf_lo(q.z), bf_hi(q.z), bf_lo(q.w), bf_hi(q.w)};
                a = dot8(w[r][i], xv, a);
            }
            acc[r][b] = warp_sum(a);
        }
}

// Generic "R sub-rows" step used by all K=1024 phases.
template <bool GLOBAL, int NB, int R>
__device__ __forceinline__ void dot_rows_k1024(Cta& c, const bf16* const (&wp)[R], const float (&xr)[32],
                                               float (&acc)[R][NB]) {
    if constexpr (NB == 1) {
        float a[R];
        dot_subrows_xreg<GLOBAL, R>(wp, xr, c.lane, a);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r][0] = a[r];
    } else {
        const uint32_t* xseg[R];
#pragma unroll
        for (int r = 0; r < R; ++r) xseg[r] = c.xs;
        dot_subrows_smem<GLOBAL, NB, R>(wp, xseg, c.lane, acc);
    }
}

// ---- GEMV tiles on the tensor cores --------------------------------------------------------------------
// One warp multiplies 16 weight rows x 256 columns with the activations of up to eight sequences: D[row, seq] as
// sixteen m16n8k16 MMAs, the sequences as the N dimension (at batch 1 seven of the eight columns repeat the first and
// are ignored).  A lane reads 8 consecutive weights of row g and of row g + 8 per 32-column window (one 128-bit access
// each) and the matching 8 activations of sequence g; which of the window's columns an MMA k-index stands for is free
// as long as A and B agree, so no transposing load is needed.  Rows past `n_rows` repeat the last row (their results
// are dropped by the caller).  `W`: row-major slice in shared memory, `ld` elements per row; `xs`: packed bf16 pairs,
// FF/2 words per sequence.  Replaces 12 instructions per 8 weights (unpack + packed FMAs) by 3 per 128.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <int NB>
__device__ __forceinline__ void gemv_tile(const bf16* W, int ld, int r0, int n_rows, const uint32_t* xs, int k0, int lane, float (&d)[4]) {
    const int g = lane >> 2, t = lane & 3;
    const int ra = r0 + g < n_rows ? r0 + g : n_rows - 1, rb = r0 + g + 8 < n_rows ? r0 + g + 8 : n_rows - 1;
    const bf16* pa = W + (size_t)ra * ld + k0 + 8 * t;
    const bf16* pb = W + (size_t)rb * ld + k0 + 8 * t;
    const uint32_t* px = xs + (g % NB) * (FF / 2) + (k0 >> 1) + 4 * t;
    float e[4] = {0.f, 0.f, 0.f, 0.f}, f[4] = {0.f, 0.f, 0.f, 0.f}, h[4] = {0.f, 0.f, 0.f, 0.f};
    d[0] = 0.f; d[1] = 0.f; d[2] = 0.f; d[3] = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w += 2) {                 // four independent accumulation chains of four MMAs each
        const uint4 va = *reinterpret_cast<const uint4*>(pa + 32 * w), va2 = *reinterpret_cast<const uint4*>(pa + 32 * w + 32);
        const uint4 vb = *reinterpret_cast<const uint4*>(pb + 32 * w), vb2 = *reinterpret_cast<const uint4*>(pb + 32 * w + 32);
        const uint4 vx = *reinterpret_cast<const uint4*>(px + 16 * w), vx2 = *reinterpret_cast<const uint4*>(px + 16 * w + 16);
        mma_bf16_16816(d, va.x, vb.x, va.y, vb.y, vx.x, vx.y);      // columns 8t .. 8t+3 of the window
        mma_bf16_16816(e, va.z, vb.z, va.w, vb.w, vx.z, vx.w);      // columns 8t+4 .. 8t+7
        mma_bf16_16816(f, va2.x, vb2.x, va2.y, vb2.y, vx2.x, vx2.y);
        mma_bf16_16816(h, va2.z, vb2.z, va2.w, vb2.w, vx2.z, vx2.w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = (d[i] + e[i]) + (f[i] + h[i]);
}
// Lane (g, t) holds rows g, g + 8 of sequences 2t, 2t + 1: part[(task * 16 + row) * NB + seq].
template <int NB>
__device__ __forceinline__ void gemv_store(float* part, int task, int lane, const float (&d)[4]) {
    const int g = lane >> 2, t = lane & 3;
    float* p0 = part + (size_t)(task * 16 + g) * NB;
    float* p1 = part + (size_t)(task * 16 + g + 8) * NB;
    if (2 * t < NB) { p0[2 * t] = d[0]; p1[2 * t] = d[2]; }
    if (2 * t + 1 < NB) { p0[2 * t + 1] = d[1]; p1[2 * t + 1] = d[3]; }
}
// Sum of the NK column-block partials of local row `row` for sequence b, in fixed order.
template <int NB, int NK>
__device__ __forceinline__ float gemv_sum(const float* part, int row, int b) {
    const int blk = row >> 4, rr = row & 15;
    float v[NK];
#pragma unroll
    for (int kq = 0; kq < NK; ++kq) v[kq] = part[(size_t)((blk * NK + kq) * 16 + rr) * NB + b];
    float s = v[0];
#pragma unroll
    for (int kq = 1; kq < NK; ++kq) s += v[kq];
    return s;
}

// ---- phase: embed gather (layer 0) + RMSNorm + QKV GEMV ------------------------------------------------
template <int NB>
__device__ bool phase_qkv(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t tag = tag_of(c, c.step, l);
    const uint32_t gw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const bf16*>(p.ln1) + (size_t)l * D + 2 * c.tid);
    uint32_t u[NB];
    bool ok = true;
    if (l == 0) {
#pragma unroll
        for (int b = 0; b < NB; ++b) u[b] = ldcg32(reinterpret_cast<const bf16*>(p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * c.tid);
    } else {
        ok = wait_words<NB>(c.w, c.ws.h + c.tid, D / 2, tag, u, ITTAI_PH_QKV);
    }
    int p0, p1;
    split_range(DQKV / 4, c.ncta, c.cta, p0, p1);    // 128-bit words: two row pairs (four outputs) each
    p0 *= 2; p1 *= 2;
    const bf16* W = nullptr;                                   // this CTA's rows [2*p0, 2*p1), contiguous in the ring
    if (!norm_pairs_to_smem<NB>(c, u, gw, ok, p1 > p0 ? &W : nullptr)) return false;
    if (p1 == p0) return true;
    if constexpr (NB == 1) {
        // one sequence: a row pair per warp on the fp32 pipes (the tensor-core tiles below are no faster here)
        float xr[32];
        if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
        uint32_t* pub = reinterpret_cast<uint32_t*>(c.hdr->sub);      // this CTA's packed outputs, [row pair][sequence]
        for (int pr = p0 + c.warp; pr < p1; pr += kWarps) {
            const bf16* wp[2] = {W + (size_t)(2 * (pr - p0)) * D, W + (size_t)(2 * (pr - p0) + 1) * D};
            float acc[2][NB];
            dot_rows_k1024<false, NB, 2>(c, wp, xr, acc);
            if (c.lane == 0) {
#pragma unroll
                for (int b = 0; b < NB; ++b) pub[(pr - p0) * NB + b] = pack_bf16x2(acc[0][b], acc[1][b]);
            }
        }
        stream_release(c.st, 1);                         // its barrier also publishes `pub` to the CTA
        for (int i = c.tid; i < (p1 - p0) / 2 * NB; i += kThreads) {
            const int wq = i / NB, b = i % NB;
            st_flagged128(reinterpret_cast<uint4*>(c.ws.qkv) + (size_t)b * (DQKV / 4) + p0 / 2 + wq,
                          pub[(2 * wq) * NB + b], pub[(2 * wq + 1) * NB + b], 0u, tag);
        }
    } else {
        // tiles of 16 rows x 256 columns over the warps; the four column blocks of a row meet in shared memory
        const int n_rows = 2 * (p1 - p0), n_tasks = (n_rows + 15) / 16 * 4;
        float* part = c.hdr->sub;
        for (int task = c.warp; task < n_tasks; task += kWarps) {
            float d[4];
            gemv_tile<NB>(W, D, (task >> 2) * 16, n_rows, c.xs, (task & 3) * 256, c.lane, d);
            gemv_store<NB>(part, task, c.lane, d);
        }
        stream_release(c.st, 1);                         // its barrier also publishes `part` to the CTA
        for (int i = c.tid; i < (p1 - p0) / 2 * NB; i += kThreads) {     // four rows leave as one 128-bit word
            const int wq = i / NB, b = i % NB;
            const float r0 = gemv_sum<NB, 4>(part, 4 * wq, b), r1 = gemv_sum<NB, 4>(part, 4 * wq + 1, b);
            const float r2 = gemv_sum<NB, 4>(part, 4 * wq + 2, b), r3 = gemv_sum<NB, 4>(part, 4 * wq + 3, b);
            st_flagged128(reinterpret_cast<uint4*>(c.ws.qkv) + (size_t)b * (DQKV / 4) + p0 / 2 + wq,
                          pack_bf16x2(r0, r1), pack_bf16x2(r2, r3), 0u, tag);
        }
    }
    return true;
}

// 2^x on the special-function unit without exp2f's range fix-ups (2^-inf = 0; arguments here are differences of
// finite log2-domain scores or -inf).
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- phase: QK-RMSNorm + RoPE + KV append + split-K GQA attention + merge -----------------------------
// Work item = (sequence b, kv head g, split s) = CTA index.  Scores live in the log2 domain with the softmax scale
// folded into q, as the reference does (src/ittai/qwen3/config.py:6-7).  Old cache rows arrive through the ring in tiles
// of 128 positions (a K entry and a V entry per tile); the row of the token being computed is taken from shared memory
// and appended to the cache by the split that owns its position.  Each split publishes (m, l, o[2][128]); the first
// `nc` splits of a head then each merge a slice of the 256 outputs.
template <int NB>
__device__ bool phase_attn(Cta& c, int l) {
    // Four or more sequences: a CTA walks many tiles, and the scores q k of a tile come from the tensor cores (below).
    // One sequence keeps the fp32 dot products (its two tiles per CTA run at the memory rate as they are), and so do
    // two (measured 1.4 % slower per step with the tensor-core scores).
    constexpr bool kMmaScores = NB >= 4;
    const IttaiQwen3Decode& p = c.p;
    const int B = p.batch;
    const int n_splits = attn_splits(c.ncta, B);
    const uint32_t tag = tag_of(c, c.step, l);
    SmemAttn* at = c.at;
    const AttnItem it = attn_item(c, c.step);
    if (it.active) {
        const int b = it.b, g = it.g, pos = it.pos;
        const bool has_new = it.has_new;
        const size_t head_off = ((((size_t)l * B + b) * NKV + g) * (size_t)p.kv_cap) * HD;
        bf16* kc = reinterpret_cast<bf16*>(p.kcache) + head_off;
        bf16* vc = reinterpret_cast<bf16*>(p.vcache) + head_off;

        // -- norm + rotate q (warps 0,1) and the new key (warp 2); copy the new value (warp 3).
        //    The row arrives as 32 words of four values: a lane owns elements 4*lane .. 4*lane+3, and the rotation
        //    partner (element +-64) of each sits in lane ^ 16.  Gains and the rotary row are fetched before the wait, so
        //    their latency hides behind it.
        const uint4* qw = reinterpret_cast<const uint4*>(c.ws.qkv) + (size_t)b * (DQKV / 4);
        bool ok = true;
        if (c.warp < 3 && (c.warp < 2 || has_new)) {
            const bool is_k = c.warp == 2;
            const int e0 = is_k ? DQ + g * HD : (2 * g + c.warp) * HD;
            const bf16* gain = reinterpret_cast<const bf16*>(is_k ? p.kn : p.qn) + (size_t)l * HD;
            const bf16* rp = reinterpret_cast<const bf16*>(p.rope) + (size_t)pos * HD;
            const int hi_half = c.lane >> 4, ei = 4 * (c.lane & 15);        // rotation index of this lane's first element
            const uint2 gq = *reinterpret_cast<const uint2*>(gain + 4 * c.lane);
            const uint2 cq = *reinterpret_cast<const uint2*>(rp + ei);
            const uint2 sq = *reinterpret_cast<const uint2*>(rp + HD / 2 + ei);
            uint32_t ua = 0, ub = 0, uc = 0;
            ok = wait_word128(c.w, qw + e0 / 4 + c.lane, tag, ua, ub, uc, ITTAI_PH_ATTN);
            float x[4] = {bf_lo(ua), bf_hi(ua), bf_lo(ub), bf_hi(ub)};
            const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
            const float rstd = 1.0f / sqrtf(ss * (1.0f / HD) + p.eps);
            const float gn[4] = {bf_lo(gq.x), bf_hi(gq.x), bf_lo(gq.y), bf_hi(gq.y)};
            const float cs[4] = {bf_lo(cq.x), bf_hi(cq.x), bf_lo(cq.y), bf_hi(cq.y)};
            const float sn[4] = {bf_lo(sq.x), bf_hi(sq.x), bf_lo(sq.y), bf_hi(sq.y)};
            float r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                x[j] = bf16r(bf16r(x[j] * rstd) * gn[j]);
                const float y = __shfl_xor_sync(0xffffffffu, x[j], 16);      // element j +- 64
                // pair (i, i+64): out[i] = x_i cos_i - x_{i+64} sin_i,  out[i+64] = x_{i+64} cos_i + x_i sin_i
                r[j] = hi_half ? bf16r(bf16r(x[j] * cs[j]) + bf16r(y * sn[j])) : bf16r(bf16r(x[j] * cs[j]) + bf16r(-y * sn[j]));
            }
            if (is_k) {
                const uint2 wk = make_uint2(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]));
                *reinterpret_cast<uint2*>(at->knew + 4 * c.lane) = wk;
                if (ok) {
                    *reinterpret_cast<uint2*>(kc + (size_t)pos * HD + 4 * c.lane) = wk;
                    __threadfence();
                    fence_proxy_async();       // later tokens read this row through the TMA unit
                }
            } else {
                const float qscale = 0.08838834764831845f * kLog2e;   // head_dim^-0.5 * log2(e)
                if constexpr (kMmaScores)     // the rotated query as it is (bf16 values), the scale goes onto the scores
                    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(at->qs[c.warp]) + 4 * c.lane) = make_uint2(pack_bf16x2(r[0], r[1]), pack_bf16x2(r[2], r[3]));
                else
                    *reinterpret_cast<float4*>(&at->qs[c.warp][4 * c.lane]) = make_float4(r[0] * qscale, r[1] * qscale, r[2] * qscale, r[3] * qscale);
            }
        } else if (c.warp == 3 && has_new) {
            const int e0 = DQ + DKV + g * HD;
            uint32_t ua = 0, ub = 0, uc = 0;
            ok = wait_word128(c.w, qw + e0 / 4 + c.lane, tag, ua, ub, uc, ITTAI_PH_ATTN);
            *reinterpret_cast<uint2*>(at->vnew + 4 * c.lane) = make_uint2(ua, ub);
            if (ok) {
                *reinterpret_cast<uint2*>(vc + (size_t)pos * HD + 4 * c.lane) = make_uint2(ua, ub);
                __threadfence();
                fence_proxy_async();
            }
        }
        if (!all_ok(ok)) return false;
        mark_ready(c);

        // -- every half-warp runs its own online softmax over the positions it owns (position index = 2*warp + half
        //    modulo 32), with no CTA-wide barrier inside a tile; the 32 private (m, l, o) are merged once at the end.
        const int half = c.lane >> 4, sub = c.lane & 15;
        float q0[8], q1[8], acc0[8], acc1[8];
        // Tensor-core scores: a warp owns 8 consecutive positions of a tile, rows 0-7 of an m16n8k16 A operand read
        // straight from the tile (rows 8-15 are zero); the two query heads are N columns.  Rows of a tile are 256 bytes
        // apart, so rows g and g + 1 read at the same columns would meet in the same banks: even rows read the first 32
        // dims of a 64-dim window while odd rows read the second 32, then the other way round, with N columns 0, 1
        // carrying the heads' values of the half the even rows hold and columns 2, 3 those of the half the odd rows
        // hold.  Row g's scores end up in D[g][2 (g & 1) + head], in lane 4 g + (g & 1).
        const int mg = c.lane >> 2, mt = c.lane & 3;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if constexpr (!kMmaScores) {
                q0[e] = at->qs[0][sub * 8 + e];
                q1[e] = at->qs[1][sub * 8 + e];
            }
            acc0[e] = 0.f; acc1[e] = 0.f;
        }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        // positions of this split: n_old rows from the ring, then (has_new) the current token's row
        const int n_pos = it.n_old + (has_new ? 1 : 0);
        const int n_ring_tiles = (it.n_old + kTile - 1) / kTile;
        int rel = 0;                 // ring tiles already handed back
        bool okr = true;
        // two tiles (K and V of each: 128 KB) are held before they go back, when the ring has room for that and more and
        // the split is those two tiles; a longer split hands every tile back at once, so that the feeding lane can stay
        // two tiles ahead instead of waiting for 128 KB to come free in one piece
        const int hold = (c.st.ring_bytes >= 5u * kTile * HD * 2 && n_ring_tiles <= kHoldMaxTiles) ? 2 : 1;
        for (int j = 0; j * kTile < n_pos; ++j) {
            const int ring_rows = it.n_old - j * kTile < 0 ? 0 : (it.n_old - j * kTile < kTile ? it.n_old - j * kTile : kTile);
            const bool from_ring = j < n_ring_tiles;
            const bf16* kt = nullptr;
            const bf16* vt = nullptr;
            if (from_ring) {
                const unsigned char* pk = stream_wait(c.st, c.st.consumed + 2 * (j - rel), c.w);
                const unsigned char* pv = stream_wait(c.st, c.st.consumed + 2 * (j - rel) + 1, c.w);
                // warp-uniform exit (the shuffles below need every lane); the CTA's verdict is collected at the next barrier
                if (__any_sync(0xffffffffu, pk == nullptr || pv == nullptr)) { okr = false; break; }
                kt = reinterpret_cast<const bf16*>(pk);
                vt = reinterpret_cast<const bf16*>(pv);
            }
            bool valid[kTile / 32];
            float s0[kTile / 32], s1[kTile / 32];
            if constexpr (kMmaScores) {
                const int tg = c.warp * 8 + mg;                  // the position whose key is row mg of this warp's A operand
                const bf16* krow = tg < ring_rows ? kt + (size_t)tg * HD : at->knew;
                const bool live = tg < ring_rows || (has_new && j * kTile + tg == it.n_old);
                float d[4] = {0.f, 0.f, 0.f, 0.f}, e4[4] = {0.f, 0.f, 0.f, 0.f};
                // the query fragments come from shared memory every tile (four broadcast reads): kept in registers across
                // the loop they are 16 of the 96 a thread has, and the loop spills
                const bf16* qrow = reinterpret_cast<const bf16*>(at->qs[mg & 1]) + 8 * mt;
#pragma unroll
                for (int wi = 0; wi < 2; ++wi)
#pragma unroll
                    for (int st = 0; st < 2; ++st) {
                        uint4 va = make_uint4(0u, 0u, 0u, 0u), qf = make_uint4(0u, 0u, 0u, 0u);
                        if (live) va = *reinterpret_cast<const uint4*>(krow + 64 * wi + 32 * ((mg & 1) ^ st) + 8 * mt);
                        if (mg < 4) qf = *reinterpret_cast<const uint4*>(qrow + 64 * wi + 32 * ((mg >> 1) ^ st));
                        mma_bf16_16816(d, va.x, 0u, va.y, 0u, qf.x, qf.y);
                        mma_bf16_16816(e4, va.z, 0u, va.w, 0u, qf.z, qf.w);
                    }
                const float qscale = 0.08838834764831845f * kLog2e;
                const float sa = (d[0] + e4[0]) * qscale, sb = (d[1] + e4[1]) * qscale;
#pragma unroll
                for (int r = 0; r < kTile / 32; ++r) {           // this half-warp's position of round r is row 2 r + half
                    const int tl = c.warp * 8 + 2 * r + half;
                    valid[r] = j * kTile + tl < n_pos;
                    const float a0 = __shfl_sync(0xffffffffu, sa, 8 * r + 5 * half), a1 = __shfl_sync(0xffffffffu, sb, 8 * r + 5 * half);
                    s0[r] = valid[r] ? a0 : -INFINITY;
                    s1[r] = valid[r] ? a1 : -INFINITY;
                }
            } else {
                uint4 kk[kTile / 32];
#pragma unroll
                for (int r = 0; r < kTile / 32; ++r) {
                    const int tl = r * 32 + c.warp * 2 + half;
                    valid[r] = j * kTile + tl < n_pos;
                    if (tl < ring_rows) kk[r] = *reinterpret_cast<const uint4*>(kt + (size_t)tl * HD + sub * 8);
                    else if (has_new && j * kTile + tl == it.n_old) kk[r] = *reinterpret_cast<const uint4*>(at->knew + sub * 8);
                    else kk[r] = make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int r = 0; r < kTile / 32; ++r) {
                    float a0 = dot8(kk[r], q0, 0.f), a1 = dot8(kk[r], q1, 0.f);
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) {
                        a0 += __shfl_xor_sync(0xffffffffu, a0, o);
                        a1 += __shfl_xor_sync(0xffffffffu, a1, o);
                    }
                    s0[r] = valid[r] ? a0 : -INFINITY;
                    s1[r] = valid[r] ? a1 : -INFINITY;
                }
            }
            float mt0 = m0, mt1 = m1;
#pragma unroll
            for (int r = 0; r < kTile / 32; ++r) { mt0 = fmaxf(mt0, s0[r]); mt1 = fmaxf(mt1, s1[r]); }
            const float ms0 = mt0 == -INFINITY ? 0.f : mt0, ms1 = mt1 == -INFINITY ? 0.f : mt1;   // no (-inf) - (-inf)
            const float c0 = ex2_approx(m0 - ms0), c1 = ex2_approx(m1 - ms1);
            l0 *= c0; l1 *= c1;
#pragma unroll
            for (int e = 0; e < 8; ++e) { acc0[e] *= c0; acc1[e] *= c1; }
#pragma unroll
            for (int r = 0; r < kTile / 32; ++r) {
                const float p0 = ex2_approx(s0[r] - ms0), p1 = ex2_approx(s1[r] - ms1);
                l0 += p0; l1 += p1;
                const int tl = kMmaScores ? c.warp * 8 + 2 * r + half : r * 32 + c.warp * 2 + half;
                uint4 vr = make_uint4(0, 0, 0, 0);
                if (tl < ring_rows) vr = *reinterpret_cast<const uint4*>(vt + (size_t)tl * HD + sub * 8);
                else if (has_new && j * kTile + tl == it.n_old) vr = *reinterpret_cast<const uint4*>(at->vnew + sub * 8);
                const uint32_t vw[4] = {vr.x, vr.y, vr.z, vr.w};
                const float2 pp0 = make_float2(p0, p0), pp1 = make_float2(p1, p1);
#pragma unroll
                for (int e = 0; e < 4; ++e) {       // packed fp32 FMAs: two dims per instruction
                    const float2 ve = make_float2(bf_lo(vw[e]), bf_hi(vw[e]));
                    const float2 r0 = __ffma2_rn(pp0, ve, make_float2(acc0[2 * e], acc0[2 * e + 1]));
                    const float2 r1 = __ffma2_rn(pp1, ve, make_float2(acc1[2 * e], acc1[2 * e + 1]));
                    acc0[2 * e] = r0.x; acc0[2 * e + 1] = r0.y; acc1[2 * e] = r1.x; acc1[2 * e + 1] = r1.y;
                }
            }
            m0 = mt0; m1 = mt1;
            // the half-warps never synchronise inside a tile; ring entries go back two tiles at a time (one CTA barrier
            // per 128 KB instead of two per tile), which is everything at batch 1
            if (from_ring && j - rel == hold - 1) { stream_release(c.st, 2 * hold); rel += hold; }
        }
        if (n_ring_tiles > rel) stream_release(c.st, 2 * (n_ring_tiles - rel));
        // -- merge the two halves of each warp, then the 16 warps, and publish (m, l, o) of this split
        {
            const float pm0 = __shfl_xor_sync(0xffffffffu, m0, 16), pm1 = __shfl_xor_sync(0xffffffffu, m1, 16);
            const float pl0 = __shfl_xor_sync(0xffffffffu, l0, 16), pl1 = __shfl_xor_sync(0xffffffffu, l1, 16);
            const float M0 = fmaxf(m0, pm0), M1 = fmaxf(m1, pm1);
            const float S0 = M0 == -INFINITY ? 0.f : M0, S1 = M1 == -INFINITY ? 0.f : M1;
            const float w0 = ex2_approx(m0 - S0), w1 = ex2_approx(m1 - S1), v0 = ex2_approx(pm0 - S0), v1 = ex2_approx(pm1 - S1);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float o0 = __shfl_xor_sync(0xffffffffu, acc0[e], 16), o1 = __shfl_xor_sync(0xffffffffu, acc1[e], 16);
                acc0[e] = acc0[e] * w0 + o0 * v0;
                acc1[e] = acc1[e] * w1 + o1 * v1;
            }
            if (half == 0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) { at->ored[c.warp][0][sub * 8 + e] = acc0[e]; at->ored[c.warp][1][sub * 8 + e] = acc1[e]; }
                if (sub == 0) {
                    at->wm[c.warp][0] = M0; at->wm[c.warp][1] = M1;
                    at->wl[c.warp][0] = l0 * w0 + pl0 * v0; at->wl[c.warp][1] = l1 * w1 + pl1 * v1;
                }
            }
        }
        if (cta_or(!okr)) return false;
        uint64_t* part = c.ws.part + (size_t)c.cta * Q3_PART_WORDS;
        if (c.tid < 2 * HD) {
            const int h = c.tid / HD, d = c.tid % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) M = fmaxf(M, at->wm[w][h]);
            const float Ms = M == -INFINITY ? 0.f : M;
            float o = 0.f, ls = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float sc = ex2_approx(at->wm[w][h] - Ms);
                o = fmaf(at->ored[w][h][d], sc, o);
                ls = fmaf(at->wl[w][h], sc, ls);
            }
            st_flagged(part + 4 + h * HD + d, __float_as_uint(o), tag);
            if (d == 0) {
                st_flagged(part + h, __float_as_uint(M), tag);
                st_flagged(part + 2 + h, __float_as_uint(ls), tag);
            }
        }
        cta_sync();
    } else {
        mark_ready(c);
    }
    // -- merge across splits: split s < nc of each (b, g) gathers, from every split of that head, the running max and
    //    sum and its own slice of the outputs
    int nc = 1;
    while (nc * 2 <= n_splits && nc < 16) nc *= 2;
    const int dpc = HD / nc, W = 4 + 2 * dpc;
    if (it.active && it.s < nc) {
        // a warp per pair of adjacent outputs, lanes = splits: each lane fetches (m, l, o, o) of its split in one round
        // trip, then three warp reductions finish the pair
        const int b = it.b, g = it.g, d0 = it.s * dpc;
        const uint64_t* base = c.ws.part + (size_t)(b * NKV + g) * n_splits * Q3_PART_WORDS;
        bool ok = true;
        for (int pr = c.warp; pr < dpc; pr += kWarps) {
            const int h = pr / (dpc / 2), dd = (pr % (dpc / 2)) * 2;
            float m = -INFINITY, l = 0.f, o0 = 0.f, o1 = 0.f;
            if (c.lane < n_splits) {
                const uint64_t* pk = base + (size_t)c.lane * Q3_PART_WORDS;
                const uint64_t* w4[4] = {pk + h, pk + 2 + h, pk + 4 + h * HD + d0 + dd, pk + 4 + h * HD + d0 + dd + 1};
                uint32_t spins = 0;
                for (;;) {
                    const uint64_t v0 = ld_flagged(w4[0]), v1 = ld_flagged(w4[1]), v2 = ld_flagged(w4[2]), v3 = ld_flagged(w4[3]);
                    if ((uint32_t)(v0 >> 32) == tag && (uint32_t)(v1 >> 32) == tag && (uint32_t)(v2 >> 32) == tag && (uint32_t)(v3 >> 32) == tag) {
                        m = __uint_as_float((uint32_t)v0); l = __uint_as_float((uint32_t)v1);
                        o0 = __uint_as_float((uint32_t)v2); o1 = __uint_as_float((uint32_t)v3);
                        break;
                    }
                    if (((++spins) & 1023u) == 0u &&
                        !keep_waiting(c.w.sync, c.w.status, c.w.limit, spins, 16 + ITTAI_PH_ATTN, (uint32_t)(v0 >> 32), tag)) { ok = false; break; }
                }
            }
            const float M = warp_max(m);
            const float wk = ex2_approx(m - (M == -INFINITY ? 0.f : M));
            const float Ls = warp_sum(l * wk), O0 = warp_sum(o0 * wk), O1 = warp_sum(o1 * wk);
            if (c.lane == 0) at->pub[pr] = pack_bf16x2(O0 / Ls, O1 / Ls);
        }
        if (!all_ok(ok)) return false;
        // two adjacent pairs (four outputs of one head) leave as one 128-bit word
        if (c.tid < dpc / 2) {
            const int h = c.tid / (dpc / 4), k4 = c.tid % (dpc / 4);
            st_flagged128(reinterpret_cast<uint4*>(c.ws.attn) + (size_t)b * (DQ / 4) + ((2 * g + h) * HD + d0) / 4 + k4,
                          at->pub[2 * c.tid], at->pub[2 * c.tid + 1], 0u, tag);
        }
    }
    return true;
}

// ---- phases: O-proj + residual, down-proj + residual ---------------------------------------------------
// K is 2048 or 3072: rows are cut into 1024-column sub-rows spread over the warps, partial sums meet in shared
// memory and are added in a fixed order.  out = bf16(resid + bf16(W x)) (reference base.py:110-123).
// `res_src` == nullptr takes the residual from the embedding row (layer 0's o_proj).
template <int NB, int K>
__device__ bool phase_proj_residual(Cta& c, int what, const uint64_t* x_src, uint32_t x_tag, const uint64_t* res_src,
                                    uint32_t res_tag, uint64_t* dst, uint32_t dst_tag, uint32_t epoch) {
    constexpr int S = K / 1024;
    constexpr int kSlots = 60;               // sub-rows finished per pass: a multiple of 4 and of 6, so row pairs stay whole
    int p0, p1;
    split_range(D / 2, c.ncta, c.cta, p0, p1);
    // The residual rows this CTA owns were published phases ago: fetch them now, not after the GEMV.
    bool ok = true;
    uint32_t rw_early = 0;
    const int early_pairs = (2 * (p1 - p0) * S < kSlots ? 2 * (p1 - p0) * S : kSlots) / (2 * S);
    if (c.tid < early_pairs * NB) {
        const int pair = p0 + c.tid / NB, b = c.tid % NB;
        if (res_src == nullptr)
            rw_early = ldcg32(reinterpret_cast<const bf16*>(c.p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * pair);
        else
            ok = wait_word(c.w, res_src + (size_t)b * (D / 2) + pair, res_tag, rw_early, 32 + what);
    }
    const bf16* W = nullptr;                                   // this CTA's rows [2*p0, 2*p1), contiguous in the ring
    if (!wait_rows_to_smem<NB, K>(c, x_src, x_tag, what, p1 > p0 ? &W : nullptr)) return false;
    mark_ready(c);
    // The whole attention output of (step, layer) is here, so every cache row appended up to (step, layer) is in place:
    // the feeding lane may fetch the tiles of (step + 1, layer).
    if (epoch != 0u && c.tid == 0) st_release_cta(&c.st.sh->kv_epoch, epoch);
    if (p1 == p0) return all_ok(ok);
    if constexpr (NB > 1) {
        // several sequences: tiles of up to 16 rows x 256 columns on the tensor cores, one column block per warp
        constexpr int NK = K / 256;
        const int n_rows = 2 * (p1 - p0);            // at most 16: the launch requires 128 CTAs or more
        float* part = c.hdr->sub;
        for (int task = c.warp; task < NK; task += kWarps) {
            float d[4];
            gemv_tile<NB>(W, K, 0, n_rows, c.xs, task * 256, c.lane, d);
            gemv_store<NB>(part, task, c.lane, d);
        }
        cta_sync();
        for (int i = c.tid; i < (p1 - p0) * NB; i += kThreads) {
            const int pp = i / NB, b = i % NB, pair = p0 + pp;
            const float s0 = gemv_sum<NB, NK>(part, 2 * pp, b), s1 = gemv_sum<NB, NK>(part, 2 * pp + 1, b);
            uint32_t rw = rw_early;
            if (i != c.tid || i >= early_pairs * NB) {
                if (res_src == nullptr)
                    rw = ldcg32(reinterpret_cast<const bf16*>(c.p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * pair);
                else
                    ok = ok && wait_word(c.w, res_src + (size_t)b * (D / 2) + pair, res_tag, rw, 32 + what);
            }
            st_flagged(dst + (size_t)b * (D / 2) + pair, pack_bf16x2(bf_lo(rw) + bf16r(s0), bf_hi(rw) + bf16r(s1)), dst_tag);
        }
        stream_release(c.st, 1);
        return all_ok(ok);
    }
    const int n_sub = 2 * (p1 - p0) * S;
    float* sub = c.hdr->sub;
    for (int base = 0; base < n_sub; base += kSlots) {
        const int cnt = n_sub - base < kSlots ? n_sub - base : kSlots;
        for (int sr = c.warp; sr < cnt; sr += kWarps) {
            const int gsr = base + sr;
            const int seg = gsr % S;
            const bf16* wp[1] = {W + (size_t)gsr * 1024};
            const uint32_t* xseg[1] = {c.xs + seg * 512};
            float acc[1][NB];
            dot_subrows_smem<false, NB, 1>(wp, xseg, c.lane, acc);
            if (c.lane == 0) {
#pragma unroll
                for (int b = 0; b < NB; ++b) sub[sr * NB + b] = acc[0][b];
            }
        }
        cta_sync();
        const int pairs_here = cnt / (2 * S);
        for (int i = c.tid; i < pairs_here * NB; i += kThreads) {
            const int pp = i / NB, b = i % NB;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int k = 0; k < S; ++k) { s0 += sub[((2 * pp) * S + k) * NB + b]; s1 += sub[((2 * pp + 1) * S + k) * NB + b]; }
            const int pair = p0 + base / (2 * S) + pp;
            uint32_t rw = rw_early;
            if (base != 0 || i != c.tid) {       // only reached with fewer CTAs than a B200 has
                if (res_src == nullptr)
                    rw = ldcg32(reinterpret_cast<const bf16*>(c.p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * pair);
                else
                    ok = ok && wait_word(c.w, res_src + (size_t)b * (D / 2) + pair, res_tag, rw, 32 + what);
            }
            st_flagged(dst + (size_t)b * (D / 2) + pair, pack_bf16x2(bf_lo(rw) + bf16r(s0), bf_hi(rw) + bf16r(s1)), dst_tag);
        }
        cta_sync();
    }
    stream_release(c.st, 1);
    return all_ok(ok);
}

// ---- phase: RMSNorm + gate/up GEMV + SwiGLU -----------------------------------------------------------
// act = bf16(bf16(silu(bf16 gate)) * bf16 up); gate and up rows are adjacent (reference base.py:124-129).
__device__ __forceinline__ float swiglu(float gate_acc, float up_acc) {
    const float gte = bf16r(gate_acc), up = bf16r(up_acc);
    return bf16r(gte / (1.0f + expf(-gte))) * up;
}

template <int NB>
__device__ bool phase_gu(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t tag = tag_of(c, c.step, l);
    const uint32_t gw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const bf16*>(p.ln2) + (size_t)l * D + 2 * c.tid);
    uint32_t u[NB];
    bool ok = wait_words<NB>(c.w, c.ws.hmid + c.tid, D / 2, tag, u, ITTAI_PH_GU);
    int u0, u1;
    split_range(FF / 6, c.ncta, c.cta, u0, u1);      // 128-bit words: three units of two activations = four weight rows each
    u0 *= 3; u1 *= 3;
    const bf16* W = nullptr;
    if (!norm_pairs_to_smem<NB>(c, u, gw, ok, u1 > u0 ? &W : nullptr)) return false;
    if (u1 == u0) return true;
    if constexpr (NB == 1) {
        float xr[32];
        if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
        uint32_t* pub = reinterpret_cast<uint32_t*>(c.hdr->sub);      // this CTA's packed outputs, [unit][sequence]
        for (int un = u0 + c.warp; un < u1; un += kWarps) {
            const bf16* wu = W + (size_t)(4 * (un - u0)) * D;
            float a0[NB], a1[NB];
            if constexpr (NB == 1) {
                // two rows at a time: four rows' worth of weights in flight (64 registers) next to the 32 of xr spills
                const bf16* wa[2] = {wu, wu + D};
                const bf16* wb[2] = {wu + 2 * D, wu + 3 * D};
                float acc[2][NB], acd[2][NB];
                dot_rows_k1024<false, NB, 2>(c, wa, xr, acc);
                dot_rows_k1024<false, NB, 2>(c, wb, xr, acd);
                a0[0] = swiglu(acc[0][0], acc[1][0]);
                a1[0] = swiglu(acd[0][0], acd[1][0]);
            } else {
#pragma unroll
                for (int hsel = 0; hsel < 2; ++hsel) {
                    const bf16* wp[2] = {wu + (2 * hsel) * D, wu + (2 * hsel + 1) * D};
                    float acc[2][NB];
                    dot_rows_k1024<false, NB, 2>(c, wp, xr, acc);
#pragma unroll
                    for (int b = 0; b < NB; ++b) (hsel ? a1[b] : a0[b]) = swiglu(acc[0][b], acc[1][b]);
                }
            }
            if (c.lane == 0) {
#pragma unroll
                for (int b = 0; b < NB; ++b) pub[(un - u0) * NB + b] = pack_bf16x2(a0[b], a1[b]);
            }
        }
        stream_release(c.st, 1);                         // its barrier also publishes `pub` to the CTA
        // three units (six activations) leave as one 128-bit word
        for (int i = c.tid; i < (u1 - u0) / 3 * NB; i += kThreads) {
            const int wq = i / NB, b = i % NB;
            st_flagged128(reinterpret_cast<uint4*>(c.ws.act) + (size_t)b * (FF / 6) + u0 / 3 + wq,
                          pub[(3 * wq) * NB + b], pub[(3 * wq + 1) * NB + b], pub[(3 * wq + 2) * NB + b], tag);
        }
    } else {
        const int n_rows = 4 * (u1 - u0), n_tasks = (n_rows + 15) / 16 * 4;
        float* part = c.hdr->sub;
        for (int task = c.warp; task < n_tasks; task += kWarps) {
            float d[4];
            gemv_tile<NB>(W, D, (task >> 2) * 16, n_rows, c.xs, (task & 3) * 256, c.lane, d);
            gemv_store<NB>(part, task, c.lane, d);
        }
        stream_release(c.st, 1);                         // its barrier also publishes `part` to the CTA
        // a lane per unit (four rows, two activations) in groups of four lanes, the fourth idle: the first lane of a group
        // collects its neighbours' pairs and sends the three units (six activations) off as one 128-bit word
        const int n_words = (u1 - u0) / 3 * NB;
        for (int i0 = 0; i0 < n_words * 4; i0 += kThreads) {
            const int i = i0 + c.tid, wi = i >> 2, k = i & 3;
            const bool live = wi < n_words && k < 3;
            const int wq = live ? wi / NB : 0, b = live ? wi % NB : 0;
            const int r = 12 * wq + 4 * k;               // rows: gate, up, gate, up of two adjacent activations
            uint32_t w = 0;
            if (live) w = pack_bf16x2(swiglu(gemv_sum<NB, 4>(part, r, b), gemv_sum<NB, 4>(part, r + 1, b)),
                                      swiglu(gemv_sum<NB, 4>(part, r + 2, b), gemv_sum<NB, 4>(part, r + 3, b)));
            const uint32_t w1 = __shfl_down_sync(0xffffffffu, w, 1), w2 = __shfl_down_sync(0xffffffffu, w, 2);
            if (live && k == 0) st_flagged128(reinterpret_cast<uint4*>(c.ws.act) + (size_t)b * (FF / 6) + u0 / 3 + wq, w, w1, w2, tag);
        }
    }
    return true;
}

// ---- phase: final RMSNorm + tied lm_head GEMV + argmax ------------------------------------------------
// logits = bf16(W_embed x); argmax over the bf16 values, lowest index wins ties (torch semantics).  The table is read
// straight from HBM with streaming loads (2 MB per CTA: far more than the ring holds, and nothing waits behind it).
// Every CTA publishes its best (value, index); every CTA then gathers all of them, so each knows the next token at once.
template <int NB>
__device__ bool phase_head(Cta& c) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t gw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const bf16*>(p.fin_w) + 2 * c.tid);
    uint32_t u[NB];
    bool ok = wait_words<NB>(c.w, c.ws.h + c.tid, D / 2, tag_of(c, c.step, p.n_layers), u, ITTAI_PH_HEAD);
    if (!norm_pairs_to_smem<NB>(c, u, gw, ok)) return false;
    float xr[32];
    if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
    bf16* logits = reinterpret_cast<bf16*>(p.logits);
    int r0, r1;
    split_range(p.vocab, c.ncta, c.cta, r0, r1);
    constexpr int R = kHeadRows / kWarps;        // rows of one streamed entry per warp
    float bv[NB];
    int bi[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) { bv[b] = -INFINITY; bi[b] = 0x7fffffff; }
    for (int e0 = r0; e0 < r1; e0 += kHeadRows) {
        bool okw;
        const bf16* W = stream_acquire(c, c.st.consumed, okw);     // rows [e0, e0 + kHeadRows) of the table
        if (!okw) return false;
        const int rows_here = r1 - e0 < kHeadRows ? r1 - e0 : kHeadRows;
        if constexpr (NB > 1) {
            // several sequences: the entry's 32 rows as two 16-row blocks x four column blocks on the tensor cores, then
            // warp b scans sequence b's 32 logits (lane = row) for the entry's best
            static_assert(kHeadRows == 32, "one lane per row of an entry");
            float* part = c.hdr->sub;
            if (c.warp < 8) {
                float d[4];
                gemv_tile<NB>(W, D, (c.warp >> 2) * 16, rows_here, c.xs, (c.warp & 3) * 256, c.lane, d);
                gemv_store<NB>(part, c.warp, c.lane, d);
            }
            cta_sync();
            if (c.warp < NB) {
                const int b = c.warp, row = e0 + c.lane;
                const bool live = c.lane < rows_here;
                float v = live ? bf16r(gemv_sum<NB, 4>(part, c.lane, b)) : -INFINITY;
                if (live && p.write_logits) logits[(size_t)b * p.vocab + row] = __float2bfloat16_rn(v);
                int ix = live ? row : 0x7fffffff;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {       // highest value, lowest row on ties
                    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, ix, o);
                    if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
                }
#pragma unroll
                for (int bb = 0; bb < NB; ++bb)
                    if (bb == b && v > bv[bb]) { bv[bb] = v; bi[bb] = ix; }      // entries ascend: the first maximum is kept
            }
            stream_release(c.st, 1);
            continue;
        }
        const int lr = c.warp * R;                                 // this warp's first row inside the entry
        if (lr < rows_here) {
            const bf16* wp[R];
#pragma unroll
            for (int r = 0; r < R; ++r) wp[r] = W + (size_t)(lr + r < rows_here ? lr + r : rows_here - 1) * D;
            float acc[R][NB];
            dot_rows_k1024<false, NB, R>(c, wp, xr, acc);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (lr + r < rows_here) {
                    const int row = e0 + lr + r;
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        const float v = bf16r(acc[r][b]);
                        if (v > bv[b]) { bv[b] = v; bi[b] = row; }   // rows ascend within a warp: first max kept
                        if (p.write_logits && c.lane == 0) logits[(size_t)b * p.vocab + row] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
        stream_release(c.st, 1);
    }
    const uint32_t tag = (uint32_t)c.step + 1u;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        if (c.lane == 0) { c.hdr->bestv[c.warp] = bv[b]; c.hdr->besti[c.warp] = bi[b]; }
        cta_sync();
        if (c.tid == 0) {
            float v = c.hdr->bestv[0];
            int ix = c.hdr->besti[0];
            for (int w = 1; w < kWarps; ++w) {
                const float vw = c.hdr->bestv[w];
                const int iw = c.hdr->besti[w];
                if (vw > v || (vw == v && iw < ix)) { v = vw; ix = iw; }
            }
            st_flagged(c.ws.cand_val + c.cta * ITTAI_MAX_BATCH + b, __float_as_uint(v), tag);
            st_flagged(c.ws.cand_idx + c.cta * ITTAI_MAX_BATCH + b, (uint32_t)ix, tag);
        }
        cta_sync();
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        bool okb = true;
        for (int k = c.tid; k < c.ncta; k += kThreads) {
            uint32_t uv = 0, ui = 0;
            okb = okb && wait_word(c.w, c.ws.cand_val + k * ITTAI_MAX_BATCH + b, tag, uv, 16 + ITTAI_PH_HEAD);
            okb = okb && wait_word(c.w, c.ws.cand_idx + k * ITTAI_MAX_BATCH + b, tag, ui, 16 + ITTAI_PH_HEAD);
            c.hdr->candv[k] = __uint_as_float(uv);
            c.hdr->candi[k] = (int)ui;
        }
        if (!all_ok(okb)) return false;
        if (c.warp == 0) {
            float v = -INFINITY;
            int ix = 0x7fffffff;
            for (int k = c.lane; k < c.ncta; k += 32) {
                const float vk = c.hdr->candv[k];
                const int ik = c.hdr->candi[k];
                if (vk > v || (vk == v && ik < ix)) { v = vk; ix = ik; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float vo = __shfl_xor_sync(0xffffffffu, v, o);
                const int io = __shfl_xor_sync(0xffffffffu, ix, o);
                if (vo > v || (vo == v && io < ix)) { v = vo; ix = io; }
            }
            if (c.lane == 0) {
                // no logit compared greater than -inf (a row of NaNs): report it instead of feeding the sentinel back
                if (ix == 0x7fffffff && c.cta == 0)
                    report_status(p.status, c.ws.sync, ITTAI_ST_BAD_TOKEN, (uint32_t)ix, (uint32_t)c.step, (uint32_t)c.hdr->pos_s[b], (uint32_t)b);
                c.hdr->tok_s[b] = ix;
                if (c.cta == 0) {
                    p.next_id[b] = ix;
                    p.out_ids[(size_t)c.step * p.batch + b] = ix;
                }
            }
        }
        cta_sync();
    }
    return true;
}

// ---- per-step set-up: positions and input ids ----------------------------------------------------------
// Returns false (uniformly over the grid) when an id or a position is out of range.
__device__ bool step_setup(Cta& c, int step, bool ids_from_head) {
    const IttaiQwen3Decode& p = c.p;
    if (c.tid < p.batch) {
        const int b = c.tid;
        c.hdr->pos_s[b] = c.hdr->pos0[b] + step;
        if (step < p.n_forced) c.hdr->tok_s[b] = p.forced[(size_t)step * p.batch + b];
        else if (!ids_from_head) c.hdr->tok_s[b] = p.next_id[b];
        // else: the head of the previous step left the id in tok_s
    }
    cta_sync();
    bool ok = true;
    for (int b = 0; b < p.batch; ++b) {
        const int t = c.hdr->tok_s[b], ps = c.hdr->pos_s[b];
        if (t < 0 || t >= p.vocab || ps < 0 || ps >= p.kv_cap) {
            if (c.tid == 0 && c.cta == 0)
                report_status(p.status, c.ws.sync, ITTAI_ST_BAD_TOKEN, (uint32_t)t, (uint32_t)step, (uint32_t)ps, (uint32_t)b);
            ok = false;
        }
    }
    return ok;
}

template <int NB>
__device__ __forceinline__ bool run_phase(Cta& c, int phase, int l) {
    const uint32_t tag = tag_of(c, c.step, l);
    switch (phase) {
        case ITTAI_PH_QKV: return phase_qkv<NB>(c, l);
        case ITTAI_PH_ATTN: return phase_attn<NB>(c, l);
        case ITTAI_PH_OPROJ:
            return phase_proj_residual<NB, DQ>(c, ITTAI_PH_OPROJ, c.ws.attn, tag, l == 0 ? nullptr : c.ws.h, tag, c.ws.hmid, tag,
                                               (uint32_t)(c.step * c.p.n_layers + l) + 1u);
        case ITTAI_PH_GU: return phase_gu<NB>(c, l);
        case ITTAI_PH_DOWN:
            return phase_proj_residual<NB, FF>(c, ITTAI_PH_DOWN, c.ws.act, tag, c.ws.hmid, tag, c.ws.h, tag_of(c, c.step, l + 1), 0u);
        default: return phase_head<NB>(c);
    }
}

// The per-CTA context is brace-initialised inside each kernel.  nvcc 12.9 mis-infers the shared state space for the
// global pointers of a struct returned by value from a helper that also receives the shared-memory base, so there is
// deliberately no make_cta() function.
// The workspace pointers: held by reference to the kernel parameter they cost no registers (nine 64-bit pointers live
// across every phase otherwise), which at batch 1 is worth 5 % of the token time (611 -> 579 us) and removes the batch-8
// kernel's spills; the batch-8 step is 2.4 % slower that way at cache length 2048 all the same, so the larger batches keep
// a register copy.
#define ITTAI_MAKE_CTA(p, wsp, smem, nb, ring_bytes)                                                              \
    const Q3Workspace ws_copy = wsp;                                                                              \
    const Q3Workspace& ws_sel = (nb) >= 4 ? ws_copy : wsp;                                                        \
    Cta c{p, ws_sel, reinterpret_cast<SmemHdr*>(smem), reinterpret_cast<uint32_t*>(smem + kHdrBytes),                \
          reinterpret_cast<SmemAttn*>(smem + kHdrBytes), (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x,       \
          (int)(threadIdx.x & 31), (int)(threadIdx.x >> 5),                                                       \
          Waiter{wsp.sync, p.status, p.spin_limit > 0 ? (uint32_t)p.spin_limit : kSpinLimit},                     \
          Stream{&reinterpret_cast<SmemHdr*>(smem)->stream, smem + q3_fixed_smem_bytes(nb), ring_bytes, 0u},      \
          0}

template <int NB>
__global__ void __launch_bounds__(kBlock, 1) q3_decode_kernel(const __grid_constant__ IttaiQwen3Decode p,
                                                                const __grid_constant__ Q3Workspace wsp,
                                                                uint32_t ring_bytes) {
    extern __shared__ __align__(256) unsigned char smem[];
    ITTAI_MAKE_CTA(p, wsp, smem, NB, ring_bytes);
    if ((p.flags & ITTAI_F_TEST_DROP_CTA) != 0 && c.cta == 0) return;
    if (c.tid < p.batch) c.hdr->pos0[c.tid] = p.pos[c.tid];
    stream_init(c.st, c.tid);
    if (c.tid >= kThreads) {     // the stream-feeding warp: one lane issues, the others have nothing to do
        if (c.tid == kThreads) stream_feed(c, 0, p.n_steps * (kStreamPhases * p.n_layers + 1));
        return;
    }
    const bool prof = p.phase_clk != nullptr && c.cta == 0 && c.tid == 0;
    bool prev_head = false, ok = true;

    for (int step = 0; step < p.n_steps && ok; ++step) {
        c.step = step;
        ok = step_setup(c, step, prev_head);
        if (!ok) break;
        const bool run_head = step >= p.n_forced - 1;
        if (!run_head && c.cta == 0 && c.tid < p.batch) p.out_ids[(size_t)step * p.batch + c.tid] = -1;
        if (step > 0 && !prev_head) {
            // No head ran, so nothing yet orders this token after the previous one: wait for its last layer's output
            // before any buffer of the chain is written again.
            bool okw = true;
            for (int b = 0; b < p.batch; ++b) {
                uint32_t u;
                okw = okw && wait_word(c.w, c.ws.h + b * (D / 2) + c.tid, tag_of(c, step - 1, p.n_layers), u, 64);
            }
            ok = all_ok(okw);
            if (!ok) break;
        }
        for (int l = 0; l < p.n_layers && ok; ++l) {
#pragma unroll 1
            for (int phase = ITTAI_PH_QKV; phase <= ITTAI_PH_DOWN && ok; ++phase) {
                ok = run_phase<NB>(c, phase, l);
                if (prof && ok) {
                    const size_t slot = ((size_t)step * (5 * p.n_layers + 1) + l * 5 + phase) * 2;
                    p.phase_clk[slot] = (uint64_t)c.hdr->t_ready;
                    p.phase_clk[slot + 1] = (uint64_t)clock64();
                }
            }
        }
        if (run_head && ok) {
            ok = phase_head<NB>(c);
            if (prof && ok) {
                const size_t slot = ((size_t)step * (5 * p.n_layers + 1) + 5 * p.n_layers) * 2;
                p.phase_clk[slot] = (uint64_t)c.hdr->t_ready;
                p.phase_clk[slot + 1] = (uint64_t)clock64();
            }
        }
        prev_head = run_head;
        if (ok && p.step_ns != nullptr && c.cta == 0 && c.tid == 0) p.step_ns[step] = globaltimer_ns();
    }
    if (!ok) {                   // leaving early: the feeding lane stops issuing and waits for its copies in flight
        if (c.tid == 0) c.st.sh->stop = 1u;
        return;
    }
    if (c.cta == 0 && c.tid < p.batch) p.pos[c.tid] = c.hdr->pos0[c.tid] + p.n_steps;
}

// One phase on its own at step 0 (tags of step 0): unit tests and per-phase profiles.  Inputs must carry the tag of
// (step 0, layer); launched cooperatively because the attention merge and the head wait on other CTAs.
template <int NB>
__global__ void __launch_bounds__(kBlock, 1) q3_phase_kernel(const __grid_constant__ IttaiQwen3Decode p,
                                                               const __grid_constant__ Q3Workspace wsp,
                                                               uint32_t ring_bytes, int phase, int l) {
    extern __shared__ __align__(256) unsigned char smem[];
    ITTAI_MAKE_CTA(p, wsp, smem, NB, ring_bytes);
    if (c.tid < p.batch) c.hdr->pos0[c.tid] = p.pos[c.tid];
    stream_init(c.st, c.tid);
    if (c.tid >= kThreads) {
        const int k = phase == ITTAI_PH_HEAD ? kStreamPhases * p.n_layers : l * kStreamPhases + phase;
        if (c.tid == kThreads) stream_feed(c, k, k + 1);
        return;
    }
    bool ok = step_setup(c, 0, false);
    if (ok) ok = run_phase<NB>(c, phase, l);
    if (!ok && c.tid == 0) c.st.sh->stop = 1u;
}

// ---- host side ---------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

static int check_args(const IttaiQwen3Decode* p) {
    if (!p) { set_error("null IttaiQwen3Decode"); return ITTAI_E_ARG; }
    if (p->batch != 1 && p->batch != 2 && p->batch != 4 && p->batch != 8) { set_error("batch %d: supported sizes are 1, 2, 4, 8", p->batch); return ITTAI_E_ARG; }
    if (p->n_layers < 1 || p->vocab < 1 || p->kv_cap < 1 || p->n_steps < 1) { set_error("n_layers, vocab, kv_cap and n_steps must be positive"); return ITTAI_E_ARG; }
    if (p->n_forced < 0 || p->n_forced > p->n_steps) { set_error("n_forced %d outside 0..n_steps", p->n_forced); return ITTAI_E_ARG; }
    if (p->n_forced > 0 && !p->forced) { set_error("n_forced > 0 with forced == NULL"); return ITTAI_E_ARG; }
    if (p->write_logits && !p->logits) { set_error("write_logits set with logits == NULL"); return ITTAI_E_ARG; }
    if ((long long)p->n_steps * (kStreamPhases * p->n_layers + 1) >= (1ll << 31)) { set_error("n_steps * (n_layers + 1) * 5 must stay below 2^31"); return ITTAI_E_ARG; }
    const void* req[] = {p->wqkv, p->wo, p->wgu, p->wd, p->ln1, p->ln2, p->qn, p->kn, p->fin_w, p->embed, p->rope,
                         p->kcache, p->vcache, p->pos, p->next_id, p->out_ids, p->workspace, p->status};
    for (const void* q : req) if (!q) { set_error("null device pointer in IttaiQwen3Decode"); return ITTAI_E_ARG; }
    const void* al16[] = {p->wqkv, p->wo, p->wgu, p->wd, p->embed, p->kcache, p->vcache, p->ln1, p->ln2, p->fin_w, p->rope};
    for (const void* q : al16) if (((uintptr_t)q & 15u) != 0) { set_error("weight / cache pointers must be 16-byte aligned"); return ITTAI_E_ARG; }
    if (((uintptr_t)p->workspace & 255u) != 0) { set_error("workspace must be 256-byte aligned"); return ITTAI_E_ARG; }
    return ITTAI_OK;
}

struct DeviceInfo { int dev = -1; int n_sms = 0; int smem_optin = 0; bool attr_set[4] = {false, false, false, false}; };
static thread_local DeviceInfo g_info;

static int device_info() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (g_info.dev != dev) {
        int sms = 0, optin = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(sm count)");
        e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(shared memory)");
        g_info = DeviceInfo();
        g_info.dev = dev;
        g_info.n_sms = sms;
        g_info.smem_optin = optin;
    }
    return ITTAI_OK;
}

template <int NB>
static int launch_nb(const IttaiQwen3Decode* p, int phase, int layer, cudaStream_t st) {
    int rc = device_info();
    if (rc != ITTAI_OK) return rc;
    const int grid = g_info.n_sms < Q3_MAX_CTAS ? g_info.n_sms : Q3_MAX_CTAS;
    if (grid < 128) { set_error("the decode kernel's GEMV tiling needs at least 128 SMs (found %d)", grid); return ITTAI_E_DEVICE; }
    if (grid < p->batch * NKV) { set_error("%d SMs cannot hold one attention item per CTA at batch %d", grid, p->batch); return ITTAI_E_DEVICE; }
    // all the shared memory a CTA may have: header + activations + the weight ring
    const size_t fixed = q3_fixed_smem_bytes(NB);
    const size_t smem = (size_t)g_info.smem_optin;
    if (smem < fixed + 96 * 1024) { set_error("%zu bytes of shared memory per CTA leave no room for the weight ring", smem); return ITTAI_E_DEVICE; }
    uint32_t ring_bytes = (uint32_t)((smem - fixed) / 1024 * 1024);
    {   // every slice must fit the ring on its own (an empty ring restarts at its base), and the attention phase holds two K
        // and two V tiles before it hands any back
        int lo, hi;
        size_t slice = 4 * (size_t)kTile * HD * 2;
        for (int c = 0; c < grid; ++c) {
            split_range(DQKV / 4, grid, c, lo, hi);
            const size_t qkv = (size_t)(hi - lo) * 4 * D * 2;
            split_range(D / 2, grid, c, lo, hi);
            const size_t down = (size_t)(hi - lo) * 2 * FF * 2;
            split_range(FF / 6, grid, c, lo, hi);
            const size_t gu = (size_t)(hi - lo) * 12 * D * 2;
            const size_t m = qkv > down ? (qkv > gu ? qkv : gu) : (down > gu ? down : gu);
            slice = m > slice ? m : slice;
        }
        if (slice > ring_bytes) {
            set_error("a %zu-byte weight slice does not fit the %u-byte shared-memory ring (%d CTAs)", slice, ring_bytes, grid);
            return ITTAI_E_DEVICE;
        }
    }
    const void* fn_decode = (const void*)q3_decode_kernel<NB>;
    const void* fn_phase = (const void*)q3_phase_kernel<NB>;
    constexpr int slot = NB == 1 ? 0 : NB == 2 ? 1 : NB == 4 ? 2 : 3;
    if (!g_info.attr_set[slot]) {
        cudaError_t e = cudaFuncSetAttribute(fn_decode, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(decode)");
        e = cudaFuncSetAttribute(fn_phase, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(phase)");
        int occ = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, q3_decode_kernel<NB>, kBlock, smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
        if (occ < 1) { set_error("device cannot hold one persistent CTA per SM (%zu bytes of shared memory)", smem); return ITTAI_E_DEVICE; }
        g_info.attr_set[slot] = true;
    }
    Q3Workspace ws;
    q3_ws_layout(p->batch, reinterpret_cast<char*>(p->workspace), &ws);
    cudaError_t e = cudaMemsetAsync(ws.sync, 0, Q3_SYNC_WORDS * sizeof(uint32_t), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(sync)");
    if (phase < 0) {   // a phase launch keeps the flagged words its caller prepared
        e = cudaMemsetAsync(ws.h, 0, ws.flagged_bytes, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(flagged words)");
    }
    e = cudaMemsetAsync(p->status, 0, ITTAI_STATUS_WORDS * sizeof(uint32_t), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
    if (phase < 0) {
        void* args[] = {(void*)p, (void*)&ws, (void*)&ring_bytes};
        e = cudaLaunchCooperativeKernel(fn_decode, dim3(grid), dim3(kBlock), args, smem, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchCooperativeKernel(q3_decode_kernel)");
    } else {
        void* args[] = {(void*)p, (void*)&ws, (void*)&ring_bytes, (void*)&phase, (void*)&layer};
        e = cudaLaunchCooperativeKernel(fn_phase, dim3(grid), dim3(kBlock), args, smem, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchCooperativeKernel(q3_phase_kernel)");
    }
    return ITTAI_OK;
}

static int launch(const IttaiQwen3Decode* p, int phase, int layer, void* stream) {
    int rc = check_args(p);
    if (rc != ITTAI_OK) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (p->batch) {
        case 1: return launch_nb<1>(p, phase, layer, st);
        case 2: return launch_nb<2>(p, phase, layer, st);
        case 4: return launch_nb<4>(p, phase, layer, st);
        default: return launch_nb<8>(p, phase, layer, st);
    }
}

}  // namespace ittai

extern "C" int ittai_qwen3_decode_workspace_bytes(int batch, size_t* bytes) {
    if (!bytes || (batch != 1 && batch != 2 && batch != 4 && batch != 8)) { ittai::set_error("batch must be 1, 2, 4 or 8 and the output non-null"); return ITTAI_E_ARG; }
    ittai::Q3Workspace ws;
    *bytes = ittai::q3_ws_layout(batch, nullptr, &ws);
    return ITTAI_OK;
}

extern "C" int ittai_qwen3_decode_launch(const IttaiQwen3Decode* p, void* stream) { return ittai::launch(p, -1, 0, stream); }

extern "C" int ittai_qwen3_phase_launch(const IttaiQwen3Decode* p, int phase, int layer, void* stream) {
    if (phase < ITTAI_PH_QKV || phase > ITTAI_PH_HEAD) { ittai::set_error("phase %d outside 0..5", phase); return ITTAI_E_ARG; }
    if (p && (layer < 0 || layer >= p->n_layers)) { ittai::set_error("layer %d outside 0..%d", layer, p->n_layers - 1); return ITTAI_E_ARG; }
    return ittai::launch(p, phase, layer, stream);
}

// ---- decode launch for callers that cannot allocate device memory ---------------------------------------------
// Some hosts of this library have no way to get scratch memory at call time: a serving process that handed the whole
// GPU to its own pool at start-up (so a later cudaMalloc fails or fragments it), a C or Rust runtime that binds this
// ABI without an allocator of its own, or a latency-critical loop in which cudaMalloc's device-wide synchronisation is
// not acceptable.  For them the decode kernel's workspace (flagged words, split-K partials, argmax candidates,
// abort flag) lives in this file-scope device array instead of a caller buffer.  Every GPU that loads the library
// holds these bytes until the process exits.
namespace ittai {

constexpr int kStaticMaxBatch = ITTAI_STATIC_DECODE_MAX_BATCH;
// q3_ws_layout(kStaticMaxBatch) rounded up: 128 B sync + (512+2048+1024+512+1536) words per sequence + partials + candidates
constexpr size_t kStaticScratchBytes = 256 + (size_t)kStaticMaxBatch * 5632 * 8 + 1280 +
                                       (size_t)Q3_MAX_CTAS * Q3_PART_WORDS * 8 + 2 * (size_t)Q3_MAX_CTAS * ITTAI_MAX_BATCH * 8;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// In host code `g_decode_scratch` is only a handle for the runtime, not a device address: the address the kernel needs
// comes from cudaGetSymbolAddress, asked once per device with that device current.  Two host threads that make their
// first call on one device at the same time both look the address up and both store the same value: harmless.
static void* g_scratch_addr[64] = {nullptr};

static int static_scratch(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) { set_error("device ordinal %d outside 0..63", dev); return ITTAI_E_DEVICE; }
    if (g_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_decode_scratch)");
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return ITTAI_OK;
}

}  // namespace ittai

extern "C" int ittai_qwen3_decode_launch_static(const IttaiQwen3Decode* p, void* stream) {
    if (!p) { ittai::set_error("null IttaiQwen3Decode"); return ITTAI_E_ARG; }
    if (p->batch > ittai::kStaticMaxBatch) {
        ittai::set_error("batch %d exceeds the built-in scratch, which holds at most %d sequences (%zu bytes); "
                         "use ittai_qwen3_decode_launch with a caller workspace", p->batch, ittai::kStaticMaxBatch,
                         ittai::kStaticScratchBytes);
        return ITTAI_E_ARG;
    }
    ittai::Q3Workspace ws;
    if (p->batch >= 1 && ittai::q3_ws_layout(p->batch, nullptr, &ws) > ittai::kStaticScratchBytes) {
        ittai::set_error("built-in scratch of %zu bytes is smaller than the workspace batch %d needs", ittai::kStaticScratchBytes, p->batch);
        return ITTAI_E_ARG;
    }
    void* scratch = nullptr;
    const int rc = ittai::static_scratch(&scratch);
    if (rc != ITTAI_OK) return rc;
    IttaiQwen3Decode q = *p;
    q.workspace = scratch;       // the launch below zeroes the words that must start at zero, as for a caller buffer
    return ittai::launch(&q, -1, 0, stream);
}
