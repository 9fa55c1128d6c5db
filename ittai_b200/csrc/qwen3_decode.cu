// Qwen3-0.6B decode: one persistent cooperative kernel per launch runs n_steps tokens; the chosen token id is fed
// back on the device.
//
//  * Data flow instead of grid barriers: every vector one phase hands to the next travels as 128-bit mail words
//    (payload + tag of the producing step and layer) that the producer writes into a private mailbox of every CTA
//    that needs them, and a consumer polls exactly the words of its own mailbox (qwen3_ws.h).
//  * Weight stream: each CTA's slices of the layer matrices and of the KV cache are pulled into a shared-memory ring by
//    TMA bulk copies issued far ahead of use (weight_stream.cuh), so HBM keeps streaming while phases wait on each other.
//  * Batch-1 decode is HBM-bound (about 1.4 flop per weight byte): each warp multiplies whole weight sub-rows with
//    128-bit accesses and reduces with shuffles.  With several sequences the GEMV phases use warp-level
//    tensor-core tiles with the sequences as the N dimension (gemv_tile).
//
// Rounding points follow the eager modules: every Linear output, norm output, rotary product and sum, SiLU, gate*up
// product and residual sum is rounded to bf16 exactly once.  The math per phase mirrors the fused epilogues of the
// reference's megakernel (src/ittai/qwen3/base.py:80-129 for qkv / residual / gate-up, :147-162 for the embedding row),
// re-cut for one token: the row-norm scale is applied before the GEMV instead of after the GEMM, and keys and values go
// straight into the cache instead of a staging matrix.  KV cache, split-K decode attention, lm_head and argmax have no
// counterpart in the reference.
#include <cstdio>

#include "common.cuh"
#include "qwen3_ws.h"
#include "weight_stream.cuh"

namespace ittai {

constexpr int D = ITTAI_Q3_D, NKV = ITTAI_Q3_NKV, HD = ITTAI_Q3_HD, FF = ITTAI_Q3_FF;
constexpr int DQ = ITTAI_Q3_DQ, DQKV = ITTAI_Q3_DQKV, DGU = ITTAI_Q3_DGU;
constexpr int MS = Q3_MAIL_STRIDE;
constexpr int kTile = 128;                       // cache positions per attention tile = one ring entry of K and one of V
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kPartFloats = 12 * 16;             // at most 12 tiles (16 rows x 256 columns) per CTA and phase
constexpr int kStreamPhases = 5;                 // phases of a layer whose weights or cache rows come through the ring
constexpr int kPubHalves = 32;                   // outputs of one CTA and sequence in a GEMV phase (at most 28)
constexpr int kMsgFloats = 4 + 2 * HD;           // one split's partial: m[2], l[2], o[2][128]

// ---- shared-memory plan (dynamic): header | activations or attention scratch | weight ring -----------------
struct SmemHdr {
    StreamShared stream;
    int pos0[ITTAI_MAX_BATCH];                   // cache lengths at kernel entry
    int pos_s[ITTAI_MAX_BATCH];
    int tok_s[ITTAI_MAX_BATCH];
    float bestv[kWarps];
    int besti[kWarps];
    float sub[kPartFloats * ITTAI_MAX_BATCH];    // partial dot products: [task] at batch 1, [task][16 rows][sequence] for the tiles
    uint16_t pub[kPubHalves * ITTAI_MAX_BATCH];  // this CTA's bf16 outputs of the running phase, [sequence][row]
    uint16_t res[8 * ITTAI_MAX_BATCH];           // the residual rows this CTA owns, [sequence][row]
    float candv[Q3_MAX_CTAS];                    // argmax candidates of every CTA
    int candi[Q3_MAX_CTAS];
};
struct SmemAttn {
    float qs[2][HD];                             // rotated, pre-scaled queries of the two heads of a group
    float wm[kWarps][2], wl[kWarps][2];          // per-warp running max and sum
    bf16 knew[HD];
    bf16 vnew[HD];
    float msg[kMsgFloats];                       // this split's partial as it is mailed: m[2], l[2], o[2][128]
    float ored[kWarps][2][HD];                   // per-warp outputs; later the partials of all splits, [split][3 * words]
};
constexpr size_t kHdrBytes = (sizeof(SmemHdr) + 255) / 256 * 256;
__host__ __device__ constexpr size_t q3_fixed_smem_bytes(int nb) {
    size_t xs = (size_t)nb * (FF / 2) * sizeof(uint32_t);      // activations as packed bf16 pairs
    size_t at = sizeof(SmemAttn);
    return kHdrBytes + ((xs > at ? xs : at) + 255) / 256 * 256;
}
static_assert(Q3_PART_WORDS * 3 <= kWarps * 2 * HD, "the partials of all splits must fit the per-warp output scratch");

struct Cta {
    const IttaiQwen3Decode& p;
    Q3Workspace ws;
    SmemHdr* hdr;
    uint32_t* xs;       // [NB][FF/2] activations of the current GEMV as packed bf16 pairs (they are bf16 values: half the
                        // shared-memory traffic of fp32 and conflict-free 128-bit reads)
    SmemAttn* at;       // aliases xs
    int cta, ncta, tid, lane, warp;
    Waiter w;
    Stream st;
    int step;           // token index inside this launch
    long long t_ready;  // cycle counter when the current phase had its inputs (in-kernel profile)
};

// Tag of the data a (step, layer) produces; layer n_layers names the stream entering the head.  Never zero, and two
// versions of a word that follow each other (one layer or one step apart) never share a tag.
__device__ __forceinline__ uint32_t tag_of(const Cta& c, int step, int l) { return 1u + (uint32_t)(step * (c.p.n_layers + 1) + l) % 65535u; }

// CTA-uniform verdict on per-thread waits.
__device__ __forceinline__ bool all_ok(bool ok) { return !cta_or(!ok); }

__host__ __device__ __forceinline__ void split_range(int n, int parts, int i, int& lo, int& hi) {
    lo = (int)(((unsigned)n * (unsigned)i) / (unsigned)parts);          // n * parts stays far below 2^32
    hi = (int)(((unsigned)n * (unsigned)(i + 1)) / (unsigned)parts);
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
    const int B = c.p.batch, n_splits = q3_attn_splits(c.ncta, B);
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

// This CTA's rows of each layer matrix: quads of projection rows, rows of the two residual projections, SwiGLU outputs
// (two weight rows each).
__host__ __device__ __forceinline__ void qkv_rows(int ncta, int cta, int& r0, int& r1) { split_range(DQKV / 4, ncta, cta, r0, r1); r0 *= 4; r1 *= 4; }
__host__ __device__ __forceinline__ void res_rows(int ncta, int cta, int& r0, int& r1) { split_range(D, ncta, cta, r0, r1); }
__host__ __device__ __forceinline__ void act_cols(int ncta, int cta, int& a0, int& a1) { split_range(FF, ncta, cta, a0, a1); }

// The issuing lane's whole life: walk phases [k_begin, k_end) in execution order, launch every slice as soon as the
// ring has room, then wait for the last copies to land.  It stops early when the compute threads raise `stop`.
// Slice addresses are linear in the layer index, so everything but one small division per step is hoisted.
//
// Cache tiles and the row appended one step earlier: the K/V tiles of (step s, layer l) contain the row that some CTA
// appended at (step s - 1, layer l).  That store is ordered before the attention output of (s - 1, l) (the appending
// thread fences before its CTA publishes its partial, and the output needs every partial), so the tiles are held back
// until this CTA's compute threads have received that whole output (`kv_epoch`), and a fence pair orders the copy
// after what they observed.  The hold costs nothing: the condition was met a whole token ago.
__device__ void stream_feed(const Cta& c, int k_begin, int k_end) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t limit = c.w.limit;
    const int L = p.n_layers, PS = kStreamPhases * L + 1;
    int lo, hi;
    // per-phase: base of this CTA's slice in layer 0, bytes between layers, bytes of the slice
    const char* base[kStreamPhases];
    size_t stride[kStreamPhases];
    uint32_t nbytes[kStreamPhases];
    qkv_rows(c.ncta, c.cta, lo, hi);
    base[ITTAI_PH_QKV] = reinterpret_cast<const char*>(p.wqkv) + (size_t)lo * D * 2;
    stride[ITTAI_PH_QKV] = (size_t)DQKV * D * 2; nbytes[ITTAI_PH_QKV] = (uint32_t)(hi - lo) * D * 2;
    res_rows(c.ncta, c.cta, lo, hi);
    base[ITTAI_PH_OPROJ] = reinterpret_cast<const char*>(p.wo) + (size_t)lo * DQ * 2;
    stride[ITTAI_PH_OPROJ] = (size_t)D * DQ * 2; nbytes[ITTAI_PH_OPROJ] = (uint32_t)(hi - lo) * DQ * 2;
    base[ITTAI_PH_DOWN] = reinterpret_cast<const char*>(p.wd) + (size_t)lo * FF * 2;
    stride[ITTAI_PH_DOWN] = (size_t)D * FF * 2; nbytes[ITTAI_PH_DOWN] = (uint32_t)(hi - lo) * FF * 2;
    act_cols(c.ncta, c.cta, lo, hi);
    base[ITTAI_PH_GU] = reinterpret_cast<const char*>(p.wgu) + (size_t)2 * lo * D * 2;
    stride[ITTAI_PH_GU] = (size_t)DGU * D * 2; nbytes[ITTAI_PH_GU] = (uint32_t)(hi - lo) * 2 * D * 2;
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
                while (c.st.sh->kv_epoch < need) {
                    if (c.st.sh->stop != 0u || ++spins > (limit << 4)) { stream_drain(c.st, limit); return; }
                }
                asm volatile("fence.acq_rel.gpu;" ::: "memory");
                fence_proxy_async();
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

// ---- mail helpers ------------------------------------------------------------------------------------
// Seven bf16 values of a word into consecutive halves of shared memory (`cnt` of them are real).
__device__ __forceinline__ void unpack7(const uint32_t (&v)[4], uint16_t* d, int cnt) {
#pragma unroll
    for (int e = 0; e < 7; ++e)
        if (e < cnt) d[e] = (uint16_t)(v[e >> 1] >> ((e & 1) * 16));
}
// Up to seven bf16 values from shared memory as one word.
__device__ __forceinline__ void send7(void* dst, const uint16_t* s, int cnt, uint32_t tag) {
    uint32_t h[7];
#pragma unroll
    for (int e = 0; e < 7; ++e) h[e] = e < cnt ? (uint32_t)s[e] : 0u;
    st_mail(dst, h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6], tag);
}

// Collects an N-value bf16 vector per sequence that arrives as K words of up to seven values from every producer CTA
// (producer p owns values split_range(N, ncta, p)) into dst[b * FF + i].  `mail`: this CTA's mailbox, [NB][MS][K].
// Returns this thread's verdict; the caller's next barrier collects the verdicts and publishes the values.
template <int NB, int K>
__device__ __forceinline__ bool gather7(Cta& c, const uint4* mail, int N, uint32_t tag, int what, uint16_t* dst) {
    const int per = c.ncta * K;
    for (int i = c.tid; i < per * NB; i += kThreads) {
        const int b = NB == 1 ? 0 : i / per, r = i - b * per, pr = r / K, j = r - pr * K;
        int lo, hi;
        split_range(N, c.ncta, pr, lo, hi);
        const int start = lo + 7 * j;
        uint32_t v[4];
        if (!wait_mail(c.w, mail + ((size_t)b * MS + pr) * K + j, tag, v, what)) return false;
        unpack7(v, dst + b * FF + start, hi - start);
    }
    return true;
}

// Entry number n of the stream, with a CTA-uniform verdict.
__device__ __forceinline__ const bf16* stream_acquire(Cta& c, uint32_t n, bool& ok) {
    const unsigned char* ptr = stream_wait(c.st, n, c.w);
    ok = all_ok(ptr != nullptr);
    return reinterpret_cast<const bf16*>(ptr);
}

// ---- activations of one 1024-wide row in registers ---------------------------------------------------------
// Lane owns the 16-byte chunks lane, lane+32, lane+64, lane+96 of a row: 32 values.
__device__ __forceinline__ void unpack8(const uint4& q, float* x) {
    x[0] = bf_lo(q.x); x[1] = bf_hi(q.x); x[2] = bf_lo(q.y); x[3] = bf_hi(q.y);
    x[4] = bf_lo(q.z); x[5] = bf_hi(q.z); x[6] = bf_lo(q.w); x[7] = bf_hi(q.w);
}
__device__ __forceinline__ void load_gains(const bf16* gain, int lane, uint4 (&gq)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) gq[i] = *reinterpret_cast<const uint4*>(gain + (lane + 32 * i) * 8);
}
// RMSNorm of the row on the way into registers: xr = bf16(bf16(x * rstd) * gain), the value the following Linear sees
// in the eager model.  The lanes of a warp hold the whole row between them, so every warp reduces the sum of squares
// itself and the norm costs no CTA barrier.  `gq`: this lane's gains, loaded by the caller BEFORE it waits for the
// input: a global load issued after the wait would put a memory round trip on the critical path of every layer.
__device__ __forceinline__ void load_xreg_norm(const uint32_t* xs, const uint4 (&gq)[4], float eps, int lane, float (&xr)[32]) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        unpack8(*reinterpret_cast<const uint4*>(xs + (lane + 32 * i) * 4), &xr[i * 8]);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(xr[i * 8 + e], xr[i * 8 + e], ss);
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss * (1.0f / D) + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float g[8];
        unpack8(gq[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) xr[i * 8 + e] = bf16r(bf16r(xr[i * 8 + e] * rstd) * g[e]);
    }
}
// Several sequences: the rows are normalised in place in shared memory (a warp per row), for the tensor-core tiles.
template <int NB>
__device__ __forceinline__ void norm_rows_smem(Cta& c, const bf16* gain) {
    for (int b = c.warp; b < NB; b += kWarps) {
        uint32_t* row = c.xs + b * (FF / 2);
        uint4 gq[4];
        float xr[32];
        load_gains(gain, c.lane, gq);
        load_xreg_norm(row, gq, c.p.eps, c.lane, xr);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(row + (c.lane + 32 * i) * 4) =
                make_uint4(pack_bf16x2(xr[i * 8], xr[i * 8 + 1]), pack_bf16x2(xr[i * 8 + 2], xr[i * 8 + 3]),
                           pack_bf16x2(xr[i * 8 + 4], xr[i * 8 + 5]), pack_bf16x2(xr[i * 8 + 6], xr[i * 8 + 7]));
    }
    cta_sync();
}

// ---- sub-row dot products ------------------------------------------------------------------------------
// R rows of 1024 columns against the lane's 32 activations: four independent 128-bit accesses per row.
template <int R>
__device__ __forceinline__ void dot_rows_xreg(const bf16* const (&wp)[R], const float (&xr)[32], int lane, float (&acc)[R]) {
    uint4 w[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[r][i] = *reinterpret_cast<const uint4*>(wp[r] + (lane + 32 * i) * 8);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = dot8(w[r][i], &xr[i * 8], 0.f);      // four independent chains
        acc[r] = warp_sum((a[0] + a[1]) + (a[2] + a[3]));
    }
}
// One sub-row of CH * 256 columns against activations in shared memory (packed bf16 pairs).
template <int CH>
__device__ __forceinline__ float dot_subrow_smem(const bf16* w, const uint32_t* x, int lane) {
    uint4 wv[CH], xv[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        wv[i] = *reinterpret_cast<const uint4*>(w + (lane + 32 * i) * 8);
        xv[i] = *reinterpret_cast<const uint4*>(x + (lane + 32 * i) * 4);
    }
    float a[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        float xf[8];
        unpack8(xv[i], xf);
        a[i] = dot8(wv[i], xf, 0.f);
    }
    float s = a[0];
#pragma unroll
    for (int i = 1; i < CH; ++i) s += a[i];
    return warp_sum(s);
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
// This CTA's rows are whole quads (four consecutive outputs, which never straddle a head); a quad travels as one word
// to every CTA whose attention item belongs to the quad's kv head.
template <int NB>
__device__ bool phase_qkv(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t tag = tag_of(c, c.step, l);
    const bf16* gain = reinterpret_cast<const bf16*>(p.ln1) + (size_t)l * D;
    uint4 gq[4];
    if constexpr (NB == 1) load_gains(gain, c.lane, gq);
    bool ok = true;
    if (l == 0) {
        for (int i = c.tid; i < NB * (D / 2); i += kThreads) {
            const int b = i / (D / 2), t = i - b * (D / 2);
            c.xs[b * (FF / 2) + t] = ldcg32(reinterpret_cast<const bf16*>(p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * t);
        }
    } else {
        ok = gather7<NB, Q3_ROW_WORDS>(c, c.ws.mail_h + (size_t)c.cta * NB * MS, D, tag, ITTAI_PH_QKV, reinterpret_cast<uint16_t*>(c.xs));
    }
    int r0, r1;
    qkv_rows(c.ncta, c.cta, r0, r1);
    const bf16* W = nullptr;                                   // this CTA's rows [r0, r1), contiguous in the ring
    if (r1 > r0) {
        W = reinterpret_cast<const bf16*>(stream_wait(c.st, c.st.consumed, c.w));
        ok = ok && W != nullptr;
    }
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
    if constexpr (NB > 1) norm_rows_smem<NB>(c, gain);
    if (r1 == r0) return true;
    const int n_rows = r1 - r0;
    uint32_t* pub = reinterpret_cast<uint32_t*>(c.hdr->pub);      // packed output pairs, [sequence][kPubHalves / 2]
    if constexpr (NB == 1) {
        // one sequence: a row pair per warp on the fp32 pipes (the tensor-core tiles below are no faster here)
        float xr[32];
        load_xreg_norm(c.xs, gq, p.eps, c.lane, xr);
        for (int pr = c.warp; 2 * pr < n_rows; pr += kWarps) {
            const bf16* wp[2] = {W + (size_t)(2 * pr) * D, W + (size_t)(2 * pr + 1) * D};
            float acc[2];
            dot_rows_xreg<2>(wp, xr, c.lane, acc);
            if (c.lane == 0) pub[pr] = pack_bf16x2(acc[0], acc[1]);
        }
        stream_release(c.st, 1);                         // its barrier also publishes `pub` to the CTA
    } else {
        // tiles of 16 rows x 256 columns over the warps; the four column blocks of a row meet in shared memory
        const int n_tasks = (n_rows + 15) / 16 * 4;
        float* part = c.hdr->sub;
        for (int task = c.warp; task < n_tasks; task += kWarps) {
            float d[4];
            gemv_tile<NB>(W, D, (task >> 2) * 16, n_rows, c.xs, (task & 3) * 256, c.lane, d);
            gemv_store<NB>(part, task, c.lane, d);
        }
        stream_release(c.st, 1);                         // its barrier also publishes `part` to the CTA
        for (int i = c.tid; i < n_rows / 2 * NB; i += kThreads) {
            const int b = i / (n_rows / 2), pr = i - b * (n_rows / 2);
            pub[b * (kPubHalves / 2) + pr] = pack_bf16x2(gemv_sum<NB, 4>(part, 2 * pr, b), gemv_sum<NB, 4>(part, 2 * pr + 1, b));
        }
        cta_sync();
    }
    // quad q of sequence b -> the n_splits CTAs of (b, kv head of the quad)
    const int n_splits = q3_attn_splits(c.ncta, p.batch), n_quads = n_rows / 4;
    for (int i = c.tid; i < n_quads * n_splits * NB; i += kThreads) {
        const int s = i % n_splits, r = i / n_splits, qi = r % n_quads, b = r / n_quads;
        const int q = r0 / 4 + qi, head = q >> 5;                  // 32 quads per head; heads: 16 q | 8 k | 8 v
        const int g = head < 16 ? head >> 1 : (head - 16) & 7, which = head < 16 ? head & 1 : (head < 24 ? 2 : 3);
        const int dst = (b * NKV + g) * n_splits + s;
        st_mail(c.ws.mail_qkv + (size_t)dst * Q3_QKV_WORDS + which * 32 + (q & 31),
                pub[b * (kPubHalves / 2) + 2 * qi], pub[b * (kPubHalves / 2) + 2 * qi + 1], 0u, 0u, tag);
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
// and appended to the cache by the split that owns its position.  Each split mails (m, l, o-slice) to the first `nc`
// splits of its head, which each merge a slice of the 256 outputs and mail it to every CTA.
__device__ bool phase_attn(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const int B = p.batch;
    const int n_splits = q3_attn_splits(c.ncta, B), nc = q3_merge_ctas(n_splits), dpc = HD / nc;
    const int MW = q3_part_words_per_msg(nc), WPO = q3_attn_words_per_owner(nc);
    const uint32_t tag = tag_of(c, c.step, l);
    SmemAttn* at = c.at;
    const AttnItem it = attn_item(c, c.step);
    if (!it.active) { c.t_ready = clock64(); return true; }
    const int b = it.b, g = it.g, pos = it.pos;
    {
        const bool has_new = it.has_new;
        const size_t head_off = ((((size_t)l * B + b) * NKV + g) * (size_t)p.kv_cap) * HD;
        bf16* kc = reinterpret_cast<bf16*>(p.kcache) + head_off;
        bf16* vc = reinterpret_cast<bf16*>(p.vcache) + head_off;

        // -- norm + rotate q (warps 0,1) and the new key (warp 2); copy the new value (warp 3).
        //    A head's row arrives as 32 words of four values: a lane owns elements 4*lane .. 4*lane+3, and the rotation
        //    partner (element +-64) of each sits in lane ^ 16.  Gains and the rotary row are fetched before the wait, so
        //    their latency hides behind it.
        const uint4* qw = c.ws.mail_qkv + (size_t)c.cta * Q3_QKV_WORDS;
        bool ok = true;
        if (c.warp < 3 && (c.warp < 2 || has_new)) {
            const bool is_k = c.warp == 2;
            const bf16* gain = reinterpret_cast<const bf16*>(is_k ? p.kn : p.qn) + (size_t)l * HD;
            const bf16* rp = reinterpret_cast<const bf16*>(p.rope) + (size_t)pos * HD;
            const int hi_half = c.lane >> 4, ei = 4 * (c.lane & 15);        // rotation index of this lane's first element
            const uint2 gq = *reinterpret_cast<const uint2*>(gain + 4 * c.lane);
            const uint2 cq = *reinterpret_cast<const uint2*>(rp + ei);
            const uint2 sq = *reinterpret_cast<const uint2*>(rp + HD / 2 + ei);
            uint32_t u[4] = {0, 0, 0, 0};
            ok = wait_mail(c.w, qw + c.warp * 32 + c.lane, tag, u, ITTAI_PH_ATTN);
            float x[4] = {bf_lo(u[0]), bf_hi(u[0]), bf_lo(u[1]), bf_hi(u[1])};
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
                *reinterpret_cast<float4*>(&at->qs[c.warp][4 * c.lane]) = make_float4(r[0] * qscale, r[1] * qscale, r[2] * qscale, r[3] * qscale);
            }
        } else if (c.warp == 3 && has_new) {
            uint32_t u[4] = {0, 0, 0, 0};
            ok = wait_mail(c.w, qw + 3 * 32 + c.lane, tag, u, ITTAI_PH_ATTN);
            *reinterpret_cast<uint2*>(at->vnew + 4 * c.lane) = make_uint2(u[0], u[1]);
            if (ok) {
                *reinterpret_cast<uint2*>(vc + (size_t)pos * HD + 4 * c.lane) = make_uint2(u[0], u[1]);
                __threadfence();
                fence_proxy_async();
            }
        }
        if (!all_ok(ok)) return false;
        c.t_ready = clock64();

        // -- every half-warp runs its own online softmax over the positions it owns (position index = 2*warp + half
        //    modulo 32), with no CTA-wide barrier inside a tile; the 32 private (m, l, o) are merged once at the end.
        const int half = c.lane >> 4, sub = c.lane & 15;
        float q0[8], q1[8], acc0[8], acc1[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            q0[e] = at->qs[0][sub * 8 + e];
            q1[e] = at->qs[1][sub * 8 + e];
            acc0[e] = 0.f; acc1[e] = 0.f;
        }
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        // positions of this split: n_old rows from the ring, then (has_new) the current token's row
        const int n_pos = it.n_old + (has_new ? 1 : 0);
        const int n_ring_tiles = (it.n_old + kTile - 1) / kTile;
        int rel = 0;                 // ring tiles already handed back
        bool okr = true;
        // two tiles (K and V of each: 128 KB) are held before they go back, when the ring has room for that and more
        const int hold = c.st.ring_bytes >= 5u * kTile * HD * 2 ? 2 : 1;
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
            uint4 kk[kTile / 32];
            bool valid[kTile / 32];
#pragma unroll
            for (int r = 0; r < kTile / 32; ++r) {
                const int tl = r * 32 + c.warp * 2 + half;
                valid[r] = j * kTile + tl < n_pos;
                if (tl < ring_rows) kk[r] = *reinterpret_cast<const uint4*>(kt + (size_t)tl * HD + sub * 8);
                else if (has_new && j * kTile + tl == it.n_old) kk[r] = *reinterpret_cast<const uint4*>(at->knew + sub * 8);
                else kk[r] = make_uint4(0, 0, 0, 0);
            }
            float s0[kTile / 32], s1[kTile / 32];
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
                const int tl = r * 32 + c.warp * 2 + half;
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
        // -- merge the two halves of each warp, then the 16 warps: (m, l, o) of this split
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
        // this barrier publishes the per-warp partials, collects the ring verdicts and hands the last tiles back
        if (cta_or(!okr)) return false;
        if (n_ring_tiles > rel) stream_release_synced(c.st, 2 * (n_ring_tiles - rel));
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
            at->msg[4 + h * HD + d] = o;
            if (d == 0) { at->msg[h] = M; at->msg[2 + h] = ls; }
        }
        cta_sync();
        // -- mail the partial: owner j gets m[2], l[2] and its dpc dims of both heads, three floats per word
        for (int i = c.tid; i < nc * MW; i += kThreads) {
            const int j = i / MW, w = i - j * MW;
            float f[3];
#pragma unroll
            for (int e = 0; e < 3; ++e) {
                const int k = 3 * w + e, v = k - 4;
                f[e] = k < 4 ? at->msg[k] : (v < 2 * dpc ? at->msg[4 + (v / dpc) * HD + j * dpc + v % dpc] : 0.f);
            }
            const int owner = (b * NKV + g) * n_splits + j;
            st_mail(c.ws.mail_part + (size_t)owner * Q3_PART_WORDS + it.s * MW + w,
                    __float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), 0u, tag);
        }
    }
    // -- merge across splits: split s < nc of each (b, g) gathers, from every split of that head, the running max and
    //    sum and its own slice of the outputs
    if (it.s < nc) {
        float* pm = &at->ored[0][0][0];              // [split][3 * MW]: the messages as sent (all threads are past their reads of ored)
        bool ok = true;
        for (int i = c.tid; i < n_splits * MW; i += kThreads) {
            uint32_t v[4];
            if (!wait_mail(c.w, c.ws.mail_part + (size_t)c.cta * Q3_PART_WORDS + i, tag, v, 16 + ITTAI_PH_ATTN)) { ok = false; break; }
            pm[3 * i] = __uint_as_float(v[0]); pm[3 * i + 1] = __uint_as_float(v[1]); pm[3 * i + 2] = __uint_as_float(v[2]);
        }
        if (!all_ok(ok)) return false;
        // a warp per output, lanes = splits: three warp reductions finish it
        uint16_t* pub = c.hdr->pub;
        for (int v = c.warp; v < 2 * dpc; v += kWarps) {
            const int h = v / dpc;
            float m = -INFINITY, ls = 0.f, o = 0.f;
            if (c.lane < n_splits) {
                const float* ms = pm + c.lane * 3 * MW;
                m = ms[h]; ls = ms[2 + h]; o = ms[4 + v];
            }
            const float M = warp_max(m);
            const float wk = ex2_approx(m - (M == -INFINITY ? 0.f : M));
            const float Ls = warp_sum(ls * wk), O = warp_sum(o * wk);
            if (c.lane == 0) pub[v] = __bfloat16_as_ushort(__float2bfloat16_rn(O / Ls));
        }
        cta_sync();
        // the slice leaves as WPO words of seven values to every CTA
        for (int i = c.tid; i < c.ncta * WPO; i += kThreads) {
            const int dst = i / WPO, k = i - dst * WPO;
            send7(c.ws.mail_attn + (((size_t)dst * B + b) * NKV + g) * Q3_ATTN_WORDS + it.s * WPO + k, pub + 7 * k, 2 * dpc - 7 * k, tag);
        }
    }
    return true;
}

// Collects the attention output of every (sequence, kv head) from this CTA's mailbox into xs[b][2048].
template <int NB>
__device__ __forceinline__ bool gather_attn(Cta& c, uint32_t tag) {
    const int n_splits = q3_attn_splits(c.ncta, c.p.batch), nc = q3_merge_ctas(n_splits), dpc = HD / nc;
    const int WPO = q3_attn_words_per_owner(nc), per = nc * WPO;
    uint16_t* dst = reinterpret_cast<uint16_t*>(c.xs);
    const uint4* mail = c.ws.mail_attn + (size_t)c.cta * NB * NKV * Q3_ATTN_WORDS;
    for (int i = c.tid; i < NB * NKV * per; i += kThreads) {
        const int bg = i / per, r = i - bg * per, j = r / WPO, k = r - j * WPO;
        const int b = bg / NKV, g = bg - b * NKV;
        uint32_t v[4];
        if (!wait_mail(c.w, mail + (size_t)bg * Q3_ATTN_WORDS + r, tag, v, ITTAI_PH_OPROJ)) return false;
#pragma unroll
        for (int e = 0; e < 7; ++e) {
            const int x = 7 * k + e;                 // index into the owner's 2 * dpc values: head-major
            if (x < 2 * dpc) dst[b * FF + (2 * g + x / dpc) * HD + j * dpc + x % dpc] = (uint16_t)(v[e >> 1] >> ((e & 1) * 16));
        }
    }
    return true;
}

// ---- phases: O-proj + residual, down-proj + residual ---------------------------------------------------
// K is 2048 or 3072: each of this CTA's six or seven rows is cut into two sub-rows, one per warp; the two partial sums
// meet in shared memory.  out = bf16(resid + bf16(W x)) (reference base.py:110-123).  The residual rows are the ones
// this CTA produced itself one phase pair earlier; they come back from its own mailbox (`res_mail` == nullptr takes
// them from the embedding row: layer 0's o_proj).  The result leaves as one word per sequence to every CTA.
enum { kFromAttn = 0, kFromAct = 1 };
template <int NB, int K, int SRC>
__device__ bool phase_proj_residual(Cta& c, int what, int l, uint32_t x_tag, const uint4* res_mail, uint32_t res_tag,
                                    uint4* dst_mail, uint32_t dst_tag) {
    constexpr int CH = K / 512;              // 16-byte chunks per lane of a half row (K / 2 columns)
    int r0, r1;
    res_rows(c.ncta, c.cta, r0, r1);
    const int n_rows = r1 - r0;
    // The residual rows were published phases ago: fetch them now, not after the GEMV.
    bool ok = true;
    if (c.tid < NB) {
        const int b = c.tid;
        uint16_t* res = c.hdr->res + b * 8;
        if (res_mail == nullptr) {
            for (int e = 0; e < n_rows; ++e)
                res[e] = __bfloat16_as_ushort(reinterpret_cast<const bf16*>(c.p.embed)[(size_t)c.hdr->tok_s[b] * D + r0 + e]);
        } else {
            uint32_t v[4] = {0, 0, 0, 0};
            ok = wait_mail(c.w, res_mail + ((size_t)c.cta * NB + b) * MS + c.cta, res_tag, v, 32 + what);
            unpack7(v, res, n_rows);
        }
    }
    if constexpr (SRC == kFromAttn) ok = gather_attn<NB>(c, x_tag) && ok;
    else ok = gather7<NB, Q3_ACT_WORDS>(c, c.ws.mail_act + (size_t)c.cta * NB * MS * Q3_ACT_WORDS, FF, x_tag, what, reinterpret_cast<uint16_t*>(c.xs)) && ok;
    const bf16* W = nullptr;                                   // this CTA's rows [r0, r1), contiguous in the ring
    if (n_rows > 0) {
        W = reinterpret_cast<const bf16*>(stream_wait(c.st, c.st.consumed, c.w));
        ok = ok && W != nullptr;
    }
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
    // every cache row appended up to (step, l) is ordered before what this CTA has now seen: the feeding lane may
    // fetch the tiles of (step + 1, l)
    if (SRC == kFromAttn && c.tid == 0) c.st.sh->kv_epoch = (uint32_t)(c.step * c.p.n_layers + l) + 1u;
    if (n_rows == 0) return true;
    float* sub = c.hdr->sub;
    if constexpr (NB == 1) {
        for (int t = c.warp; t < 2 * n_rows; t += kWarps) {
            const int row = t >> 1, half = t & 1;
            const float s = dot_subrow_smem<CH>(W + (size_t)row * K + half * (K / 2), c.xs + half * (K / 4), c.lane);
            if (c.lane == 0) sub[t] = s;
        }
    } else {
        // several sequences: tiles of up to 16 rows x 256 columns on the tensor cores, one column block per warp
        constexpr int NK = K / 256;
        for (int task = c.warp; task < NK; task += kWarps) {
            float d[4];
            gemv_tile<NB>(W, K, 0, n_rows, c.xs, task * 256, c.lane, d);
            gemv_store<NB>(sub, task, c.lane, d);
        }
    }
    cta_sync();
    stream_release_synced(c.st, 1);
    // every sending thread finishes the CTA's rows of its sequence itself (a dozen additions) and mails one word
    for (int i = c.tid; i < c.ncta * NB; i += kThreads) {
        const int dst = i / NB, b = i - dst * NB;
        const uint16_t* res = c.hdr->res + b * 8;
        uint32_t h[7];
#pragma unroll
        for (int e = 0; e < 7; ++e) {
            float s = 0.f;
            if (e < n_rows) {
                if constexpr (NB == 1) s = sub[2 * e] + sub[2 * e + 1];
                else s = gemv_sum<NB, K / 256>(sub, e, b);
            }
            const float y = __uint_as_float((uint32_t)res[e] << 16) + bf16r(s);
            h[e] = e < n_rows ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y)) : 0u;
        }
        st_mail(dst_mail + ((size_t)dst * NB + b) * MS + c.cta, h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6], dst_tag);
    }
    return true;
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
    const bf16* gain = reinterpret_cast<const bf16*>(p.ln2) + (size_t)l * D;
    uint4 gq[4];
    if constexpr (NB == 1) load_gains(gain, c.lane, gq);
    bool ok = gather7<NB, Q3_ROW_WORDS>(c, c.ws.mail_hmid + (size_t)c.cta * NB * MS, D, tag, ITTAI_PH_GU, reinterpret_cast<uint16_t*>(c.xs));
    int a0, a1;
    act_cols(c.ncta, c.cta, a0, a1);             // this CTA's SwiGLU outputs: weight rows 2 a0 .. 2 a1
    const int n_act = a1 - a0;
    const bf16* W = nullptr;
    if (n_act > 0) {
        W = reinterpret_cast<const bf16*>(stream_wait(c.st, c.st.consumed, c.w));
        ok = ok && W != nullptr;
    }
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
    if constexpr (NB > 1) norm_rows_smem<NB>(c, gain);
    if (n_act == 0) return true;
    uint16_t* pub = c.hdr->pub;                  // [sequence][kPubHalves]
    if constexpr (NB == 1) {
        float xr[32];
        load_xreg_norm(c.xs, gq, p.eps, c.lane, xr);
        for (int un = c.warp; 2 * un < n_act; un += kWarps) {        // two outputs = four weight rows per warp
            const bool two = 2 * un + 1 < n_act;
            const bf16* wu = W + (size_t)(4 * un) * D;
            const bf16* wp[4] = {wu, wu + D, two ? wu + 2 * D : wu, two ? wu + 3 * D : wu + D};
            float acc[4];
            dot_rows_xreg<4>(wp, xr, c.lane, acc);
            if (c.lane == 0) {
                pub[2 * un] = __bfloat16_as_ushort(__float2bfloat16_rn(swiglu(acc[0], acc[1])));
                if (two) pub[2 * un + 1] = __bfloat16_as_ushort(__float2bfloat16_rn(swiglu(acc[2], acc[3])));
            }
        }
        stream_release(c.st, 1);                         // its barrier also publishes `pub` to the CTA
    } else {
        const int n_rows = 2 * n_act, n_tasks = (n_rows + 15) / 16 * 4;
        float* part = c.hdr->sub;
        for (int task = c.warp; task < n_tasks; task += kWarps) {
            float d[4];
            gemv_tile<NB>(W, D, (task >> 2) * 16, n_rows, c.xs, (task & 3) * 256, c.lane, d);
            gemv_store<NB>(part, task, c.lane, d);
        }
        stream_release(c.st, 1);                         // its barrier also publishes `part` to the CTA
        for (int i = c.tid; i < n_act * NB; i += kThreads) {
            const int b = i / n_act, a = i - b * n_act;
            pub[b * kPubHalves + a] = __bfloat16_as_ushort(__float2bfloat16_rn(
                swiglu(gemv_sum<NB, 4>(part, 2 * a, b), gemv_sum<NB, 4>(part, 2 * a + 1, b))));
        }
        cta_sync();
    }
    // the outputs leave as three words of seven values per sequence to every CTA
    for (int i = c.tid; i < c.ncta * Q3_ACT_WORDS * NB; i += kThreads) {
        const int k = i % Q3_ACT_WORDS, r = i / Q3_ACT_WORDS, b = r % NB, dst = r / NB;
        send7(c.ws.mail_act + (((size_t)dst * NB + b) * MS + c.cta) * Q3_ACT_WORDS + k, pub + b * kPubHalves + 7 * k, n_act - 7 * k, tag);
    }
    return true;
}

// ---- phase: final RMSNorm + tied lm_head GEMV + argmax ------------------------------------------------
// logits = bf16(W_embed x); argmax over the bf16 values, lowest index wins ties (torch semantics).  The table rows come
// through the ring in entries of 32.  Every CTA mails its best (value, index) to every CTA, so each knows the next token
// at once.
template <int NB>
__device__ bool phase_head(Cta& c) {
    const IttaiQwen3Decode& p = c.p;
    const bf16* gain = reinterpret_cast<const bf16*>(p.fin_w);
    uint4 gq[4];
    if constexpr (NB == 1) load_gains(gain, c.lane, gq);
    bool ok = gather7<NB, Q3_ROW_WORDS>(c, c.ws.mail_h + (size_t)c.cta * NB * MS, D, tag_of(c, c.step, p.n_layers), ITTAI_PH_HEAD,
                                        reinterpret_cast<uint16_t*>(c.xs));
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
    float xr[32];
    if constexpr (NB == 1) load_xreg_norm(c.xs, gq, p.eps, c.lane, xr);
    else norm_rows_smem<NB>(c, gain);
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
        } else {
            const int lr = c.warp * R;                                 // this warp's first row inside the entry
            if (lr < rows_here) {
                const bf16* wp[R];
#pragma unroll
                for (int r = 0; r < R; ++r) wp[r] = W + (size_t)(lr + r < rows_here ? lr + r : rows_here - 1) * D;
                float acc[R];
                dot_rows_xreg<R>(wp, xr, c.lane, acc);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (lr + r < rows_here) {
                        const int row = e0 + lr + r;
                        const float v = bf16r(acc[r]);
                        if (v > bv[0]) { bv[0] = v; bi[0] = row; }   // rows ascend within a warp: first max kept
                        if (p.write_logits && c.lane == 0) logits[row] = __float2bfloat16_rn(v);
                    }
                }
            }
            stream_release(c.st, 1);
        }
    }
    const uint32_t tag = 1u + (uint32_t)c.step % 65535u;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        if (c.lane == 0) { c.hdr->bestv[c.warp] = bv[b]; c.hdr->besti[c.warp] = bi[b]; }
        cta_sync();
        bool okb = true;
        if (c.tid < c.ncta) {
            // every sending thread folds the warps' candidates itself and mails the CTA's best to CTA `tid` ...
            float v = c.hdr->bestv[0];
            int ix = c.hdr->besti[0];
            for (int w = 1; w < kWarps; ++w) {
                const float vw = c.hdr->bestv[w];
                const int iw = c.hdr->besti[w];
                if (vw > v || (vw == v && iw < ix)) { v = vw; ix = iw; }
            }
            st_mail(c.ws.mail_cand + ((size_t)c.tid * NB + b) * MS + c.cta, __float_as_uint(v), (uint32_t)ix, 0u, 0u, tag);
            // ... and collects the best of CTA `tid`
            uint32_t u[4] = {0, 0, 0, 0};
            okb = wait_mail(c.w, c.ws.mail_cand + ((size_t)c.cta * NB + b) * MS + c.tid, tag, u, 16 + ITTAI_PH_HEAD);
            c.hdr->candv[c.tid] = __uint_as_float(u[0]);
            c.hdr->candi[c.tid] = (int)u[1];
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
        case ITTAI_PH_ATTN: return phase_attn(c, l);
        case ITTAI_PH_OPROJ:
            return phase_proj_residual<NB, DQ, kFromAttn>(c, ITTAI_PH_OPROJ, l, tag, l == 0 ? nullptr : c.ws.mail_h, tag, c.ws.mail_hmid, tag);
        case ITTAI_PH_GU: return phase_gu<NB>(c, l);
        case ITTAI_PH_DOWN:
            return phase_proj_residual<NB, FF, kFromAct>(c, ITTAI_PH_DOWN, l, tag, c.ws.mail_hmid, tag, c.ws.mail_h, tag_of(c, c.step, l + 1));
        default: return phase_head<NB>(c);
    }
}

// The per-CTA context is brace-initialised inside each kernel.  nvcc 12.9 mis-infers the shared state space for the
// global pointers of a struct returned by value from a helper that also receives the shared-memory base, so there is
// deliberately no make_cta() function.
#define ITTAI_MAKE_CTA(p, wsp, smem, nb, ring_bytes)                                                              \
    Cta c{p, wsp, reinterpret_cast<SmemHdr*>(smem), reinterpret_cast<uint32_t*>(smem + kHdrBytes),                   \
          reinterpret_cast<SmemAttn*>(smem + kHdrBytes), (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x,       \
          (int)(threadIdx.x & 31), (int)(threadIdx.x >> 5),                                                       \
          Waiter{wsp.sync, p.status, p.spin_limit > 0 ? (uint32_t)p.spin_limit : kSpinLimit},                     \
          Stream{&reinterpret_cast<SmemHdr*>(smem)->stream, smem + q3_fixed_smem_bytes(nb), ring_bytes, 0u},      \
          0, 0}

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
            // before any mailbox of the chain is written again.
            ok = all_ok(gather7<NB, Q3_ROW_WORDS>(c, c.ws.mail_h + (size_t)c.cta * NB * MS, D, tag_of(c, step - 1, p.n_layers), 64,
                                                 reinterpret_cast<uint16_t*>(c.xs)));
            if (!ok) break;
        }
        for (int l = 0; l < p.n_layers && ok; ++l) {
#pragma unroll 1
            for (int phase = ITTAI_PH_QKV; phase <= ITTAI_PH_DOWN && ok; ++phase) {
                ok = run_phase<NB>(c, phase, l);
                if (prof && ok) {
                    const size_t slot = ((size_t)step * (5 * p.n_layers + 1) + l * 5 + phase) * 2;
                    p.phase_clk[slot] = (uint64_t)c.t_ready;
                    p.phase_clk[slot + 1] = (uint64_t)clock64();
                }
            }
        }
        if (run_head && ok) {
            ok = phase_head<NB>(c);
            if (prof && ok) {
                const size_t slot = ((size_t)step * (5 * p.n_layers + 1) + 5 * p.n_layers) * 2;
                p.phase_clk[slot] = (uint64_t)c.t_ready;
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

// One phase on its own at step 0 (tags of step 0): unit tests and per-phase profiles.  The inputs must sit in the
// mailboxes with the tag of (step 0, layer); launched cooperatively because the attention merge and the head wait on
// other CTAs.
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

// What the kernel's fixed-size buffers assume about the grid: checked on the host so that a device the plan does not
// fit is refused instead of overrunning a mailbox or waiting for a slice the ring can never hold.
int q3_check_plan(int grid, int batch, uint32_t ring_bytes, char* why, size_t why_len) {
    int lo, hi, rows_max = 0, act_max = 0, qkv_max = 0;
    for (int c = 0; c < grid; ++c) {
        res_rows(grid, c, lo, hi); rows_max = hi - lo > rows_max ? hi - lo : rows_max;
        act_cols(grid, c, lo, hi); act_max = hi - lo > act_max ? hi - lo : act_max;
        qkv_rows(grid, c, lo, hi); qkv_max = hi - lo > qkv_max ? hi - lo : qkv_max;
    }
    if (grid < 1 || grid > Q3_MAX_CTAS) { snprintf(why, why_len, "grid %d outside 1..%d", grid, Q3_MAX_CTAS); return ITTAI_E_DEVICE; }
    if (rows_max > 7 * Q3_ROW_WORDS || act_max > 7 * Q3_ACT_WORDS || qkv_max > kPubHalves) {
        snprintf(why, why_len, "%d CTAs leave %d residual rows, %d SwiGLU outputs, %d projection rows to one CTA: more than its mail words hold", grid, rows_max, act_max, qkv_max);
        return ITTAI_E_DEVICE;
    }
    if (grid < batch * NKV) { snprintf(why, why_len, "%d SMs cannot hold one attention item per CTA at batch %d", grid, batch); return ITTAI_E_DEVICE; }
    const int n_splits = q3_attn_splits(grid, batch), nc = q3_merge_ctas(n_splits);
    if (n_splits * q3_part_words_per_msg(nc) > Q3_PART_WORDS || nc * q3_attn_words_per_owner(nc) > Q3_ATTN_WORDS) {
        snprintf(why, why_len, "%d cache splits merged by %d CTAs do not fit the attention mailboxes", n_splits, nc);
        return ITTAI_E_DEVICE;
    }
    // Every slice must fit the ring on its own (an empty ring restarts at its base), and the attention phase holds two
    // K and two V tiles before it hands any back.
    size_t slice = (size_t)qkv_max * D * 2;
    const size_t cand[] = {(size_t)act_max * 2 * D * 2, (size_t)rows_max * DQ * 2, (size_t)rows_max * FF * 2, (size_t)kHeadRows * D * 2,
                           (size_t)4 * kTile * HD * 2};
    for (size_t s : cand) slice = s > slice ? s : slice;
    if (slice > ring_bytes) { snprintf(why, why_len, "a %zu-byte weight slice does not fit the %u-byte shared-memory ring", slice, ring_bytes); return ITTAI_E_DEVICE; }
    return ITTAI_OK;
}
static int check_plan(int grid, int batch, uint32_t ring_bytes) {
    char why[200];
    const int rc = q3_check_plan(grid, batch, ring_bytes, why, sizeof why);
    if (rc != ITTAI_OK) set_error("%s", why);
    return rc;
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
    if (grid < Q3_MIN_CTAS) {
        set_error("the decode kernel's mailboxes are sized for one CTA on each of a B200's %d SMs (found %d)", Q3_MAX_CTAS, g_info.n_sms);
        return ITTAI_E_DEVICE;
    }
    // all the shared memory a CTA may have: header + activations + the weight ring
    const size_t fixed = q3_fixed_smem_bytes(NB);
    const size_t smem = (size_t)g_info.smem_optin;
    if (smem < fixed + 96 * 1024) { set_error("%zu bytes of shared memory per CTA leave no room for the weight ring", smem); return ITTAI_E_DEVICE; }
    uint32_t ring_bytes = (uint32_t)((smem - fixed) / 1024 * 1024);
    rc = check_plan(grid, p->batch, ring_bytes);
    if (rc != ITTAI_OK) return rc;
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
    if (phase < 0) {   // a phase launch keeps the mail its caller prepared
        e = cudaMemsetAsync(ws.mail_h, 0, ws.mail_bytes, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(mailboxes)");
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

extern "C" int ittai_qwen3_decode_layout(int batch, int n_sms, IttaiQwen3Layout* out) {
    if (!out || (batch != 1 && batch != 2 && batch != 4 && batch != 8)) { ittai::set_error("batch must be 1, 2, 4 or 8 and the output non-null"); return ITTAI_E_ARG; }
    const int grid = n_sms < ittai::Q3_MAX_CTAS ? n_sms : ittai::Q3_MAX_CTAS;
    char why[200];
    if (ittai::q3_check_plan(grid, batch, 0xffffffffu, why, sizeof why) != ITTAI_OK || grid < ittai::Q3_MIN_CTAS) {
        ittai::set_error("no decode plan for %d SMs at batch %d", n_sms, batch);
        return ITTAI_E_DEVICE;
    }
    ittai::Q3Workspace ws;
    size_t offs[ittai::Q3_N_REGIONS];
    out->bytes = ittai::q3_ws_layout(batch, nullptr, &ws, offs);
    out->off_h = offs[1]; out->off_hmid = offs[2]; out->off_act = offs[3]; out->off_attn = offs[4];
    out->off_qkv = offs[5]; out->off_part = offs[6]; out->off_cand = offs[7];
    out->n_ctas = grid;
    out->mail_stride = ittai::Q3_MAIL_STRIDE;
    out->act_words = ittai::Q3_ACT_WORDS;
    out->attn_words = ittai::Q3_ATTN_WORDS;
    out->qkv_words = ittai::Q3_QKV_WORDS;
    out->n_splits = ittai::q3_attn_splits(grid, batch);
    out->merge_ctas = ittai::q3_merge_ctas(out->n_splits);
    out->attn_words_per_owner = ittai::q3_attn_words_per_owner(out->merge_ctas);
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
// not acceptable.  For them the decode kernel's workspace (the CTAs' mailboxes and the abort flag) lives in this
// file-scope device array instead of a caller buffer.  Every GPU that loads the library
// holds these bytes until the process exits.
namespace ittai {

constexpr int kStaticMaxBatch = ITTAI_STATIC_DECODE_MAX_BATCH;
constexpr size_t kStaticScratchBytes = q3_ws_bytes(kStaticMaxBatch);      // the mailboxes of two sequences: about 7.5 MB
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
