// Qwen3-0.6B decode: one persistent cooperative kernel per launch runs n_steps tokens; the chosen token id is fed
// back on the device.  The phases of a layer are chained by data flow, not by grid barriers: every vector one phase
// hands to the next travels as flagged 64-bit words (payload + tag of the producing step and layer), and a consumer
// polls exactly the words it needs (see qwen3_ws.h).
//
// Batch-1 decode is HBM-bound (about 1.4 flop per weight byte), so there are no tensor-core tiles here: each warp
// streams whole 1024-column weight sub-rows with 128-bit coalesced loads and reduces with shuffles.  Rounding points
// follow the eager modules: every Linear output, norm output, rotary product and sum, SiLU, gate*up product and
// residual sum is rounded to bf16 exactly once.
//
// The math per phase mirrors the fused epilogues of the reference's megakernel (src/ittai/qwen3/base.py:80-129 for
// qkv / residual / gate-up, :147-162 for the embedding row), re-cut for one token: the row-norm scale is applied before
// the GEMV instead of after the GEMM, and keys and values go straight into the cache instead of a staging matrix.
// KV cache, split-K decode attention, lm_head and argmax have no counterpart in the reference.
#include "common.cuh"
#include "qwen3_ws.h"

namespace ittai {

constexpr int D = ITTAI_Q3_D, NKV = ITTAI_Q3_NKV, HD = ITTAI_Q3_HD, FF = ITTAI_Q3_FF;
constexpr int DQ = ITTAI_Q3_DQ, DKV = ITTAI_Q3_DKV, DQKV = ITTAI_Q3_DQKV, DGU = ITTAI_Q3_DGU;
constexpr int kTile = 256;                       // cache positions scored per attention tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kCombMax = 640;                    // floats the combine step gathers (worst case over split counts)

// ---- shared-memory plan (dynamic) ----------------------------------------------------------------------
struct SmemHdr {
    float red[32];
    float m_s[2], l_s[2], corr_s[2];
    int pos_s[ITTAI_MAX_BATCH];
    int tok_s[ITTAI_MAX_BATCH];
    float bestv[kWarps];
    int besti[kWarps];
    float sub[64 * ITTAI_MAX_BATCH];             // per-sub-row partial dot products
    float comb[kCombMax];                        // split-K partials gathered by the combine step
    float candv[Q3_MAX_CTAS];                    // argmax candidates of every CTA
    int candi[Q3_MAX_CTAS];
};
struct SmemAttn {
    float sc[2][kTile];                          // scores, then probabilities, of the two query heads of a group
    float qs[2][HD];                             // rotated, pre-scaled queries
    bf16 knew[HD];
    bf16 vnew[HD];
    float ored[kWarps][2][HD];
};
constexpr size_t kHdrBytes = (sizeof(SmemHdr) + 255) / 256 * 256;
__host__ __device__ constexpr size_t q3_smem_bytes(int nb) {
    size_t xs = (size_t)nb * FF * sizeof(float);
    size_t at = sizeof(SmemAttn);
    return kHdrBytes + (xs > at ? xs : at);
}

struct Cta {
    const IttaiQwen3Decode& p;
    Q3Workspace ws;
    SmemHdr* hdr;
    float* xs;          // [NB][FF] activations of the current GEMV
    SmemAttn* at;       // aliases xs
    int cta, ncta, tid, lane, warp;
    Waiter w;
    int step;           // token index inside this launch
    long long t_ready;  // cycle counter when the current phase had its inputs (in-kernel profile)
};

// Tag of the data a (step, layer) produces; layer n_layers names the stream entering the head.  Never zero.
__device__ __forceinline__ uint32_t tag_of(const Cta& c, int step, int l) { return (uint32_t)(step * (c.p.n_layers + 1) + l + 1); }

// CTA-uniform verdict on per-thread waits.
__device__ __forceinline__ bool all_ok(bool ok) { return __syncthreads_or(ok ? 0 : 1) == 0; }

// ---- RMSNorm of one row (already in registers, one bf16 pair per thread) into shared memory --------------
// xs[i] = bf16(bf16(x*rstd) * gain): the value the following Linear sees in the eager model.
__device__ __forceinline__ void norm_pair_to_smem(Cta& c, uint32_t u, const bf16* gain, float* xs_row) {
    static_assert(kThreads * 2 == D, "one bf16 pair per thread");
    const uint32_t gw = *reinterpret_cast<const uint32_t*>(gain + 2 * c.tid);
    const float x0 = bf_lo(u), x1 = bf_hi(u);
    const float tot = block_sum(x0 * x0 + x1 * x1, c.hdr->red);
    const float rstd = 1.0f / sqrtf(tot * (1.0f / D) + c.p.eps);
    xs_row[2 * c.tid] = bf16r(bf16r(x0 * rstd) * bf_lo(gw));
    xs_row[2 * c.tid + 1] = bf16r(bf16r(x1 * rstd) * bf_hi(gw));
}

// Waits for NB rows of K bf16 values in flagged-word format and spreads them into xs as fp32.
template <int NB, int K>
__device__ __forceinline__ bool wait_rows_to_smem(Cta& c, const uint64_t* src, uint32_t tag, int what) {
    bool ok = true;
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int i = 0; i < K / 2 / kThreads; ++i) {
            const int wd = c.tid + i * kThreads;
            uint32_t u = 0;
            ok = ok && wait_word(c.w, src + (size_t)b * (K / 2) + wd, tag, u, what);
            c.xs[b * FF + 2 * wd] = bf_lo(u);
            c.xs[b * FF + 2 * wd + 1] = bf_hi(u);
        }
    return all_ok(ok);
}

// ---- 1024-column sub-row dot products ------------------------------------------------------------------
// Lane owns the 16-byte chunks lane, lane+32, lane+64, lane+96 of a sub-row: four independent 128-bit loads per
// sub-row, R sub-rows in flight.  Batch 1 keeps its 32 activations in registers; larger batches read shared memory.
__device__ __forceinline__ void load_xreg(const float* xs, int lane, float (&xr)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(xs + (lane + 32 * i) * 8);
        const float4 b = *reinterpret_cast<const float4*>(xs + (lane + 32 * i) * 8 + 4);
        xr[i * 8 + 0] = a.x; xr[i * 8 + 1] = a.y; xr[i * 8 + 2] = a.z; xr[i * 8 + 3] = a.w;
        xr[i * 8 + 4] = b.x; xr[i * 8 + 5] = b.y; xr[i * 8 + 6] = b.z; xr[i * 8 + 7] = b.w;
    }
}

template <int R>
__device__ __forceinline__ void dot_subrows_xreg(const bf16* const (&wp)[R], const float (&xr)[32], int lane,
                                                 float (&acc)[R]) {
    uint4 w[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[r][i] = ldg_stream(wp[r] + (lane + 32 * i) * 8);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) a = dot8(w[r][i], &xr[i * 8], a);
        acc[r] = warp_sum(a);
    }
}

// xseg points at the 1024-float segment this sub-row multiplies, for batch row 0; batch rows are FF floats apart.
template <int NB, int R>
__device__ __forceinline__ void dot_subrows_smem(const bf16* const (&wp)[R], const float* const (&xseg)[R], int lane,
                                                 float (&acc)[R][NB]) {
    uint4 w[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) w[r][i] = ldg_stream(wp[r] + (lane + 32 * i) * 8);
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float* x = xseg[r] + b * FF + (lane + 32 * i) * 8;
                float xv[8];
                *reinterpret_cast<float4*>(xv) = *reinterpret_cast<const float4*>(x);
                *reinterpret_cast<float4*>(xv + 4) = *reinterpret_cast<const float4*>(x + 4);
                a = dot8(w[r][i], xv, a);
            }
            acc[r][b] = warp_sum(a);
        }
}

// Generic "R sub-rows" step used by all K=1024 phases.
template <int NB, int R>
__device__ __forceinline__ void dot_rows_k1024(Cta& c, const bf16* const (&wp)[R], const float (&xr)[32],
                                               float (&acc)[R][NB]) {
    if constexpr (NB == 1) {
        float a[R];
        dot_subrows_xreg<R>(wp, xr, c.lane, a);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r][0] = a[r];
    } else {
        const float* xseg[R];
#pragma unroll
        for (int r = 0; r < R; ++r) xseg[r] = c.xs;
        dot_subrows_smem<NB, R>(wp, xseg, c.lane, acc);
    }
}

__device__ __forceinline__ void split_range(int n, int parts, int i, int& lo, int& hi) {
    lo = (int)(((long long)n * i) / parts);
    hi = (int)(((long long)n * (i + 1)) / parts);
}

__device__ __forceinline__ int attn_splits(int ncta, int batch) {
    int s = ncta / (batch * NKV);
    return s < 1 ? 1 : (s > Q3_MAX_SPLITS ? Q3_MAX_SPLITS : s);
}
// Cache range [start, end) of split s at context length n_ctx, in multiples of 32 positions.
__device__ __forceinline__ void attn_range(int n_ctx, int n_splits, int s, int& start, int& end, int& chunk) {
    chunk = (((n_ctx + n_splits - 1) / n_splits) + 31) & ~31;
    start = s * chunk;
    end = start + chunk < n_ctx ? start + chunk : n_ctx;
}

// ---- L2 prefetch ------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_bytes(const Cta& c, const void* base, size_t bytes) {
    constexpr uint32_t kPiece = 4096;
    const char* p = reinterpret_cast<const char*>(base);
    for (size_t off = (size_t)c.tid * kPiece; off < bytes; off += (size_t)kThreads * kPiece) {
        const size_t n = bytes - off < kPiece ? bytes - off : kPiece;
        l2_prefetch(p + off, (uint32_t)n);
    }
}
// rows are split over CTAs in multiples of `unit` rows exactly as the phases do
__device__ __forceinline__ void prefetch_slice(const Cta& c, const bf16* base, size_t row_bytes, int n_rows, int unit) {
    int lo, hi;
    split_range(n_rows / unit, c.ncta, c.cta, lo, hi);
    prefetch_bytes(c, reinterpret_cast<const char*>(base) + (size_t)lo * unit * row_bytes, (size_t)(hi - lo) * unit * row_bytes);
}

// ---- phase: embed gather (layer 0) + RMSNorm + QKV GEMV ------------------------------------------------
template <int NB>
__device__ bool phase_qkv(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const uint32_t tag = tag_of(c, c.step, l);
    uint32_t u[NB];
    bool ok = true;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        if (l == 0) u[b] = ldcg32(reinterpret_cast<const bf16*>(p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * c.tid);
        else ok = ok && wait_word(c.w, c.ws.h + b * (D / 2) + c.tid, tag, u[b], ITTAI_PH_QKV);
    }
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
#pragma unroll
    for (int b = 0; b < NB; ++b) norm_pair_to_smem(c, u[b], reinterpret_cast<const bf16*>(p.ln1) + (size_t)l * D, c.xs + b * FF);
    __syncthreads();
    float xr[32];
    if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
    const bf16* W = reinterpret_cast<const bf16*>(p.wqkv) + (size_t)l * DQKV * D;
    int p0, p1;
    split_range(DQKV / 2, c.ncta, c.cta, p0, p1);
    for (int pr = p0 + c.warp; pr < p1; pr += kWarps) {
        const bf16* wp[2] = {W + (size_t)(2 * pr) * D, W + (size_t)(2 * pr + 1) * D};
        float acc[2][NB];
        dot_rows_k1024<NB, 2>(c, wp, xr, acc);
        if (c.lane == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) st_flagged(c.ws.qkv + b * (DQKV / 2) + pr, pack_bf16x2(acc[0][b], acc[1][b]), tag);
        }
    }
    return true;
}

// ---- phase: QK-RMSNorm + RoPE + KV append + split-K GQA attention + combine ---------------------------
// Work item = (sequence b, kv head g, split s); CTA i takes item i.  Scores live in the log2 domain with the
// softmax scale folded into q, as the reference does (src/ittai/qwen3/config.py:6-7).  Each split publishes
// (m, l, o[2][128]); the first `nc` splits of a head then each merge a slice of the 256 outputs.
__device__ bool phase_attn(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const int B = p.batch;
    const int n_splits = attn_splits(c.ncta, B);
    const int n_items = B * NKV * n_splits;
    const uint32_t tag = tag_of(c, c.step, l);
    SmemAttn* at = c.at;
    bool first = true;
    for (int item = c.cta; item < n_items; item += c.ncta) {
        const int b = item / (NKV * n_splits), g = (item / n_splits) % NKV, s = item % n_splits;
        const int pos = c.hdr->pos_s[b], n_ctx = pos + 1;
        int start, end, chunk;
        attn_range(n_ctx, n_splits, s, start, end, chunk);
        const bool has_new = pos >= start && pos < start + chunk;
        const uint64_t* qw = c.ws.qkv + (size_t)b * (DQKV / 2);
        const size_t head_off = ((((size_t)l * B + b) * NKV + g) * (size_t)p.kv_cap) * HD;
        bf16* kc = reinterpret_cast<bf16*>(p.kcache) + head_off;
        bf16* vc = reinterpret_cast<bf16*>(p.vcache) + head_off;

        // -- norm + rotate q (warps 0,1) and the new key (warp 2); copy the new value (warp 3).
        //    A lane owns elements 2*lane, 2*lane+1 and their rotation partners 64 + the same.
        bool ok = true;
        if (c.warp < 3 && (c.warp < 2 || has_new)) {
            const bool is_k = c.warp == 2;
            const int e0 = is_k ? DQ + g * HD : (2 * g + c.warp) * HD;
            const bf16* gain = reinterpret_cast<const bf16*>(is_k ? p.kn : p.qn) + (size_t)l * HD;
            uint32_t ua = 0, ub = 0;
            ok = wait_word(c.w, qw + e0 / 2 + c.lane, tag, ua, ITTAI_PH_ATTN);
            ok = ok && wait_word(c.w, qw + e0 / 2 + 32 + c.lane, tag, ub, ITTAI_PH_ATTN);
            float x[4] = {bf_lo(ua), bf_hi(ua), bf_lo(ub), bf_hi(ub)};
            const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
            const float rstd = 1.0f / sqrtf(ss * (1.0f / HD) + p.eps);
            const uint32_t ga = *reinterpret_cast<const uint32_t*>(gain + 2 * c.lane);
            const uint32_t gb = *reinterpret_cast<const uint32_t*>(gain + HD / 2 + 2 * c.lane);
            x[0] = bf16r(bf16r(x[0] * rstd) * bf_lo(ga));
            x[1] = bf16r(bf16r(x[1] * rstd) * bf_hi(ga));
            x[2] = bf16r(bf16r(x[2] * rstd) * bf_lo(gb));
            x[3] = bf16r(bf16r(x[3] * rstd) * bf_hi(gb));
            const bf16* rp = reinterpret_cast<const bf16*>(p.rope) + (size_t)pos * HD;
            const uint32_t cw = *reinterpret_cast<const uint32_t*>(rp + 2 * c.lane);
            const uint32_t sw = *reinterpret_cast<const uint32_t*>(rp + HD / 2 + 2 * c.lane);
            float lo[2], hi[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {      // pair (i, i+64), i = 2*lane + j
                const float cs = j ? bf_hi(cw) : bf_lo(cw), sn = j ? bf_hi(sw) : bf_lo(sw);
                const float a = x[j], bb = x[j + 2];
                lo[j] = bf16r(bf16r(a * cs) + bf16r(-bb * sn));
                hi[j] = bf16r(bf16r(bb * cs) + bf16r(a * sn));
            }
            if (is_k) {
                const uint32_t wlo = pack_bf16x2(lo[0], lo[1]), whi = pack_bf16x2(hi[0], hi[1]);
                *reinterpret_cast<uint32_t*>(at->knew + 2 * c.lane) = wlo;
                *reinterpret_cast<uint32_t*>(at->knew + HD / 2 + 2 * c.lane) = whi;
                if (ok) {
                    *reinterpret_cast<uint32_t*>(kc + (size_t)pos * HD + 2 * c.lane) = wlo;
                    *reinterpret_cast<uint32_t*>(kc + (size_t)pos * HD + HD / 2 + 2 * c.lane) = whi;
                    __threadfence();
                }
            } else {
                const float qscale = 0.08838834764831845f * kLog2e;   // head_dim^-0.5 * log2(e)
                at->qs[c.warp][2 * c.lane] = lo[0] * qscale;
                at->qs[c.warp][2 * c.lane + 1] = lo[1] * qscale;
                at->qs[c.warp][HD / 2 + 2 * c.lane] = hi[0] * qscale;
                at->qs[c.warp][HD / 2 + 2 * c.lane + 1] = hi[1] * qscale;
            }
        } else if (c.warp == 3 && has_new) {
            const int e0 = DQ + DKV + g * HD;
            uint32_t ua = 0, ub = 0;
            ok = wait_word(c.w, qw + e0 / 2 + c.lane, tag, ua, ITTAI_PH_ATTN);
            ok = ok && wait_word(c.w, qw + e0 / 2 + 32 + c.lane, tag, ub, ITTAI_PH_ATTN);
            *reinterpret_cast<uint32_t*>(at->vnew + 2 * c.lane) = ua;
            *reinterpret_cast<uint32_t*>(at->vnew + HD / 2 + 2 * c.lane) = ub;
            if (ok) {
                *reinterpret_cast<uint32_t*>(vc + (size_t)pos * HD + 2 * c.lane) = ua;
                *reinterpret_cast<uint32_t*>(vc + (size_t)pos * HD + HD / 2 + 2 * c.lane) = ub;
                __threadfence();
            }
        }
        if (c.tid < 2) { c.hdr->m_s[c.tid] = -INFINITY; c.hdr->l_s[c.tid] = 0.f; }
        if (!all_ok(ok)) return false;
        if (first) { c.t_ready = clock64(); first = false; }

        const int half = c.lane >> 4, sub = c.lane & 15;
        float q0[8], q1[8], acc0[8], acc1[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            q0[e] = at->qs[0][sub * 8 + e];
            q1[e] = at->qs[1][sub * 8 + e];
            acc0[e] = 0.f; acc1[e] = 0.f;
        }

        for (int tile0 = start; tile0 < end; tile0 += kTile) {
            // -- scores: a half-warp reads one 256-byte key row; 8 rows in flight per lane
            uint4 kv[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int t = tile0 + r * 32 + c.warp * 2 + half;
                if (t < end) {
                    if (has_new && t == pos) kv[r] = *reinterpret_cast<const uint4*>(at->knew + sub * 8);
                    else kv[r] = ldcg128(kc + (size_t)t * HD + sub * 8);
                } else kv[r] = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int tl = r * 32 + c.warp * 2 + half;
                float s0 = dot8(kv[r], q0, 0.f), s1 = dot8(kv[r], q1, 0.f);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
                    s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                }
                if (sub == 0) {
                    const bool valid = tile0 + tl < end;
                    at->sc[0][tl] = valid ? s0 : -INFINITY;
                    at->sc[1][tl] = valid ? s1 : -INFINITY;
                }
            }
            __syncthreads();
            // -- running max / sum for each of the two heads (warp 0 -> head 0, warp 1 -> head 1)
            if (c.warp < 2) {
                float v[kTile / 32], mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < kTile / 32; ++j) { v[j] = at->sc[c.warp][c.lane + 32 * j]; mx = fmaxf(mx, v[j]); }
                mx = warp_max(mx);
                const float m_old = c.hdr->m_s[c.warp];
                const float m_new = fmaxf(m_old, mx);
                float ps = 0.f;
#pragma unroll
                for (int j = 0; j < kTile / 32; ++j) {
                    const float e = exp2f(v[j] - m_new);
                    at->sc[c.warp][c.lane + 32 * j] = e;
                    ps += e;
                }
                ps = warp_sum(ps);
                if (c.lane == 0) {
                    const float corr = exp2f(m_old - m_new);
                    c.hdr->corr_s[c.warp] = corr;
                    c.hdr->l_s[c.warp] = c.hdr->l_s[c.warp] * corr + ps;
                    c.hdr->m_s[c.warp] = m_new;
                }
            }
            __syncthreads();
            // -- O += P V
            const float c0 = c.hdr->corr_s[0], c1 = c.hdr->corr_s[1];
#pragma unroll
            for (int e = 0; e < 8; ++e) { acc0[e] *= c0; acc1[e] *= c1; }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int t = tile0 + r * 32 + c.warp * 2 + half;
                if (t < end) {
                    if (has_new && t == pos) kv[r] = *reinterpret_cast<const uint4*>(at->vnew + sub * 8);
                    else kv[r] = ldcg128(vc + (size_t)t * HD + sub * 8);
                } else kv[r] = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int tl = r * 32 + c.warp * 2 + half;
                const float p0 = at->sc[0][tl], p1 = at->sc[1][tl];
                const float vv[8] = {bf_lo(kv[r].x), bf_hi(kv[r].x), bf_lo(kv[r].y), bf_hi(kv[r].y),
                                     bf_lo(kv[r].z), bf_hi(kv[r].z), bf_lo(kv[r].w), bf_hi(kv[r].w)};
#pragma unroll
                for (int e = 0; e < 8; ++e) { acc0[e] = fmaf(p0, vv[e], acc0[e]); acc1[e] = fmaf(p1, vv[e], acc1[e]); }
            }
            __syncthreads();
        }
        // -- fold the 32 per-(warp, half) partial outputs and publish (m, l, o) of this split
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            acc0[e] += __shfl_xor_sync(0xffffffffu, acc0[e], 16);
            acc1[e] += __shfl_xor_sync(0xffffffffu, acc1[e], 16);
        }
        if (half == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) { at->ored[c.warp][0][sub * 8 + e] = acc0[e]; at->ored[c.warp][1][sub * 8 + e] = acc1[e]; }
        }
        __syncthreads();
        uint64_t* part = c.ws.part + (size_t)item * Q3_PART_WORDS;
        if (c.tid < 2 * HD) {
            const int h = c.tid / HD, d = c.tid % HD;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) o += at->ored[w][h][d];
            st_flagged(part + 4 + h * HD + d, __float_as_uint(o), tag);
            if (d == 0) {
                st_flagged(part + h, __float_as_uint(c.hdr->m_s[h]), tag);
                st_flagged(part + 2 + h, __float_as_uint(c.hdr->l_s[h]), tag);
            }
        }
        __syncthreads();
    }
    // -- merge: split s < nc of each (b, g) gathers, from every split of that head, the running max and sum and its
    //    own slice of the outputs.  All partials are published before any CTA waits here, so CTAs that own several
    //    items cannot wait on each other in a cycle.
    int nc = 1;
    while (nc * 2 <= n_splits && nc < 16) nc *= 2;
    const int dpc = HD / nc, W = 4 + 2 * dpc;
    for (int item = c.cta; item < n_items; item += c.ncta) {
        const int b = item / (NKV * n_splits), g = (item / n_splits) % NKV, s = item % n_splits;
        if (s >= nc) continue;
        const int d0 = s * dpc;
        const uint64_t* base = c.ws.part + (size_t)(b * NKV + g) * n_splits * Q3_PART_WORDS;
        bool ok = true;
        for (int idx = c.tid; idx < n_splits * W; idx += kThreads) {
            const int k = idx / W, j = idx % W;
            const int src = j < 4 ? j : 4 + ((j - 4) / dpc) * HD + d0 + (j - 4) % dpc;
            uint32_t u = 0;
            ok = ok && wait_word(c.w, base + (size_t)k * Q3_PART_WORDS + src, tag, u, 16 + ITTAI_PH_ATTN);
            c.hdr->comb[idx] = __uint_as_float(u);
        }
        if (!all_ok(ok)) return false;
        const bool valid = c.tid < 2 * dpc;
        const int tt = valid ? c.tid : 0, h = tt / dpc, dd = tt % dpc;
        float M = -INFINITY;
        for (int k = 0; k < n_splits; ++k) M = fmaxf(M, c.hdr->comb[k * W + h]);
        float Ls = 0.f, O = 0.f;
        for (int k = 0; k < n_splits; ++k) {
            const float wk = exp2f(c.hdr->comb[k * W + h] - M);
            Ls = fmaf(c.hdr->comb[k * W + 2 + h], wk, Ls);
            O = fmaf(c.hdr->comb[k * W + 4 + h * dpc + dd], wk, O);
        }
        const float out = O / Ls;
        const float nb = __shfl_down_sync(0xffffffffu, out, 1);
        if (valid && (dd & 1) == 0)
            st_flagged(c.ws.attn + (size_t)b * (DQ / 2) + ((2 * g + h) * HD + d0 + dd) / 2, pack_bf16x2(out, nb), tag);
        __syncthreads();
    }
    return true;
}

// ---- phases: O-proj + residual, down-proj + residual ---------------------------------------------------
// K is 2048 or 3072: rows are cut into 1024-column sub-rows spread over the warps, partial sums meet in shared
// memory and are added in a fixed order.  out = bf16(resid + bf16(W x)) (reference base.py:110-123).
// `res_src` == nullptr takes the residual from the embedding row (layer 0's o_proj).
template <int NB, int K>
__device__ bool phase_proj_residual(Cta& c, int what, const bf16* W, const uint64_t* x_src, uint32_t x_tag,
                                    const uint64_t* res_src, uint32_t res_tag, uint64_t* dst, uint32_t dst_tag) {
    constexpr int S = K / 1024;
    if (!wait_rows_to_smem<NB, K>(c, x_src, x_tag, what)) return false;
    c.t_ready = clock64();
    int p0, p1;
    split_range(D / 2, c.ncta, c.cta, p0, p1);
    const int r0 = 2 * p0, n_sub = 2 * (p1 - p0) * S;
    constexpr int kSlots = 60;               // sub-rows finished per pass: a multiple of 4 and of 6, so row pairs stay whole
    float* sub = c.hdr->sub;
    bool ok = true;
    for (int base = 0; base < n_sub; base += kSlots) {
        const int cnt = n_sub - base < kSlots ? n_sub - base : kSlots;
        for (int sr = c.warp; sr < cnt; sr += kWarps) {
            const int gsr = base + sr;
            const int row = r0 + gsr / S, seg = gsr % S;
            const bf16* wp[1] = {W + (size_t)row * K + seg * 1024};
            const float* xseg[1] = {c.xs + seg * 1024};
            float acc[1][NB];
            dot_subrows_smem<NB, 1>(wp, xseg, c.lane, acc);
            if (c.lane == 0) {
#pragma unroll
                for (int b = 0; b < NB; ++b) sub[sr * NB + b] = acc[0][b];
            }
        }
        __syncthreads();
        const int pairs_here = cnt / (2 * S);
        for (int i = c.tid; i < pairs_here * NB; i += kThreads) {
            const int pp = i / NB, b = i % NB;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int k = 0; k < S; ++k) { s0 += sub[((2 * pp) * S + k) * NB + b]; s1 += sub[((2 * pp + 1) * S + k) * NB + b]; }
            const int pair = p0 + base / (2 * S) + pp;
            uint32_t rw = 0;
            if (res_src == nullptr)
                rw = ldcg32(reinterpret_cast<const bf16*>(c.p.embed) + (size_t)c.hdr->tok_s[b] * D + 2 * pair);
            else
                ok = ok && wait_word(c.w, res_src + (size_t)b * (D / 2) + pair, res_tag, rw, 32 + what);
            st_flagged(dst + (size_t)b * (D / 2) + pair, pack_bf16x2(bf_lo(rw) + bf16r(s0), bf_hi(rw) + bf16r(s1)), dst_tag);
        }
        __syncthreads();
    }
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
    uint32_t u[NB];
    bool ok = true;
#pragma unroll
    for (int b = 0; b < NB; ++b) ok = ok && wait_word(c.w, c.ws.hmid + b * (D / 2) + c.tid, tag, u[b], ITTAI_PH_GU);
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
#pragma unroll
    for (int b = 0; b < NB; ++b) norm_pair_to_smem(c, u[b], reinterpret_cast<const bf16*>(p.ln2) + (size_t)l * D, c.xs + b * FF);
    __syncthreads();
    float xr[32];
    if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
    const bf16* W = reinterpret_cast<const bf16*>(p.wgu) + (size_t)l * DGU * D;
    int u0, u1;
    split_range(FF / 2, c.ncta, c.cta, u0, u1);      // unit = two activations = four weight rows = one flagged word
    for (int un = u0 + c.warp; un < u1; un += kWarps) {
        float a0[NB], a1[NB];
        if constexpr (NB == 1) {
            const bf16* wp[4] = {W + (size_t)(4 * un) * D, W + (size_t)(4 * un + 1) * D, W + (size_t)(4 * un + 2) * D,
                                 W + (size_t)(4 * un + 3) * D};
            float acc[4][NB];
            dot_rows_k1024<NB, 4>(c, wp, xr, acc);
            a0[0] = swiglu(acc[0][0], acc[1][0]);
            a1[0] = swiglu(acc[2][0], acc[3][0]);
        } else {
#pragma unroll
            for (int hsel = 0; hsel < 2; ++hsel) {
                const bf16* wp[2] = {W + (size_t)(4 * un + 2 * hsel) * D, W + (size_t)(4 * un + 2 * hsel + 1) * D};
                float acc[2][NB];
                dot_rows_k1024<NB, 2>(c, wp, xr, acc);
#pragma unroll
                for (int b = 0; b < NB; ++b) (hsel ? a1[b] : a0[b]) = swiglu(acc[0][b], acc[1][b]);
            }
        }
        if (c.lane == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) st_flagged(c.ws.act + (size_t)b * (FF / 2) + un, pack_bf16x2(a0[b], a1[b]), tag);
        }
    }
    return true;
}

// ---- phase: final RMSNorm + tied lm_head GEMV + argmax ------------------------------------------------
// logits = bf16(W_embed x); argmax over the bf16 values, lowest index wins ties (torch semantics).  Every CTA
// publishes its best (value, index); every CTA then gathers all of them, so each knows the next token at once.
template <int NB>
__device__ bool phase_head(Cta& c) {
    const IttaiQwen3Decode& p = c.p;
    uint32_t u[NB];
    bool ok = true;
#pragma unroll
    for (int b = 0; b < NB; ++b)
        ok = ok && wait_word(c.w, c.ws.h + b * (D / 2) + c.tid, tag_of(c, c.step, p.n_layers), u[b], ITTAI_PH_HEAD);
    if (!all_ok(ok)) return false;
    c.t_ready = clock64();
#pragma unroll
    for (int b = 0; b < NB; ++b) norm_pair_to_smem(c, u[b], reinterpret_cast<const bf16*>(p.fin_w), c.xs + b * FF);
    __syncthreads();
    float xr[32];
    if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
    const bf16* W = reinterpret_cast<const bf16*>(p.embed);
    bf16* logits = reinterpret_cast<bf16*>(p.logits);
    int r0, r1;
    split_range(p.vocab, c.ncta, c.cta, r0, r1);
    constexpr int R = (NB == 1) ? 4 : 2;
    float bv[NB];
    int bi[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) { bv[b] = -INFINITY; bi[b] = 0x7fffffff; }
    for (int row = r0 + c.warp * R; row < r1; row += kWarps * R) {
        const bf16* wp[R];
#pragma unroll
        for (int r = 0; r < R; ++r) wp[r] = W + (size_t)(row + r < r1 ? row + r : r1 - 1) * D;
        float acc[R][NB];
        dot_rows_k1024<NB, R>(c, wp, xr, acc);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row + r < r1) {
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const float v = bf16r(acc[r][b]);
                    if (v > bv[b]) { bv[b] = v; bi[b] = row + r; }   // rows ascend within a warp: first max kept
                    if (p.write_logits && c.lane == 0) logits[(size_t)b * p.vocab + row + r] = __float2bfloat16_rn(v);
                }
            }
        }
    }
    const uint32_t tag = (uint32_t)c.step + 1u;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        if (c.lane == 0) { c.hdr->bestv[c.warp] = bv[b]; c.hdr->besti[c.warp] = bi[b]; }
        __syncthreads();
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
        __syncthreads();
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
                c.hdr->tok_s[b] = ix;
                if (c.cta == 0) {
                    p.next_id[b] = ix;
                    p.out_ids[(size_t)c.step * p.batch + b] = ix;
                }
            }
        }
        __syncthreads();
    }
    return true;
}

// ---- L2 prefetch one layer ahead ------------------------------------------------------------------------
// While phase (l, ph) runs, ask L2 for this CTA's slice of the same phase of the next layer (layer 0 of the next
// token after the last layer).  126 MB of L2 hold a layer's 31 MB of weights plus its cache slice several times over.
__device__ void prefetch_ahead(const Cta& c, int ph, int l) {
    const IttaiQwen3Decode& p = c.p;
    const int lt = l + 1 < p.n_layers ? l + 1 : 0;
    switch (ph) {
        case ITTAI_PH_QKV: prefetch_slice(c, reinterpret_cast<const bf16*>(p.wqkv) + (size_t)lt * DQKV * D, D * 2, DQKV, 2); break;
        case ITTAI_PH_ATTN: {
            const int n_splits = attn_splits(c.ncta, p.batch);
            const int item = c.cta;
            if (item < p.batch * NKV * n_splits) {
                const int b = item / (NKV * n_splits), g = (item / n_splits) % NKV, s = item % n_splits;
                int start, end, chunk;
                attn_range(c.hdr->pos_s[b] + 1, n_splits, s, start, end, chunk);
                if (end > start) {
                    const size_t off = (((((size_t)lt * p.batch + b) * NKV + g) * (size_t)p.kv_cap) + start) * HD;
                    prefetch_bytes(c, reinterpret_cast<const bf16*>(p.kcache) + off, (size_t)(end - start) * HD * 2);
                    prefetch_bytes(c, reinterpret_cast<const bf16*>(p.vcache) + off, (size_t)(end - start) * HD * 2);
                }
            }
            break;
        }
        case ITTAI_PH_OPROJ: prefetch_slice(c, reinterpret_cast<const bf16*>(p.wo) + (size_t)lt * D * DQ, DQ * 2, D, 2); break;
        case ITTAI_PH_GU: prefetch_slice(c, reinterpret_cast<const bf16*>(p.wgu) + (size_t)lt * DGU * D, D * 2, DGU, 4); break;
        case ITTAI_PH_DOWN: prefetch_slice(c, reinterpret_cast<const bf16*>(p.wd) + (size_t)lt * D * FF, FF * 2, D, 2); break;
        default: break;
    }
}

// ---- per-step set-up: positions and input ids ----------------------------------------------------------
// Returns false (uniformly over the grid) when an id or a position is out of range.
__device__ bool step_setup(Cta& c, int step, const int* pos0, bool ids_from_head) {
    const IttaiQwen3Decode& p = c.p;
    if (c.tid < p.batch) {
        const int b = c.tid;
        c.hdr->pos_s[b] = pos0[b] + step;
        if (step < p.n_forced) c.hdr->tok_s[b] = p.forced[(size_t)step * p.batch + b];
        else if (!ids_from_head) c.hdr->tok_s[b] = p.next_id[b];
        // else: the head of the previous step left the id in tok_s
    }
    __syncthreads();
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
    const IttaiQwen3Decode& p = c.p;
    const uint32_t tag = tag_of(c, c.step, l);
    switch (phase) {
        case ITTAI_PH_QKV: return phase_qkv<NB>(c, l);
        case ITTAI_PH_ATTN: return phase_attn(c, l);
        case ITTAI_PH_OPROJ:
            return phase_proj_residual<NB, DQ>(c, ITTAI_PH_OPROJ, reinterpret_cast<const bf16*>(p.wo) + (size_t)l * D * DQ,
                                               c.ws.attn, tag, l == 0 ? nullptr : c.ws.h, tag, c.ws.hmid, tag);
        case ITTAI_PH_GU: return phase_gu<NB>(c, l);
        case ITTAI_PH_DOWN:
            return phase_proj_residual<NB, FF>(c, ITTAI_PH_DOWN, reinterpret_cast<const bf16*>(p.wd) + (size_t)l * D * FF,
                                               c.ws.act, tag, c.ws.hmid, tag, c.ws.h, tag_of(c, c.step, l + 1));
        default: return phase_head<NB>(c);
    }
}

// The per-CTA context is brace-initialised inside each kernel.  nvcc 12.9 mis-infers the shared state space for the
// global pointers of a struct returned by value from a helper that also receives the shared-memory base, so there is
// deliberately no make_cta() function.
#define ITTAI_MAKE_CTA(p, wsp, smem)                                                                              \
    Cta c{p, wsp, reinterpret_cast<SmemHdr*>(smem), reinterpret_cast<float*>(smem + kHdrBytes),                   \
          reinterpret_cast<SmemAttn*>(smem + kHdrBytes), (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x,       \
          (int)(threadIdx.x & 31), (int)(threadIdx.x >> 5),                                                       \
          Waiter{wsp.sync, p.status, p.spin_limit > 0 ? (uint32_t)p.spin_limit : kSpinLimit}, 0, 0}

template <int NB>
__global__ void __launch_bounds__(kThreads, 1) q3_decode_kernel(const __grid_constant__ IttaiQwen3Decode p,
                                                                const __grid_constant__ Q3Workspace wsp) {
    extern __shared__ __align__(256) unsigned char smem[];
    ITTAI_MAKE_CTA(p, wsp, smem);
    if ((p.flags & ITTAI_F_TEST_DROP_CTA) != 0 && c.cta == 0) return;
    __shared__ int pos0[ITTAI_MAX_BATCH];
    if (c.tid < p.batch) pos0[c.tid] = p.pos[c.tid];
    __syncthreads();
    const bool prefetch = (p.flags & ITTAI_F_L2_PREFETCH) != 0;
    const bool prof = p.phase_clk != nullptr && c.cta == 0 && c.tid == 0;
    bool prev_head = false;

    for (int step = 0; step < p.n_steps; ++step) {
        c.step = step;
        if (!step_setup(c, step, pos0, prev_head)) return;
        const bool run_head = step >= p.n_forced - 1;
        if (!run_head && c.cta == 0 && c.tid < p.batch) p.out_ids[(size_t)step * p.batch + c.tid] = -1;
        if (step > 0 && !prev_head) {
            // No head ran, so nothing yet orders this token after the previous one: wait for its last layer's output
            // before any buffer of the chain is written again.
            bool ok = true;
            for (int b = 0; b < p.batch; ++b) {
                uint32_t u;
                ok = ok && wait_word(c.w, c.ws.h + b * (D / 2) + c.tid, tag_of(c, step - 1, p.n_layers), u, 64);
            }
            if (!all_ok(ok)) return;
        }
        for (int l = 0; l < p.n_layers; ++l) {
#pragma unroll 1
            for (int phase = ITTAI_PH_QKV; phase <= ITTAI_PH_DOWN; ++phase) {
                if (prefetch) prefetch_ahead(c, phase, l);
                if (!run_phase<NB>(c, phase, l)) return;
                if (prof) {
                    const size_t slot = ((size_t)step * (5 * p.n_layers + 1) + l * 5 + phase) * 2;
                    p.phase_clk[slot] = (uint64_t)c.t_ready;
                    p.phase_clk[slot + 1] = (uint64_t)clock64();
                }
            }
        }
        if (run_head) {
            if (!phase_head<NB>(c)) return;
            if (prof) {
                const size_t slot = ((size_t)step * (5 * p.n_layers + 1) + 5 * p.n_layers) * 2;
                p.phase_clk[slot] = (uint64_t)c.t_ready;
                p.phase_clk[slot + 1] = (uint64_t)clock64();
            }
        }
        prev_head = run_head;
        if (p.step_ns != nullptr && c.cta == 0 && c.tid == 0) p.step_ns[step] = globaltimer_ns();
    }
    if (c.cta == 0 && c.tid < p.batch) p.pos[c.tid] = pos0[c.tid] + p.n_steps;
}

// One phase on its own at step 0 (tags of step 0): unit tests and per-phase profiles.  Inputs must carry the tag of
// (step 0, layer); launched cooperatively because the attention merge and the head wait on other CTAs.
template <int NB>
__global__ void __launch_bounds__(kThreads, 1) q3_phase_kernel(const __grid_constant__ IttaiQwen3Decode p,
                                                               const __grid_constant__ Q3Workspace wsp, int phase, int l) {
    extern __shared__ __align__(256) unsigned char smem[];
    ITTAI_MAKE_CTA(p, wsp, smem);
    __shared__ int pos0[ITTAI_MAX_BATCH];
    if (c.tid < p.batch) pos0[c.tid] = p.pos[c.tid];
    __syncthreads();
    if (!step_setup(c, 0, pos0, false)) return;
    run_phase<NB>(c, phase, l);
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
    if ((long long)p->n_steps * (p->n_layers + 1) >= (1ll << 31)) { set_error("n_steps * (n_layers + 1) must stay below 2^31"); return ITTAI_E_ARG; }
    const void* req[] = {p->wqkv, p->wo, p->wgu, p->wd, p->ln1, p->ln2, p->qn, p->kn, p->fin_w, p->embed, p->rope,
                         p->kcache, p->vcache, p->pos, p->next_id, p->out_ids, p->workspace, p->status};
    for (const void* q : req) if (!q) { set_error("null device pointer in IttaiQwen3Decode"); return ITTAI_E_ARG; }
    const void* al16[] = {p->wqkv, p->wo, p->wgu, p->wd, p->embed, p->kcache, p->vcache, p->ln1, p->ln2, p->fin_w, p->rope};
    for (const void* q : al16) if (((uintptr_t)q & 15u) != 0) { set_error("weight / cache pointers must be 16-byte aligned"); return ITTAI_E_ARG; }
    if (((uintptr_t)p->workspace & 255u) != 0) { set_error("workspace must be 256-byte aligned"); return ITTAI_E_ARG; }
    return ITTAI_OK;
}

struct DeviceInfo { int dev = -1; int n_sms = 0; bool attr_set[4] = {false, false, false, false}; };
static thread_local DeviceInfo g_info;

static int device_info(int* n_sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (g_info.dev != dev) {
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        g_info = DeviceInfo();
        g_info.dev = dev;
        g_info.n_sms = sms;
    }
    *n_sms = g_info.n_sms;
    return ITTAI_OK;
}

template <int NB>
static int launch_nb(const IttaiQwen3Decode* p, int phase, int layer, cudaStream_t st) {
    int n_sms = 0;
    int rc = device_info(&n_sms);
    if (rc != ITTAI_OK) return rc;
    const size_t smem = q3_smem_bytes(NB) + 256;   // slack: the dynamic region starts on a 256-byte boundary after the static words
    const void* fn_decode = (const void*)q3_decode_kernel<NB>;
    const void* fn_phase = (const void*)q3_phase_kernel<NB>;
    constexpr int slot = NB == 1 ? 0 : NB == 2 ? 1 : NB == 4 ? 2 : 3;
    if (!g_info.attr_set[slot]) {
        cudaError_t e = cudaFuncSetAttribute(fn_decode, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(decode)");
        e = cudaFuncSetAttribute(fn_phase, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(phase)");
        int occ = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, q3_decode_kernel<NB>, kThreads, smem);
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
    const int grid = n_sms < Q3_MAX_CTAS ? n_sms : Q3_MAX_CTAS;
    if (phase < 0) {
        void* args[] = {(void*)p, (void*)&ws};
        e = cudaLaunchCooperativeKernel(fn_decode, dim3(grid), dim3(kThreads), args, smem, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchCooperativeKernel(q3_decode_kernel)");
    } else {
        void* args[] = {(void*)p, (void*)&ws, (void*)&phase, (void*)&layer};
        e = cudaLaunchCooperativeKernel(fn_phase, dim3(grid), dim3(kThreads), args, smem, st);
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
    if (!bytes || batch < 1 || batch > ITTAI_MAX_BATCH) { ittai::set_error("bad batch or null output"); return ITTAI_E_ARG; }
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
