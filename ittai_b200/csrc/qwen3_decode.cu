// Qwen3-0.6B decode: one persistent cooperative kernel per launch runs n_steps tokens, every layer phase
// separated by a bounded grid barrier, the chosen token id fed back on the device.
//
// Batch-1 decode is HBM-bound (about 1.4 flop per weight byte), so there are no tensor-core tiles here:
// each warp streams whole 1024-column weight sub-rows with 128-bit coalesced loads and reduces with
// shuffles.  Rounding points follow the eager modules: every Linear output, norm output, rotary product
// and sum, SiLU, gate*up product and residual sum is rounded to bf16 exactly once.
//
// The math per phase mirrors the fused epilogues of the reference's megakernel
// (src/ittai/qwen3/base.py:80-129 for qkv / residual / gate-up, :147-162 for the embedding row), re-cut
// for one token: the row-norm scale is applied before the GEMV instead of after the GEMM, and keys and
// values go straight into the cache instead of a staging matrix.  KV cache, split-K decode attention,
// lm_head and argmax have no counterpart in the reference.
#include "common.cuh"
#include "qwen3_ws.h"

namespace ittai {

constexpr int D = ITTAI_Q3_D, NH = ITTAI_Q3_NH, NKV = ITTAI_Q3_NKV, HD = ITTAI_Q3_HD, FF = ITTAI_Q3_FF;
constexpr int DQ = ITTAI_Q3_DQ, DKV = ITTAI_Q3_DKV, DQKV = ITTAI_Q3_DQKV, DGU = ITTAI_Q3_DGU;
constexpr int kTile = 256;                       // cache positions scored per attention tile
constexpr float kLog2e = 1.4426950408889634f;

// ---- shared-memory plan (dynamic) ----------------------------------------------------------------------
struct SmemHdr {
    float red[32];
    float m_s[2], l_s[2], corr_s[2];
    int last_s, ok_s;
    int pos_s[ITTAI_MAX_BATCH];
    int tok_s[ITTAI_MAX_BATCH];
    float bestv[kWarps];
    int besti[kWarps];
    float sub[64 * ITTAI_MAX_BATCH];             // per-sub-row partial dot products
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
};

// ---- RMSNorm of NB rows into shared memory -----------------------------------------------------------
// xs[b][i] = bf16(bf16(x*rstd) * gain): the value the following Linear sees in the eager model.
template <int NB>
__device__ __forceinline__ void norm_rows_to_smem(Cta& c, const bf16* const* src, const bf16* gain) {
    static_assert(kThreads * 2 == D, "one bf16 pair per thread");
    const uint32_t gw = *reinterpret_cast<const uint32_t*>(gain + 2 * c.tid);
    const float g0 = bf_lo(gw), g1 = bf_hi(gw);
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const uint32_t u = ldcg32(src[b] + 2 * c.tid);
        const float x0 = bf_lo(u), x1 = bf_hi(u);
        const float tot = block_sum(x0 * x0 + x1 * x1, c.hdr->red);
        const float rstd = 1.0f / sqrtf(tot * (1.0f / D) + c.p.eps);
        c.xs[b * FF + 2 * c.tid] = bf16r(bf16r(x0 * rstd) * g0);
        c.xs[b * FF + 2 * c.tid + 1] = bf16r(bf16r(x1 * rstd) * g1);
    }
    __syncthreads();
}

// Copies NB bf16 rows of length K (multiple of 1024) into xs as fp32.
template <int NB, int K>
__device__ __forceinline__ void copy_rows_to_smem(Cta& c, const bf16* src, int row_stride) {
#pragma unroll
    for (int b = 0; b < NB; ++b)
        for (int i = c.tid; i < K / 2; i += kThreads) {
            const uint32_t u = ldcg32(src + (size_t)b * row_stride + 2 * i);
            c.xs[b * FF + 2 * i] = bf_lo(u);
            c.xs[b * FF + 2 * i + 1] = bf_hi(u);
        }
    __syncthreads();
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

// xs points at the 1024-float segment this sub-row multiplies, for batch row 0; batch rows are FF floats apart.
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

// ---- L2 prefetch of the slice of weights this CTA reads in a coming phase ------------------------------
__device__ __forceinline__ void prefetch_slice(const Cta& c, const bf16* base, size_t row_bytes, int n_rows, int unit) {
    // rows are split over CTAs in multiples of `unit` rows exactly as the phases do
    int lo, hi;
    split_range(n_rows / unit, c.ncta, c.cta, lo, hi);
    const char* p = reinterpret_cast<const char*>(base) + (size_t)lo * unit * row_bytes;
    const size_t bytes = (size_t)(hi - lo) * unit * row_bytes;
    constexpr uint32_t kPiece = 8192;
    for (size_t off = (size_t)c.tid * kPiece; off < bytes; off += (size_t)kThreads * kPiece) {
        const size_t n = bytes - off < kPiece ? bytes - off : kPiece;
        l2_prefetch(p + off, (uint32_t)n);
    }
}

// ---- phase: embed gather (layer 0) + RMSNorm + QKV GEMV ------------------------------------------------
template <int NB>
__device__ void phase_qkv(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const bf16* src[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b)
        src[b] = (l == 0) ? reinterpret_cast<const bf16*>(p.embed) + (size_t)c.hdr->tok_s[b] * D : c.ws.h + b * D;
    norm_rows_to_smem<NB>(c, src, reinterpret_cast<const bf16*>(p.ln1) + (size_t)l * D);
    float xr[32];
    if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
    const bf16* W = reinterpret_cast<const bf16*>(p.wqkv) + (size_t)l * DQKV * D;
    int r0, r1;
    split_range(DQKV, c.ncta, c.cta, r0, r1);
    for (int row = r0 + c.warp * 2; row < r1; row += kWarps * 2) {
        const int row1 = row + 1 < r1 ? row + 1 : row;
        const bf16* wp[2] = {W + (size_t)row * D, W + (size_t)row1 * D};
        float acc[2][NB];
        dot_rows_k1024<NB, 2>(c, wp, xr, acc);
        if (c.lane == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                c.ws.qkv[b * DQKV + row] = __float2bfloat16_rn(acc[0][b]);
                if (row1 != row) c.ws.qkv[b * DQKV + row1] = __float2bfloat16_rn(acc[1][b]);
            }
        }
    }
}

// ---- phase: QK-RMSNorm + RoPE + KV append + split-K GQA attention + combine ---------------------------
// Work item = (sequence b, kv head g, split s); CTA i takes item i.  Scores live in the log2 domain with the
// softmax scale folded into q, as the reference does (src/ittai/qwen3/config.py:6-7).
__device__ __forceinline__ int attn_splits(int ncta, int batch) {
    int s = ncta / (batch * NKV);
    return s < 1 ? 1 : (s > Q3_MAX_SPLITS ? Q3_MAX_SPLITS : s);
}

__device__ void phase_attn(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const int B = p.batch;
    const int n_splits = attn_splits(c.ncta, B);
    const int n_items = B * NKV * n_splits;
    // With fewer CTAs than (b, g) pairs a CTA walks several items.
    for (int item = c.cta; item < n_items; item += c.ncta) {
        const int b = item / (NKV * n_splits), g = (item / n_splits) % NKV, s = item % n_splits;
        const int pos = c.hdr->pos_s[b], n_ctx = pos + 1;
        const int chunk = (((n_ctx + n_splits - 1) / n_splits) + 31) & ~31;
        const int start = s * chunk;
        const int end = start + chunk < n_ctx ? start + chunk : n_ctx;
        const bool has_new = pos >= start && pos < start + chunk;
        const bf16* qkv = c.ws.qkv + b * DQKV;
        const size_t head_off = ((((size_t)l * B + b) * NKV + g) * (size_t)p.kv_cap) * HD;
        bf16* kc = reinterpret_cast<bf16*>(p.kcache) + head_off;
        bf16* vc = reinterpret_cast<bf16*>(p.vcache) + head_off;
        SmemAttn* at = c.at;

        // -- norm + rotate q (warps 0,1) and the new key (warp 2); copy the new value (warp 3)
        if (c.warp < 3 && (c.warp < 2 || has_new)) {
            const bool is_k = c.warp == 2;
            const bf16* x_src = is_k ? qkv + DQ + g * HD : qkv + (2 * g + c.warp) * HD;
            const bf16* gain = reinterpret_cast<const bf16*>(is_k ? p.kn : p.qn) + (size_t)l * HD;
            float x[4], ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) { x[j] = ldcg_bf16(x_src + c.lane + 32 * j); ss += x[j] * x[j]; }
            ss = warp_sum(ss);
            const float rstd = 1.0f / sqrtf(ss * (1.0f / HD) + p.eps);
#pragma unroll
            for (int j = 0; j < 4; ++j) x[j] = bf16r(bf16r(x[j] * rstd) * bf2f(gain[c.lane + 32 * j]));
            const bf16* rp = reinterpret_cast<const bf16*>(p.rope) + (size_t)pos * HD;
#pragma unroll
            for (int j = 0; j < 2; ++j) {      // pair (i, i+64), i = lane + 32 j
                const int i = c.lane + 32 * j;
                const float cs = bf2f(rp[i]), sn = bf2f(rp[HD / 2 + i]);
                const float a = x[j], bb = x[j + 2];
                const float lo = bf16r(bf16r(a * cs) + bf16r(-bb * sn));
                const float hi = bf16r(bf16r(bb * cs) + bf16r(a * sn));
                if (is_k) {
                    at->knew[i] = __float2bfloat16_rn(lo);
                    at->knew[i + HD / 2] = __float2bfloat16_rn(hi);
                    kc[(size_t)pos * HD + i] = __float2bfloat16_rn(lo);
                    kc[(size_t)pos * HD + i + HD / 2] = __float2bfloat16_rn(hi);
                } else {
                    const float qscale = 0.08838834764831845f * kLog2e;   // head_dim^-0.5 * log2(e)
                    at->qs[c.warp][i] = lo * qscale;
                    at->qs[c.warp][i + HD / 2] = hi * qscale;
                }
            }
        } else if (c.warp == 3 && has_new) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = c.lane + 32 * j;
                const unsigned short raw = (unsigned short)(__float_as_uint(ldcg_bf16(qkv + DQ + DKV + g * HD + i)) >> 16);
                const bf16 v = __ushort_as_bfloat16(raw);
                at->vnew[i] = v;
                vc[(size_t)pos * HD + i] = v;
            }
        }
        if (c.tid < 2) { c.hdr->m_s[c.tid] = -INFINITY; c.hdr->l_s[c.tid] = 0.f; }
        __syncthreads();

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
        // -- fold the 32 per-(warp, half) partial outputs
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
        float* part = c.ws.part + (size_t)item * Q3_PART_FLOATS;
        if (c.tid < 2 * HD) {
            const int h = c.tid / HD, d = c.tid % HD;
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) o += at->ored[w][h][d];
            part[4 + h * HD + d] = o;
            if (d == 0) { part[h] = c.hdr->m_s[h]; part[2 + h] = c.hdr->l_s[h]; }
        }
        __syncthreads();
        // -- the last split of (b, g) to arrive merges all of them
        if (c.tid == 0) {
            __threadfence();
            const uint32_t old = atomicAdd(&c.ws.sync[Q3_SYNC_HEADCNT + b * NKV + g], 1u);
            c.hdr->last_s = (old % (uint32_t)n_splits) == (uint32_t)(n_splits - 1);
        }
        __syncthreads();
        if (c.hdr->last_s) {
            __threadfence();
            if (c.tid < 2 * HD) {
                const int h = c.tid / HD, d = c.tid % HD;
                const float* base = c.ws.part + (size_t)(b * NKV + g) * n_splits * Q3_PART_FLOATS;
                float M = -INFINITY;
                for (int k = 0; k < n_splits; ++k) M = fmaxf(M, ldcgf(base + (size_t)k * Q3_PART_FLOATS + h));
                float Ls = 0.f, O = 0.f;
                for (int k = 0; k < n_splits; ++k) {
                    const float* pk = base + (size_t)k * Q3_PART_FLOATS;
                    const float w = exp2f(ldcgf(pk + h) - M);
                    Ls = fmaf(ldcgf(pk + 2 + h), w, Ls);
                    O = fmaf(ldcgf(pk + 4 + h * HD + d), w, O);
                }
                c.ws.attn[b * DQ + (2 * g + h) * HD + d] = __float2bfloat16_rn(O / Ls);
            }
        }
        __syncthreads();
    }
}

// ---- phases: O-proj + residual, down-proj + residual ---------------------------------------------------
// K is 2048 or 3072: rows are cut into 1024-column sub-rows spread over the warps, partial sums meet in shared
// memory and are added in a fixed order.  h <- bf16(resid + bf16(W x)), in place (reference base.py:110-123).
template <int NB, int K>
__device__ void phase_proj_residual(Cta& c, int l, const bf16* W, const bf16* x_src, bool resid_from_embed) {
    constexpr int S = K / 1024;
    copy_rows_to_smem<NB, K>(c, x_src, K);
    int r0, r1;
    split_range(D, c.ncta, c.cta, r0, r1);
    const int n_sub = (r1 - r0) * S;
    constexpr int kSlots = 60;               // sub-rows finished per pass: a multiple of 2 and of 3, so rows stay whole
    float* sub = c.hdr->sub;
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
        const int rows_here = cnt / S;
        for (int i = c.tid; i < rows_here * NB; i += kThreads) {
            const int rr = i / NB, b = i % NB;
            float sum = 0.f;
#pragma unroll
            for (int k = 0; k < S; ++k) sum += sub[(rr * S + k) * NB + b];
            const int row = r0 + base / S + rr;
            const bf16* rs = resid_from_embed
                                 ? reinterpret_cast<const bf16*>(c.p.embed) + (size_t)c.hdr->tok_s[b] * D
                                 : c.ws.h + b * D;
            const float res = ldcg_bf16(rs + row);
            c.ws.h[b * D + row] = __float2bfloat16_rn(res + bf16r(sum));
        }
        __syncthreads();
    }
}

// ---- phase: RMSNorm + gate/up GEMV + SwiGLU -----------------------------------------------------------
// act = bf16(bf16(silu(bf16 gate)) * bf16 up); gate and up rows are adjacent (reference base.py:124-129).
template <int NB>
__device__ void phase_gu(Cta& c, int l) {
    const IttaiQwen3Decode& p = c.p;
    const bf16* src[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) src[b] = c.ws.h + b * D;
    norm_rows_to_smem<NB>(c, src, reinterpret_cast<const bf16*>(p.ln2) + (size_t)l * D);
    float xr[32];
    if constexpr (NB == 1) load_xreg(c.xs, c.lane, xr);
    const bf16* W = reinterpret_cast<const bf16*>(p.wgu) + (size_t)l * DGU * D;
    int p0, p1;
    split_range(FF, c.ncta, c.cta, p0, p1);
    for (int pr = p0 + c.warp; pr < p1; pr += kWarps) {
        const bf16* wp[2] = {W + (size_t)(2 * pr) * D, W + (size_t)(2 * pr + 1) * D};
        float acc[2][NB];
        dot_rows_k1024<NB, 2>(c, wp, xr, acc);
        if (c.lane == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const float gte = bf16r(acc[0][b]), up = bf16r(acc[1][b]);
                const float sl = bf16r(gte / (1.0f + expf(-gte)));
                c.ws.act[b * FF + pr] = __float2bfloat16_rn(sl * up);
            }
        }
    }
}

// ---- phase: final RMSNorm + tied lm_head GEMV + argmax ------------------------------------------------
// logits = bf16(W_embed x); argmax over the bf16 values, lowest index wins ties (torch semantics).
template <int NB>
__device__ void phase_head(Cta& c, int step) {
    const IttaiQwen3Decode& p = c.p;
    const bf16* src[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) src[b] = c.ws.h + b * D;
    norm_rows_to_smem<NB>(c, src, reinterpret_cast<const bf16*>(p.fin_w));
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
    // CTA-level argmax, then the last CTA to arrive folds the per-CTA candidates
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
            c.ws.cand_val[c.cta * ITTAI_MAX_BATCH + b] = v;
            c.ws.cand_idx[c.cta * ITTAI_MAX_BATCH + b] = ix;
        }
        __syncthreads();
    }
    if (c.tid == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(&c.ws.sync[Q3_SYNC_HEADARRIVE], 1u);
        c.hdr->last_s = (old % (uint32_t)c.ncta) == (uint32_t)(c.ncta - 1);
    }
    __syncthreads();
    if (c.hdr->last_s && c.warp < NB) {
        __threadfence();
        const int b = c.warp;
        float v = -INFINITY;
        int ix = 0x7fffffff;
        for (int k = c.lane; k < c.ncta; k += 32) {
            const float vk = ldcgf(c.ws.cand_val + k * ITTAI_MAX_BATCH + b);
            const int ik = (int)ldcg32(c.ws.cand_idx + k * ITTAI_MAX_BATCH + b);
            if (vk > v || (vk == v && ik < ix)) { v = vk; ix = ik; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float vo = __shfl_xor_sync(0xffffffffu, v, o);
            const int io = __shfl_xor_sync(0xffffffffu, ix, o);
            if (vo > v || (vo == v && io < ix)) { v = vo; ix = io; }
        }
        if (c.lane == 0) {
            p.next_id[b] = ix;
            p.out_ids[(size_t)step * p.batch + b] = ix;
        }
    }
    __syncthreads();
}

// ---- per-step set-up: positions and input ids ----------------------------------------------------------
// Returns false (uniformly over the grid) when an id or a position is out of range.
__device__ bool step_setup(Cta& c, int step, const int* pos0) {
    const IttaiQwen3Decode& p = c.p;
    if (c.tid < p.batch) {
        const int b = c.tid;
        c.hdr->pos_s[b] = pos0[b] + step;
        c.hdr->tok_s[b] = (step < p.n_forced) ? p.forced[(size_t)step * p.batch + b] : (int)ldcg32(p.next_id + b);
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
__device__ __forceinline__ void run_phase(Cta& c, int phase, int l, int step) {
    const IttaiQwen3Decode& p = c.p;
    switch (phase) {
        case ITTAI_PH_QKV: phase_qkv<NB>(c, l); break;
        case ITTAI_PH_ATTN: phase_attn(c, l); break;
        case ITTAI_PH_OPROJ:
            phase_proj_residual<NB, DQ>(c, l, reinterpret_cast<const bf16*>(p.wo) + (size_t)l * D * DQ, c.ws.attn, l == 0);
            break;
        case ITTAI_PH_GU: phase_gu<NB>(c, l); break;
        case ITTAI_PH_DOWN:
            phase_proj_residual<NB, FF>(c, l, reinterpret_cast<const bf16*>(p.wd) + (size_t)l * D * FF, c.ws.act, false);
            break;
        case ITTAI_PH_HEAD: phase_head<NB>(c, step); break;
    }
}

// Weights of the phase after (phase, l), prefetched into L2 while (phase, l) computes and waits.
__device__ void prefetch_next(const Cta& c, int phase, int l, bool head_follows) {
    const IttaiQwen3Decode& p = c.p;
    const bf16* wqkv = reinterpret_cast<const bf16*>(p.wqkv);
    const bf16* wo = reinterpret_cast<const bf16*>(p.wo);
    const bf16* wgu = reinterpret_cast<const bf16*>(p.wgu);
    const bf16* wd = reinterpret_cast<const bf16*>(p.wd);
    switch (phase) {
        case ITTAI_PH_QKV: break;   // attention follows: its cache slice depends on the split, fetched by the phase itself
        case ITTAI_PH_ATTN: prefetch_slice(c, wo + (size_t)l * D * DQ, DQ * 2, D, 1); break;
        case ITTAI_PH_OPROJ: prefetch_slice(c, wgu + (size_t)l * DGU * D, D * 2, DGU, 2); break;
        case ITTAI_PH_GU: prefetch_slice(c, wd + (size_t)l * D * FF, FF * 2, D, 1); break;
        case ITTAI_PH_DOWN:
            if (l + 1 < p.n_layers) prefetch_slice(c, wqkv + (size_t)(l + 1) * DQKV * D, D * 2, DQKV, 1);
            else if (!head_follows) prefetch_slice(c, wqkv, D * 2, DQKV, 1);
            break;
        default: prefetch_slice(c, wqkv, D * 2, DQKV, 1); break;
    }
}

// The per-CTA context is brace-initialised inside each kernel.  nvcc 12.9 mis-infers the shared state space for the
// global pointers of a struct returned by value from a helper that also receives the shared-memory base, so there is
// deliberately no make_cta() function.
#define ITTAI_MAKE_CTA(p, wsp, smem)                                                                              \
    Cta c{p, wsp, reinterpret_cast<SmemHdr*>(smem), reinterpret_cast<float*>(smem + kHdrBytes),                   \
          reinterpret_cast<SmemAttn*>(smem + kHdrBytes), (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x,       \
          (int)(threadIdx.x & 31), (int)(threadIdx.x >> 5)}

template <int NB>
__global__ void __launch_bounds__(kThreads, 1) q3_decode_kernel(const __grid_constant__ IttaiQwen3Decode p,
                                                                const __grid_constant__ Q3Workspace wsp) {
    extern __shared__ __align__(256) unsigned char smem[];
    ITTAI_MAKE_CTA(p, wsp, smem);
    GridSync gs{c.ws.sync, p.status, 0u, (uint32_t)gridDim.x, p.spin_limit > 0 ? (uint32_t)p.spin_limit : kSpinLimit};
    if ((p.flags & ITTAI_F_TEST_DROP_ARRIVAL) != 0 && c.cta == 0) return;
    __shared__ int pos0[ITTAI_MAX_BATCH];
    if (c.tid < p.batch) pos0[c.tid] = p.pos[c.tid];
    __syncthreads();
    const bool prefetch = (p.flags & ITTAI_F_L2_PREFETCH) != 0;

    for (int step = 0; step < p.n_steps; ++step) {
        if (!step_setup(c, step, pos0)) return;
        const bool run_head = step >= p.n_forced - 1;
        if (!run_head && c.cta == 0 && c.tid < p.batch) p.out_ids[(size_t)step * p.batch + c.tid] = -1;
        for (int l = 0; l < p.n_layers; ++l) {
#pragma unroll 1
            for (int phase = ITTAI_PH_QKV; phase <= ITTAI_PH_DOWN; ++phase) {
                if (prefetch) prefetch_next(c, phase, l, run_head);
                run_phase<NB>(c, phase, l, step);
                if (!grid_barrier(gs, step * 1024 + l * 8 + phase, &c.hdr->ok_s)) return;
            }
        }
        if (run_head) {
            if (prefetch) prefetch_next(c, ITTAI_PH_HEAD, 0, false);
            phase_head<NB>(c, step);
            if (!grid_barrier(gs, step * 1024 + 1023, &c.hdr->ok_s)) return;
        }
        if (p.step_ns != nullptr && c.cta == 0 && c.tid == 0) p.step_ns[step] = globaltimer_ns();
    }
    if (c.cta == 0 && c.tid < p.batch) p.pos[c.tid] = pos0[c.tid] + p.n_steps;
}

// One phase on its own (no grid barrier): unit tests and per-phase profiles.
template <int NB>
__global__ void __launch_bounds__(kThreads, 1) q3_phase_kernel(const __grid_constant__ IttaiQwen3Decode p,
                                                               const __grid_constant__ Q3Workspace wsp, int phase, int l) {
    extern __shared__ __align__(256) unsigned char smem[];
    ITTAI_MAKE_CTA(p, wsp, smem);
    __shared__ int pos0[ITTAI_MAX_BATCH];
    if (c.tid < p.batch) pos0[c.tid] = p.pos[c.tid];
    __syncthreads();
    if (!step_setup(c, 0, pos0)) return;
    run_phase<NB>(c, phase, l, 0);
}

// ---- host side ---------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

static int check_args(const IttaiQwen3Decode* p) {
    if (!p) { set_error("null IttaiQwen3Decode"); return ITTAI_E_ARG; }
    if (p->batch < 1 || p->batch > ITTAI_MAX_BATCH) { set_error("batch %d outside 1..%d", p->batch, ITTAI_MAX_BATCH); return ITTAI_E_ARG; }
    if (p->batch != 1 && p->batch != 2 && p->batch != 4 && p->batch != 8) { set_error("batch %d: supported sizes are 1, 2, 4, 8", p->batch); return ITTAI_E_ARG; }
    if (p->n_layers < 1 || p->vocab < 1 || p->kv_cap < 1 || p->n_steps < 1) { set_error("n_layers, vocab, kv_cap and n_steps must be positive"); return ITTAI_E_ARG; }
    if (p->n_forced < 0 || p->n_forced > p->n_steps) { set_error("n_forced %d outside 0..n_steps", p->n_forced); return ITTAI_E_ARG; }
    if (p->n_forced > 0 && !p->forced) { set_error("n_forced > 0 with forced == NULL"); return ITTAI_E_ARG; }
    if (p->write_logits && !p->logits) { set_error("write_logits set with logits == NULL"); return ITTAI_E_ARG; }
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
    e = cudaMemsetAsync(p->status, 0, ITTAI_STATUS_WORDS * sizeof(uint32_t), st);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status)");
    const int grid = n_sms < Q3_MAX_CTAS ? n_sms : Q3_MAX_CTAS;
    if (phase < 0) {
        void* args[] = {(void*)p, (void*)&ws};
        e = cudaLaunchCooperativeKernel(fn_decode, dim3(grid), dim3(kThreads), args, smem, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchCooperativeKernel(q3_decode_kernel)");
    } else {
        q3_phase_kernel<NB><<<grid, kThreads, smem, st>>>(*p, ws, phase, layer);
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "launch q3_phase_kernel");
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
