// Row-wise kernels around the tensor-core GEMMs of the prefill and SigLIP paths: RMSNorm, LayerNorm, Qwen3
// QK-norm + RoPE + cache scatter, SigLIP patch gather, last-token pooling.  All are memory-bound passes over a
// [rows, width] bf16 matrix, one warp per row, 128-bit accesses.
//
// The reference folds these into GEMM epilogues (row statistics finished by the last arriving tile,
// src/ittai/qwen3/base.py:59-78, :84-109; src/ittai/siglip/kernel.py:266-364).  Here they are separate passes so that
// every rounding point is the eager module's (norm output rounded to bf16 before the Linear reads it).
#include "common.cuh"
#include "launch.h"

namespace ittai {

constexpr int kRowThreads = 256;     // 8 rows per CTA

// y = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * gain), width 1024.
__global__ void __launch_bounds__(kRowThreads) rmsnorm_rows_kernel(const bf16* __restrict__ x, int ld_x, const bf16* __restrict__ gain,
                                                                     bf16* __restrict__ y, int ld_y, int rows, float eps) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    uint4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = *reinterpret_cast<const uint4*>(x + (size_t)row * ld_x + (lane + 32 * i) * 8);
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) ss += bf_lo(w[j]) * bf_lo(w[j]) + bf_hi(w[j]) * bf_hi(w[j]);
    }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss * (1.0f / 1024.f) + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 gq = *reinterpret_cast<const uint4*>(gain + (lane + 32 * i) * 8);
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, gw[4] = {gq.x, gq.y, gq.z, gq.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = pack_bf16x2(bf16r(bf_lo(w[j]) * rstd) * bf_lo(gw[j]), bf16r(bf_hi(w[j]) * rstd) * bf_hi(gw[j]));
        *reinterpret_cast<uint4*>(y + (size_t)row * ld_y + (lane + 32 * i) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// y = bf16((x - mean) * rsqrt(var + eps) * gain + beta); width a multiple of 8, at most NCH * 256; gain/beta fp32.
// A warp walks rows with a grid stride, holding its slice of gain and beta in registers (re-reading them per row costs
// four times the row's own bytes) and loading the next row while it reduces the current one.
template <int NCH>
__global__ void __launch_bounds__(kRowThreads) layernorm_rows_kernel(const bf16* __restrict__ x, int ld_x, const float* __restrict__ gain,
                                                                       const float* __restrict__ beta, bf16* __restrict__ y, int ld_y,
                                                                       int rows, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int n_chunks = width / 8, stride = gridDim.x * (kRowThreads / 32);
    int row = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float gg[NCH][8], bb[NCH][8];
    uint4 cur[NCH], nxt[NCH];
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int ch = lane + 32 * i;
        if (ch < n_chunks) {
            const float4 g0 = *reinterpret_cast<const float4*>(gain + ch * 8), g1 = *reinterpret_cast<const float4*>(gain + ch * 8 + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(beta + ch * 8), b1 = *reinterpret_cast<const float4*>(beta + ch * 8 + 4);
            gg[i][0] = g0.x; gg[i][1] = g0.y; gg[i][2] = g0.z; gg[i][3] = g0.w; gg[i][4] = g1.x; gg[i][5] = g1.y; gg[i][6] = g1.z; gg[i][7] = g1.w;
            bb[i][0] = b0.x; bb[i][1] = b0.y; bb[i][2] = b0.z; bb[i][3] = b0.w; bb[i][4] = b1.x; bb[i][5] = b1.y; bb[i][6] = b1.z; bb[i][7] = b1.w;
            cur[i] = *reinterpret_cast<const uint4*>(x + (size_t)row * ld_x + ch * 8);
        }
    }
    const float inv_w = 1.0f / (float)width;
    for (; row < rows; row += stride) {
        const int next = row + stride;
        if (next < rows) {
#pragma unroll
            for (int i = 0; i < NCH; ++i)
                if (lane + 32 * i < n_chunks) nxt[i] = *reinterpret_cast<const uint4*>(x + (size_t)next * ld_x + (lane + 32 * i) * 8);
        }
        float v[NCH][8];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NCH; ++i)
            if (lane + 32 * i < n_chunks) {
                const uint32_t w[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) { v[i][2 * j] = bf_lo(w[j]); v[i][2 * j + 1] = bf_hi(w[j]); s += v[i][2 * j] + v[i][2 * j + 1]; }
            }
        const float mean = warp_sum(s) * inv_w;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < NCH; ++i)
            if (lane + 32 * i < n_chunks) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; sq += d * d; }
            }
        const float rstd = 1.0f / sqrtf(warp_sum(sq) * inv_w + eps);
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int ch = lane + 32 * i;
            if (ch < n_chunks) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    o[j] = pack_bf16x2((v[i][2 * j] - mean) * rstd * gg[i][2 * j] + bb[i][2 * j], (v[i][2 * j + 1] - mean) * rstd * gg[i][2 * j + 1] + bb[i][2 * j + 1]);
                *reinterpret_cast<uint4*>(y + (size_t)row * ld_y + ch * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
#pragma unroll
        for (int i = 0; i < NCH; ++i) cur[i] = nxt[i];
    }
}

// stats[row] = (mean, rstd) over `width` columns: what a GEMM with a folded LayerNorm applies in its epilogue (the
// reference's row statistics, src/ittai/siglip/kernel.py:335-364).  Two passes over registers, like the LayerNorm above.
template <int NCH>
__global__ void __launch_bounds__(kRowThreads) row_stats_kernel(const bf16* __restrict__ x, int ld_x, float* __restrict__ stats,
                                                                  int rows, int width, float eps) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int n_chunks = width / 8;
    float v[NCH][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int ch = lane + 32 * i;
        if (ch < n_chunks) {
            const uint4 q = *reinterpret_cast<const uint4*>(x + (size_t)row * ld_x + ch * 8);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[i][2 * j] = bf_lo(w[j]); v[i][2 * j + 1] = bf_hi(w[j]); s += v[i][2 * j] + v[i][2 * j + 1]; }
        }
    }
    const float mean = warp_sum(s) / (float)width;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NCH; ++i)
        if (lane + 32 * i < n_chunks) {
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; sq += d * d; }
        }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
    if (lane == 0) *reinterpret_cast<float2*>(stats + 2 * (size_t)row) = make_float2(mean, rstd);
}

// Qwen3 prefill: per token and head, RMSNorm over the 128 head dims + half-split RoPE in bf16 steps (the arithmetic of
// the decode phase), Q rotated in place in the qkv matrix, K and V written to cache row slot[t] of sequence seq[t]
// (the rotary position pos[t] and the cache row differ when sequences are packed into one cache).
// Eight lanes per (token, head), four heads per warp: heads 0..15 = q, 16..23 = k, 24..31 = v.  A lane owns elements
// 8*sub .. 8*sub+7 and their rotation partners 64 + the same, as two 16-byte accesses.
__global__ void __launch_bounds__(kRowThreads) qk_rope_scatter_kernel(bf16* __restrict__ qkv, const bf16* __restrict__ qn,
                                                                        const bf16* __restrict__ kn, const bf16* __restrict__ rope,
                                                                        const int* __restrict__ pos, const int* __restrict__ seq,
                                                                        const int* __restrict__ slot,
                                                                        bf16* __restrict__ kc, bf16* __restrict__ vc, int n_tokens,
                                                                        int kv_cap, float eps) {
    pdl_trigger();
    pdl_wait();
    constexpr int HD = ITTAI_Q3_HD, NKV = ITTAI_Q3_NKV, DQKV = ITTAI_Q3_DQKV;
    const int gw = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int t = gw >> 3, head = (gw & 7) * 4 + (lane >> 3), sub = lane & 7;
    if (t >= n_tokens) return;
    bf16* row = qkv + (size_t)t * DQKV + head * HD;
    const int p = pos[t], b = seq[t], sl = slot[t];   // rotary position, cache sequence, cache row
    const uint4 ua = *reinterpret_cast<const uint4*>(row + 8 * sub), ub = *reinterpret_cast<const uint4*>(row + HD / 2 + 8 * sub);
    if (head >= 24) {                                  // a warp's four heads are all q, all k or all v
        bf16* dst = vc + (((size_t)b * NKV + (head - 24)) * kv_cap + sl) * HD;
        *reinterpret_cast<uint4*>(dst + 8 * sub) = ua;
        *reinterpret_cast<uint4*>(dst + HD / 2 + 8 * sub) = ub;
        return;
    }
    const bool is_k = head >= 16;
    const bf16* gain = is_k ? kn : qn;
    const uint4 ga = *reinterpret_cast<const uint4*>(gain + 8 * sub), gb = *reinterpret_cast<const uint4*>(gain + HD / 2 + 8 * sub);
    const bf16* rp = rope + (size_t)p * HD;
    const uint4 cw = *reinterpret_cast<const uint4*>(rp + 8 * sub), sw = *reinterpret_cast<const uint4*>(rp + HD / 2 + 8 * sub);
    const uint32_t wa[4] = {ua.x, ua.y, ua.z, ua.w}, wb[4] = {ub.x, ub.y, ub.z, ub.w};
    const uint32_t wga[4] = {ga.x, ga.y, ga.z, ga.w}, wgb[4] = {gb.x, gb.y, gb.z, gb.w};
    const uint32_t wc[4] = {cw.x, cw.y, cw.z, cw.w}, ws[4] = {sw.x, sw.y, sw.z, sw.w};
    float xa[8], xb[8], ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        xa[2 * j] = bf_lo(wa[j]); xa[2 * j + 1] = bf_hi(wa[j]); xb[2 * j] = bf_lo(wb[j]); xb[2 * j + 1] = bf_hi(wb[j]);
        ss += xa[2 * j] * xa[2 * j] + xa[2 * j + 1] * xa[2 * j + 1] + xb[2 * j] * xb[2 * j] + xb[2 * j + 1] * xb[2 * j + 1];
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // the 8 lanes of this head
    const float rstd = 1.0f / sqrtf(ss * (1.0f / HD) + eps);
    uint32_t olo[4], ohi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float lo[2], hi[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float g0 = h ? bf_hi(wga[j]) : bf_lo(wga[j]), g1 = h ? bf_hi(wgb[j]) : bf_lo(wgb[j]);
            const float cs = h ? bf_hi(wc[j]) : bf_lo(wc[j]), sn = h ? bf_hi(ws[j]) : bf_lo(ws[j]);
            const float x0 = bf16r(bf16r(xa[2 * j + h] * rstd) * g0), x1 = bf16r(bf16r(xb[2 * j + h] * rstd) * g1);
            lo[h] = bf16r(bf16r(x0 * cs) + bf16r(-x1 * sn));
            hi[h] = bf16r(bf16r(x1 * cs) + bf16r(x0 * sn));
        }
        olo[j] = pack_bf16x2(lo[0], lo[1]);
        ohi[j] = pack_bf16x2(hi[0], hi[1]);
    }
    bf16* dst = is_k ? kc + (((size_t)b * NKV + (head - 16)) * kv_cap + sl) * HD : row;
    *reinterpret_cast<uint4*>(dst + 8 * sub) = make_uint4(olo[0], olo[1], olo[2], olo[3]);
    *reinterpret_cast<uint4*>(dst + HD / 2 + 8 * sub) = make_uint4(ohi[0], ohi[1], ohi[2], ohi[3]);
}

// SigLIP patch gather: fp32 pixels [B, 3, H, W] -> bf16 patches [B * (H/p) * (W/p)][ld_out], the first 3 * p * p columns of
// a row in (channel, row, col) order, the order a Conv2d weight flattens to (reference src/ittai/siglip/kernel.py:633-637);
// columns beyond are left as they are (a zero-padded K stays zero), and pixels beyond the last whole patch are dropped, as a
// Conv2d of stride p without padding drops them.  One thread per V consecutive pixels of a patch row:
// V = 4 when the patch size is a multiple of 4, else 2 (patch 14).
template <int V>
__global__ void __launch_bounds__(256) im2col_kernel(const float* __restrict__ px, bf16* __restrict__ out, int B, int H, int W, int p, int ld_out) {
    pdl_trigger();
    pdl_wait();
    // 32-bit index arithmetic (the host checks that the element count fits)
    const unsigned gw = W / p, gh = H / p, pp = p * p, kpv = 3 * pp / V, pv = p / V;
    const unsigned total = (unsigned)B * gh * gw * kpv;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const unsigned patch = i / kpv, colv = i - patch * kpv;          // element = V consecutive pixels of a patch row
        const unsigned c = colv / (pp / V), rem = colv - c * (pp / V), py = rem / pv, pxv = rem - py * pv;
        const unsigned b = patch / (gh * gw), pi = patch - b * (gh * gw), pr = pi / gw, pc = pi - pr * gw;
        const float* src = px + (((size_t)b * 3 + c) * H + pr * p + py) * W + pc * p + pxv * V;
        bf16* dst = out + (size_t)patch * ld_out + (size_t)colv * V;
        if constexpr (V == 4) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(src));
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
        } else {
            const float2 v = __ldg(reinterpret_cast<const float2*>(src));
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(v.x, v.y);
        }
    }
}

// Embedding rows: out[t] = table[ids[t]], width 1024 (reference src/ittai/qwen3/base.py:147-162).
__global__ void __launch_bounds__(kRowThreads) embed_rows_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                                                   bf16* __restrict__ out, int rows, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(out + (size_t)row * 1024 + (lane + 32 * i) * 8) =
            *reinterpret_cast<const uint4*>(table + (size_t)id * 1024 + (lane + 32 * i) * 8);
}

// Embedding head of the reference: final RMSNorm of one row per sequence in fp32, then L2 normalisation
// (reference src/ittai/qwen3/base.py:131-145).  One warp per sequence; rows[s] is the last token's row.
__global__ void __launch_bounds__(kRowThreads) final_pool_kernel(const bf16* __restrict__ h, const int* __restrict__ rows,
                                                                   const bf16* __restrict__ gain, float* __restrict__ out, int n_seq, float eps) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (s >= n_seq) return;
    const bf16* x = h + (size_t)rows[s] * 1024;
    float v[32], ss = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] = bf2f(x[lane + 32 * i]); ss += v[i] * v[i]; }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) * (1.0f / 1024.f) + eps);
    float n2 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) { v[i] = v[i] * rstd * bf2f(gain[lane + 32 * i]); n2 += v[i] * v[i]; }
    const float inv = 1.0f / fmaxf(sqrtf(warp_sum(n2)), 1e-12f);
#pragma unroll
    for (int i = 0; i < 32; ++i) out[(size_t)s * 1024 + lane + 32 * i] = v[i] * inv;
}

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
static int launched(const char* what) {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ITTAI_OK : cuda_fail(e, what);
}
static int row_grid(long long rows) { return (int)((rows + kRowThreads / 32 - 1) / (kRowThreads / 32)); }

}  // namespace ittai

using namespace ittai;

extern "C" int ittai_rmsnorm_rows(const void* x, int ld_x, const void* gain, void* y, int ld_y, int rows, float eps, void* stream) {
    if (!x || !gain || !y || rows < 1 || ld_x % 8 || ld_y % 8) { set_error("rmsnorm_rows: bad argument"); return ITTAI_E_ARG; }
    launch_pdl(rmsnorm_rows_kernel, dim3(row_grid(rows)), dim3(kRowThreads), 0, (cudaStream_t)stream, 1, (const bf16*)x, ld_x, (const bf16*)gain, (bf16*)y, ld_y, rows, eps);
    return launched("rmsnorm_rows_kernel");
}

extern "C" int ittai_layernorm_rows(const void* x, int ld_x, const void* gain, const void* beta, void* y, int ld_y, int rows, int width,
                                    float eps, void* stream) {
    if (!x || !gain || !beta || !y || rows < 1 || width < 8 || width % 8 || width > 2048 || ld_x % 8 || ld_y % 8) {
        set_error("layernorm_rows: width must be a multiple of 8 up to 2048");
        return ITTAI_E_ARG;
    }
    // a few rows per warp, so that the parameter registers are worth loading: four CTAs per SM
    const int grid = row_grid(rows) < 148 * 4 ? row_grid(rows) : 148 * 4;
    cudaStream_t st = (cudaStream_t)stream;
    if (width <= 768) launch_pdl(layernorm_rows_kernel<3>, dim3(grid), dim3(kRowThreads), 0, st, 1, (const bf16*)x, ld_x, (const float*)gain, (const float*)beta, (bf16*)y, ld_y, rows, width, eps);
    else if (width <= 1280) launch_pdl(layernorm_rows_kernel<5>, dim3(grid), dim3(kRowThreads), 0, st, 1, (const bf16*)x, ld_x, (const float*)gain, (const float*)beta, (bf16*)y, ld_y, rows, width, eps);
    else launch_pdl(layernorm_rows_kernel<8>, dim3(grid), dim3(kRowThreads), 0, st, 1, (const bf16*)x, ld_x, (const float*)gain, (const float*)beta, (bf16*)y, ld_y, rows, width, eps);
    return launched("layernorm_rows_kernel");
}

extern "C" int ittai_row_stats(const void* x, int ld_x, float* stats, int rows, int width, float eps, void* stream) {
    if (!x || !stats || rows < 1 || width < 8 || width % 8 || width > 2048 || ld_x % 8) { set_error("row_stats: bad argument"); return ITTAI_E_ARG; }
    const int grid = row_grid(rows);
    cudaStream_t st = (cudaStream_t)stream;
    if (width <= 768) launch_pdl(row_stats_kernel<3>, dim3(grid), dim3(kRowThreads), 0, st, 1, (const bf16*)x, ld_x, stats, rows, width, eps);
    else if (width <= 1280) launch_pdl(row_stats_kernel<5>, dim3(grid), dim3(kRowThreads), 0, st, 1, (const bf16*)x, ld_x, stats, rows, width, eps);
    else launch_pdl(row_stats_kernel<8>, dim3(grid), dim3(kRowThreads), 0, st, 1, (const bf16*)x, ld_x, stats, rows, width, eps);
    return launched("row_stats_kernel");
}

extern "C" int ittai_qwen3_qk_rope_scatter(void* qkv, const void* qn, const void* kn, const void* rope, const int32_t* pos,
                                           const int32_t* seq, const int32_t* slot, void* kcache_layer, void* vcache_layer,
                                           int n_tokens, int kv_cap, float eps, void* stream) {
    if (!qkv || !qn || !kn || !rope || !pos || !seq || !slot || !kcache_layer || !vcache_layer || n_tokens < 1) { set_error("qk_rope_scatter: bad argument"); return ITTAI_E_ARG; }
    launch_pdl(qk_rope_scatter_kernel, dim3(row_grid((long long)n_tokens * 8)), dim3(kRowThreads), 0, (cudaStream_t)stream, 1, 
        (bf16*)qkv, (const bf16*)qn, (const bf16*)kn, (const bf16*)rope, pos, seq, slot, (bf16*)kcache_layer, (bf16*)vcache_layer, n_tokens, kv_cap, eps);
    return launched("qk_rope_scatter_kernel");
}

extern "C" int ittai_siglip_im2col(const float* pixels, void* patches, int batch, int height, int width, int patch, int ld_out, void* stream) {
    const int row = 3 * patch * patch;
    if (ld_out == 0) ld_out = row;
    if (!pixels || !patches || batch < 1 || patch < 2 || patch % 2 || height < patch || width < patch || width % 2 || ld_out < row || ld_out % 2) {
        set_error("im2col: bad argument (even patch size and image width, ld_out >= 3 p p and even)");
        return ITTAI_E_ARG;
    }
    const int v = patch % 4 == 0 && width % 4 == 0 && ld_out % 4 == 0 ? 4 : 2;
    if ((unsigned long long)batch * height * width * 3 / v >= (1ull << 31)) { set_error("im2col: too many pixel values in one call"); return ITTAI_E_ARG; }
    const size_t total = (size_t)batch * height * width * 3 / v;
    const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (v == 4) launch_pdl(im2col_kernel<4>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, 1, pixels, (bf16*)patches, batch, height, width, patch, ld_out);
    else launch_pdl(im2col_kernel<2>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, 1, pixels, (bf16*)patches, batch, height, width, patch, ld_out);
    return launched("im2col_kernel");
}

extern "C" int ittai_embed_rows(const int32_t* ids, const void* table, void* out, int rows, int vocab, void* stream) {
    if (!ids || !table || !out || rows < 1 || vocab < 1) { set_error("embed_rows: bad argument"); return ITTAI_E_ARG; }
    launch_pdl(embed_rows_kernel, dim3(row_grid(rows)), dim3(kRowThreads), 0, (cudaStream_t)stream, 1, ids, (const bf16*)table, (bf16*)out, rows, vocab);
    return launched("embed_rows_kernel");
}

extern "C" int ittai_qwen3_final_pool(const void* h, const int32_t* rows, const void* gain, float* out, int n_seq, float eps, void* stream) {
    if (!h || !rows || !gain || !out || n_seq < 1) { set_error("final_pool: bad argument"); return ITTAI_E_ARG; }
    launch_pdl(final_pool_kernel, dim3(row_grid(n_seq)), dim3(kRowThreads), 0, (cudaStream_t)stream, 1, (const bf16*)h, rows, (const bf16*)gain, out, n_seq, eps);
    return launched("final_pool_kernel");
}
