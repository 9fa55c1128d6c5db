// Row-wise kernels around the tensor-core GEMMs of the prefill and SigLIP paths: RMSNorm, LayerNorm, Qwen3
// QK-norm + RoPE + cache scatter, SigLIP patch gather, last-token pooling.  All are memory-bound passes over a
// [rows, width] bf16 matrix, one warp per row, 128-bit accesses.
//
// The reference folds these into GEMM epilogues (row statistics finished by the last arriving tile,
// src/ittai/qwen3/base.py:59-78, :84-109; src/ittai/siglip/kernel.py:266-364).  Here they are separate passes so that
// every rounding point is the eager module's (norm output rounded to bf16 before the Linear reads it).
#include "common.cuh"

namespace ittai {

constexpr int kRowThreads = 256;     // 8 rows per CTA

// y = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * gain), width 1024.
__global__ void __launch_bounds__(kRowThreads) rmsnorm_rows_kernel(const bf16* __restrict__ x, int ld_x, const bf16* __restrict__ gain,
                                                                     bf16* __restrict__ y, int ld_y, int rows, float eps) {
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
template <int NCH>
__global__ void __launch_bounds__(kRowThreads) layernorm_rows_kernel(const bf16* __restrict__ x, int ld_x, const float* __restrict__ gain,
                                                                       const float* __restrict__ beta, bf16* __restrict__ y, int ld_y,
                                                                       int rows, int width, float eps) {
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
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int ch = lane + 32 * i;
        if (ch < n_chunks) {
            const float4 g0 = *reinterpret_cast<const float4*>(gain + ch * 8), g1 = *reinterpret_cast<const float4*>(gain + ch * 8 + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(beta + ch * 8), b1 = *reinterpret_cast<const float4*>(beta + ch * 8 + 4);
            const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                o[j] = pack_bf16x2((v[i][2 * j] - mean) * rstd * gg[2 * j] + bb[2 * j], (v[i][2 * j + 1] - mean) * rstd * gg[2 * j + 1] + bb[2 * j + 1]);
            *reinterpret_cast<uint4*>(y + (size_t)row * ld_y + ch * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// Qwen3 prefill: per token and head, RMSNorm over the 128 head dims + half-split RoPE in bf16 steps (the arithmetic of
// the decode phase), Q rotated in place in the qkv matrix, K and V written to cache row slot[t] of sequence seq[t]
// (the rotary position pos[t] and the cache row differ when sequences are packed into one cache).
// One warp per (token, head): heads 0..15 = q, 16..23 = k, 24..31 = v.
__global__ void __launch_bounds__(kRowThreads) qk_rope_scatter_kernel(bf16* __restrict__ qkv, const bf16* __restrict__ qn,
                                                                        const bf16* __restrict__ kn, const bf16* __restrict__ rope,
                                                                        const int* __restrict__ pos, const int* __restrict__ seq,
                                                                        const int* __restrict__ slot,
                                                                        bf16* __restrict__ kc, bf16* __restrict__ vc, int n_tokens,
                                                                        int kv_cap, float eps) {
    constexpr int HD = ITTAI_Q3_HD, NKV = ITTAI_Q3_NKV, DQ = ITTAI_Q3_DQ, DKV = ITTAI_Q3_DKV, DQKV = ITTAI_Q3_DQKV;
    const int gw = blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int t = gw >> 5, head = gw & 31;
    if (t >= n_tokens) return;
    bf16* row = qkv + (size_t)t * DQKV + head * HD;
    const int p = pos[t], b = seq[t], sl = slot[t];   // rotary position, cache sequence, cache row
    // elements 2*lane, 2*lane+1 and their rotation partners 64 + the same
    const uint32_t ua = *reinterpret_cast<const uint32_t*>(row + 2 * lane), ub = *reinterpret_cast<const uint32_t*>(row + HD / 2 + 2 * lane);
    if (head >= 24) {
        const int g = head - 24;
        bf16* dst = vc + (((size_t)b * NKV + g) * kv_cap + sl) * HD;
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = ua;
        *reinterpret_cast<uint32_t*>(dst + HD / 2 + 2 * lane) = ub;
        return;
    }
    const bool is_k = head >= 16;
    const bf16* gain = is_k ? kn : qn;
    float x[4] = {bf_lo(ua), bf_hi(ua), bf_lo(ub), bf_hi(ub)};
    const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    const float rstd = 1.0f / sqrtf(ss * (1.0f / HD) + eps);
    const uint32_t ga = *reinterpret_cast<const uint32_t*>(gain + 2 * lane), gb = *reinterpret_cast<const uint32_t*>(gain + HD / 2 + 2 * lane);
    x[0] = bf16r(bf16r(x[0] * rstd) * bf_lo(ga)); x[1] = bf16r(bf16r(x[1] * rstd) * bf_hi(ga));
    x[2] = bf16r(bf16r(x[2] * rstd) * bf_lo(gb)); x[3] = bf16r(bf16r(x[3] * rstd) * bf_hi(gb));
    const bf16* rp = rope + (size_t)p * HD;
    const uint32_t cw = *reinterpret_cast<const uint32_t*>(rp + 2 * lane), sw = *reinterpret_cast<const uint32_t*>(rp + HD / 2 + 2 * lane);
    float lo[2], hi[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float cs = j ? bf_hi(cw) : bf_lo(cw), sn = j ? bf_hi(sw) : bf_lo(sw);
        lo[j] = bf16r(bf16r(x[j] * cs) + bf16r(-x[j + 2] * sn));
        hi[j] = bf16r(bf16r(x[j + 2] * cs) + bf16r(x[j] * sn));
    }
    bf16* dst = is_k ? kc + (((size_t)b * NKV + (head - 16)) * kv_cap + sl) * HD : row;
    *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16x2(lo[0], lo[1]);
    *reinterpret_cast<uint32_t*>(dst + HD / 2 + 2 * lane) = pack_bf16x2(hi[0], hi[1]);
    (void)DQ; (void)DKV;
}

// SigLIP patch gather: fp32 pixels [B, 3, H, W] -> bf16 patches [B * (H/p) * (W/p), 3 * p * p] in (channel, row, col)
// order, the order a Conv2d weight flattens to (reference src/ittai/siglip/kernel.py:633-637).  One thread per
// 4 consecutive pixels of a patch row.
__global__ void im2col_kernel(const float* __restrict__ px, bf16* __restrict__ out, int B, int H, int W, int p) {
    const int gw = W / p, gh = H / p, kp = 3 * p * p;
    const size_t total = (size_t)B * gh * gw * kp / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t e = i * 4;
        const int col = (int)(e % kp);
        const size_t patch = e / kp;
        const int c = col / (p * p), py = (col / p) % p, pxx = col % p;
        const int b = (int)(patch / (gh * gw)), pr = (int)(patch % (gh * gw)) / gw, pc = (int)(patch % gw);
        const float4 v = *reinterpret_cast<const float4*>(px + (((size_t)b * 3 + c) * H + pr * p + py) * W + pc * p + pxx);
        *reinterpret_cast<uint2*>(out + e) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    }
}

// Embedding rows: out[t] = table[ids[t]], width 1024 (reference src/ittai/qwen3/base.py:147-162).
__global__ void __launch_bounds__(kRowThreads) embed_rows_kernel(const int* __restrict__ ids, const bf16* __restrict__ table,
                                                                   bf16* __restrict__ out, int rows, int vocab) {
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
    rmsnorm_rows_kernel<<<row_grid(rows), kRowThreads, 0, (cudaStream_t)stream>>>((const bf16*)x, ld_x, (const bf16*)gain, (bf16*)y, ld_y, rows, eps);
    return launched("rmsnorm_rows_kernel");
}

extern "C" int ittai_layernorm_rows(const void* x, int ld_x, const void* gain, const void* beta, void* y, int ld_y, int rows, int width,
                                    float eps, void* stream) {
    if (!x || !gain || !beta || !y || rows < 1 || width < 8 || width % 8 || width > 2048 || ld_x % 8 || ld_y % 8) {
        set_error("layernorm_rows: width must be a multiple of 8 up to 2048");
        return ITTAI_E_ARG;
    }
    const int grid = row_grid(rows);
    cudaStream_t st = (cudaStream_t)stream;
    if (width <= 768) layernorm_rows_kernel<3><<<grid, kRowThreads, 0, st>>>((const bf16*)x, ld_x, (const float*)gain, (const float*)beta, (bf16*)y, ld_y, rows, width, eps);
    else if (width <= 1280) layernorm_rows_kernel<5><<<grid, kRowThreads, 0, st>>>((const bf16*)x, ld_x, (const float*)gain, (const float*)beta, (bf16*)y, ld_y, rows, width, eps);
    else layernorm_rows_kernel<8><<<grid, kRowThreads, 0, st>>>((const bf16*)x, ld_x, (const float*)gain, (const float*)beta, (bf16*)y, ld_y, rows, width, eps);
    return launched("layernorm_rows_kernel");
}

extern "C" int ittai_qwen3_qk_rope_scatter(void* qkv, const void* qn, const void* kn, const void* rope, const int32_t* pos,
                                           const int32_t* seq, const int32_t* slot, void* kcache_layer, void* vcache_layer,
                                           int n_tokens, int kv_cap, float eps, void* stream) {
    if (!qkv || !qn || !kn || !rope || !pos || !seq || !slot || !kcache_layer || !vcache_layer || n_tokens < 1) { set_error("qk_rope_scatter: bad argument"); return ITTAI_E_ARG; }
    qk_rope_scatter_kernel<<<row_grid((long long)n_tokens * 32), kRowThreads, 0, (cudaStream_t)stream>>>(
        (bf16*)qkv, (const bf16*)qn, (const bf16*)kn, (const bf16*)rope, pos, seq, slot, (bf16*)kcache_layer, (bf16*)vcache_layer, n_tokens, kv_cap, eps);
    return launched("qk_rope_scatter_kernel");
}

extern "C" int ittai_siglip_im2col(const float* pixels, void* patches, int batch, int height, int width, int patch, void* stream) {
    if (!pixels || !patches || batch < 1 || patch % 4 || height % patch || width % patch) { set_error("im2col: bad argument"); return ITTAI_E_ARG; }
    const size_t total = (size_t)batch * height * width * 3 / 4;
    const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    im2col_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(pixels, (bf16*)patches, batch, height, width, patch);
    return launched("im2col_kernel");
}

extern "C" int ittai_embed_rows(const int32_t* ids, const void* table, void* out, int rows, int vocab, void* stream) {
    if (!ids || !table || !out || rows < 1 || vocab < 1) { set_error("embed_rows: bad argument"); return ITTAI_E_ARG; }
    embed_rows_kernel<<<row_grid(rows), kRowThreads, 0, (cudaStream_t)stream>>>(ids, (const bf16*)table, (bf16*)out, rows, vocab);
    return launched("embed_rows_kernel");
}

extern "C" int ittai_qwen3_final_pool(const void* h, const int32_t* rows, const void* gain, float* out, int n_seq, float eps, void* stream) {
    if (!h || !rows || !gain || !out || n_seq < 1) { set_error("final_pool: bad argument"); return ITTAI_E_ARG; }
    final_pool_kernel<<<row_grid(n_seq), kRowThreads, 0, (cudaStream_t)stream>>>((const bf16*)h, rows, (const bf16*)gain, out, n_seq, eps);
    return launched("final_pool_kernel");
}
