// Softmax attention for the prefill and SigLIP paths: flash-style, 64 query rows x 64 keys per step, causal (Qwen3,
// grouped-query, head_dim 128) or dense with a key-length mask (SigLIP, head_dim 64).  Same schedule as the
// reference's attention tasks (src/ittai/qwen3/sm80.py:274-403, src/ittai/siglip/kernel.py:366-500): Q tile resident,
// K/V blocks streamed, scores and softmax in fp32 in the log2 domain, P rounded to bf16 for the PV product.
// Tensor-core path: warp-level mma.sync m16n8k16 (bf16 in, fp32 accumulate) on ldmatrix fragments from swizzled
// shared memory.  Attention is a few percent of SigLIP's FLOPs and a third of a 4k prefill's.
#include "common.cuh"
#include "launch.h"

namespace ittai {

struct AttnArgs {
    const bf16* q; const bf16* k; const bf16* v; bf16* o;
    long long q_row, q_head, k_row, k_head, k_seq, v_row, v_head, v_seq, o_row, o_head;   // strides in elements
    const int4* seqs;     // per sequence: {first q/o row, q rows, first k/v row, k/v rows}
    int group;            // query heads per kv head
    float scale_log2;     // head_dim^-0.5 * log2(e)
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int kAttnBN = 64;     // keys per step; query rows per CTA = 16 per warp, 4 warps (head_dim 128) or 8 (head_dim 64)

// element offset of 16-byte chunk `ch` of row `r` in a [rows][HD] tile whose chunks are XOR-swizzled by the row
template <int HD>
__device__ __forceinline__ int sw(int r, int ch) { return r * HD + ((ch ^ (r & 7)) << 3); }

template <int HD, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src, long long row_stride, int rows_valid, int tid) {
    constexpr int CH = HD / 8;
    for (int i = tid; i < ROWS * CH; i += THREADS) {
        const int r = i / CH, ch = i % CH;
        cp_async16(dst + sw<HD>(r, ch), src + (long long)r * row_stride + ch * 8, r < rows_valid);
    }
}

template <int HD, bool CAUSAL, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) attn_fwd_kernel(const AttnArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int kAttnBM = 16 * WARPS, kAttnThreads = 32 * WARPS;
    // shared memory: Q tile, then two (K, V) tile pairs so that block kb+1 streams in while block kb is multiplied
    extern __shared__ __align__(128) unsigned char attn_smem[];
    bf16* sq = reinterpret_cast<bf16*>(attn_smem);
    bf16* skv = sq + kAttnBM * HD;                                    // [2][K | V][64 * HD]
    const int4 sinfo = a.seqs[blockIdx.z];
    const int q_len = sinfo.y, kv_len = sinfo.w;
    const int qb = blockIdx.x * kAttnBM;
    if (qb >= q_len) return;
    const int head = blockIdx.y, kvh = head / a.group;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const bf16* qp = a.q + (long long)(sinfo.x + qb) * a.q_row + (long long)head * a.q_head;
    const bf16* kp = a.k + (long long)blockIdx.z * a.k_seq + (long long)kvh * a.k_head + (long long)sinfo.z * a.k_row;
    const bf16* vp = a.v + (long long)blockIdx.z * a.v_seq + (long long)kvh * a.v_head + (long long)sinfo.z * a.v_row;
    const int q_rows = q_len - qb < kAttnBM ? q_len - qb : kAttnBM;
    const int shift = kv_len - q_len;                       // query i sees keys j <= i + shift
    int kv_end = kv_len;
    if (CAUSAL) { const int lim = qb + q_rows + shift; kv_end = lim < kv_len ? lim : kv_len; }
    const bool warp_live = warp * 16 < q_rows;              // a warp whose 16 rows are all padding only helps loading

    auto load_kv = [&](int kb, int buf) {
        const int rows_valid = kv_len - kb < kAttnBN ? kv_len - kb : kAttnBN;
        load_tile<HD, kAttnBN, kAttnThreads>(skv + (size_t)buf * 2 * kAttnBN * HD, kp + (long long)kb * a.k_row, a.k_row, rows_valid, tid);
        load_tile<HD, kAttnBN, kAttnThreads>(skv + (size_t)buf * 2 * kAttnBN * HD + kAttnBN * HD, vp + (long long)kb * a.v_row, a.v_row, rows_valid, tid);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile<HD, kAttnBM, kAttnThreads>(sq, qp, a.q_row, q_rows, tid);
    if (kv_end > 0) load_kv(0, 0); else asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldsm_x4(qf[ks], sq + sw<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows g and g + 8 of this warp's 16
    const int row0 = qb + warp * 16 + g, row1 = row0 + 8;

    int buf = 0;
    for (int kb = 0; kb < kv_end; kb += kAttnBN, buf ^= 1) {
        // block kb is in `buf` (waited for below or before the loop); start fetching the next one into the other half
        if (kb + kAttnBN < kv_end) load_kv(kb + kAttnBN, buf ^ 1);
        const bf16* sk = skv + (size_t)buf * 2 * kAttnBN * HD;
        const bf16* sv = sk + kAttnBN * HD;
        const int rows_valid = kv_len - kb < kAttnBN ? kv_len - kb : kAttnBN;
        const int n16 = (rows_valid + 15) / 16;              // 16-key groups that hold at least one real key
        if (warp_live) {
            // ---- S = Q K^T
            float s[kAttnBN / 8][4];
#pragma unroll
            for (int i = 0; i < kAttnBN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
                for (int np = 0; np < kAttnBN / 16; ++np) {
                    if (np < n16) {
                        uint32_t kf[4];
                        ldsm_x4(kf, sk + sw<HD>(np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                        mma16816(s[2 * np], qf[ks], kf[0], kf[1]);
                        mma16816(s[2 * np + 1], qf[ks], kf[2], kf[3]);
                    }
                }
            }
            // ---- mask, scale, online softmax
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < kAttnBN / 8; ++i) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = kb + i * 8 + 2 * t + (e & 1), r = (e < 2) ? row0 : row1;
                    const bool vis = j < kv_len && (!CAUSAL || j <= r + shift);
                    s[i][e] = vis ? s[i][e] * a.scale_log2 : -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
                mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
            m0 = mn0; m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
            uint32_t pf[kAttnBN / 16][4];
#pragma unroll
            for (int i = 0; i < kAttnBN / 8; ++i) {
                const float p0 = exp2f(s[i][0] - ms0), p1 = exp2f(s[i][1] - ms0), p2 = exp2f(s[i][2] - ms1), p3 = exp2f(s[i][3] - ms1);
                ps0 += p0 + p1; ps1 += p2 + p3;
                pf[i / 2][(i & 1) * 2] = pack_bf16x2(p0, p1);
                pf[i / 2][(i & 1) * 2 + 1] = pack_bf16x2(p2, p3);
            }
            l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
            // ---- O += P V
#pragma unroll
            for (int ks = 0; ks < kAttnBN / 16; ++ks) {
                if (ks < n16) {
#pragma unroll
                    for (int dp = 0; dp < HD / 16; ++dp) {
                        uint32_t vf[4];
                        ldsm_x4_t(vf, sv + sw<HD>(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
                        mma16816(o[2 * dp], pf[ks], vf[0], vf[1]);
                        mma16816(o[2 * dp + 1], pf[ks], vf[2], vf[3]);
                    }
                }
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");   // the next block has landed
        __syncthreads();                                      // and everyone is done reading this one
    }
    if (!warp_live) return;
    // ---- normalise and store
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    bf16* op = a.o + (long long)sinfo.x * a.o_row + (long long)head * a.o_head;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * t;
        if (row0 < q_len) *reinterpret_cast<uint32_t*>(op + (long long)row0 * a.o_row + d) = pack_bf16x2(o[i][0] * i0, o[i][1] * i0);
        if (row1 < q_len) *reinterpret_cast<uint32_t*>(op + (long long)row1 * a.o_row + d) = pack_bf16x2(o[i][2] * i1, o[i][3] * i1);
    }
}

// Short sequences (at most 256 keys, dense): one CTA per (sequence, head) keeps the whole K and V in shared memory,
// loaded once, and every warp runs its 16 query rows against all keys with no CTA-wide barrier after the load: 13 warps
// for SigLIP's 196 tokens, two CTAs per SM.  K and V are read from HBM once per head instead of once per query block.
constexpr int kShortKeys = 256;
template <int HD>
__global__ void __launch_bounds__(512) attn_short_kernel(const AttnArgs a, int warps) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char attn_smem[];
    const int4 sinfo = a.seqs[blockIdx.z];
    const int q_len = sinfo.y, kv_len = sinfo.w;
    const int head = blockIdx.y, kvh = head / a.group;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int q_rows_pad = warps * 16, threads = warps * 32;
    bf16* sq = reinterpret_cast<bf16*>(attn_smem);
    bf16* sk = sq + q_rows_pad * HD;
    bf16* sv = sk + kShortKeys * HD;
    const bf16* qp = a.q + (long long)sinfo.x * a.q_row + (long long)head * a.q_head;
    const bf16* kp = a.k + (long long)blockIdx.z * a.k_seq + (long long)kvh * a.k_head + (long long)sinfo.z * a.k_row;
    const bf16* vp = a.v + (long long)blockIdx.z * a.v_seq + (long long)kvh * a.v_head + (long long)sinfo.z * a.v_row;
    constexpr int CH = HD / 8;
    const int kv_pad = (kv_len + 15) & ~15;
    for (int i = tid; i < q_rows_pad * CH; i += threads) {
        const int r = i / CH, ch = i % CH;
        cp_async16(sq + sw<HD>(r, ch), qp + (long long)r * a.q_row + ch * 8, r < q_len);
    }
    for (int i = tid; i < kv_pad * CH; i += threads) {
        const int r = i / CH, ch = i % CH;
        cp_async16(sk + sw<HD>(r, ch), kp + (long long)r * a.k_row + ch * 8, r < kv_len);
        cp_async16(sv + sw<HD>(r, ch), vp + (long long)r * a.v_row + ch * 8, r < kv_len);
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (warp * 16 >= q_len) return;
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
        ldsm_x4(qf[ks], sq + sw<HD>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    for (int kb = 0; kb < kv_len; kb += kAttnBN) {
        const int rows_valid = kv_len - kb < kAttnBN ? kv_len - kb : kAttnBN;
        const int n16 = (rows_valid + 15) / 16;
        float s[kAttnBN / 8][4];
#pragma unroll
        for (int i = 0; i < kAttnBN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < kAttnBN / 16; ++np) {
                if (np < n16) {
                    uint32_t kf[4];
                    ldsm_x4(kf, sk + sw<HD>(kb + np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                    mma16816(s[2 * np], qf[ks], kf[0], kf[1]);
                    mma16816(s[2 * np + 1], qf[ks], kf[2], kf[3]);
                }
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < kAttnBN / 8; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kb + i * 8 + 2 * t + (e & 1);
                s[i][e] = j < kv_len ? s[i][e] * a.scale_log2 : -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
            mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);       // every block holds a real key, so mn is finite
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t pf[kAttnBN / 16][4];
#pragma unroll
        for (int i = 0; i < kAttnBN / 8; ++i) {
            const float p0 = exp2f(s[i][0] - mn0), p1 = exp2f(s[i][1] - mn0), p2 = exp2f(s[i][2] - mn1), p3 = exp2f(s[i][3] - mn1);
            ps0 += p0 + p1; ps1 += p2 + p3;
            pf[i / 2][(i & 1) * 2] = pack_bf16x2(p0, p1);
            pf[i / 2][(i & 1) * 2 + 1] = pack_bf16x2(p2, p3);
        }
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
#pragma unroll
        for (int ks = 0; ks < kAttnBN / 16; ++ks) {
            if (ks < n16) {
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    uint32_t vf[4];
                    ldsm_x4_t(vf, sv + sw<HD>(kb + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
                    mma16816(o[2 * dp], pf[ks], vf[0], vf[1]);
                    mma16816(o[2 * dp + 1], pf[ks], vf[2], vf[3]);
                }
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
    const int row0 = warp * 16 + g, row1 = row0 + 8;
    bf16* op = a.o + (long long)sinfo.x * a.o_row + (long long)head * a.o_head;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * t;
        if (row0 < q_len) *reinterpret_cast<uint32_t*>(op + (long long)row0 * a.o_row + d) = pack_bf16x2(o[i][0] * i0, o[i][1] * i0);
        if (row1 < q_len) *reinterpret_cast<uint32_t*>(op + (long long)row1 * a.o_row + d) = pack_bf16x2(o[i][2] * i1, o[i][3] * i1);
    }
}

// One query per sequence (the SigLIP MAP head: a learned probe attends over the tokens), head_dim 64: a CTA of 4 warps
// per (sequence, head); 8 lanes share a key (8 dims each, one 16-byte load), so a warp scores 4 keys per step; each
// 8-lane group keeps a private online softmax over its keys and the 16 groups are merged once through shared memory.
__global__ void __launch_bounds__(128) attn_q1_kernel(const AttnArgs a) {
    pdl_trigger();
    pdl_wait();
    const int head = blockIdx.x, kvh = head / a.group;
    const int4 sinfo = a.seqs[blockIdx.y];
    const int kv_len = sinfo.w;
    const int grp = threadIdx.x >> 3, sub = threadIdx.x & 7;          // 16 groups of 8 lanes
    __shared__ float s_m[16], s_l[16], s_o[16][64];
    const bf16* qp = a.q + (long long)sinfo.x * a.q_row + (long long)head * a.q_head + 8 * sub;
    const uint4 qw = *reinterpret_cast<const uint4*>(qp);
    const uint32_t qq[4] = {qw.x, qw.y, qw.z, qw.w};
    float q[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { q[2 * j] = bf_lo(qq[j]) * a.scale_log2; q[2 * j + 1] = bf_hi(qq[j]) * a.scale_log2; }
    const bf16* kb = a.k + (long long)blockIdx.y * a.k_seq + (long long)kvh * a.k_head + (long long)sinfo.z * a.k_row + 8 * sub;
    const bf16* vb = a.v + (long long)blockIdx.y * a.v_seq + (long long)kvh * a.v_head + (long long)sinfo.z * a.v_row + 8 * sub;
    float m = -INFINITY, l = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j0 = 0; j0 < kv_len; j0 += 16) {
        const int j = j0 + grp;
        const bool valid = j < kv_len;
        uint4 kw = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0);
        if (valid) {
            kw = *reinterpret_cast<const uint4*>(kb + (long long)j * a.k_row);
            vw = *reinterpret_cast<const uint4*>(vb + (long long)j * a.v_row);
        }
        const uint32_t kk[4] = {kw.x, kw.y, kw.z, kw.w}, vv[4] = {vw.x, vw.y, vw.z, vw.w};
        float sc = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) sc += q[2 * e] * bf_lo(kk[e]) + q[2 * e + 1] * bf_hi(kk[e]);
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        if (valid) {
            const float mn = fmaxf(m, sc), c = exp2f(m - mn), pr = exp2f(sc - mn);
            l = l * c + pr;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[2 * e] = acc[2 * e] * c + pr * bf_lo(vv[e]);
                acc[2 * e + 1] = acc[2 * e + 1] * c + pr * bf_hi(vv[e]);
            }
            m = mn;
        }
    }
    if (sub == 0) { s_m[grp] = m; s_l[grp] = l; }
#pragma unroll
    for (int e = 0; e < 8; ++e) s_o[grp][8 * sub + e] = acc[e];
    __syncthreads();
    if (threadIdx.x < 64) {
        float M = -INFINITY;
#pragma unroll
        for (int g = 0; g < 16; ++g) M = fmaxf(M, s_m[g]);
        float o = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int g = 0; g < 16; ++g) {
                const float w = exp2f(s_m[g] - M);        // a group without keys has m = -inf: weight 0
                o = fmaf(s_o[g][threadIdx.x], w, o);
                L = fmaf(s_l[g], w, L);
            }
        }
        a.o[(long long)sinfo.x * a.o_row + (long long)head * a.o_head + threadIdx.x] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
    }
}

static int attn_short_launch(const AttnArgs& a, int max_q_len, int n_heads, int n_seqs, cudaStream_t st) {
    const int warps = (max_q_len + 15) / 16;
    const size_t smem = (size_t)(warps * 16 + 2 * kShortKeys) * 64 * 2;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(attn_short_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((16 * 16 + 2 * kShortKeys) * 64 * 2));
        if (e != cudaSuccess) return (int)e;
        attr_dev = dev;
    }
    launch_pdl(attn_short_kernel<64>, dim3(1, n_heads, n_seqs), dim3(warps * 32), smem, st, 1, a, warps);
    return 0;
}

template <int HD, bool CAUSAL, int WARPS>
static int attn_launch(const AttnArgs& a, int max_q_len, int n_heads, int n_seqs, cudaStream_t st) {
    constexpr size_t smem = (size_t)(16 * WARPS + 4 * kAttnBN) * HD * 2;
    const dim3 grid((max_q_len + 16 * WARPS - 1) / (16 * WARPS), n_heads, n_seqs);
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<HD, CAUSAL, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_dev = dev;
    }
    launch_pdl(attn_fwd_kernel<HD, CAUSAL, WARPS>, grid, dim3(WARPS * 32), smem, st, 1, a);
    return 0;
}

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
bool attn_tc_supported(const IttaiAttention* p);          // attention_sm100.cu
int attn_tc_launch(const IttaiAttention* p, cudaStream_t st);
bool attn_fa_supported(const IttaiAttention* p);          // attention_fa_sm100.cu
int attn_fa_launch(const IttaiAttention* p, cudaStream_t st);

}  // namespace ittai

using namespace ittai;

extern "C" int ittai_attention_launch(const IttaiAttention* p, void* stream) {
    if (!p || !p->q || !p->k || !p->v || !p->o || !p->seqs) { set_error("attention: null pointer"); return ITTAI_E_ARG; }
    if (p->head_dim != 64 && p->head_dim != 128) { set_error("attention: head_dim %d (64 or 128)", p->head_dim); return ITTAI_E_ARG; }
    if (p->n_seqs < 1 || p->n_heads < 1 || p->group < 1 || p->max_q_len < 1) { set_error("attention: bad sizes"); return ITTAI_E_ARG; }
    const long long strides[] = {p->q_row, p->q_head, p->k_row, p->k_head, p->k_seq, p->v_row, p->v_head, p->v_seq, p->o_row};
    for (long long s : strides) if (s % 8) { set_error("attention: strides must be multiples of 8 elements"); return ITTAI_E_ARG; }
    if (attn_tc_supported(p)) return attn_tc_launch(p, (cudaStream_t)stream);
    if (attn_fa_supported(p)) return attn_fa_launch(p, (cudaStream_t)stream);
    AttnArgs a;
    a.q = (const bf16*)p->q; a.k = (const bf16*)p->k; a.v = (const bf16*)p->v; a.o = (bf16*)p->o;
    a.q_row = p->q_row; a.q_head = p->q_head; a.k_row = p->k_row; a.k_head = p->k_head; a.k_seq = p->k_seq;
    a.v_row = p->v_row; a.v_head = p->v_head; a.v_seq = p->v_seq; a.o_row = p->o_row; a.o_head = p->o_head;
    a.seqs = (const int4*)p->seqs; a.group = p->group;
    a.scale_log2 = 1.4426950408889634f / sqrtf((float)p->head_dim);
    cudaStream_t st = (cudaStream_t)stream;
    const int ql = p->max_q_len, nh = p->n_heads, ns = p->n_seqs;
    int rc;
    if (p->head_dim == 64 && !p->causal && ql == 1) {
        const cudaError_t e1 = launch_pdl(attn_q1_kernel, dim3(nh, ns), dim3(128), 0, st, 1, a);
        return e1 == cudaSuccess ? ITTAI_OK : cuda_fail(e1, "launch attn_q1_kernel");
    }
    if (p->head_dim == 128) rc = p->causal ? attn_launch<128, true, 4>(a, ql, nh, ns, st) : attn_launch<128, false, 4>(a, ql, nh, ns, st);
    else if (!p->causal && ql > 64 && ql <= 256 && p->max_kv_len > 0 && p->max_kv_len <= kShortKeys) rc = attn_short_launch(a, ql, nh, ns, st);
    else if (ql <= 64) rc = p->causal ? attn_launch<64, true, 4>(a, ql, nh, ns, st) : attn_launch<64, false, 4>(a, ql, nh, ns, st);
    else rc = p->causal ? attn_launch<64, true, 8>(a, ql, nh, ns, st) : attn_launch<64, false, 8>(a, ql, nh, ns, st);
    if (rc != 0) return cuda_fail((cudaError_t)rc, "cudaFuncSetAttribute(attn_fwd_kernel)");
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ITTAI_OK : cuda_fail(e, "launch attn_fwd_kernel");
}
