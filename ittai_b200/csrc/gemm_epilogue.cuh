// Pieces shared by the tensor-core GEMM kernels: launch arguments and the fused epilogue arithmetic (bias, GELU-tanh,
// SwiGLU, residual add with the eager modules' rounding points; reference src/ittai/qwen3/base.py:110-129,
// src/ittai/siglip/kernel.py:266-333).
#pragma once
#include "tcgen05.cuh"

namespace ittai {

struct GemmArgs {
    int M, N, K;
    int epi;                 // ITTAI_EPI_*
    const float* bias;       // [N] or nullptr
    const bf16* residual;    // [M, ld_res] or nullptr
    int ld_res;
    bf16* out;               // [M, ld_out]  (SwiGLU: N/2 columns)
    int ld_out;
    uint32_t* status;        // device status words
    const float* row_stats;  // [M][2] (mean, rstd) of the rows of A, or nullptr: LayerNorm folded into the GEMM
    const float* col_sums;   // [N] column sums of the folded weight
    float* stats_out;        // [M][N/128][2] (sum, sum of squares) per 128-column slice of the output rows, or nullptr
    int stats_parts;         // > 0: row_stats holds [M][parts][2] partial sums over K instead of (mean, rstd)
    float stats_eps;
    int stats_k;             // columns the folded LayerNorm's statistics are over (A may be zero-padded beyond them); 0 = K
    int stats_rms;           // 1: the folded norm is an RMSNorm (mean 0, rstd from the sum of squares alone)
    IttaiQkRope rope;        // ITTAI_EPI_QKROPE only
};

// GELU-tanh as the reference writes it (src/ittai/siglip/kernel.py:289-291); the hardware tanh approximation is good
// to about 2^-11, well inside the bf16 rounding of the result.
__device__ __forceinline__ float gelu_tanh(float y) {
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.7978845608028654f * (y + 0.044715f * y * y * y)));
    return 0.5f * y * (1.0f + th);
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One 32-column slice of an accumulator row: bias, activation, residual, rounding, 128-bit stores.
__device__ __forceinline__ void epilogue_chunk(const GemmArgs& g, const uint32_t (&r)[32], int row, int col) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
    if (g.bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(g.bias + col + i);
            v[i] += b4.x; v[i + 1] += b4.y; v[i + 2] += b4.z; v[i + 3] += b4.w;
        }
    }
    if (g.epi == ITTAI_EPI_SWIGLU) {
        // adjacent columns are (gate, up): act = bf16(bf16(silu(bf16 gate)) * bf16 up)
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const float g0 = bf16r(v[2 * i]), u0 = bf16r(v[2 * i + 1]);
            const float g1 = bf16r(v[2 * i + 2]), u1 = bf16r(v[2 * i + 3]);
            o[i / 2] = pack_bf16x2(bf16r(g0 / (1.0f + expf(-g0))) * u0, bf16r(g1 / (1.0f + expf(-g1))) * u1);
        }
        uint4* dst = reinterpret_cast<uint4*>(g.out + (size_t)row * g.ld_out + col / 2);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        return;
    }
    if (g.epi == ITTAI_EPI_GELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(bf16r(v[i]));   // the Linear output is rounded before the activation
    }
    if (g.residual != nullptr) {
        // out = bf16(residual + bf16(acc [+ bias])): the module output is rounded before the add
        const uint4* rs = reinterpret_cast<const uint4*>(g.residual + (size_t)row * g.ld_res + col);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 rr = rs[i];
            const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[i * 8 + 2 * j] = bf_lo(w[j]) + bf16r(v[i * 8 + 2 * j]);
                v[i * 8 + 2 * j + 1] = bf_hi(w[j]) + bf16r(v[i * 8 + 2 * j + 1]);
            }
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(g.out + (size_t)row * g.ld_out + col);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        dst[i] = make_uint4(pack_bf16x2(v[i * 8], v[i * 8 + 1]), pack_bf16x2(v[i * 8 + 2], v[i * 8 + 3]),
                            pack_bf16x2(v[i * 8 + 4], v[i * 8 + 5]), pack_bf16x2(v[i * 8 + 6], v[i * 8 + 7]));
}

// Same arithmetic without the residual and without the store: 32 accumulator columns of one row -> packed bf16 of the
// module output (16 words; SwiGLU: 8 words for 16 output columns).  `bias32` points at the 32 bias values of these
// columns (shared or global memory) or is null.  The caller adds the residual afterwards, on the rounded values, as the
// eager modules do.
__device__ __forceinline__ void epilogue_pack(const GemmArgs& g, const uint32_t (&r)[32], const float* bias32, uint32_t (&o)[16],
                                              const float* csum32 = nullptr, float mean = 0.f, float rstd = 1.f) {
    // arithmetic on fp32 pairs: one packed instruction does two columns
    float2 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    if (csum32 != nullptr) {
        // folded LayerNorm: rstd * (acc - mean * column sum)
        const float2 nm = make_float2(-mean, -mean), rs = make_float2(rstd, rstd);
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const float4 c4 = *reinterpret_cast<const float4*>(csum32 + 2 * i);
            v[i] = __fmul2_rn(rs, __ffma2_rn(nm, make_float2(c4.x, c4.y), v[i]));
            v[i + 1] = __fmul2_rn(rs, __ffma2_rn(nm, make_float2(c4.z, c4.w), v[i + 1]));
        }
    }
    if (bias32 != nullptr) {
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const float4 b4 = *reinterpret_cast<const float4*>(bias32 + 2 * i);
            v[i] = __fadd2_rn(v[i], make_float2(b4.x, b4.y));
            v[i + 1] = __fadd2_rn(v[i + 1], make_float2(b4.z, b4.w));
        }
    }
    if (g.epi == ITTAI_EPI_SWIGLU) {
        // adjacent columns are (gate, up): act = bf16(bf16(silu(bf16 gate)) * bf16 up), silu(x) = x / (1 + 2^(-x log2 e)) with
        // the hardware exponential and reciprocal (their error is far below the bf16 rounding of the result); the
        // roundings of the Linear outputs run on the integer pipe
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            float gt[2], up[2], sl[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                gt[h] = __uint_as_float(bf16r_bits(__float_as_uint(v[i + h].x)));
                up[h] = __uint_as_float(bf16r_bits(__float_as_uint(v[i + h].y)));
                float e, rc;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(gt[h] * -1.4426950408889634f));
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(1.0f + e));
                sl[h] = __uint_as_float(bf16r_bits(__float_as_uint(gt[h] * rc)));
            }
            o[i / 2] = pack_bf16x2(sl[0] * up[0], sl[1] * up[1]);
        }
        return;
    }
    if (g.epi == ITTAI_EPI_GELU) {
        // 0.5 y (1 + tanh(0.79788456 (y + 0.044715 y^3))) on the Linear output rounded to bf16, written as
        // hy + hy * tanh(y * (c0 + c1 y^2)) with hy = y / 2
        const float2 c0 = make_float2(0.7978845608028654f, 0.7978845608028654f);
        const float2 c1 = make_float2(0.7978845608028654f * 0.044715f, 0.7978845608028654f * 0.044715f);
        const float2 half2 = make_float2(0.5f, 0.5f);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            // rounded on the integer pipe: the conversion unit is busy with tanh and the output packing
            const float2 y = make_float2(__uint_as_float(bf16r_bits(__float_as_uint(v[i].x))), __uint_as_float(bf16r_bits(__float_as_uint(v[i].y))));
            const float2 u = __fmul2_rn(y, __ffma2_rn(__fmul2_rn(y, y), c1, c0));
            float2 th;
            asm("tanh.approx.f32 %0, %1;" : "=f"(th.x) : "f"(u.x));
            asm("tanh.approx.f32 %0, %1;" : "=f"(th.y) : "f"(u.y));
            const float2 hy = __fmul2_rn(y, half2);
            v[i] = __ffma2_rn(hy, th, hy);
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = pack_bf16x2(v[i].x, v[i].y);
}

}  // namespace ittai
