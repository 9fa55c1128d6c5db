// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T (+ fused epilogue), fp32 accumulation in
// tensor memory.  Both operands are K-major, as the reference stores them (activations [M,K], weights [N,K]:
// src/ittai/qwen3/sm80.py:175-237, src/ittai/siglip/kernel.py:197-264), and the epilogues fuse what the reference's
// GEMM epilogues fuse (src/ittai/qwen3/base.py:110-129, src/ittai/siglip/kernel.py:266-333): bias, residual add,
// GELU-tanh, SwiGLU on interleaved gate/up columns.
//
// This file: argument checking and dispatch (M > 128 goes to the two-SM kernel of gemm2_sm100.cu), and the one-SM
// kernel for M <= 128.  Persistent, one CTA per SM, looping over 128 x TN output tiles (tile t = blockIdx.x +
// i * gridDim.x, N fastest, the reference's "N-tile outer, M-block inner" grouping: src/ittai/qwen3/engine.py:53-63).
// Warp 0 (one lane) streams 128 x 64 A tiles and TN x 64 W tiles through a ring of shared-memory stages with TMA
// (128-byte swizzle); warp 1 owns the TMEM columns as two TN-column accumulators and (one lane) issues four
// tcgen05.mma (M128 N=TN K16) per stage, releasing the stage with tcgen05.commit; warps 2-9 read a finished
// accumulator with tcgen05.ld (each warp its own 32 TMEM lanes = 32 output rows, two warps per lane quarter splitting
// the columns) and run the epilogue while the MMA warp already fills the other accumulator.  Every wait is bounded; a
// wait that runs out raises the abort flag, all roles fall through to the common exit and TMEM is freed.
#include <cuda.h>

#include "gemm_epilogue.cuh"
#include "tmap.h"
#include "launch.h"

namespace ittai {

constexpr int GM = 128, GN = 256, GK = 64;     // GN: tile width of the wide kernel and the granularity N must have
constexpr int kGemmThreads = 320;        // TMA warp, MMA warp, 8 epilogue warps
constexpr uint32_t kStageBytesA = GM * GK * 2;
// Instantiated with tiles 128 x 64 and 8 stages: this kernel serves M <= 128 (larger problems go to the two-SM kernel),
// where a GEMM has one row tile and only the number of column tiles puts CTAs to work (the MAP head: N = 768 would be 3
// tiles of 256 columns but is 12 of 64).
template <int TN, int STAGES>
struct GemmCfg {
    static constexpr uint32_t kStageBytesB = TN * GK * 2;
    static constexpr uint32_t kSmem = STAGES * (kStageBytesA + kStageBytesB) + 1024 /*alignment*/ + 256 /*barriers*/;
};
constexpr uint32_t kGemmSpin = 1u << 24;
constexpr uint32_t kTmemCols = 512;

template <int TN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmArgs g) {
    extern __shared__ __align__(1024) unsigned char gsm_raw[];
    unsigned char* gsm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sa = gsm;                                         // [stages][128 rows][128 B]
    unsigned char* sb = gsm + STAGES * kStageBytesA;            // [stages][256 rows][128 B]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sb + STAGES * GemmCfg<TN, STAGES>::kStageBytesB);
    unsigned long long* full = bars;                                 // [stages]  TMA -> MMA
    unsigned long long* empty = bars + STAGES;                  // [stages]  MMA -> TMA
    unsigned long long* acc_full = bars + 2 * STAGES;           // [2]       MMA -> epilogue
    unsigned long long* acc_empty = bars + 2 * STAGES + 2;      // [2]       epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = g.N / TN, tiles_m = (g.M + GM - 1) / GM, n_tiles = tiles_m * tiles_n;
    const int n_kb = g.K / GK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    pdl_trigger();
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();                                                      // operands come from the kernels before this one
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer: one running k-block counter across all of this CTA's tiles
            int it = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !*abort_flag; tile += gridDim.x) {
                const int tile_m = tile / tiles_n, tile_n = tile % tiles_n;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES, use = it / STAGES;
                    if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1, kGemmSpin)) { *abort_flag = 1; break; }
                    if (*abort_flag) break;
                    mbar_expect_tx(&full[s], kStageBytesA + GemmCfg<TN, STAGES>::kStageBytesB);
                    tma_load_2d(sa + s * kStageBytesA, &tm_a, kb * GK, tile_m * GM, &full[s]);
                    tma_load_2d(sb + s * GemmCfg<TN, STAGES>::kStageBytesB, &tm_b, kb * GK, tile_n * TN, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            constexpr uint32_t idesc = umma_idesc_bf16(GM, TN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
                const int buf = local & 1, round = local >> 1;
                // the epilogue must have drained this accumulator (passes at once on its first use)
                ok = (round == 0 || mbar_wait_bounded(&acc_empty[buf], (round - 1) & 1, kGemmSpin)) && !*abort_flag;
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * TN);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % STAGES, use = it / STAGES;
                    ok = mbar_wait_bounded(&full[s], use & 1, kGemmSpin) && !*abort_flag;
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(sa + s * kStageBytesA), db = umma_desc_sw128(sb + s * GemmCfg<TN, STAGES>::kStageBytesB);
#pragma unroll
                    for (int k = 0; k < GK / 16; ++k)      // 16 bf16 = 32 bytes = 2 descriptor address units per step
                        umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);                // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[buf]);               // accumulator complete
            }
            if (!ok) *abort_flag = 1;
        }
    } else {
        // ---- epilogue: warp w may touch TMEM lanes 32*(w%4)..+31 = 32 rows of the tile; the two warps that share a lane
        //      quarter split the 256 columns, so every scheduler has two epilogue warps to interleave
        const int q = warp & 3, col_half = (warp - 2) >> 2;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1, round = local >> 1;
            const int tile_m = tile / tiles_n, tile_n = tile % tiles_n;
            bool ok = true;
            {   // bounded wait that also gives up when another role aborted
                uint32_t spins = 0;
                while (!mbar_try_wait_parked(&acc_full[buf], round & 1)) {
                    if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kGemmSpin)) { ok = false; break; }
                }
            }
            if (!ok) { *abort_flag = 1; break; }
            tc_fence_after();
            const int row = tile_m * GM + q * 32 + lane;
#pragma unroll 1
            for (int c0 = col_half * (TN / 2); c0 < (col_half + 1) * (TN / 2); c0 += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * TN + c0), r);
                tmem_ld_wait();
                if (row < g.M) epilogue_chunk(g, r, row, tile_n * TN + c0);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (atomicCAS(&g.status[0], 0u, (uint32_t)ITTAI_ST_GEMM_TIMEOUT) == 0u) { g.status[1] = blockIdx.x; g.status[2] = (uint32_t)n_kb; }
            // let copies that may still be in flight land before the shared memory is handed back
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---- host side ---------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

int gemm2_bf16_launch(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const GemmArgs& g, cudaStream_t st);   // gemm2_sm100.cu

// Checks one IttaiGemm and turns it into kernel arguments and the operand tensor maps (`pair`: the two-SM kernel's W box).
int gemm_args_from_abi(const IttaiGemm* a, GemmArgs* gp, CUtensorMap* tm_a, CUtensorMap* tm_b, bool pair) {
    if (!a || !a->a || !a->w || !a->out || !a->status) { set_error("null pointer in IttaiGemm"); return ITTAI_E_ARG; }
    if (a->m < 1 || a->n < GN || a->n % GN != 0 || a->k < GK || a->k % GK != 0) {
        set_error("gemm shape M=%d N=%d K=%d: N must be a multiple of %d and K of %d", a->m, a->n, a->k, GN, GK);
        return ITTAI_E_ARG;
    }
    if (a->epi < ITTAI_EPI_NONE || a->epi > ITTAI_EPI_QKROPE) { set_error("unknown epilogue %d", a->epi); return ITTAI_E_ARG; }
    if (a->epi == ITTAI_EPI_QKROPE) {
        const IttaiQkRope* r = a->qk_rope;
        if (a->n != ITTAI_Q3_DQKV || a->m <= GM || a->bias || a->residual || (a->row_stats && !(a->stats_rms && a->stats_parts > 0)) || a->stats_out ||
            !r || !r->qn || !r->kn || !r->rope ||
            !r->pos || !r->seq || !r->slot || !r->kcache_layer || !r->vcache_layer || r->kv_cap < 1) {
            set_error("the QK-norm + RoPE epilogue needs N = %d, M > %d, no bias / residual / output statistics, row statistics only as RMS partial sums, and a complete IttaiQkRope", ITTAI_Q3_DQKV, GM);
            return ITTAI_E_ARG;
        }
    }
    if (a->epi == ITTAI_EPI_SWIGLU && a->residual) { set_error("SwiGLU epilogue takes no residual"); return ITTAI_E_ARG; }
    if ((a->row_stats == nullptr) != (a->col_sums == nullptr) || (a->row_stats != nullptr && a->m <= GM)) {
        set_error("a folded LayerNorm needs both row_stats and col_sums, and M > %d", GM);
        return ITTAI_E_ARG;
    }
    if (a->stats_out != nullptr && (a->m <= GM || a->epi == ITTAI_EPI_SWIGLU)) { set_error("stats_out needs M > %d and no SwiGLU", GM); return ITTAI_E_ARG; }
    if (a->stats_parts < 0 || a->stats_parts > 64) { set_error("stats_parts %d out of range", a->stats_parts); return ITTAI_E_ARG; }
    if (a->stats_k < 0 || a->stats_k > a->k) { set_error("stats_k %d: between 0 and K", a->stats_k); return ITTAI_E_ARG; }
    if (a->stats_rms != 0 && (a->stats_rms != 1 || a->stats_parts <= 0)) { set_error("stats_rms is 0 or 1 and needs partial sums (stats_parts > 0)"); return ITTAI_E_ARG; }
    const int ld_a = a->ld_a ? a->ld_a : a->k, ld_w = a->ld_w ? a->ld_w : a->k;
    const int n_out = a->epi == ITTAI_EPI_SWIGLU ? a->n / 2 : a->n;
    const int ld_out = a->ld_out ? a->ld_out : n_out, ld_res = a->ld_res ? a->ld_res : a->n;
    if (((uintptr_t)a->a & 15) || ((uintptr_t)a->w & 15) || ((uintptr_t)a->out & 15) || ((uintptr_t)a->residual & 15) ||
        ((uintptr_t)a->bias & 15) || ld_a % 8 || ld_w % 8 || ld_out % 8 || ld_res % 8) {
        set_error("gemm operands must be 16-byte aligned with leading dimensions that are multiples of 8");
        return ITTAI_E_ARG;
    }
    int rc = make_tmap_bf16(tm_a, a->a, a->m, a->k, ld_a, GM);
    if (rc != ITTAI_OK) return rc;
    rc = make_tmap_bf16(tm_b, a->w, a->n, a->k, ld_w, pair ? GN / 2 : 64);
    if (rc != ITTAI_OK) return rc;
    GemmArgs& g = *gp;
    g.M = a->m; g.N = a->n; g.K = a->k; g.epi = a->epi;
    g.bias = reinterpret_cast<const float*>(a->bias);
    g.residual = reinterpret_cast<const bf16*>(a->residual);
    g.ld_res = ld_res;
    g.out = reinterpret_cast<bf16*>(a->out);
    g.ld_out = ld_out;
    g.status = a->status;
    g.row_stats = a->row_stats;
    g.col_sums = a->col_sums;
    g.stats_out = a->stats_out;
    g.stats_parts = a->stats_parts;
    g.stats_eps = a->stats_eps;
    g.stats_k = a->stats_k;
    g.stats_rms = a->stats_rms;
    if (a->epi == ITTAI_EPI_QKROPE) g.rope = *a->qk_rope; else g.rope = IttaiQkRope{};
    return ITTAI_OK;
}

int gemm_bf16_launch(const IttaiGemm* a, cudaStream_t st) {
    // more than one 128-row tile: the two-SM kernel (each CTA of a pair loads 128 rows of A and 128 rows of W per stage)
    const bool pair = a != nullptr && a->m > GM;
    CUtensorMap tm_a, tm_b;
    GemmArgs g;
    const int rc = gemm_args_from_abi(a, &g, &tm_a, &tm_b, pair);
    if (rc != ITTAI_OK) return rc;
    static thread_local int attr_dev = -1, n_sms = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<64, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GemmCfg<64, 8>::kSmem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm)");
        e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(sm count)");
        attr_dev = dev;
    }
    if (pair) return gemm2_bf16_launch(tm_a, tm_b, g, st);
    const int tiles = ((a->m + GM - 1) / GM) * (a->n / 64);
    cudaError_t e = launch_pdl(gemm_bf16_kernel<64, 8>, dim3(tiles < n_sms ? tiles : n_sms), dim3(kGemmThreads), GemmCfg<64, 8>::kSmem, st, 1, tm_a, tm_b, g);
    if (e != cudaSuccess) return cuda_fail(e, "launch gemm_bf16_kernel");
    return ITTAI_OK;
}

}  // namespace ittai

extern "C" int ittai_gemm_bf16_launch(const IttaiGemm* a, void* stream) {
    return ittai::gemm_bf16_launch(a, reinterpret_cast<cudaStream_t>(stream));
}
