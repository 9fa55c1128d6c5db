// A chain of up to four dependent two-SM GEMMs in ONE persistent launch: GEMM i + 1 reads GEMM i's output as its A
// operand (and may read its output statistics, or an older output as residual).  The reference runs a whole forward as
// one persistent kernel whose CTAs claim tasks from a list and wait on per-row-block counters
// (src/ittai/siglip/kernel.py:197-333, src/ittai/qwen3/engine.py:17-84); launched one GEMM at a time, every boundary
// costs the drain of the last tiles' epilogues, the refill of the load pipeline and the wait for the slowest cluster.
// Here the tiles of all GEMMs form one list (GEMM after GEMM, row block after row block, column tile fastest) dealt
// round-robin to the co-resident clusters, and a tile waits only for the row block it reads:
//
//   flags[g][2 * tile_m + rank]   counts the epilogue warps that have finished a tile of GEMM g in that 128-row block
//                                 (their TMA stores complete, then a gpu-scope release); 8 per column tile.
//   producer of a tile of GEMM g+1, CTA `rank`   acquires flags[g][2 * tile_m + rank] == 8 * column tiles of GEMM g,
//                                 fences the async proxy, then issues its loads.
//
// A task depends only on tasks earlier in the list and every cluster walks the list in order, so the earliest
// unfinished task can always run; every wait is bounded all the same.  In-place residuals are safe under the same
// flags: the tile of GEMM g+1 that overwrites rows of a matrix starts after every tile of GEMM g that read those rows.
// Kernel roles, tile shape, pipeline and epilogue arithmetic are those of gemm2_bf16_kernel; residual chunks are
// prefetched inside a tile only (the next tile may belong to a GEMM whose inputs are not complete yet), and the row
// statistics of a folded LayerNorm are read after the accumulator is ready (their producer is then known complete).
#include "gemm2_common.cuh"

namespace ittai {

constexpr int kChainMax = 4;

struct ChainParams {
    CUtensorMap tm_a[kChainMax], tm_b[kChainMax], tm_out[kChainMax], tm_res[kChainMax];
    GemmArgs g[kChainMax];
    int n;
    uint32_t* flags;          // [n][2 * tiles_m], zero at launch (the caller clears them)
};

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kThreads2, 1)
gemm2_chain_kernel(const __grid_constant__ ChainParams P) {
    extern __shared__ __align__(1024) unsigned char gsm_raw[];
    unsigned char* gsm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gsm_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sa = gsm;                                         // [stages][128 rows][128 B]
    unsigned char* sb = gsm + kStages2 * kHalfA;                     // [stages][128 rows][128 B]
    unsigned char* sout = sb + kStages2 * kHalfB;                    // [epilogue warps] staging tiles, then their bias slices
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sout + kEpiWarps * kStageOut + 2 * 4096);
    unsigned long long* full = bars;                                 // [stages]  both producers -> leader's MMA
    unsigned long long* empty = bars + kStages2;                     // [stages]  MMA -> this CTA's producer
    unsigned long long* acc_full = bars + 2 * kStages2;              // [2]       MMA -> this CTA's epilogue
    unsigned long long* acc_empty = bars + 2 * kStages2 + 2;         // [2]       both epilogues -> leader's MMA
    unsigned long long* res_bars = bars + 2 * kStages2 + 4;          // [epilogue warps][2] residual chunk landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages2 + 4 + 2 * kEpiWarps);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                         // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_g = P.n;
    const int tiles_m = (P.g[0].M + PM - 1) / PM;                    // every GEMM of the chain has the same rows
    // first list index of each GEMM (unused entries: past the end)
    const int c1 = tiles_m * (P.g[0].N / PN);
    const int c2 = n_g > 1 ? c1 + tiles_m * (P.g[1].N / PN) : c1;
    const int c3 = n_g > 2 ? c2 + tiles_m * (P.g[2].N / PN) : c2;
    const int total = n_g > 3 ? c3 + tiles_m * (P.g[3].N / PN) : c3;
    // list index -> (GEMM, tile inside it)
    auto locate = [&](int t, int& gi, int& tile) {
        gi = (n_g > 1 && t >= c1 ? 1 : 0) + (n_g > 2 && t >= c2 ? 1 : 0) + (n_g > 3 && t >= c3 ? 1 : 0);
        tile = t - (gi == 0 ? 0 : gi == 1 ? c1 : gi == 2 ? c2 : c3);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * kEpiWarps); }
        for (int b = 0; b < 2 * kEpiWarps; ++b) mbar_init(&res_bars[b], 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&P.tm_a[0]);
        tma_prefetch_desc(&P.tm_b[0]);
    }
    pdl_trigger();
    if (warp == 1) tmem_alloc_pair(tmem_slot, kTmemCols2);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                              // the peer's barriers exist before anything targets them
    tc_fence_after();
    pdl_wait();                                                      // the chain's inputs come from the kernels before this one
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer for this CTA's halves; one running k-block counter across all of the pair's tiles
            int it = 0;
            for (int t = pair; t < total && !*abort_flag; t += n_pairs) {
                int gi, tile;
                locate(t, gi, tile);
                const int tiles_n = P.g[gi].N / PN, n_kb = P.g[gi].K / PK;
                const int tile_m = tile / tiles_n, tile_n = tile % tiles_n;
                if (gi > 0) {
                    // this CTA's 128 rows of A are the rows the same rank of the pairs of GEMM gi - 1 wrote
                    const uint32_t* f = P.flags + (size_t)(gi - 1) * 2 * tiles_m + 2 * tile_m + rank;
                    const uint32_t want = (uint32_t)(kEpiWarps * (P.g[gi - 1].N / PN));
                    uint32_t spins = 0;
                    while (ld_acquire_gpu_u32(f) < want) {
                        __nanosleep(100);                            // a poll is an L2 round trip: no need to keep several in flight
                        if (((++spins) & 63u) == 0u && (*abort_flag || spins >= (kSpin2 >> 4))) { *abort_flag = 1; break; }
                    }
                    if (*abort_flag) break;
                    fence_proxy_async();                             // the loads below go through the async proxy
                }
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages2, use = it / kStages2;
                    if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1, kSpin2)) { *abort_flag = 1; break; }
                    if (*abort_flag) break;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * (kHalfA + kHalfB));
                    const uint32_t leader_full = map_to_cta(&full[s], 0);
                    tma_load_2d_pair(sa + s * kHalfA, &P.tm_a[gi], kb * PK, tile_m * PM + (int)rank * 128, leader_full);
                    tma_load_2d_pair(sb + s * kHalfB, &P.tm_b[gi], kb * PK, tile_n * PN + (int)rank * 128, leader_full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (leader only)
            constexpr uint32_t idesc = umma_idesc_bf16(PM, PN);
            int it = 0, local = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += n_pairs, ++local) {
                int gi, tile;
                locate(t, gi, tile);
                const int n_kb = P.g[gi].K / PK;
                const int buf = local & 1, round = local >> 1;
                ok = (round == 0 || mbar_wait_bounded(&acc_empty[buf], (round - 1) & 1, kSpin2)) && !*abort_flag;
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * PN);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages2, use = it / kStages2;
                    ok = mbar_wait_bounded(&full[s], use & 1, kSpin2) && !*abort_flag;
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(sa + s * kHalfA), db = umma_desc_sw128(sb + s * kHalfB);
#pragma unroll
                    for (int k = 0; k < PK / 16; ++k)
                        umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s]);               // both CTAs' producers may refill the stage
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[buf]);              // both CTAs' epilogues may read their rows
            }
            if (!ok) *abort_flag = 1;
        }
    } else {
        // ---- epilogue: warp w may touch TMEM lanes 32*(w%4)..+31 = 32 rows of this CTA's half tile; the two warps that
        //      share a lane quarter split the 256 columns
        const int ew = warp - 2, q = warp & 3, cq = ew >> 2;         // TMEM lane quarter, column slice (kEpiCols columns)
        unsigned char* so = sout + ew * kStageOut;                   // three [32 rows][64 B] tiles, 64-byte swizzle
        float* sbias = reinterpret_cast<float*>(sout + kEpiWarps * kStageOut) + ew * kEpiCols;   // this warp's bias values
        float* scsum = sbias + kEpiWarps * kEpiCols;                 // and, with a folded LayerNorm, its column sums
        unsigned long long* res_bar = res_bars + 2 * ew;
        const int swz = (lane >> 1) & 3;                             // 64-byte swizzle of this thread's staging row
        constexpr uint32_t kChunks = kEpiCols / 32;                  // 32-column chunks per tile for this warp
        uint32_t cc = 0, rcnt = 0;                                   // chunks stored / residual chunks consumed so far
        int local = 0;
        bool ok = true;
        for (int t = pair; t < total && ok; t += n_pairs, ++local) {
            int gi, tile;
            locate(t, gi, tile);
            const GemmArgs& g = P.g[gi];
            const int tiles_n = g.N / PN;
            const int buf = local & 1, round = local >> 1;
            const int tile_m = tile / tiles_n, tile_n = tile % tiles_n;
            const int row0 = tile_m * PM + (int)rank * 128 + q * 32;  // first row of this warp
            const int col0 = tile_n * PN + kEpiCols * cq;             // first accumulator column of this warp
            const bool fold = g.row_stats != nullptr, has_res = g.residual != nullptr;
            const float* bias = g.bias;
            // weights' bias and column sums do not depend on the chain: fetched before waiting for the accumulator
            if (bias != nullptr && lane < kEpiCols / 4) *reinterpret_cast<float4*>(sbias + 4 * lane) = *reinterpret_cast<const float4*>(bias + col0 + 4 * lane);
            if (fold && lane < kEpiCols / 4) *reinterpret_cast<float4*>(scsum + 4 * lane) = *reinterpret_cast<const float4*>(g.col_sums + col0 + 4 * lane);
            __syncwarp();
            {
                uint32_t spins = 0;
                while (!mbar_try_wait_parked(&acc_full[buf], round & 1)) {
                    if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kSpin2)) { ok = false; break; }
                }
            }
            if (!ok) { *abort_flag = 1; break; }
            tc_fence_after();
            // The accumulator exists, so this CTA's producer saw the row block of GEMM gi - 1 complete; take the same
            // acquire here for the statistics and the residual this warp reads itself.
            if (gi > 0 && (fold || has_res)) {
                if (lane == 0) {
                    (void)ld_acquire_gpu_u32(P.flags + (size_t)(gi - 1) * 2 * tiles_m + 2 * tile_m + rank);
                    fence_proxy_async();
                }
                __syncwarp();
            }
            auto prefetch_res = [&](uint32_t n, uint32_t ch) {       // chunk `ch` of this tile, n-th residual chunk of the warp
                mbar_expect_tx(&res_bar[n & 1], 2048);
                tma_load_2d(so + 2048 + (n & 1) * 2048, &P.tm_res[gi], col0 + 32 * (int)ch, row0, &res_bar[n & 1]);
            };
            if (has_res && lane == 0) {
                tma_store_wait_read<0>();                             // staging tiles 1-2 become load targets
                prefetch_res(rcnt, 0); prefetch_res(rcnt + 1, 1);
            }
            float mean = 0.f, rstd = 1.f;
            if (fold && row0 + lane < g.M) {
                if (g.stats_parts == 0) {
                    const float2 ms = *reinterpret_cast<const float2*>(g.row_stats + 2 * (size_t)(row0 + lane));
                    mean = ms.x; rstd = ms.y;
                } else {
                    // partial (sum, sum of squares) of the K columns in slices, added in slice order
                    const float2* ps = reinterpret_cast<const float2*>(g.row_stats) + (size_t)(row0 + lane) * g.stats_parts;
                    float s1 = 0.f, s2 = 0.f;
                    for (int i = 0; i < g.stats_parts; ++i) { const float2 tt = ps[i]; s1 += tt.x; s2 += tt.y; }
                    const float inv_k = 1.0f / (float)(g.stats_k > 0 ? g.stats_k : g.K);
                    mean = g.stats_rms ? 0.f : s1 * inv_k;
                    rstd = rsqrtf(fmaxf(s2 * inv_k - mean * mean, 0.f) + g.stats_eps);
                }
            }
            float st1 = 0.f, st2 = 0.f;                               // statistics of this row's output slice
#pragma unroll 1
            for (uint32_t ch = 0; ch < kChunks && ok; ++ch, ++cc) {
                // 32 accumulator columns of this thread's row -> bias, activation, rounding -> 16 packed words
                uint32_t r[32], o[16];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * PN + kEpiCols * cq + 32 * ch), r);
                tmem_ld_wait();
                epilogue_pack(g, r, bias != nullptr ? sbias + 32 * ch : nullptr, o, fold ? scsum + 32 * ch : nullptr, mean, rstd);
                if (has_res) {
                    // out = bf16(residual + bf16(module output)); this thread's row piece of the TMA-filled buffer
                    const uint32_t n = rcnt + ch, b = n & 1;
                    uint32_t spins = 0;
                    while (!mbar_try_wait_parked(&res_bar[b], (n >> 1) & 1)) {
                        if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kSpin2)) { ok = false; break; }
                    }
                    if (!ok) { *abort_flag = 1; break; }
                    const unsigned char* rrow = so + 2048 + b * 2048 + lane * 64;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 rs = *reinterpret_cast<const uint4*>(rrow + ((j ^ swz) << 4));
                        o[4 * j] = pack_bf16x2(bf_lo(rs.x) + bf_lo(o[4 * j]), bf_hi(rs.x) + bf_hi(o[4 * j]));
                        o[4 * j + 1] = pack_bf16x2(bf_lo(rs.y) + bf_lo(o[4 * j + 1]), bf_hi(rs.y) + bf_hi(o[4 * j + 1]));
                        o[4 * j + 2] = pack_bf16x2(bf_lo(rs.z) + bf_lo(o[4 * j + 2]), bf_hi(rs.z) + bf_hi(o[4 * j + 2]));
                        o[4 * j + 3] = pack_bf16x2(bf_lo(rs.w) + bf_lo(o[4 * j + 3]), bf_hi(rs.w) + bf_hi(o[4 * j + 3]));
                    }
                    __syncwarp();                                     // every lane has consumed the buffer: refill it
                    if (lane == 0 && ch + 2 < kChunks) prefetch_res(n + 2, ch + 2);
                }
                if (g.stats_out != nullptr) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float lo = bf_lo(o[i]), hi = bf_hi(o[i]);
                        st1 += lo + hi;
                        st2 = fmaf(lo, lo, fmaf(hi, hi, st2));
                    }
                }
                // the store that last used this staging tile must have finished reading it
                unsigned char* sto = has_res ? so : so + (cc % 3u) * 2048;
                if (lane == 0) { if (has_res) tma_store_wait_read<0>(); else tma_store_wait_read<2>(); }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(sto + lane * 64 + ((j ^ swz) << 4)) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { tma_store_2d(&P.tm_out[gi], sto, col0 + 32 * (int)ch, row0); tma_store_commit(); }
            }
            if (!ok) break;
            if (has_res) rcnt += kChunks;
            if (g.stats_out != nullptr && row0 + lane < g.M)
                *reinterpret_cast<float2*>(g.stats_out + 2 * ((size_t)(row0 + lane) * (g.N / 128) + col0 / 128)) = make_float2(st1, st2);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[buf], 0));
            if (gi + 1 < n_g) {
                // publish: this warp's stores of the tile are complete (bulk stores and the statistics of all its lanes)
                if (lane == 0) {
                    tma_store_wait_all();
                    fence_proxy_async();
                    __threadfence();
                    atomicAdd(P.flags + (size_t)gi * 2 * tiles_m + 2 * tile_m + rank, 1u);
                }
                __syncwarp();
            }
        }
        if (lane == 0) tma_store_wait_all();                          // shared memory stays valid until the stores are done
    }
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            if (atomicCAS(&P.g[0].status[0], 0u, (uint32_t)ITTAI_ST_GEMM_TIMEOUT) == 0u) { P.g[0].status[1] = blockIdx.x; P.g[0].status[2] = (uint32_t)total; }
            // let copies that may still be in flight land before the shared memory is handed back
            const long long t0 = clock64();
            while (clock64() - t0 < 2000000) {}
        }
        __syncthreads();
    }
    // neither CTA leaves while the other may still read its shared memory or signal its barriers
    cluster_sync_all();
    if (warp == 1) { __syncwarp(); tmem_dealloc_pair(tmem_base, kTmemCols2); }
}

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
int gemm_args_from_abi(const IttaiGemm* a, GemmArgs* g, CUtensorMap* tm_a, CUtensorMap* tm_b, bool pair);   // gemm_sm100.cu

int gemm2_chain_launch(const IttaiGemm* gemms, int n, uint32_t* flags, cudaStream_t st) {
    if (!gemms || !flags || n < 1 || n > kChainMax) { set_error("a GEMM chain holds 1 to %d GEMMs and needs a flag buffer", kChainMax); return ITTAI_E_ARG; }
    static thread_local ChainParams C;       // 3 KB of tensor maps and arguments, handed to the launch by value
    C.n = n;
    C.flags = flags;
    for (int i = 0; i < n; ++i) {
        const IttaiGemm* a = gemms + i;
        if (a->m <= 128 || a->m != gemms[0].m) { set_error("every GEMM of a chain needs the same M > 128"); return ITTAI_E_ARG; }
        if (a->epi != ITTAI_EPI_NONE && a->epi != ITTAI_EPI_GELU) { set_error("a GEMM chain takes the plain and GELU epilogues only"); return ITTAI_E_ARG; }
        if (i > 0 && (a->a != gemms[i - 1].out || a->k != gemms[i - 1].n)) { set_error("GEMM %d of the chain must read GEMM %d's output as A", i, i - 1); return ITTAI_E_ARG; }
        int rc = gemm_args_from_abi(a, &C.g[i], &C.tm_a[i], &C.tm_b[i], true);
        if (rc != ITTAI_OK) return rc;
        rc = make_tmap_bf16(&C.tm_out[i], C.g[i].out, C.g[i].M, C.g[i].N, C.g[i].ld_out, 32, 32);
        if (rc != ITTAI_OK) return rc;
        if (C.g[i].residual != nullptr) rc = make_tmap_bf16(&C.tm_res[i], C.g[i].residual, C.g[i].M, C.g[i].N, C.g[i].ld_res, 32, 32);
        else C.tm_res[i] = C.tm_out[i];
        if (rc != ITTAI_OK) return rc;
    }
    for (int i = n; i < kChainMax; ++i) { C.g[i] = C.g[0]; C.tm_a[i] = C.tm_a[0]; C.tm_b[i] = C.tm_b[0]; C.tm_out[i] = C.tm_out[0]; C.tm_res[i] = C.tm_res[0]; }
    static thread_local int attr_dev = -1, max_pairs = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(gemm2_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm2_chain)");
        int n_sms = 0;
        e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(sm count)");
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.blockDim = dim3(kThreads2);
        cfg.dynamicSmemBytes = kSmem2;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cfg.gridDim = dim3(n_sms & ~1);
        int n_clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&n_clusters, gemm2_chain_kernel, &cfg);
        if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters(gemm2_chain)");
        // every cluster must be resident: a tile may wait for a tile of another cluster
        max_pairs = n_clusters < 1 ? 1 : (n_clusters > n_sms / 2 ? n_sms / 2 : n_clusters);
        attr_dev = dev;
    }
    const int tiles_m = (C.g[0].M + PM - 1) / PM;
    int total = 0;
    for (int i = 0; i < n; ++i) total += tiles_m * (C.g[i].N / PN);
    const cudaError_t e = launch_pdl(gemm2_chain_kernel, dim3(2 * (total < max_pairs ? total : max_pairs)), dim3(kThreads2), kSmem2, st, 2, C);
    if (e != cudaSuccess) return cuda_fail(e, "launch gemm2_chain_kernel");
    return ITTAI_OK;
}

}  // namespace ittai

extern "C" int ittai_gemm_chain_launch(const IttaiGemm* gemms, int32_t n, uint32_t* flags, void* stream) {
    return ittai::gemm2_chain_launch(gemms, n, flags, reinterpret_cast<cudaStream_t>(stream));
}
