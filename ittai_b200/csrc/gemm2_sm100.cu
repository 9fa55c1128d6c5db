// Two-SM bf16 GEMM: C[M,N] = A[M,K] * W[N,K]^T (+ fused epilogue) with tcgen05.mma.cta_group::2.  A cluster of two CTAs
// owns a 256 x 256 output tile: each CTA loads 128 rows of A and 128 rows of W per 64-wide k-block (32 KB instead of the
// 48 KB a lone CTA needs for its 128 x 256 tile, which is what bounds the one-SM kernel: the L2 cannot feed 96 bytes
// per clock to every SM), the leader CTA issues M256 N256 K16 MMAs that read both CTAs' shared memory, and each CTA
// keeps the accumulator rows of its own 128 rows of A in its own tensor memory (two 256-column buffers, so the epilogue of
// one tile overlaps the main loop of the next).
//
// Roles per CTA: warp 0 (one lane) TMA producer for this CTA's half of every stage, completion counted on the LEADER's
// full barrier; warp 1 allocates tensor memory and, in the leader only, issues the MMAs, releasing stages and
// publishing accumulators with multicast commits that arrive in both CTAs; warps 2-9 are the epilogue, 32 columns at a
// time: accumulator -> bias / activation / rounding in the row-per-thread layout tcgen05.ld gives -> residual add from
// a TMA-prefetched tile -> a swizzled staging tile in shared memory -> TMA store (row-per-thread global stores write
// half sectors of 32 different lines per instruction and slow the main loop's loads down).  The peer's epilogue warps
// arrive on the leader's accumulator-free barrier through the cluster's shared window.  Every wait is bounded.
#include "gemm2_common.cuh"

namespace ittai {

// ITTAI_EPI_QKROPE: one warp = 32 tokens x one head (its 128 accumulator columns).  The thread that owns a token's row
// rounds the 128 values to bf16 (the Linear output), and for q / k heads applies the head RMSNorm and the half-split
// rotary embedding with the rounding steps of the eager modules (the arithmetic of qk_rope_scatter_kernel); q goes
// to the output matrix through the staging tile and a TMA store, k and v go to their cache rows through the staging
// tile with four lanes per 64-byte row piece (whole sectors), each lane having looked up the rows it stores.
__device__ __forceinline__ void epilogue_qkrope(const GemmArgs& g, const CUtensorMap* tm_out, uint32_t t_addr, unsigned char* so,
                                                const uint32_t* sgain, uint32_t& cc, int row0, int col0, int lane, float row_scale) {
    constexpr int HD = ITTAI_Q3_HD, NKV = ITTAI_Q3_NKV;
    const int head = col0 / HD, t = row0 + lane;
    const bool valid = t < g.M;
    uint32_t pk[64];
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + 32 * ch, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[16 * ch + i] = pack_bf16x2(__uint_as_float(r[2 * i]) * row_scale, __uint_as_float(r[2 * i + 1]) * row_scale);   // a folded RMSNorm's rstd of the row, else 1
    }
    if (head < 24) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) { const float lo = bf_lo(pk[i]), hi = bf_hi(pk[i]); ss = fmaf(lo, lo, fmaf(hi, hi, ss)); }
        const float rstd = 1.0f / sqrtf(ss * (1.0f / HD) + g.rope.eps);
        const bf16* rp = reinterpret_cast<const bf16*>(g.rope.rope) + (size_t)(valid ? g.rope.pos[t] : 0) * HD;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {                  // elements 8jj .. 8jj+7 and their partners 64 + the same
            const uint4 cw = *reinterpret_cast<const uint4*>(rp + 8 * jj), sw = *reinterpret_cast<const uint4*>(rp + HD / 2 + 8 * jj);
            const uint4 ga = *reinterpret_cast<const uint4*>(sgain + 4 * jj), gb = *reinterpret_cast<const uint4*>(sgain + 32 + 4 * jj);
            const uint32_t wc[4] = {cw.x, cw.y, cw.z, cw.w}, ws[4] = {sw.x, sw.y, sw.z, sw.w};
            const uint32_t wga[4] = {ga.x, ga.y, ga.z, ga.w}, wgb[4] = {gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float lo[2], hi[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float xa = h ? bf_hi(pk[4 * jj + j]) : bf_lo(pk[4 * jj + j]), xb = h ? bf_hi(pk[32 + 4 * jj + j]) : bf_lo(pk[32 + 4 * jj + j]);
                    const float g0 = h ? bf_hi(wga[j]) : bf_lo(wga[j]), g1 = h ? bf_hi(wgb[j]) : bf_lo(wgb[j]);
                    const float cs = h ? bf_hi(wc[j]) : bf_lo(wc[j]), sn = h ? bf_hi(ws[j]) : bf_lo(ws[j]);
                    const float x0 = bf16r(bf16r(xa * rstd) * g0), x1 = bf16r(bf16r(xb * rstd) * g1);
                    lo[h] = bf16r(bf16r(x0 * cs) + bf16r(-x1 * sn));
                    hi[h] = bf16r(bf16r(x1 * cs) + bf16r(x0 * sn));
                }
                pk[4 * jj + j] = pack_bf16x2(lo[0], lo[1]);
                pk[32 + 4 * jj + j] = pack_bf16x2(hi[0], hi[1]);
            }
        }
    }
    const int swz = (lane >> 1) & 3;
    // cache rows of the four tokens this lane stores pieces of (k / v heads)
    bf16* dst[4] = {nullptr, nullptr, nullptr, nullptr};
    if (head >= 16) {
        bf16* cache = reinterpret_cast<bf16*>(head < 24 ? g.rope.kcache_layer : g.rope.vcache_layer);
        const int kvh = head < 24 ? head - 16 : head - 24;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int tt = row0 + (lane >> 2) + 8 * i;
            if (tt < g.M) dst[i] = cache + (((size_t)g.rope.seq[tt] * NKV + kvh) * g.rope.kv_cap + g.rope.slot[tt]) * HD + 8 * (lane & 3);
        }
    }
#pragma unroll
    for (int ch = 0; ch < 4; ++ch, ++cc) {
        unsigned char* sto = so + (cc % 3u) * 2048;
        if (lane == 0) tma_store_wait_read<2>();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(sto + lane * 64 + ((j ^ swz) << 4)) = make_uint4(pk[16 * ch + 4 * j], pk[16 * ch + 4 * j + 1], pk[16 * ch + 4 * j + 2], pk[16 * ch + 4 * j + 3]);
        if (head < 16) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) { tma_store_2d(tm_out, sto, col0 + 32 * ch, row0); tma_store_commit(); }
        } else {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int rr = (lane >> 2) + 8 * i;
                const uint4 val = *reinterpret_cast<const uint4*>(sto + rr * 64 + (((lane & 3) ^ ((rr >> 1) & 3)) << 4));
                if (dst[i] != nullptr) *reinterpret_cast<uint4*>(dst[i] + 32 * ch) = val;
            }
            __syncwarp();
        }
    }
}

__global__ void __launch_bounds__(kThreads2, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                  const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_res, const GemmArgs g) {
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
    const int tiles_n = g.N / PN, tiles_m = (g.M + PM - 1) / PM, n_tiles = tiles_m * tiles_n;
    const int n_kb = g.K / PK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * kEpiWarps); }
        for (int b = 0; b < 2 * kEpiWarps; ++b) mbar_init(&res_bars[b], 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    pdl_trigger();
    if (warp == 1) tmem_alloc_pair(tmem_slot, kTmemCols2);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                              // the peer's barriers exist before anything targets them
    tc_fence_after();
    pdl_wait();                                                      // operands come from the kernels before this one
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer for this CTA's halves; one running k-block counter across all of the pair's tiles
            int it = 0;
            for (int tile = pair; tile < n_tiles && !*abort_flag; tile += n_pairs) {
                const int tile_m = TILE_M(tile), tile_n = TILE_N(tile);
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kStages2, use = it / kStages2;
                    if (use > 0 && !mbar_wait_bounded(&empty[s], (use - 1) & 1, kSpin2)) { *abort_flag = 1; break; }
                    if (*abort_flag) break;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * (kHalfA + kHalfB));
                    const uint32_t leader_full = map_to_cta(&full[s], 0);
                    tma_load_2d_pair(sa + s * kHalfA, &tm_a, kb * PK, tile_m * PM + (int)rank * 128, leader_full);
                    tma_load_2d_pair(sb + s * kHalfB, &tm_b, kb * PK, tile_n * PN + (int)rank * 128, leader_full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (leader only)
            constexpr uint32_t idesc = umma_idesc_bf16(PM, PN);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local) {
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
        const bool fold = g.row_stats != nullptr;
        unsigned long long* res_bar = res_bars + 2 * ew;
        const bool swiglu = g.epi == ITTAI_EPI_SWIGLU, has_res = g.residual != nullptr;
        const int swz = (lane >> 1) & 3;                             // 64-byte swizzle of this thread's staging row
        constexpr uint32_t kChunks = kEpiCols / 32;                  // 32-column chunks per tile for this warp
        // With a residual, tile 0 stages the output and tiles 1-2 receive residual chunks by TMA, two chunks ahead of
        // their use and across tile boundaries: chunk n of this warp's running sequence is chunk n % kChunks of its
        // (n / kChunks)-th tile and lands in buffer n % 2.  Without one, the three tiles rotate as output staging.
        auto prefetch_res = [&](uint32_t n) {
            const int t = pair + (int)(n / kChunks) * n_pairs;
            if (t < n_tiles) {
                mbar_expect_tx(&res_bar[n & 1], 2048);
                tma_load_2d(so + 2048 + (n & 1) * 2048, &tm_res, TILE_N(t) * PN + kEpiCols * cq + 32 * (int)(n % kChunks),
                            TILE_M(t) * PM + (int)rank * 128 + q * 32, &res_bar[n & 1]);
            }
        };
        if (has_res && lane == 0) { prefetch_res(0); prefetch_res(1); }
        uint32_t cc = 0;
        int local = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++local) {
            const int buf = local & 1, round = local >> 1;
            const int tile_m = TILE_M(tile), tile_n = TILE_N(tile);
            const int row0 = tile_m * PM + (int)rank * 128 + q * 32;  // first row of this warp
            const int col0 = tile_n * PN + kEpiCols * cq;             // first accumulator column of this warp
            // the bias slice does not depend on the accumulator: fetched before waiting for it
            if (g.bias != nullptr && lane < kEpiCols / 4) *reinterpret_cast<float4*>(sbias + 4 * lane) = *reinterpret_cast<const float4*>(g.bias + col0 + 4 * lane);
            float mean = 0.f, rstd = 1.f;
            if (fold) {
                if (lane < kEpiCols / 4) *reinterpret_cast<float4*>(scsum + 4 * lane) = *reinterpret_cast<const float4*>(g.col_sums + col0 + 4 * lane);
                if (row0 + lane < g.M) {
                    if (g.stats_parts == 0) {
                        const float2 ms = *reinterpret_cast<const float2*>(g.row_stats + 2 * (size_t)(row0 + lane));
                        mean = ms.x; rstd = ms.y;
                    } else {
                        // partial (sum, sum of squares) of the K columns in slices, added in slice order
                        const float2* ps = reinterpret_cast<const float2*>(g.row_stats) + (size_t)(row0 + lane) * g.stats_parts;
                        float s1 = 0.f, s2 = 0.f;
                        for (int i = 0; i < g.stats_parts; ++i) { const float2 t = ps[i]; s1 += t.x; s2 += t.y; }
                        const float inv_k = 1.0f / (float)(g.stats_k > 0 ? g.stats_k : g.K);
                        mean = g.stats_rms ? 0.f : s1 * inv_k;
                        rstd = rsqrtf(fmaxf(s2 * inv_k - mean * mean, 0.f) + g.stats_eps);
                    }
                }
            }
            float st1 = 0.f, st2 = 0.f;                               // statistics of this row's output slice
            if (g.epi == ITTAI_EPI_QKROPE && col0 < ITTAI_Q3_DQ + ITTAI_Q3_DKV && lane < 16)   // this head's norm gain, 128 bf16
                *reinterpret_cast<uint4*>(sbias + 4 * lane) = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(col0 < ITTAI_Q3_DQ ? g.rope.qn : g.rope.kn) + 8 * lane);
            __syncwarp();
            bool ok = true;
            {
                uint32_t spins = 0;
                while (!mbar_try_wait_parked(&acc_full[buf], round & 1)) {
                    if (((++spins) & 255u) == 0u && (*abort_flag || spins >= kSpin2)) { ok = false; break; }
                }
            }
            if (!ok) { *abort_flag = 1; break; }
            tc_fence_after();
            if (g.epi == ITTAI_EPI_QKROPE) {
                epilogue_qkrope(g, &tm_out, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * PN + kEpiCols * cq), so,
                                reinterpret_cast<const uint32_t*>(sbias), cc, row0, col0, lane, rstd);
            } else
#pragma unroll 1
            for (uint32_t ch = 0; ch < kChunks && ok; ++ch, ++cc) {
                // 32 accumulator columns of this thread's row -> bias, activation, rounding -> 16 packed words
                uint32_t r[32], o[16];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * PN + kEpiCols * cq + 32 * ch), r);
                tmem_ld_wait();
                epilogue_pack(g, r, g.bias != nullptr ? sbias + 32 * ch : nullptr, o, fold ? scsum + 32 * ch : nullptr, mean, rstd);
                if (swiglu) {
                    // 16 output columns per chunk: two consecutive chunks fill one 32-column staging tile, then one TMA store
                    const uint32_t half = ch & 1;
                    unsigned char* sto = so + ((cc >> 1) % 3u) * 2048;
                    if (half == 0) {
                        if (lane == 0) tma_store_wait_read<2>();
                        __syncwarp();
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        *reinterpret_cast<uint4*>(sto + lane * 64 + (((2 * half + j) ^ swz) << 4)) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                    if (half == 1) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) { tma_store_2d(&tm_out, sto, (col0 + 32 * ((int)ch - 1)) / 2, row0); tma_store_commit(); }
                    }
                    continue;
                }
                if (has_res) {
                    // out = bf16(residual + bf16(module output)); this thread's row piece of the TMA-filled buffer
                    const uint32_t b = cc & 1;
                    uint32_t spins = 0;
                    while (!mbar_try_wait_parked(&res_bar[b], (cc >> 1) & 1)) {
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
                    if (lane == 0) prefetch_res(cc + 2);
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
                if (lane == 0) { tma_store_2d(&tm_out, sto, col0 + 32 * (int)ch, row0); tma_store_commit(); }
            }
            if (!ok) break;
            if (g.stats_out != nullptr && row0 + lane < g.M)
                *reinterpret_cast<float2*>(g.stats_out + 2 * ((size_t)(row0 + lane) * (g.N / 128) + col0 / 128)) = make_float2(st1, st2);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[buf], 0));
        }
        if (lane == 0) tma_store_wait_all();                          // shared memory stays valid until the stores are done
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
    // neither CTA leaves while the other may still read its shared memory or signal its barriers
    cluster_sync_all();
    if (warp == 1) { __syncwarp(); tmem_dealloc_pair(tmem_base, kTmemCols2); }
}

int cuda_fail(cudaError_t e, const char* what);

int gemm2_bf16_launch(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const GemmArgs& g, cudaStream_t st) {
    // the epilogue stores 32-row x 32-column boxes through TMA (rows past M are dropped) and fetches the residual the same way
    CUtensorMap tm_out, tm_res;
    const bool swiglu = g.epi == ITTAI_EPI_SWIGLU;
    int rc = make_tmap_bf16(&tm_out, g.out, g.M, swiglu ? g.N / 2 : g.N, g.ld_out, 32, 32);
    if (rc != ITTAI_OK) return rc;
    if (g.residual != nullptr) rc = make_tmap_bf16(&tm_res, g.residual, g.M, g.N, g.ld_res, 32, 32);
    else tm_res = tm_out;
    if (rc != ITTAI_OK) return rc;
    static thread_local int attr_dev = -1, max_pairs = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(gemm2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(gemm2)");
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
        e = cudaOccupancyMaxActiveClusters(&n_clusters, gemm2_bf16_kernel, &cfg);
        if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters(gemm2)");
        max_pairs = n_clusters < 1 ? 1 : (n_clusters > n_sms / 2 ? n_sms / 2 : n_clusters);
        attr_dev = dev;
    }
    const int tiles = ((g.M + PM - 1) / PM) * (g.N / PN);
    const cudaError_t e = launch_pdl(gemm2_bf16_kernel, dim3(2 * (tiles < max_pairs ? tiles : max_pairs)), dim3(kThreads2), kSmem2, st, 2, tm_a, tm_b, tm_out, tm_res, g);
    if (e != cudaSuccess) return cuda_fail(e, "launch gemm2_bf16_kernel");
    return ITTAI_OK;
}

}  // namespace ittai
