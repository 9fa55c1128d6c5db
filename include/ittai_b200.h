/*
 * ittai_b200 — C ABI of the B200 (sm_100a) inference kernels behind the Python engines.
 *
 * The reference has no FFI layer: its device code is CuTe-DSL Python compiled at run time and
 * launched from `Engine.forward` (reference src/ittai/qwen3/engine.py:141,153-187 and
 * src/ittai/siglip/kernel.py:614-620,651-664).  These entry points replace that compile-and-launch
 * step.  Conventions for every function:
 *   - returns 0 on success, a negative ITTAI_E_* code otherwise; ittai_last_error() gives the text;
 *   - all data pointers are DEVICE pointers borrowed from the caller (torch owns every buffer, as the
 *     reference's Engine owns its tensors: src/ittai/qwen3/engine.py:123-140);
 *   - `stream` is a cudaStream_t passed as void*; launch functions enqueue work and return, they do not
 *     synchronise, allocate or read device memory on the host;
 *   - device-side waits are bounded: a wait that runs out records a code in the `status` words of the
 *     call's struct and every CTA leaves the kernel; the host decodes it with ittai_decode_status().
 *
 * Model widths are compile-time (Qwen3-0.6B: reference src/ittai/qwen3/config.py:1-5); layer count,
 * vocabulary, batch and cache capacity are run-time.
 */
#ifndef ITTAI_B200_H
#define ITTAI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ITTAI_ABI_VERSION 1

/* Qwen3-0.6B widths (reference src/ittai/qwen3/config.py:1-5). */
#define ITTAI_Q3_D 1024
#define ITTAI_Q3_NH 16
#define ITTAI_Q3_NKV 8
#define ITTAI_Q3_HD 128
#define ITTAI_Q3_FF 3072
#define ITTAI_Q3_DQ 2048
#define ITTAI_Q3_DKV 1024
#define ITTAI_Q3_DQKV 4096
#define ITTAI_Q3_DGU 6144

#define ITTAI_MAX_BATCH 8

/* IttaiQwen3Decode.flags */
#define ITTAI_F_TEST_DROP_CTA 2 /* test hook: CTA 0 leaves at once, so the words it would publish never arrive and
                                  the other CTAs' bounded waits run out and report ITTAI_ST_FLAG_TIMEOUT */

enum {
    ITTAI_OK = 0,
    ITTAI_E_ARG = -1,     /* bad argument (null pointer, size out of range, misaligned pointer) */
    ITTAI_E_CUDA = -2,    /* a CUDA runtime call failed; see ittai_last_error() */
    ITTAI_E_DEVICE = -3,  /* not an sm_100 device, or it cannot co-schedule the persistent grid */
    ITTAI_E_STATUS = -4   /* the device status words report a failed wait */
};

/* Device status words written by a kernel whose bounded wait ran out (status[0] != 0). */
#define ITTAI_STATUS_WORDS 8
enum {
    ITTAI_ST_OK = 0,
    ITTAI_ST_BARRIER_TIMEOUT = 1, /* reserved */
    ITTAI_ST_FLAG_TIMEOUT = 2,    /* status[1]=what was awaited (phase id, +16 merge, +32 residual, 64 step order),
                                     status[2]=CTA, status[3]=tag seen, status[4]=tag expected */
    ITTAI_ST_BAD_TOKEN = 3,       /* status[1]=token id, status[2]=step, status[3]=position, status[4]=sequence */
    ITTAI_ST_STREAM_TIMEOUT = 4,  /* a weight-stream copy did not land: status[1]=entry, status[2]=CTA */
    ITTAI_ST_GEMM_TIMEOUT = 5     /* a pipeline wait of a tensor-core kernel (GEMM, attention) ran out: status[1]=CTA */
};

/* Phases of one decoded token, in execution order inside a layer (ids used by ittai_qwen3_phase_launch). */
enum {
    ITTAI_PH_QKV = 0,   /* embed gather (layer 0) + RMSNorm + QKV GEMV                         */
    ITTAI_PH_ATTN = 1,  /* QK-RMSNorm + RoPE + in-place KV append + split-K GQA attention + combine */
    ITTAI_PH_OPROJ = 2, /* O-proj GEMV + residual                                              */
    ITTAI_PH_GU = 3,    /* RMSNorm + gate/up GEMV + SwiGLU                                     */
    ITTAI_PH_DOWN = 4,  /* down-proj GEMV + residual                                           */
    ITTAI_PH_HEAD = 5   /* final RMSNorm + tied lm_head GEMV + argmax                          */
};

/*
 * Everything one Qwen3 decode launch needs.  Weight layout follows the reference's packed engine
 * (src/ittai/qwen3/engine.py:100-117) except that the norm gains stay separate (so the bf16 rounding
 * points are those of the eager modules) and Q/K rows keep the half-split RoPE order, so the cache holds
 * keys exactly as the eager model's cache does.
 * All matrices are bf16, row-major [out_features, in_features], stacked over layers.
 */
typedef struct IttaiQwen3Decode {
    int32_t n_layers;   /* L                                                                   */
    int32_t vocab;      /* V                                                                   */
    int32_t kv_cap;     /* cache capacity in tokens per sequence                               */
    int32_t batch;      /* B: 1, 2, 4 or 8                                                     */
    int32_t n_steps;    /* tokens to run in this launch (>= 1)                                 */
    int32_t n_forced;   /* first n_forced steps take their input id from `forced` (prompt feeding);
                           lm_head + argmax run only from step n_forced-1 on                   */
    float eps;          /* RMSNorm epsilon                                                     */
    int32_t write_logits; /* non-zero: store bf16 logits of the last step that ran the head    */
    int32_t flags;      /* ITTAI_F_* bits                                                      */
    int32_t spin_limit; /* polls before a device wait gives up; 0 = library default (about a second) */

    const void* wqkv;   /* [L, 4096, 1024] rows: q(2048) | k(1024) | v(1024)                   */
    const void* wo;     /* [L, 1024, 2048]                                                     */
    const void* wgu;    /* [L, 6144, 1024] gate row i at 2i, up row i at 2i+1 (engine.py:110-111) */
    const void* wd;     /* [L, 1024, 3072]                                                     */
    const void* ln1;    /* [L, 1024] input_layernorm gain                                      */
    const void* ln2;    /* [L, 1024] post_attention_layernorm gain                             */
    const void* qn;     /* [L, 128] q_norm gain                                                */
    const void* kn;     /* [L, 128] k_norm gain                                                */
    const void* fin_w;  /* [1024] final norm gain                                              */
    const void* embed;  /* [V, 1024] embedding table = tied lm_head                            */
    const void* rope;   /* [kv_cap, 128] bf16: cos[0..63] | sin[0..63] per position            */

    void* kcache;       /* [L, B, 8, kv_cap, 128] bf16                                         */
    void* vcache;       /* [L, B, 8, kv_cap, 128] bf16                                         */
    int32_t* pos;       /* [B] tokens already in each sequence's cache; advanced by n_steps    */
    int32_t* next_id;   /* [B] input id of the first free-running step; holds the last argmax after the launch */
    const int32_t* forced; /* [n_forced, B] or NULL                                            */
    int32_t* out_ids;   /* [n_steps, B] argmax of each step (-1 where the head did not run)    */
    void* logits;       /* [B, V] bf16 (may be NULL when write_logits == 0)                    */

    void* workspace;    /* ittai_qwen3_decode_workspace_bytes() bytes, 256-byte aligned        */
    uint32_t* status;   /* [ITTAI_STATUS_WORDS] device words, zeroed by the launch             */
    uint64_t* step_ns;  /* [n_steps] device: globaltimer at the end of each step, or NULL      */
    uint64_t* phase_clk; /* [n_steps, 5*L+1, 2] device, or NULL: CTA 0's SM cycle counter when each phase had
                            its inputs and when it finished (in-kernel profile)                  */
} IttaiQwen3Decode;

/* ---- library ------------------------------------------------------------------------------------ */

/* ABI version of the loaded library (ITTAI_ABI_VERSION). */
int ittai_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* ittai_last_error(void);

/* Checks that `device` is an sm_100 part able to run the persistent grid; fills *n_sms (may be NULL).
 * Replaces the capability probe of reference src/ittai/qwen3/model.py:22-24. */
int ittai_device_check(int device, int* n_sms);

/* Turns a host copy of the device status words into text.  Returns 0 when status[0]==0,
 * ITTAI_E_STATUS otherwise.  The reference has no counterpart: its device waits are unbounded
 * (src/ittai/qwen3/base.py:53-57). */
int ittai_decode_status(const uint32_t* status_host, char* msg, size_t msg_len);

/* ---- Qwen3 decode ------------------------------------------------------------------------------- */

/* Scratch bytes the decode kernels need for `batch` (1, 2, 4 or 8) sequences (activations, split-K partials, argmax
 * candidates, barrier and arrival counters).  Replaces the buffer plan of engine.py:123-134. */
int ittai_qwen3_decode_workspace_bytes(int batch, size_t* bytes);

/* One persistent cooperative launch that runs p->n_steps tokens: per layer RMSNorm+QKV, QK-norm+RoPE+
 * KV append + split-K GQA attention, O-proj+residual, gate/up SwiGLU, down+residual, then final norm +
 * tied lm_head + argmax, with the chosen id fed back on the device.  Replaces the launch of
 * engine.py:153-155 (`_graph_body`) for the decode loop the reference does not have.  One CTA per SM; a device with
 * fewer than 128 SMs is refused with ITTAI_E_DEVICE (the per-CTA weight slices are sized for a B200's 148). */
int ittai_qwen3_decode_launch(const IttaiQwen3Decode* p, void* stream);

/* The same launch for callers that cannot allocate device memory at call time (a process whose GPU memory was all handed
 * to a pool at start-up, a host runtime without a device allocator, a loop that cannot afford cudaMalloc's device-wide
 * synchronisation).  p->workspace is ignored: the scratch is a static device array inside the library, at most
 * ITTAI_STATIC_DECODE_MAX_BATCH sequences (about 2.3 MB, held by every GPU that loads the library until the process
 * exits); a larger p->batch is rejected with ITTAI_E_ARG.  The call itself allocates nothing (no cudaMalloc / cudaFree,
 * no allocating library routine).  Its first call on a device looks up the array's device address
 * (cudaGetSymbolAddress): make that first call outside any stream capture.  All calls share the one array and it keeps
 * the previous call's contents; the launch clears the words that must start at zero, and two calls whose kernels overlap
 * on the GPU (different streams, or different threads) race on it.  Two host threads may make their first call on one
 * device at the same time: both look the address up and store the same value.  No counterpart in the reference. */
#define ITTAI_STATIC_DECODE_MAX_BATCH 2
int ittai_qwen3_decode_launch_static(const IttaiQwen3Decode* p, void* stream);

/* Runs ONE phase (ITTAI_PH_*) of layer `layer` as its own kernel with the same grid and the same device
 * code as the persistent kernel, for unit parity tests and per-phase profiling.  `pos`/`next_id` are
 * read, not advanced. */
int ittai_qwen3_phase_launch(const IttaiQwen3Decode* p, int phase, int layer, void* stream);

/* ---- dense bf16 GEMM on tcgen05 / TMEM (Qwen3 prefill, SigLIP encoder) ------------------------------- */

/* Fused epilogues, the ones the reference's GEMM epilogues apply (src/ittai/qwen3/base.py:110-129,
 * src/ittai/siglip/kernel.py:266-333).  Bias and residual are independent of `epi`: they apply when non-NULL. */
enum {
    ITTAI_EPI_NONE = 0,   /* out = bf16(acc [+ bias]) [then + residual, rounded again]                  */
    ITTAI_EPI_GELU = 1,   /* out = bf16(gelu_tanh(bf16(acc + bias)))                                      */
    ITTAI_EPI_SWIGLU = 2, /* columns (2i, 2i+1) = (gate, up): out[:, i] = bf16(bf16(silu(gate)) * up); N/2 columns */
    ITTAI_EPI_QKROPE = 3  /* Qwen3 QKV projection (N = 4096 = 16 q | 8 k | 8 v heads of 128, M > 128, no bias / residual):
                             the work of ittai_qwen3_qk_rope_scatter inside the epilogue.  q heads: RMSNorm + RoPE, stored
                             to `out`; k heads: RMSNorm + RoPE, stored to the cache row of the token; v heads: copied to
                             the cache row.  The k and v columns of `out` are not written.  Needs IttaiGemm.qk_rope.
                             (reference: the qkv epilogue, src/ittai/qwen3/base.py:84-109) */
};

/* Arguments of ITTAI_EPI_QKROPE: the same arrays ittai_qwen3_qk_rope_scatter takes (all device pointers). */
typedef struct IttaiQkRope {
    const void* qn;        /* [128] bf16 q_norm gain of this layer */
    const void* kn;        /* [128] bf16 k_norm gain */
    const void* rope;      /* [positions][128] bf16: cos[0..63] | sin[0..63] */
    const int32_t* pos;    /* [M] rotary position of each token */
    const int32_t* seq;    /* [M] cache sequence of each token */
    const int32_t* slot;   /* [M] cache row of each token */
    void* kcache_layer;    /* [B, 8, kv_cap, 128] bf16 */
    void* vcache_layer;
    int32_t kv_cap;
    float eps;
} IttaiQkRope;

/* out[M, N] = a[M, K] * w[N, K]^T with fp32 accumulation.  a, w, residual, out are bf16 row-major; bias is fp32.
 * N must be a multiple of 256 and K of 64; leading dimensions of 0 mean "dense".  `status` must be zeroed by the
 * caller before a sequence of launches and decoded afterwards. */
typedef struct IttaiGemm {
    int32_t m, n, k, epi;
    int32_t ld_a, ld_w, ld_out, ld_res;
    const void* a;
    const void* w;
    const void* bias;      /* [N] fp32 or NULL */
    const void* residual;  /* [M, ld_res] bf16 or NULL */
    void* out;
    uint32_t* status;      /* [ITTAI_STATUS_WORDS] device words */
    /* LayerNorm folded into the GEMM (both NULL: off; M > 128 only).  With W' = gain (.) W along K, col_sums[n] = sum_k W'[n,k]
     * and bias' = bias + W beta, LayerNorm(x) W^T + bias = rstd_r (x W'^T - mean_r col_sums) + bias': the kernel reads the
     * un-normalised x as A and applies the row statistics in the epilogue, as the reference does
     * (src/ittai/siglip/kernel.py:284-288, 523-525).  The caller passes W' as `w`, bias' as `bias`. */
    const float* row_stats; /* stats_parts == 0: [M][2] fp32 mean, rstd of each row of A (ittai_row_stats);
                               stats_parts > 0: [M][stats_parts][2] partial (sum, sum of squares) over slices of the K columns,
                               as another GEMM's stats_out wrote them; mean and rstd are finished in the epilogue */
    const float* col_sums;  /* [N] fp32 */
    float* stats_out;       /* or NULL (M > 128, no SwiGLU): [M][N/128][2] fp32, (sum, sum of squares) of every 128-column
                               slice of each OUTPUT row, of the bf16 values as stored: the statistics of a LayerNorm over
                               this GEMM's output come for free with its epilogue (the reference finishes them in the last
                               arriving tile, src/ittai/siglip/kernel.py:335-364); plain stores, no atomics */
    int32_t stats_parts;
    float stats_eps;        /* LayerNorm epsilon, used when stats_parts > 0 */
    int32_t stats_k;        /* stats_parts > 0: the number of columns of A the statistics are over, when A is zero-padded
                               beyond its true width (the zero columns add nothing to the sums); 0 = k */
    int32_t stats_rms;      /* stats_parts > 0: 1 = the folded norm is an RMSNorm: mean = 0, rstd = 1 / sqrt(sum x^2 / k + eps)
                               (col_sums is not used and may hold zeros); the reference's Qwen3 kernels finish their norms
                               this way (src/ittai/qwen3/base.py:59-78, 84-109).  Allowed with ITTAI_EPI_QKROPE. */
    const IttaiQkRope* qk_rope; /* host pointer, read during the call; required by ITTAI_EPI_QKROPE, NULL otherwise */
} IttaiGemm;

/* Replaces the tiled GEMM main loops + epilogues of the reference's megakernels
 * (src/ittai/qwen3/sm80.py:175-272, src/ittai/qwen3/sm90.py:256-316, src/ittai/siglip/kernel.py:197-333). */
int ittai_gemm_bf16_launch(const IttaiGemm* g, void* stream);

/* A chain of 1 to 4 GEMMs in ONE persistent launch: gemms[i + 1].a must be gemms[i].out (k = the previous n), every GEMM
 * has the same M > 128, epilogues ITTAI_EPI_NONE / ITTAI_EPI_GELU with bias, residual (also in place), a folded LayerNorm
 * and stats_out as in ittai_gemm_bf16_launch; the results are bit-identical to the same GEMMs launched one by one.  The tiles
 * of all GEMMs form one task list dealt round-robin to the resident clusters; a tile of GEMM i + 1 waits on a counter per
 * 128-row block that the tiles of GEMM i bump when their stores are complete, so the next GEMM starts on a row block as
 * soon as that block exists instead of after the slowest tile of the whole GEMM.  `flags`: n * 2 * ceil(M / 256) device
 * words that are ZERO at launch (the caller clears them, e.g. once per forward for all its chains).  This is the
 * reference's device task queue with per-row-block dependency counters (src/ittai/siglip/kernel.py:197-333,
 * src/ittai/qwen3/engine.py:17-84) restricted to runs of consecutive GEMMs. */
int ittai_gemm_chain_launch(const IttaiGemm* gemms, int32_t n, uint32_t* flags, void* stream);

/* ---- softmax attention for the prefill and SigLIP paths ------------------------------------------------- */

/* Flash-style attention over `n_seqs` independent sequences.  Row r of sequence s lives at
 *   q + (seqs[s].q_row0 + r) * q_row + head * q_head           (same for o)
 *   k + s * k_seq + (head / group) * k_head + (seqs[s].kv_row0 + j) * k_row   (same for v)
 * all strides in elements, multiples of 8.  causal != 0: query r sees keys j <= r + (kv_len - q_len).
 * Replaces the attention tasks of src/ittai/qwen3/sm80.py:274-403 and src/ittai/siglip/kernel.py:366-500. */
typedef struct IttaiAttention {
    const void* q; const void* k; const void* v; void* o;          /* bf16 */
    int64_t q_row, q_head, k_row, k_head, k_seq, v_row, v_head, v_seq, o_row, o_head;
    const int32_t* seqs;   /* [n_seqs][4] device: first q row, q rows, first k/v row, k/v rows */
    int32_t n_seqs, n_heads, group, head_dim, causal, max_q_len;
    int32_t max_kv_len;    /* largest kv_rows over the sequences, or 0 if unknown (enables the short-sequence kernel) */
    /* The tensor-memory kernels address q, k and v through TMA tensor maps and need the row counts of the matrices they
     * point into, plus status words for their bounded waits; leave the three at 0/NULL to stay on the register-tile
     * kernels.  Covered: head_dim 64, dense, 65..256 queries and at most 256 keys per sequence, heads adjacent in a row
     * (q_head = k_head = v_head = 64, k_seq = v_seq = 0); and head_dim 128 with a key loop, causal or dense, q_head = 128,
     * more than 64 queries in some sequence, keys and values either as dense rows (k_row = v_row = 128, head and sequence
     * strides multiples of 128, equal for k and v: the cache layout) or packed like the queries (k_head = v_head = 128,
     * k_seq = v_seq = 0, k_row = v_row > 128: the heads of a token side by side in one row). */
    int32_t q_rows_total;  /* rows of the matrix behind q (every sequence's q_row0 + q rows lies inside) */
    int32_t kv_rows_total; /* rows of the matrices behind k and v */
    int32_t reserved0;
    uint32_t* status;      /* [ITTAI_STATUS_WORDS] device words, or NULL */
} IttaiAttention;
int ittai_attention_launch(const IttaiAttention* a, void* stream);

/* ---- row-wise passes around the GEMMs ------------------------------------------------------------------- */

/* y = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * gain) over rows of 1024 bf16 (Qwen3 RMSNorm; the reference folds the gain
 * into the next weight and applies the scale in the GEMM epilogue: src/ittai/qwen3/engine.py:106-111, base.py:84-85). */
int ittai_rmsnorm_rows(const void* x, int ld_x, const void* gain, void* y, int ld_y, int rows, float eps, void* stream);
/* stats[r] = (mean, 1/sqrt(var + eps)) of row r over `width` bf16 columns (a multiple of 8, at most 2048): the row
 * statistics a GEMM with a folded LayerNorm applies in its epilogue (reference src/ittai/siglip/kernel.py:335-364). */
int ittai_row_stats(const void* x, int ld_x, float* stats, int rows, int width, float eps, void* stream);
/* y = bf16(LayerNorm(x) * gain + beta), gain/beta fp32, width a multiple of 8 up to 2048 (SigLIP; folded into the next
 * GEMM by the reference: src/ittai/siglip/kernel.py:284-288,523-525). */
int ittai_layernorm_rows(const void* x, int ld_x, const void* gain, const void* beta, void* y, int ld_y, int rows, int width,
                         float eps, void* stream);
/* Qwen3 prefill: per-head RMSNorm + RoPE (position pos[t]) of q (in place in qkv[T, 4096]) and k, and the scatter of k
 * and v into one layer of the cache ([B, 8, kv_cap, 128]) at row slot[t] of sequence seq[t].  The reference's qkv
 * epilogue: src/ittai/qwen3/base.py:84-109. */
int ittai_qwen3_qk_rope_scatter(void* qkv, const void* qn, const void* kn, const void* rope, const int32_t* pos,
                                const int32_t* seq, const int32_t* slot, void* kcache_layer, void* vcache_layer,
                                int n_tokens, int kv_cap, float eps, void* stream);
/* fp32 pixels [B, 3, H, W] -> bf16 patch rows [B * (H/p) * (W/p)][ld_out]: the first 3 p p columns of a row, in (channel,
 * row, col) order (the torch unfold of src/ittai/siglip/kernel.py:633-637); ld_out = 0 means dense rows, a larger ld_out
 * leaves the columns beyond untouched (zero-padded K).  Even patch sizes and widths; H/p and W/p round down, the pixels
 * beyond the last whole patch are dropped (a stride-p convolution without padding). */
int ittai_siglip_im2col(const float* pixels, void* patches, int batch, int height, int width, int patch, int ld_out, void* stream);
/* out[t, :] = table[ids[t], :], rows of 1024 bf16 (src/ittai/qwen3/base.py:147-162). */
int ittai_embed_rows(const int32_t* ids, const void* table, void* out, int rows, int vocab, void* stream);
/* Embedding head: out[s] = l2_normalise(rmsnorm(h[rows[s]]) * gain) in fp32 (src/ittai/qwen3/base.py:131-145). */
int ittai_qwen3_final_pool(const void* h, const int32_t* rows, const void* gain, float* out, int n_seq, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ITTAI_B200_H */
