// Layout of the Qwen3 decode workspace, carved up on the host (size query, memset at launch); the resulting pointer
// set travels to the kernels as a launch parameter.
//
// Everything one CTA hands to another inside a launch travels as 128-bit "mail" words: up to 112 bits of payload
// (seven bf16 values, or three fp32 values) and, in the top 16 bits, a tag that names the producing (step, layer).
// A 128-bit store is single-copy atomic, so a consumer that polls a word until the tag matches has the payload too:
// one L2 round trip per dependency, no fence, no counter, no grid barrier.
//
// Every consumer CTA has a mailbox of its own for each kind of vector, and a producer writes its few words into the
// mailbox of every CTA that needs them.  The first version of this kernel kept one shared copy of each vector that all
// 148 CTAs polled: the 75 000 polls of one hand-off then queue up on the two or three dozen L2 lines of that copy, and a
// synchronised all-to-all hand-off took 2.9 us against 1.6 us with private mailboxes (measured on a B200 with a
// stand-alone exchange loop).  The launch zeroes the whole region; tags are never zero.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/ittai_b200.h"

namespace ittai {

constexpr int Q3_MAX_CTAS = 148;         // persistent grid: one CTA per SM of a B200
constexpr int Q3_MIN_CTAS = 147;         // fewer CTAs would need more words per producer than the mailboxes hold
constexpr int Q3_MAIL_STRIDE = 152;      // producer slots per mailbox row, padded so that rows start on a 128-byte line
constexpr int Q3_MAX_SPLITS = 32;        // cache splits per (sequence, kv head)
constexpr int Q3_ROW_WORDS = 1;          // words per producer of the residual stream (6-7 of 1024 values each)
constexpr int Q3_ACT_WORDS = 3;          // words per producer of the SwiGLU output (20-21 of 3072 values each)
constexpr int Q3_ATTN_WORDS = 48;        // words per (sequence, kv head) of the attention output (256 values)
constexpr int Q3_QKV_WORDS = 128;        // words per attention CTA: q head 0 | q head 1 | k | v, four values per word
constexpr int Q3_PART_WORDS = 256;       // words per merging CTA: [split][words of one split's message]
constexpr int Q3_SYNC_WORDS = 64;        // [1] abort flag; the rest is spare

struct Q3Workspace {
    uint32_t* sync;
    uint4* mail_h;      // [cta][B][MAIL_STRIDE]            residual stream entering a layer, one word per producer
    uint4* mail_hmid;   // [cta][B][MAIL_STRIDE]            residual stream after o_proj
    uint4* mail_act;    // [cta][B][MAIL_STRIDE][ACT_WORDS] SwiGLU output
    uint4* mail_attn;   // [cta][B][8][ATTN_WORDS]          attention output, by (kv head, merging CTA, word)
    uint4* mail_qkv;    // [cta][QKV_WORDS]                 projections of the kv head the CTA's attention item belongs to
    uint4* mail_part;   // [cta][PART_WORDS]                split-K partials sent to the CTA that merges them (fp32)
    uint4* mail_cand;   // [cta][B][MAIL_STRIDE]            per-CTA argmax candidates (value, index)
    size_t mail_bytes;  // bytes from `mail_h` to the end: zeroed at every launch
};

constexpr int Q3_N_REGIONS = 8;
// Host only.  With `base` == nullptr only the size is meaningful.
inline size_t q3_ws_layout(int batch, char* base, Q3Workspace* ws, size_t* offsets = nullptr) {
    const size_t B = (size_t)batch, C = Q3_MAX_CTAS, W = 16;
    const size_t sizes[Q3_N_REGIONS] = {Q3_SYNC_WORDS * sizeof(uint32_t),
                                        C * B * Q3_MAIL_STRIDE * Q3_ROW_WORDS * W,
                                        C * B * Q3_MAIL_STRIDE * Q3_ROW_WORDS * W,
                                        C * B * Q3_MAIL_STRIDE * Q3_ACT_WORDS * W,
                                        C * B * ITTAI_Q3_NKV * Q3_ATTN_WORDS * W,
                                        C * Q3_QKV_WORDS * W,
                                        C * Q3_PART_WORDS * W,
                                        C * B * Q3_MAIL_STRIDE * W};
    size_t off = 0, offs[Q3_N_REGIONS];
    for (int i = 0; i < Q3_N_REGIONS; ++i) {
        offs[i] = off;
        off += (sizes[i] + 255) / 256 * 256;
        if (offsets) offsets[i] = offs[i];
    }
    ws->sync = reinterpret_cast<uint32_t*>(base + offs[0]);
    ws->mail_h = reinterpret_cast<uint4*>(base + offs[1]);
    ws->mail_hmid = reinterpret_cast<uint4*>(base + offs[2]);
    ws->mail_act = reinterpret_cast<uint4*>(base + offs[3]);
    ws->mail_attn = reinterpret_cast<uint4*>(base + offs[4]);
    ws->mail_qkv = reinterpret_cast<uint4*>(base + offs[5]);
    ws->mail_part = reinterpret_cast<uint4*>(base + offs[6]);
    ws->mail_cand = reinterpret_cast<uint4*>(base + offs[7]);
    ws->mail_bytes = off - offs[1];
    return off;
}

// Bytes of q3_ws_layout(batch) as a constant expression (the same sum), for the built-in scratch array.
constexpr size_t q3_ws_bytes(int batch) {
    const size_t B = (size_t)batch, C = Q3_MAX_CTAS, W = 16;
    const size_t sizes[Q3_N_REGIONS] = {Q3_SYNC_WORDS * sizeof(uint32_t),
                                        C * B * Q3_MAIL_STRIDE * Q3_ROW_WORDS * W,
                                        C * B * Q3_MAIL_STRIDE * Q3_ROW_WORDS * W,
                                        C * B * Q3_MAIL_STRIDE * Q3_ACT_WORDS * W,
                                        C * B * ITTAI_Q3_NKV * Q3_ATTN_WORDS * W,
                                        C * Q3_QKV_WORDS * W,
                                        C * Q3_PART_WORDS * W,
                                        C * B * Q3_MAIL_STRIDE * W};
    size_t off = 0;
    for (int i = 0; i < Q3_N_REGIONS; ++i) off += (sizes[i] + 255) / 256 * 256;
    return off;
}

// Cache splits per (sequence, kv head), CTAs that merge them, and the message sizes that follow; shared by the kernel,
// the launch checks and (through ittai_qwen3_decode_layout) the tests.
__host__ __device__ inline int q3_attn_splits(int ncta, int batch) {
    int s = ncta / (batch * ITTAI_Q3_NKV);
    return s < 1 ? 1 : (s > Q3_MAX_SPLITS ? Q3_MAX_SPLITS : s);
}
__host__ __device__ inline int q3_merge_ctas(int n_splits) {
    int nc = 1;
    while (nc * 2 <= n_splits && nc < 16) nc *= 2;
    return nc;
}
// Words a merging CTA sends for its 2 * (128 / nc) outputs (seven bf16 per word).
__host__ __device__ inline int q3_attn_words_per_owner(int nc) { return (2 * (ITTAI_Q3_HD / nc) + 6) / 7; }
// Words of one split's message to one merging CTA: m[2], l[2], o[2][128 / nc] as fp32, three per word.
__host__ __device__ inline int q3_part_words_per_msg(int nc) { return (4 + 2 * (ITTAI_Q3_HD / nc) + 2) / 3; }

}  // namespace ittai
