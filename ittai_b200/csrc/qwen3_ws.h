// Layout of the Qwen3 decode workspace, carved up on the host (size query, memset at launch); the resulting pointer
// set travels to the kernels as a launch parameter.
//
// Every buffer that one CTA writes and another reads inside a launch is in "flagged word" format: 64-bit words whose
// low half carries the payload (two bf16 values, one fp32 or one int32) and whose high half carries a tag that
// names the producing (step, layer).  A 64-bit store is single-copy atomic, so a consumer that polls a word until the
// tag matches has the payload too: one L2 round trip per dependency, no fence, no counter, no grid barrier.
// The launch zeroes the whole region; tags start at 1.
#pragma once
#include <cuda_bf16.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/ittai_b200.h"

namespace ittai {

constexpr int Q3_MAX_CTAS = 1024;        // upper bound on the persistent grid (partials and argmax candidates are per CTA)
constexpr int Q3_MAX_SPLITS = 32;        // cache splits per (sequence, kv head)
constexpr int Q3_PART_WORDS = 4 + 2 * ITTAI_Q3_HD;   // m[2], l[2], o[2][128] of one split
constexpr int Q3_SYNC_WORDS = 64;        // [1] abort flag; the rest is spare

struct Q3Workspace {
    uint32_t* sync;
    uint64_t* h;        // [B, 512]  residual stream entering a layer (bf16 pairs)
    uint64_t* qkv;      // [B, 1024] 128-bit words: raw q|k|v projections of the current token, four bf16 per word
    uint64_t* attn;     // [B, 512] 128-bit words: attention output, four bf16 per word
    uint64_t* hmid;     // [B, 512]  residual stream after o_proj
    uint64_t* act;      // [B, 512] 128-bit words: SwiGLU output, six bf16 per word (the region keeps its 64-bit-word size)
    uint64_t* part;     // [Q3_MAX_CTAS, Q3_PART_WORDS] split-K partials (fp32 payloads)
    uint64_t* cand_val; // [Q3_MAX_CTAS, ITTAI_MAX_BATCH] per-CTA best logit (fp32 payload)
    uint64_t* cand_idx; // [Q3_MAX_CTAS, ITTAI_MAX_BATCH] its index
    size_t flagged_bytes;   // bytes from `h` to the end: zeroed at every launch
};

// Host only.
inline size_t q3_ws_layout(int batch, char* base, Q3Workspace* ws) {
    size_t off = 0;
    const size_t sizes[9] = {Q3_SYNC_WORDS * sizeof(uint32_t),
                             (size_t)batch * (ITTAI_Q3_D / 2) * 8,
                             (size_t)batch * (ITTAI_Q3_DQKV / 2) * 8,
                             (size_t)batch * (ITTAI_Q3_DQ / 2) * 8,
                             (size_t)batch * (ITTAI_Q3_D / 2) * 8,
                             (size_t)batch * (ITTAI_Q3_FF / 2) * 8,
                             (size_t)Q3_MAX_CTAS * Q3_PART_WORDS * 8,
                             (size_t)Q3_MAX_CTAS * ITTAI_MAX_BATCH * 8,
                             (size_t)Q3_MAX_CTAS * ITTAI_MAX_BATCH * 8};
    char* ptr[9];
    for (int i = 0; i < 9; ++i) {
        ptr[i] = base + off;
        off += (sizes[i] + 255) / 256 * 256;
    }
    ws->sync = reinterpret_cast<uint32_t*>(ptr[0]);
    ws->h = reinterpret_cast<uint64_t*>(ptr[1]);
    ws->qkv = reinterpret_cast<uint64_t*>(ptr[2]);
    ws->attn = reinterpret_cast<uint64_t*>(ptr[3]);
    ws->hmid = reinterpret_cast<uint64_t*>(ptr[4]);
    ws->act = reinterpret_cast<uint64_t*>(ptr[5]);
    ws->part = reinterpret_cast<uint64_t*>(ptr[6]);
    ws->cand_val = reinterpret_cast<uint64_t*>(ptr[7]);
    ws->cand_idx = reinterpret_cast<uint64_t*>(ptr[8]);
    ws->flagged_bytes = off - (size_t)(ptr[1] - base);
    return off;
}

}  // namespace ittai
