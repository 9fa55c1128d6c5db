// Layout of the Qwen3 decode workspace: carved up on the host (size query, memset of the
// synchronisation words); the resulting pointer set travels to the kernels as a launch parameter.
#pragma once
#include <cuda_bf16.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/ittai_b200.h"

namespace ittai {

constexpr int Q3_MAX_CTAS = 1024;        // upper bound on the persistent grid (partials and argmax candidates are per CTA)
constexpr int Q3_MAX_SPLITS = 32;        // cache splits per (sequence, kv head)
constexpr int Q3_PART_FLOATS = 4 + 2 * ITTAI_Q3_HD;   // m[2], l[2], o[2][128] of one split
constexpr int Q3_SYNC_WORDS = 128;       // [0] barrier arrivals, [1] abort, [2] lm_head arrivals, [16..80) per-(b,g) split arrivals
constexpr int Q3_SYNC_HEADARRIVE = 2;
constexpr int Q3_SYNC_HEADCNT = 16;

struct Q3Workspace {
    uint32_t* sync;
    __nv_bfloat16* h;      // [B, 1024] residual stream
    __nv_bfloat16* qkv;    // [B, 4096] raw projections of the current token
    __nv_bfloat16* attn;   // [B, 2048]
    __nv_bfloat16* act;    // [B, 3072]
    float* part;           // [Q3_MAX_CTAS, Q3_PART_FLOATS]
    float* cand_val;       // [Q3_MAX_CTAS, ITTAI_MAX_BATCH]
    int* cand_idx;         // [Q3_MAX_CTAS, ITTAI_MAX_BATCH]
};

// Host only: the kernels receive the finished pointer set as a launch parameter.
inline size_t q3_ws_layout(int batch, char* base, Q3Workspace* ws) {
    size_t off = 0;
    const size_t sizes[8] = {Q3_SYNC_WORDS * sizeof(uint32_t),
                             (size_t)batch * ITTAI_Q3_D * 2,
                             (size_t)batch * ITTAI_Q3_DQKV * 2,
                             (size_t)batch * ITTAI_Q3_DQ * 2,
                             (size_t)batch * ITTAI_Q3_FF * 2,
                             (size_t)Q3_MAX_CTAS * Q3_PART_FLOATS * sizeof(float),
                             (size_t)Q3_MAX_CTAS * ITTAI_MAX_BATCH * sizeof(float),
                             (size_t)Q3_MAX_CTAS * ITTAI_MAX_BATCH * sizeof(int)};
    char* ptr[8];
    for (int i = 0; i < 8; ++i) {
        ptr[i] = base + off;
        off += (sizes[i] + 255) / 256 * 256;
    }
    ws->sync = reinterpret_cast<uint32_t*>(ptr[0]);
    ws->h = reinterpret_cast<__nv_bfloat16*>(ptr[1]);
    ws->qkv = reinterpret_cast<__nv_bfloat16*>(ptr[2]);
    ws->attn = reinterpret_cast<__nv_bfloat16*>(ptr[3]);
    ws->act = reinterpret_cast<__nv_bfloat16*>(ptr[4]);
    ws->part = reinterpret_cast<float*>(ptr[5]);
    ws->cand_val = reinterpret_cast<float*>(ptr[6]);
    ws->cand_idx = reinterpret_cast<int*>(ptr[7]);
    return off;
}

}  // namespace ittai
