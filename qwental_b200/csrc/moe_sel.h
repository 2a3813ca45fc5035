// Selection record shared by the MoE kernels and the fused combine + norm kernel.
#pragma once
#include <stdint.h>

#define MOE_MAXB 64
#define MOE_MAXK 16
#define MOE_MAXE 1024

// Result of the selection, read by the gate/up, down and combine kernels (role of struct gg_sel,
// kernels/moe_gg.metal:110-116).  Groups are in expert-id order; a group's entries are in token order.
struct moe_sel {
    uint32_t U;                               // groups (distinct experts in [e_lo, e_hi) that were chosen)
    uint32_t nb, topk, pad;
    int32_t ids[MOE_MAXB][MOE_MAXK];          // chosen experts per token, rank order
    float w[MOE_MAXB][MOE_MAXK + 1];          // routed weights, then the shared gate at [topk]
    uint32_t ue[MOE_MAXE];                    // expert of group u
    uint32_t off[MOE_MAXE + 1];               // entries of group u: ent[off[u] .. off[u+1])
    uint16_t ent[MOE_MAXB * MOE_MAXK];        // token << 8 | rank
    uint32_t pre[MOE_MAXE + 2];               // passes of 8 entries in the groups before u (pre[U] = all routed passes)
};


// Scratch buffer of the fused expert-FFN kernel (k_ffn.cu): the items' counters and the finished-block counter in the first
// MOE_FFN_SYNC_BYTES (all zero between launches: the owner zeroes the buffer once), then H [item][2 planes][8 columns][I] fp16.
// An item is one pass of up to 8 tokens of one chosen expert or of the shared expert: at most 512 experts + the extra passes
// of 64 tokens x 10 choices + the shared expert's 8.
#define MOE_FFN_MAXITEMS 640
#define MOE_FFN_SYNC_BYTES 8192
// word MOE_FFN_ROWCNT + tok * (topk + 1) + rank of the same area counts the reader warps that have stored their part of output row
// (tok, rank) of Pg: 8 per tile of 128 output rows, MOE_FFN_ROW_DONE(D) when the row is complete.  The combine + norm kernel that
// follows waits on the rows of its token instead of on the whole launch, and clears them (one GPU only).
#define MOE_FFN_ROWCNT 1024
#define MOE_FFN_ROW_DONE(D) ((D) / 128 * 8)
#define MOE_FFN_SCRATCH_BYTES(I) ((size_t)MOE_FFN_SYNC_BYTES + (size_t)MOE_FFN_MAXITEMS * 16 * (I) * 2)
