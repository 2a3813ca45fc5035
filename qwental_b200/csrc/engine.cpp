// Host engine of the batched decode step: the "par" interface of the reference's engine
// (src/engine.h:77-127; implementation src/engine.c:8084-9045) written against the device interface only
// (qw_gpu.h: kernels by name, buffers and bytes bound by index, one batch and one wait per step), the way
// src/engine.c encodes its steps (par_step8, src/engine.c:8868-9045).
//
// Differences by design:
//   - one weight pass for up to 64 slots (the reference splits into groups of <= 8, src/engine.c:8783-8814);
//   - per-slot kernels (attention core, GDN recurrence, conv state) take the slot as a grid dimension and find
//     the slot's state through tables in device memory, so a step is ~12 dispatches per layer for any batch
//     (the reference issues 3 more per slot, src/engine.c:8948-8959, 8992-9007);
//   - KV lives in 256-token pages drawn from one pool; a slot owns a page list;
//   - the step's control data (token, slot id, position per row) is read once from pinned host memory and kept
//     in device memory, so consecutive greedy steps can run with no host round trip and identical steps replay
//     as CUDA graphs.
#include "../../include/qw_engine.h"
#include "../../include/qw_gpu_ext.h"
#include "moe_sel.h"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

extern "C" size_t qw_moe_sel_bytes(void);

namespace {

constexpr int PAGE = 256;
std::string g_open_error;

struct Slot {
    bool used = false;
    int pos = 0;  // tokens in the context
    std::vector<int> pages;
    unsigned long long last_use = 0;
};

struct LayerW {
    bool attn;
    size_t w_in, w_out;          // offsets into `dense`
    uint32_t n_in;               // rows of the input projection
    size_t small;                // offset into `small` (fp32 vectors)
    int idx;                     // index among layers of its kind (attention layer number / GDN layer number)
};

struct fill_args {
    uint64_t seed, count, base;
    uint32_t mode;
    float p0, p1;
};

uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// per-tensor seed = hash(master, "<layer>/<name>") -- the same function as qwental_b200/synth.py:tensor_seed
uint64_t tensor_seed(uint64_t master, int layer, const char *name) {
    char buf[128];
    snprintf(buf, sizeof buf, "%d/%s", layer, name);
    uint64_t h = master;
    for (const char *p = buf; *p; p++) h = mix64(h ^ (uint64_t)(unsigned char)*p);
    return h;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct qw_engine {
    qw_gpu *g = nullptr;
    qw_model_cfg c;
    std::string err;
    // derived shapes
    int D, L, V, E, EL, e_lo, TOPK, I, QH, KVH, HD, HK, HV, C, n_attn, n_gdn, max_pages;
    uint32_t rbD, rbI, rbKA, rbKG, rbV, qkv_rows, gdn_rows, KA, KG;  // KA / KG: inputs of the attention / GDN output projections
    std::vector<LayerW> layers;
    // weights
    qw_buf emb{}, lm_head{}, dense{}, small{}, router{}, exg{}, exu{}, exd{}, shg{}, shu{}, shd{};
    size_t small_stride = 0, final_norm = 0;
    // state
    qw_buf kvpool{}, ptab{}, sstate{}, cstate{};
    std::vector<Slot> slots;
    std::vector<int> free_pages;
    unsigned long long clock = 0;
    // scratch
    qw_buf ctl_h{}, ctl_d{}, h{}, x{}, proj{}, cv{}, la{}, be{}, gy{}, qb{}, part{}, ya{}, ob{}, mo{}, logits{}, ids{}, ids_h{}, logits_h{}, cand_h{};
    qw_buf mlog{}, msel{}, Hhi{}, Hlo{}, Pg{}, rcnt{};
    size_t sel_bytes = 0;
    // kernels
    qw_kernel *k_begin, *k_embed, *k_norm, *k_norm0, *k_norm_cmb, *k_route, *k_adv_feed, *k_qmv_in_a, *k_qmv_in_g, *k_qmv_o_a, *k_qmv_o_g, *k_lm, *k_prep, *k_attn, *k_merge, *k_epi, *k_gdn, *k_router, *k_select,
        *k_gu, *k_dn, *k_cmb, *k_argmax, *k_adv, *k_fill, *k_ar;
    bool ep_ready = false;
    // fused exchange: each rank's down projection stores its rows straight into every rank's Pg (peer memory)
    bool ep_fused = false;
    qw_buf epx{};            // [2][Pg] (double-buffered by layer parity) + flag array, exported to the other ranks
    qw_buf ep_peer[8]{};     // the other ranks' epx (ep_peer[own rank] aliases epx)
    qw_kernel *k_dn_x = nullptr, *k_norm_cmb_x = nullptr, *k_topk = nullptr;
    qw_kernel *k_norm_cmb_rc = nullptr;  // combine + norm that waits on moe_ffn's per-row counters instead of on its whole launch (one GPU)
    // gate/up + down of the expert FFN in one launch (moe_ffn), where the shapes allow it; QW_MOE_FFN=split keeps the two launches
    bool ffn_fused = false;
    // ... on expert weights re-coded once into the kernel's own stage order and bit layout (IQ3X, csrc/iq3x.cuh): lossless, 136
    // instead of 110 bytes per 256 weights; QW_MOE_FFN=fused keeps the fused kernel on the raw IQ3_S blocks
    bool ffn_iq3x = false;
    qw_buf xq_gu{}, xq_d{}, xs_gu{}, xs_d{};  // routed gate+up / down and the shared expert's, per layer
    qw_buf ffn_scr{};  // moe_ffn's scratch (moe_sel.h): per-item counters, zero between launches, and H
    size_t x_gus = 0, x_dns = 0;              // IQ3X bytes of one expert's gate+up / down
    qw_kernel *k_ffn = nullptr, *k_ffn_x = nullptr, *k_ffn_probe = nullptr, *k_pack = nullptr;
    bool moe_probe = false;  // measurement only: the copy-only twin of moe_ffn runs in its place (outputs are not produced)
    // slot sharding on top of the fused exchange: attention / GDN (their projections included) run only for the rows whose
    // slot this rank owns (slot % ep_size == ep_rank); the out-projection stores its rows into every rank's `ob` and publishes
    bool slot_shard = false;
    qw_kernel *k_qmv_o_a_x = nullptr, *k_qmv_o_g_x = nullptr, *k_norm_x = nullptr, *k_pub = nullptr;
    size_t ob_off = 0;            // offset of the gathered `ob` rows inside epx
    int perm[QW_PAR_MAX] = {};    // device row j = caller's row perm[j] (rows are ordered by owning rank)
    uint32_t row_lo = 0, row_hi = 0;  // this rank's rows of the current step
    std::vector<int32_t> ids_out;     // sampled ids in the caller's row order
    size_t pg_bytes = 0;
    // bookkeeping
    double cost[QW_PAR_MAX + 1];
    int lastB = 0;
    std::vector<int> last_sids;
    long long last_ctx = 0;
    int last_own = 0;  // rows of the last step whose token mixers ran on this rank

    bool fail(const char *fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        err = buf;
        if (g && *qw_gpu_last_error(g)) err += std::string(" [") + qw_gpu_last_error(g) + "]";
        return false;
    }
};

namespace {

bool compile(qw_engine *e, const char *family, const char *name, const std::vector<std::pair<const char *, long>> &defs, qw_kernel **out) {
    std::string src = std::string("#define QW_KERNEL ") + family + "\n#define QW_NAME " + name + "\n";
    for (auto &d : defs) src += std::string("#define ") + d.first + " " + std::to_string(d.second) + "\n";
    char msg[256];
    if (!qw_gpu_compile(e->g, src.c_str(), src.size(), msg, sizeof msg)) return e->fail("compile %s: %s", name, msg);
    *out = qw_kernel_get(e->g, name);
    return *out ? true : e->fail("kernel %s not found", name);
}

bool new_buf(qw_engine *e, qw_buf *b, size_t size, int kind = QW_BUF_DEVICE) {
    if (!qw_buf_new_kind(e->g, size, kind, b)) return e->fail("allocation of %zu bytes failed", size);
    return true;
}

void enc_fill(qw_engine *e, qw_batch *b, const qw_buf *dst, size_t off, const fill_args &a) {
    qw_batch_kernel(b, e->k_fill);
    qw_batch_buf(b, 0, dst, off);
    qw_batch_bytes(b, 1, &a, sizeof a);
    qw_batch_dispatch(b, 1, 1, 1, 256, 1, 1);
}

float d_scale_for(int K) { return K <= 512 ? 1.0f / 32 : K <= 2048 ? 1.0f / 64 : 1.0f / 128; }

bool init_weights(qw_engine *e) {
    const qw_model_cfg &c = e->c;
    const uint64_t ms = c.seed;
    qw_batch *b = qw_batch_begin(e->g, false);
    // embedding fp16 N(0,1), lm_head Q8_0 at the stated range
    enc_fill(e, b, &e->emb, 0, {tensor_seed(ms, -1, "token_embd"), (uint64_t)e->V * e->D, 0, 3, 1.0f, 0.f});
    enc_fill(e, b, &e->lm_head, 0, {tensor_seed(ms, -1, "output"), (uint64_t)e->V * e->rbV, 0, 2, 1.0f, 0.f});
    enc_fill(e, b, &e->small, e->final_norm * 4, {0, (uint64_t)e->D, 0, 5, 1.0f, 0.f});
    const size_t gu_bytes = (size_t)e->I * e->rbD, ex_bytes = (size_t)e->EL * gu_bytes;
    for (int l = 0; l < e->L; l++) {
        const LayerW &w = e->layers[l];
        const size_t sm = w.small * 4;
        enc_fill(e, b, &e->small, sm, {0, (uint64_t)2 * e->D, 0, 5, 1.0f, 0.f});  // the two block norms = 1
        if (w.attn) {
            enc_fill(e, b, &e->dense, w.w_in, {tensor_seed(ms, l, "attn_qkv"), (uint64_t)w.n_in * e->rbD, 0, 1, d_scale_for(e->D), 0.f});
            enc_fill(e, b, &e->dense, w.w_out, {tensor_seed(ms, l, "attn_output"), (uint64_t)e->D * e->rbKA, 0, 1, d_scale_for(e->KA), 0.f});
            enc_fill(e, b, &e->small, sm + 2 * e->D * 4, {0, 512, 0, 5, 1.0f, 0.f});  // q / k norm = 1
        } else {
            enc_fill(e, b, &e->dense, w.w_in, {tensor_seed(ms, l, "ssm_in"), (uint64_t)w.n_in * e->rbD, 0, 1, d_scale_for(e->D), 0.f});
            enc_fill(e, b, &e->dense, w.w_out, {tensor_seed(ms, l, "ssm_out"), (uint64_t)e->D * e->rbKG, 0, 1, d_scale_for(e->KG), 0.f});
            size_t o = sm + 2 * e->D * 4;
            enc_fill(e, b, &e->small, o, {tensor_seed(ms, l, "ssm_conv1d"), (uint64_t)e->C * 4, 0, 4, 0.5f, 0.f});
            o += (size_t)e->C * 16;
            enc_fill(e, b, &e->small, o, {0, (uint64_t)e->HV, 0, 5, -1.0f, 0.f});          // A_neg
            enc_fill(e, b, &e->small, o + e->HV * 4, {0, (uint64_t)e->HV, 0, 5, 0.0f, 0.f});  // dt_bias
            enc_fill(e, b, &e->small, o + 2 * e->HV * 4, {0, 128, 0, 5, 1.0f, 0.f});       // gated norm weight
        }
        // router fp16 N(0, 0.02) incl. the shared-gate row; experts (this rank's slice of the global tensors)
        enc_fill(e, b, &e->router, (size_t)l * (e->E + 1) * e->D * 2, {tensor_seed(ms, l, "ffn_gate_inp"), (uint64_t)(e->E + 1) * e->D, 0, 3, 0.02f, 0.f});
        const uint64_t base = (uint64_t)e->e_lo * gu_bytes;
        enc_fill(e, b, &e->exg, (size_t)l * ex_bytes, {tensor_seed(ms, l, "ffn_gate_exps"), ex_bytes, base, 1, d_scale_for(e->D), 0.f});
        enc_fill(e, b, &e->exu, (size_t)l * ex_bytes, {tensor_seed(ms, l, "ffn_up_exps"), ex_bytes, base, 1, d_scale_for(e->D), 0.f});
        enc_fill(e, b, &e->exd, (size_t)l * ex_bytes, {tensor_seed(ms, l, "ffn_down_exps"), ex_bytes, base, 1, d_scale_for(e->I), 0.f});
        enc_fill(e, b, &e->shg, (size_t)l * gu_bytes, {tensor_seed(ms, l, "ffn_gate_shexp"), gu_bytes, 0, 1, d_scale_for(e->D), 0.f});
        enc_fill(e, b, &e->shu, (size_t)l * gu_bytes, {tensor_seed(ms, l, "ffn_up_shexp"), gu_bytes, 0, 1, d_scale_for(e->D), 0.f});
        enc_fill(e, b, &e->shd, (size_t)l * gu_bytes, {tensor_seed(ms, l, "ffn_down_shexp"), gu_bytes, 0, 1, d_scale_for(e->I), 0.f});
    }
    if (qw_batch_end(b) < 0) return e->fail("weight fill failed");
    return true;
}

// Re-codes every layer's expert matrices (already in their IQ3_S buffers) into IQ3X for the fused expert-FFN kernel.
bool pack_experts(qw_engine *e) {
    const size_t gu_bytes = (size_t)e->I * e->rbD, ex_bytes = (size_t)e->EL * gu_bytes;
    struct { uint32_t mode, experts, I, D; } a;
    for (int l = 0; l < e->L; l++) {
        qw_batch *b = qw_batch_begin(e->g, false);
        auto enc = [&](uint32_t mode, uint32_t experts, const qw_buf *A, size_t ao, const qw_buf *B, size_t bo, const qw_buf *dst, size_t dofs) {
            a = {mode, experts, (uint32_t)e->I, (uint32_t)e->D};
            qw_batch_kernel(b, e->k_pack);
            qw_batch_buf(b, 0, A, ao);
            if (B) qw_batch_buf(b, 1, B, bo);
            qw_batch_buf(b, 2, dst, dofs);
            qw_batch_bytes(b, 3, &a, sizeof a);
            qw_batch_dispatch(b, 1, 1, 1, 256, 1, 1);
        };
        enc(0, (uint32_t)e->EL, &e->exg, (size_t)l * ex_bytes, &e->exu, (size_t)l * ex_bytes, &e->xq_gu, (size_t)l * e->EL * e->x_gus);
        enc(1, (uint32_t)e->EL, &e->exd, (size_t)l * ex_bytes, nullptr, 0, &e->xq_d, (size_t)l * e->EL * e->x_dns);
        enc(0, 1, &e->shg, (size_t)l * gu_bytes, &e->shu, (size_t)l * gu_bytes, &e->xs_gu, (size_t)l * e->x_gus);
        enc(1, 1, &e->shd, (size_t)l * gu_bytes, nullptr, 0, &e->xs_d, (size_t)l * e->x_dns);
        if (qw_batch_end(b) < 0) return e->fail("re-coding of the expert weights failed at layer %d", l);
    }
    return true;
}

}  // namespace

extern "C" void qw_model_cfg_default(qw_model_cfg *c) {
    memset(c, 0, sizeof *c);
    c->hidden = 2048; c->layers = 48; c->attn_every = 4; c->vocab = 151936;
    c->experts = 512; c->topk = 10; c->expert_inter = 512;
    c->qh = 16; c->kvh = 2; c->hd = 256; c->hk = 16; c->hv = 32;
    c->max_slots = 16; c->max_ctx = 49152 + 1024; c->kv_pages = 0;
    c->ep_rank = 0; c->ep_size = 1; c->fma = 0; c->seed = 0;
}

extern "C" const char *qw_engine_error(const qw_engine *e) { return e ? e->err.c_str() : g_open_error.c_str(); }
extern "C" qw_gpu *qw_engine_gpu(qw_engine *e) { return e ? e->g : nullptr; }

extern "C" void qw_engine_close(qw_engine *e) {
    if (!e) return;
    qw_buf *all[] = {&e->emb, &e->lm_head, &e->dense, &e->small, &e->router, &e->exg, &e->exu, &e->exd, &e->shg, &e->shu, &e->shd, &e->kvpool,
                     &e->ptab, &e->sstate, &e->cstate, &e->ctl_h, &e->ctl_d, &e->h, &e->x, &e->proj, &e->cv, &e->la, &e->be, &e->gy, &e->qb,
                     &e->part, &e->ya, &e->ob, &e->mo, &e->logits, &e->ids, &e->ids_h, &e->logits_h, &e->cand_h, &e->mlog, &e->msel, &e->Hhi, &e->Hlo, &e->Pg, &e->rcnt, &e->xq_gu, &e->xq_d, &e->xs_gu, &e->xs_d, &e->ffn_scr};
    // mappings of the other ranks' exchange buffers go first (their owners free the memory), then this rank's own
    for (int r = 0; r < 8; r++)
        if (r != e->c.ep_rank && e->ep_peer[r].handle) qw_buf_free(&e->ep_peer[r]);
    qw_buf_free(&e->epx);
    for (qw_buf *b : all) qw_buf_free(b);
    delete e;
}

extern "C" qw_engine *qw_engine_open_synth(qw_gpu *g, const qw_model_cfg *cfg) {
    g_open_error.clear();
    if (!g || !cfg) {
        g_open_error = "null device or config";
        return nullptr;
    }
    qw_engine *e = new qw_engine();
    e->g = g;
    e->c = *cfg;
    const qw_model_cfg &c = e->c;
    auto bad = [&](const char *m) {
        g_open_error = m;
        delete e;
        return (qw_engine *)nullptr;
    };
    if (c.hidden != 2048 && c.hidden != 256) return bad("hidden must be 2048 (or 256 for tests)");
    if (c.hd != 256 || c.qh != 8 * c.kvh) return bad("attention kernels need head_dim 256 and 8 query heads per kv head");
    if (c.max_slots < 1 || c.max_slots > QW_PAR_MAX) return bad("max_slots must be 1..64");
    if (c.ep_size < 1 || c.experts % c.ep_size || c.ep_rank < 0 || c.ep_rank >= c.ep_size) return bad("bad expert-parallel slice");
    if (c.expert_inter % 256 || c.hidden % 256 || c.vocab % 16 || c.experts % 32 || (c.experts != 512 && c.experts > 256) || c.topk < 1 || c.topk > 15)
        return bad("unsupported MoE / vocab shape (experts: 512, or a multiple of 32 up to 256)");
    if (c.hv % c.hk || c.layers < 1 || c.attn_every < 1) return bad("bad layer shape");
    e->D = c.hidden; e->L = c.layers; e->V = c.vocab; e->E = c.experts; e->EL = c.experts / c.ep_size; e->e_lo = c.ep_rank * e->EL;
    e->TOPK = c.topk; e->I = c.expert_inter; e->QH = c.qh; e->KVH = c.kvh; e->HD = c.hd; e->HK = c.hk; e->HV = c.hv;
    e->C = 2 * c.hk * 128 + c.hv * 128;
    e->KA = c.qh * c.hd; e->KG = c.hv * 128;
    e->rbD = e->D / 256 * 110; e->rbI = e->I / 256 * 110; e->rbKA = e->KA / 256 * 110; e->rbKG = e->KG / 256 * 110; e->rbV = e->D / 32 * 34;
    e->qkv_rows = c.qh * 2 * c.hd + 2 * c.kvh * c.hd;
    e->gdn_rows = e->C + c.hv * 128 + 2 * c.hv;
    if (e->qkv_rows % 16 || e->gdn_rows % 16) return bad("projection rows must be multiples of 16");
    e->max_pages = (c.max_ctx + PAGE - 1) / PAGE;
    for (int i = 0; i <= QW_PAR_MAX; i++) e->cost[i] = 0;

    // ---- layer table and offsets
    size_t dn = 0;
    e->small_stride = (size_t)2 * e->D + std::max<size_t>(512, (size_t)e->C * 4 + 2 * e->HV + 128);
    e->n_attn = e->n_gdn = 0;
    for (int l = 0; l < e->L; l++) {
        LayerW w;
        w.attn = (l % c.attn_every) == c.attn_every - 1;
        w.n_in = w.attn ? e->qkv_rows : e->gdn_rows;
        w.w_in = dn;
        dn = align_up(dn + (size_t)w.n_in * e->rbD, 256);
        w.w_out = dn;
        dn = align_up(dn + (size_t)e->D * (w.attn ? e->rbKA : e->rbKG), 256);
        w.small = (size_t)l * e->small_stride;
        w.idx = w.attn ? e->n_attn++ : e->n_gdn++;
        e->layers.push_back(w);
    }
    e->final_norm = (size_t)e->L * e->small_stride;
    const int na = std::max(1, e->n_attn), ng = std::max(1, e->n_gdn);

    // ---- kernels
    const long D = e->D, NBX = QW_PAR_MAX;
    bool ok = compile(e, "par_begin", "par_begin", {}, &e->k_begin) && compile(e, "kb_embed", "kb_embed", {}, &e->k_embed) &&
              compile(e, "add_rmsnorm", "rmsnorm", {{"ADD", 0}}, &e->k_norm0) && compile(e, "add_rmsnorm", "add_rmsnorm", {{"ADD", 1}}, &e->k_norm) &&
              compile(e, "qw_fill", "qw_fill", {}, &e->k_fill) && compile(e, "k_argmax", "k_argmax_host", {{"IDS2", 1}}, &e->k_argmax) &&
              compile(e, "par_advance", "par_advance", {{"FEED", 0}}, &e->k_adv) && compile(e, "par_advance", "par_advance_feed", {{"FEED", 1}}, &e->k_adv_feed);
    const char *qf = c.fma ? "qmv_gg" : "qmv_mma";
    ok = ok && compile(e, qf, "qmv_in_attn", {{"GF", 21}, {"KD", D}, {"NB", NBX}, {"YT_F32", 0}}, &e->k_qmv_in_a) &&
         compile(e, qf, "qmv_in_gdn", {{"GF", 21}, {"KD", D}, {"NB", NBX}, {"YT_F32", 0}}, &e->k_qmv_in_g) &&
         compile(e, qf, "qmv_out_attn", {{"GF", 21}, {"KD", (long)e->KA}, {"NB", NBX}, {"YT_F32", 0}}, &e->k_qmv_o_a) &&
         compile(e, qf, "qmv_out_gdn", {{"GF", 21}, {"KD", (long)e->KG}, {"NB", NBX}, {"YT_F32", 0}}, &e->k_qmv_o_g) &&
         compile(e, qf, "qmv_lm_head", {{"GF", 8}, {"KD", D}, {"NB", NBX}, {"YT_F32", 1}}, &e->k_lm);
    std::vector<std::pair<const char *, long>> ad = {{"QH", c.qh}, {"KVH", c.kvh}, {"HD", c.hd}};
    ok = ok && compile(e, "qsa_prep", "qsa_prep", ad, &e->k_prep) && compile(e, "qsa_attn", "qsa_attn", ad, &e->k_attn) &&
         compile(e, "qsa_merge", "qsa_merge", ad, &e->k_merge);
    const char *fm = getenv("QW_MOE_FFN");
    // moe_ffn spreads the pieces of the chosen experts over all blocks, so it is the default at every rank count;
    // QW_MOE_FFN=split keeps the two-launch family, QW_MOE_FFN=fused runs moe_ffn on the raw IQ3_S blocks
    e->ffn_fused = e->D == 2048 && e->I == 512 && !(fm && !strcmp(fm, "split"));
    e->ffn_iq3x = e->ffn_fused && !(fm && !strcmp(fm, "fused"));
    // EARLY: the GDN kernels read their per-slot state before they wait for the previous kernel.  Allowed when every layer ends in a
    // launch that fills all SMs (moe_ffn) and there are at least two layers: see gdn_fstep_k.
    std::vector<std::pair<const char *, long>> gd = {{"HK", c.hk}, {"HV", c.hv}, {"DK", 128}, {"DV", 128}, {"GDN_TILED", 1},
                                                      {"EARLY", e->ffn_fused && e->L >= 2 ? 1 : 0}};
    ok = ok && compile(e, "dn_epi", "dn_epi", gd, &e->k_epi) && compile(e, "gdn_fstep", "gdn_fstep", gd, &e->k_gdn);
    // expert-parallel: the shared expert is computed by rank 0 only, so the exchange can sum whole buffers
    std::vector<std::pair<const char *, long>> md = {{"E", e->E}, {"EL", e->EL}, {"D", D}, {"I", e->I}, {"TOPK", e->TOPK},
                                                      {"SHARED", c.ep_rank == 0 ? 1 : 0}, {"RESID", 0}};
    ok = ok && compile(e, "moe_router", "moe_router", md, &e->k_router) && compile(e, "moe_select", "moe_select", md, &e->k_select) &&
         compile(e, "moe_gu", "moe_gu", md, &e->k_gu) && compile(e, "moe_dn", "moe_dn", md, &e->k_dn) && compile(e, "moe_cmb", "moe_cmb", md, &e->k_cmb) &&
         compile(e, "moe_route", "moe_route", md, &e->k_route) &&
         compile(e, "add_rmsnorm", "cmb_add_rmsnorm", {{"CMB", 1}, {"TOPK", e->TOPK}}, &e->k_norm_cmb);
    {
        if (ok && e->ffn_fused) {
            auto mf = md;
            mf.push_back({"IQ3X", e->ffn_iq3x ? 1 : 0});
            auto mp = mf;
            mp.push_back({"PROBE", 1});
            ok = compile(e, "moe_ffn", "moe_ffn", mf, &e->k_ffn) && compile(e, "moe_ffn", "moe_ffn_copy_probe", mp, &e->k_ffn_probe) &&
                 (!e->ffn_iq3x || compile(e, "iq3x_pack", "iq3x_pack", {}, &e->k_pack));
            const char *cw = getenv("QW_CMB_WAIT");  // QW_CMB_WAIT=launch: the combine + norm waits for the FFN's whole launch, as with any other kernel
            if (ok && c.ep_size == 1 && e->D == 2048 && !(cw && !strcmp(cw, "launch")))
                ok = compile(e, "add_rmsnorm", "cmb_add_rmsnorm_rows", {{"CMB", 1}, {"TOPK", e->TOPK}, {"ROWCNT", 1}}, &e->k_norm_cmb_rc);
        }
    }
    ok = ok && compile(e, "k_topk", "k_topk", {}, &e->k_topk);
    e->k_ar = nullptr;
    if (ok && c.ep_size > 1) ok = compile(e, "ep_allreduce", "ep_allreduce", {}, &e->k_ar);
    if (!ok) {
        g_open_error = e->err;
        delete e;
        return nullptr;
    }

    // ---- memory
    const size_t gu_bytes = (size_t)e->I * e->rbD;
    const int kvp = c.kv_pages > 0 ? c.kv_pages : c.max_slots * e->max_pages;
    const size_t page_bytes = (size_t)na * 2 * c.kvh * PAGE * c.hd * 2;
    e->sel_bytes = align_up(qw_moe_sel_bytes(), 256);
    const size_t B = QW_PAR_MAX;
    ok = new_buf(e, &e->emb, (size_t)e->V * e->D * 2) && new_buf(e, &e->lm_head, (size_t)e->V * e->rbV) && new_buf(e, &e->dense, dn) &&
         new_buf(e, &e->small, ((size_t)e->L * e->small_stride + e->D) * 4) && new_buf(e, &e->router, (size_t)e->L * (e->E + 1) * e->D * 2) &&
         new_buf(e, &e->exg, (size_t)e->L * e->EL * gu_bytes) && new_buf(e, &e->exu, (size_t)e->L * e->EL * gu_bytes) &&
         new_buf(e, &e->exd, (size_t)e->L * e->EL * gu_bytes) && new_buf(e, &e->shg, (size_t)e->L * gu_bytes) &&
         new_buf(e, &e->shu, (size_t)e->L * gu_bytes) && new_buf(e, &e->shd, (size_t)e->L * gu_bytes) &&
         new_buf(e, &e->kvpool, (size_t)kvp * page_bytes) && new_buf(e, &e->ptab, (size_t)c.max_slots * e->max_pages * 4) &&
         new_buf(e, &e->sstate, (size_t)c.max_slots * ng * c.hv * 128 * 128 * 4) && new_buf(e, &e->cstate, (size_t)c.max_slots * ng * 3 * e->C * 4) &&
         new_buf(e, &e->ctl_h, 3 * 64 * 4, QW_BUF_HOSTIO) && new_buf(e, &e->ctl_d, 3 * 64 * 4) && new_buf(e, &e->h, B * e->D * 4) &&
         new_buf(e, &e->x, B * e->D * 2) && new_buf(e, &e->proj, B * std::max(e->qkv_rows, e->gdn_rows) * 2) && new_buf(e, &e->cv, B * e->C * 2) &&
         new_buf(e, &e->la, B * c.hv * 4) && new_buf(e, &e->be, B * c.hv * 4) && new_buf(e, &e->gy, B * e->KG * 2) &&
         new_buf(e, &e->qb, B * c.qh * c.hd * 2) && new_buf(e, &e->part, B * (size_t)e->max_pages * c.qh * (c.hd + 2) * 4) &&
         new_buf(e, &e->ya, B * e->KA * 2) && new_buf(e, &e->ob, B * e->D * 2) && new_buf(e, &e->mo, B * e->D * 2) &&
         new_buf(e, &e->logits, B * (size_t)e->V * 4) && new_buf(e, &e->ids, B * 4) && new_buf(e, &e->ids_h, B * 4, QW_BUF_HOSTIO) && new_buf(e, &e->cand_h, B * 256 * 8, QW_BUF_HOSTIO) &&
         new_buf(e, &e->logits_h, B * (size_t)e->V * 4, QW_BUF_HOSTIO) && new_buf(e, &e->mlog, B * (e->E + 1) * 4) &&
         new_buf(e, &e->msel, (size_t)e->L * e->sel_bytes) && new_buf(e, &e->Hhi, B * (e->TOPK + 1) * e->I * 2) &&
         new_buf(e, &e->Hlo, B * (e->TOPK + 1) * e->I * 2) && new_buf(e, &e->Pg, B * (e->TOPK + 1) * e->D * 4) && new_buf(e, &e->rcnt, 256);
    if (ok) ok = qw_buf_zero(g, &e->msel, 0, e->msel.size) && qw_buf_zero(g, &e->Pg, 0, e->Pg.size) && qw_buf_zero(g, &e->Hhi, 0, e->Hhi.size) &&
                 qw_buf_zero(g, &e->Hlo, 0, e->Hlo.size) && qw_buf_zero(g, &e->ptab, 0, e->ptab.size) &&
                 qw_buf_zero(g, &e->kvpool, 0, e->kvpool.size) && qw_buf_zero(g, &e->rcnt, 0, e->rcnt.size);  // rows past a slot's length are multiplied by probability 0: keep them finite
    if (ok && e->ffn_fused) ok = new_buf(e, &e->ffn_scr, MOE_FFN_SCRATCH_BYTES(e->I)) && qw_buf_zero(g, &e->ffn_scr, 0, e->ffn_scr.size);
    if (ok && e->ffn_iq3x) {
        e->x_gus = (size_t)(e->I / 64) * (e->D / 512) * 128 * 272;
        e->x_dns = (size_t)(e->D / 128) * (e->I / 512) * 128 * 272;
        ok = new_buf(e, &e->xq_gu, (size_t)e->L * e->EL * e->x_gus) && new_buf(e, &e->xq_d, (size_t)e->L * e->EL * e->x_dns) &&
             new_buf(e, &e->xs_gu, (size_t)e->L * e->x_gus) && new_buf(e, &e->xs_d, (size_t)e->L * e->x_dns);
    }
    if (ok) ok = init_weights(e);
    if (ok && e->ffn_iq3x) ok = pack_experts(e);
    // The step reads only the re-coded experts from here on.  A model of real size gives the raw IQ3_S blocks back (33 GB at
    // the benchmark shape: room for KV pages); small models keep them, so that tests can read the tensors they were built from.
    if (ok && e->ffn_iq3x && (size_t)e->L * e->EL * 3 * gu_bytes > ((size_t)4 << 30)) {
        qw_buf *raw[] = {&e->exg, &e->exu, &e->exd, &e->shg, &e->shu, &e->shd};
        for (qw_buf *b : raw) {
            qw_buf_free(b);
            *b = qw_buf{};
        }
    }
    if (!ok) {
        g_open_error = e->err.empty() ? "engine open failed" : e->err;
        qw_engine_close(e);
        return nullptr;
    }
    e->slots.resize(c.max_slots);
    for (int p = kvp - 1; p >= 0; p--) e->free_pages.push_back(p);
    qw_engine_sample_set_vocab(e->V);
    return e;
}

// ------------------------------------------------------------------------------------------------ slots
extern "C" int qw_engine_par_slots(qw_engine *e) { return e ? (int)e->slots.size() : 0; }

extern "C" int qw_engine_par_pick(qw_engine *e, const int32_t *, int, unsigned long long busy) {
    if (!e) return -1;
    int best = -1;
    for (int i = 0; i < (int)e->slots.size(); i++) {
        if (busy >> i & 1) continue;
        if (!e->slots[i].used) return i;
        if (best < 0 || e->slots[i].last_use < e->slots[best].last_use) best = i;
    }
    return best;
}

static void release_slot(qw_engine *e, int sid) {
    Slot &s = e->slots[sid];
    for (int p : s.pages) e->free_pages.push_back(p);
    s.pages.clear();
    s.used = false;
    s.pos = 0;
}

// make sure slot sid owns pages for positions < upto; uploads the new page-table entries
static bool reserve_pages(qw_engine *e, int sid, int upto) {
    Slot &s = e->slots[sid];
    const int need = (upto + PAGE - 1) / PAGE;
    if (need > e->max_pages) return e->fail("slot %d: context %d exceeds max_ctx", sid, upto);
    const int have = (int)s.pages.size();
    if (need <= have) return true;
    if ((int)e->free_pages.size() < need - have) return e->fail("KV pool exhausted (%d pages free, %d needed)", (int)e->free_pages.size(), need - have);
    for (int i = have; i < need; i++) {
        s.pages.push_back(e->free_pages.back());
        e->free_pages.pop_back();
    }
    if (!qw_buf_upload(e->g, &e->ptab, ((size_t)sid * e->max_pages + have) * 4, s.pages.data() + have, (size_t)(need - have) * 4))
        return e->fail("page table upload failed");
    return true;
}

extern "C" void qw_engine_par_finish(qw_engine *e, int sid, const int32_t *, int) {
    if (e && sid >= 0 && sid < (int)e->slots.size() && e->slots[sid].used) release_slot(e, sid);
}

extern "C" int qw_engine_par_pos(qw_engine *e, int sid) {
    if (!e || sid < 0 || sid >= (int)e->slots.size() || !e->slots[sid].used) return -1;
    return e->slots[sid].pos;
}

extern "C" size_t qw_engine_par_mem(qw_engine *e) {
    if (!e) return 0;
    const size_t page_bytes = (size_t)std::max(1, e->n_attn) * 2 * e->KVH * PAGE * e->HD * 2;
    size_t m = 0;
    for (const Slot &s : e->slots)
        if (s.used) m += s.pages.size() * page_bytes + (size_t)e->n_gdn * ((size_t)e->HV * 128 * 128 * 4 + (size_t)3 * e->C * 4);
    return m;
}

extern "C" int qw_engine_par_seed(qw_engine *e, int sid, int ctx_len, unsigned long long seed) {
    if (!e || sid < 0 || sid >= (int)e->slots.size() || ctx_len < 0 || ctx_len >= e->c.max_ctx) return -1;
    if (e->slots[sid].used) release_slot(e, sid);
    Slot &s = e->slots[sid];
    if (!reserve_pages(e, sid, ctx_len + 1)) return -1;
    s.used = true;
    s.pos = ctx_len;
    s.last_use = ++e->clock;
    const size_t page_halves = (size_t)std::max(1, e->n_attn) * 2 * e->KVH * PAGE * e->HD;
    qw_batch *b = qw_batch_begin(e->g, false);
    for (size_t i = 0; i < s.pages.size(); i++)
        enc_fill(e, b, &e->kvpool, (size_t)s.pages[i] * page_halves * 2, {mix64(seed ^ (0x4B56ull << 32) ^ i), page_halves, 0, 3, 1.0f, 0.f});
    const size_t sst = (size_t)std::max(1, e->n_gdn) * e->HV * 128 * 128, cst = (size_t)std::max(1, e->n_gdn) * 3 * e->C;
    enc_fill(e, b, &e->sstate, (size_t)sid * sst * 4, {mix64(seed ^ 0x5354ull), sst, 0, 4, 0.1f, 0.f});
    enc_fill(e, b, &e->cstate, (size_t)sid * cst * 4, {mix64(seed ^ 0x434Full), cst, 0, 4, 1.0f, 0.f});
    if (qw_batch_end(b) < 0) {
        e->fail("slot seeding failed");
        return -1;
    }
    return 0;
}

// Row order of a step under slot sharding (slot s belongs to rank s mod nranks): rows grouped by owning rank, stable within
// a rank, so that every rank's rows are one contiguous range [lo, hi) of the same order on every rank.  perm[j] = the
// caller's index of device row j.  Pure host logic (no device needed).
extern "C" int qw_ep_row_order(const int *sids, int B, int nranks, int rank, int *perm, int *lo, int *hi) {
    if (!sids || !perm || B < 0 || nranks < 1 || rank < 0 || rank >= nranks) return -1;
    for (int i = 0; i < B; i++) perm[i] = i;
    std::stable_sort(perm, perm + B, [&](int a, int b) { return sids[a] % nranks < sids[b] % nranks; });
    int l = 0, h = 0;
    for (int j = 0; j < B; j++) {
        const int own = sids[perm[j]] % nranks;
        if (own < rank) l++;
        if (own <= rank) h++;
    }
    if (lo) *lo = l;
    if (hi) *hi = h;
    return 0;
}

// ------------------------------------------------------------------------------------------------ the step
namespace {

struct qmv_args { uint32_t N, xstride, ystride, nb; };
struct qsa_args { uint32_t nb, layer, nlayers, qkv_stride, max_pages, max_chunks, pad0, pad1; };
struct dn_epi_args { uint32_t nb, layer, nlayers, proj_stride; };
struct gdn_args { uint32_t nb, layer, nlayers, z_stride; };
struct sel_args { uint32_t nb, e_lo, e_hi; };

void enc_qmv(qw_batch *b, qw_kernel *k, const qw_buf *W, size_t woff, uint32_t N, uint32_t K, const qw_buf *x, const qw_buf *y, uint32_t nb, uint32_t ystride,
             size_t xoff = 0) {
    const qmv_args a = {N, K, ystride, nb};
    qw_batch_kernel(b, k);
    qw_batch_buf(b, 0, W, woff);
    qw_batch_buf(b, 3, x, xoff);
    qw_batch_buf(b, 4, y, 0);
    qw_batch_bytes(b, 5, &a, sizeof a);
    qw_batch_dispatch(b, (N + 7) / 8, 1, 1, 256, 1, 1);
}

// h (+)= the previous block's output, x = rmsnorm(h) * w.  delta == &e->Pg means "the MoE combine of layer cmb_layer",
// computed inside the norm kernel from Pg and that layer's selection record.
void enc_norm(qw_engine *e, qw_batch *b, const qw_buf *delta, size_t w_off_floats, uint32_t nb, int cmb_layer = -1, size_t delta_off = 0) {
    const uint32_t a[2] = {nb, (uint32_t)e->D};
    const bool cmb = delta == &e->Pg;
    const bool gathered = delta == &e->epx;  // slot sharding: the rows were stored by the ranks that own the slots
    const bool rows = cmb && e->k_norm_cmb_rc && e->ffn_fused && !e->ep_fused && !e->moe_probe;  // the FFN counts its output rows in
    qw_batch_kernel(b, cmb ? (e->ep_fused ? e->k_norm_cmb_x : rows ? e->k_norm_cmb_rc : e->k_norm_cmb) : gathered ? e->k_norm_x : delta ? e->k_norm : e->k_norm0);
    qw_batch_buf(b, 0, &e->h, 0);
    if (cmb) {
        qw_batch_buf(b, 5, &e->msel, (size_t)cmb_layer * e->sel_bytes);
        if (e->ep_fused) {
            qw_batch_buf(b, 6, &e->epx, (size_t)(cmb_layer & 1) * e->pg_bytes);
            qw_batch_buf(b, 7, &e->epx, 2 * e->pg_bytes);
            qw_batch_buf(b, 8, &e->rcnt, 64);
        } else qw_batch_buf(b, 6, &e->Pg, 0);
        if (rows) qw_batch_buf(b, 9, &e->ffn_scr, 0);
    } else if (delta) {
        qw_batch_buf(b, 1, delta, delta_off);
        if (gathered) {
            qw_batch_buf(b, 7, &e->epx, 2 * e->pg_bytes);
            qw_batch_buf(b, 8, &e->rcnt, 64);
        }
    }
    qw_batch_buf(b, 2, &e->small, w_off_floats * 4);
    qw_batch_buf(b, 3, &e->x, 0);
    qw_batch_bytes(b, 4, a, sizeof a);
    qw_batch_dispatch(b, nb, 1, 1, 256, 1, 1);
}

// Encodes one decode step for nb rows whose control data is in ctl_d ([0..63] tok, [64..127] slot, [128..191] pos).
void encode_step(qw_engine *e, qw_batch *b, uint32_t nb, uint32_t max_chunks, bool from_host, int sample /*0 none, 1 argmax, 2 argmax + feed next*/) {
    const uint32_t D = e->D;
    const qw_buf *none = nullptr;
    if (from_host) {
        const uint32_t n = 192;
        qw_batch_kernel(b, e->k_begin);
        qw_batch_buf(b, 0, &e->ctl_h, 0);
        qw_batch_buf(b, 1, &e->ctl_d, 0);
        qw_batch_bytes(b, 2, &n, 4);
        qw_batch_dispatch(b, 1, 1, 1, 256, 1, 1);
    }
    {
        const uint32_t a[3] = {nb, D, (uint32_t)e->V};
        qw_batch_kernel(b, e->k_embed);
        qw_batch_buf(b, 0, &e->emb, 0);
        qw_batch_buf(b, 1, &e->ctl_d, 0);
        qw_batch_buf(b, 2, &e->h, 0);
        qw_batch_bytes(b, 3, a, sizeof a);
        qw_batch_dispatch(b, (D + 255) / 256, nb, 1, 256, 1, 1);
    }
    const qw_buf *pending = none;  // block output not yet added to the residual stream
    // rows of the token mixers: all of them, or (slot sharding) the rows [lo, lo + nbl) whose slots this rank owns
    const uint32_t lo = e->slot_shard ? e->row_lo : 0, nbl = e->slot_shard ? e->row_hi - e->row_lo : nb;
    const size_t xo = (size_t)lo * D * 2, co = (size_t)lo * 4;  // byte offsets of row lo in x / ob and in the control arrays
    const qw_buf *obuf = e->slot_shard ? &e->epx : &e->ob;
    const size_t obo = e->slot_shard ? e->ob_off : 0;
    // binds of a kernel that stores into every rank's buffer and publishes (moe_dn, the sharded out-projections, ep_publish)
    auto bind_peers = [&](size_t peer_off, bool with_data) {
        const uint32_t rk = (uint32_t)e->c.ep_rank;
        qw_batch_buf(b, 11, &e->rcnt, 64);
        qw_batch_bytes(b, 12, &rk, 4);
        for (int r = 0; r < e->c.ep_size; r++) {
            if (with_data) qw_batch_buf(b, 16 + r, &e->ep_peer[r], peer_off);
            qw_batch_buf(b, 24 + r, &e->ep_peer[r], 2 * e->pg_bytes);
        }
    };
    auto enc_out_proj = [&](qw_kernel *plain, qw_kernel *shared, size_t woff, uint32_t K, const qw_buf *in) {
        if (!e->slot_shard) return enc_qmv(b, plain, &e->dense, woff, D, K, in, &e->ob, nb, D);
        const qmv_args a = {D, K, D, nbl};
        qw_batch_kernel(b, shared);
        qw_batch_buf(b, 0, &e->dense, woff);
        qw_batch_buf(b, 3, in, 0);
        qw_batch_buf(b, 4, &e->epx, e->ob_off + xo);
        qw_batch_bytes(b, 5, &a, sizeof a);
        bind_peers(e->ob_off + xo, true);
        qw_batch_dispatch(b, (D + 7) / 8, 1, 1, 256, 1, 1);
    };
    for (int l = 0; l < e->L; l++) {
        const LayerW &w = e->layers[l];
        enc_norm(e, b, pending, w.small, nb, l - 1);  // h += previous block (the MoE combine of layer l-1); x = rmsnorm(h) * w1
        if (nbl == 0) {  // no row of this rank in the step: only tell the others so
            qw_batch_kernel(b, e->k_pub);
            bind_peers(0, false);
            qw_batch_dispatch(b, 1, 1, 1, 32, 1, 1);
        } else if (w.attn) {
            enc_qmv(b, e->k_qmv_in_a, &e->dense, w.w_in, e->qkv_rows, D, &e->x, &e->proj, nbl, e->qkv_rows, xo);
            const qsa_args qa = {nbl, (uint32_t)w.idx, (uint32_t)e->n_attn, e->qkv_rows, (uint32_t)e->max_pages, max_chunks, 0, 0};
            qw_batch_kernel(b, e->k_prep);
            qw_batch_buf(b, 0, &e->proj, 0);
            qw_batch_buf(b, 1, &e->small, (w.small + 2 * D) * 4);
            qw_batch_buf(b, 2, &e->small, (w.small + 2 * D + 256) * 4);
            qw_batch_buf(b, 3, &e->qb, 0);
            qw_batch_buf(b, 4, &e->kvpool, 0);
            qw_batch_buf(b, 5, &e->ptab, 0);
            qw_batch_buf(b, 6, &e->ctl_d, 128 * 4 + co);
            qw_batch_buf(b, 7, &e->ctl_d, 64 * 4 + co);
            qw_batch_bytes(b, 8, &qa, sizeof qa);
            qw_batch_dispatch(b, e->QH + e->KVH, nbl, 1, 256, 1, 1);
            qw_batch_kernel(b, e->k_attn);
            qw_batch_buf(b, 0, &e->qb, 0);
            qw_batch_buf(b, 1, &e->kvpool, 0);
            qw_batch_buf(b, 2, &e->ptab, 0);
            qw_batch_buf(b, 3, &e->ctl_d, 128 * 4 + co);
            qw_batch_buf(b, 4, &e->ctl_d, 64 * 4 + co);
            qw_batch_buf(b, 5, &e->part, 0);
            qw_batch_bytes(b, 6, &qa, sizeof qa);
            qw_batch_dispatch(b, max_chunks, e->KVH, nbl, 128, 1, 1);
            qw_batch_kernel(b, e->k_merge);
            qw_batch_buf(b, 0, &e->part, 0);
            qw_batch_buf(b, 1, &e->proj, 0);
            qw_batch_buf(b, 2, &e->ya, 0);
            qw_batch_buf(b, 3, &e->ctl_d, 128 * 4 + co);
            qw_batch_bytes(b, 4, &qa, sizeof qa);
            qw_batch_dispatch(b, e->QH, nbl, 1, 256, 1, 1);
            enc_out_proj(e->k_qmv_o_a, e->k_qmv_o_a_x, w.w_out, e->KA, &e->ya);
        } else {
            enc_qmv(b, e->k_qmv_in_g, &e->dense, w.w_in, e->gdn_rows, D, &e->x, &e->proj, nbl, e->gdn_rows, xo);
            const size_t so = (w.small + 2 * D) * 4, sa = so + (size_t)e->C * 16;
            const dn_epi_args ea = {nbl, (uint32_t)w.idx, (uint32_t)e->n_gdn, e->gdn_rows};
            qw_batch_kernel(b, e->k_epi);
            qw_batch_buf(b, 0, &e->proj, 0);
            qw_batch_buf(b, 1, &e->small, so);
            qw_batch_buf(b, 2, &e->cstate, 0);
            qw_batch_buf(b, 3, &e->small, sa);
            qw_batch_buf(b, 4, &e->small, sa + e->HV * 4);
            qw_batch_buf(b, 5, &e->cv, 0);
            qw_batch_buf(b, 6, &e->la, 0);
            qw_batch_buf(b, 7, &e->be, 0);
            qw_batch_buf(b, 8, &e->ctl_d, 64 * 4 + co);
            qw_batch_bytes(b, 9, &ea, sizeof ea);
            qw_batch_dispatch(b, (e->C + 2 * e->HV + 255) / 256, nbl, 1, 256, 1, 1);
            const gdn_args ga = {nbl, (uint32_t)w.idx, (uint32_t)e->n_gdn, e->gdn_rows};
            qw_batch_kernel(b, e->k_gdn);
            qw_batch_buf(b, 0, &e->cv, 0);
            qw_batch_buf(b, 1, &e->la, 0);
            qw_batch_buf(b, 2, &e->be, 0);
            qw_batch_buf(b, 3, &e->sstate, 0);
            qw_batch_buf(b, 4, &e->proj, (size_t)e->C * 2);
            qw_batch_buf(b, 5, &e->small, sa + 2 * e->HV * 4);
            qw_batch_buf(b, 6, &e->gy, 0);
            qw_batch_buf(b, 7, &e->ctl_d, 64 * 4 + co);
            qw_batch_bytes(b, 8, &ga, sizeof ga);
            qw_batch_dispatch(b, e->HV, nbl, 1, 512, 1, 1);
            enc_out_proj(e->k_qmv_o_g, e->k_qmv_o_g_x, w.w_out, e->KG, &e->gy);
        }
        enc_norm(e, b, obuf, w.small + D, nb, -1, obo);  // h += mixer output (all rows); x = rmsnorm(h) * w2
        // ---- MoE (gg_moe, src/engine.c:568-646)
        const size_t gu_bytes = (size_t)e->I * e->rbD, ex_bytes = (size_t)e->EL * gu_bytes, selo = (size_t)l * e->sel_bytes;
        const sel_args sa = {nb, (uint32_t)e->e_lo, (uint32_t)(e->e_lo + e->EL)};
        qw_batch_kernel(b, e->k_route);  // router logits + top-k + grouping in one launch
        qw_batch_buf(b, 0, &e->router, (size_t)l * (e->E + 1) * D * 2);
        qw_batch_buf(b, 1, &e->router, ((size_t)l * (e->E + 1) + e->E) * D * 2);
        qw_batch_buf(b, 2, &e->x, 0);
        qw_batch_buf(b, 3, &e->mlog, 0);
        qw_batch_buf(b, 4, &e->rcnt, 0);
        qw_batch_buf(b, 5, &e->msel, selo);
        qw_batch_bytes(b, 14, &sa, sizeof sa);
        qw_batch_dispatch(b, (e->E + 1 + 7) / 8, 1, 1, 1024, 1, 1);
        const uint32_t ebase = (uint32_t)e->e_lo;
        const bool zero_first = e->c.ep_size > 1 && !e->ep_fused;  // rows of experts held elsewhere must read as zero before the NCCL exchange
        // the down projection's output: Pg, or (fused exchange) Pg[layer parity] of every rank -- two buffers suffice because a rank
        // can run at most one down projection ahead of the slowest rank (its next norm waits for everybody's flags)
        auto bind_pg = [&]() {
            if (e->ep_fused) {
                const size_t po = (size_t)(l & 1) * e->pg_bytes;
                qw_batch_buf(b, 9, &e->epx, po);
                bind_peers(po, true);
            } else qw_batch_buf(b, 9, &e->Pg, 0);
            qw_batch_bytes(b, 10, &ebase, 4);
        };
        if (e->ffn_fused) {
            if (zero_first) {
                const fill_args z = {0, (uint64_t)nb * (e->TOPK + 1) * D * 4, 0, 0, 0.f, 0.f};
                enc_fill(e, b, &e->Pg, 0, z);
            }
            qw_batch_kernel(b, e->ep_fused ? e->k_ffn_x : e->moe_probe ? e->k_ffn_probe : e->k_ffn);  // gate/up, SiLU * up and down of every chosen expert in one launch
            if (e->ffn_iq3x) {
                qw_batch_buf(b, 0, &e->xq_gu, (size_t)l * e->EL * e->x_gus);
                qw_batch_buf(b, 2, &e->xs_gu, (size_t)l * e->x_gus);
                qw_batch_buf(b, 6, &e->xq_d, (size_t)l * e->EL * e->x_dns);
                qw_batch_buf(b, 7, &e->xs_d, (size_t)l * e->x_dns);
            } else {
                qw_batch_buf(b, 0, &e->exg, (size_t)l * ex_bytes);
                qw_batch_buf(b, 1, &e->exu, (size_t)l * ex_bytes);
                qw_batch_buf(b, 2, &e->shg, (size_t)l * gu_bytes);
                qw_batch_buf(b, 3, &e->shu, (size_t)l * gu_bytes);
                qw_batch_buf(b, 6, &e->exd, (size_t)l * ex_bytes);
                qw_batch_buf(b, 7, &e->shd, (size_t)l * gu_bytes);
            }
            qw_batch_buf(b, 4, &e->x, 0);
            qw_batch_buf(b, 5, &e->msel, selo);
            qw_batch_buf(b, 8, &e->ffn_scr, 0);
            bind_pg();
            qw_batch_dispatch(b, e->I / 16, nb * e->TOPK + 1, 1, 256, 1, 1);
        } else {
            qw_batch_kernel(b, e->k_gu);
            qw_batch_buf(b, 0, &e->exg, (size_t)l * ex_bytes);
            qw_batch_buf(b, 1, &e->exu, (size_t)l * ex_bytes);
            qw_batch_buf(b, 2, &e->shg, (size_t)l * gu_bytes);
            qw_batch_buf(b, 3, &e->shu, (size_t)l * gu_bytes);
            qw_batch_buf(b, 4, &e->x, 0);
            qw_batch_buf(b, 5, &e->msel, selo);
            qw_batch_buf(b, 6, &e->Hhi, 0);
            qw_batch_buf(b, 7, &e->Hlo, 0);
            qw_batch_bytes(b, 10, &ebase, 4);
            qw_batch_dispatch(b, e->I / 16, nb * e->TOPK + 1, 1, 256, 1, 1);
            if (zero_first) {
                const fill_args z = {0, (uint64_t)nb * (e->TOPK + 1) * D * 4, 0, 0, 0.f, 0.f};
                enc_fill(e, b, &e->Pg, 0, z);
            }
            qw_batch_kernel(b, e->ep_fused ? e->k_dn_x : e->k_dn);
            qw_batch_buf(b, 0, &e->exd, (size_t)l * ex_bytes);
            qw_batch_buf(b, 2, &e->shd, (size_t)l * gu_bytes);
            qw_batch_buf(b, 5, &e->msel, selo);
            qw_batch_buf(b, 6, &e->Hhi, 0);
            qw_batch_buf(b, 7, &e->Hlo, 0);
            bind_pg();
            qw_batch_dispatch(b, D / 64, nb * e->TOPK + 1, 1, 256, 1, 1);
        }
        if (e->c.ep_size > 1 && !e->ep_fused) {
            // every (token, rank) row has exactly one non-zero contributor (a routed expert's owner, or rank 0 for
            // the shared expert), so the sum reproduces the one-GPU rows bit for bit
            const uint64_t cnt = (uint64_t)nb * (e->TOPK + 1) * D;
            qw_batch_kernel(b, e->k_ar);
            qw_batch_buf(b, 0, &e->Pg, 0);
            qw_batch_bytes(b, 1, &cnt, sizeof cnt);
            qw_batch_dispatch(b, 1, 1, 1, 1, 1, 1);
        }
        pending = &e->Pg;  // combined, rounded to fp16 and added to the residual stream inside the next norm kernel
    }
    enc_norm(e, b, pending, e->final_norm, nb, e->L - 1);
    enc_qmv(b, e->k_lm, &e->lm_head, 0, (uint32_t)e->V, D, &e->x, &e->logits, nb, (uint32_t)e->V);
    if (sample == 3) {  // the 256 best (id, logit) pairs of every row, written straight into host-visible memory
        const uint32_t a[3] = {nb, (uint32_t)e->V, 256};
        qw_batch_kernel(b, e->k_topk);
        qw_batch_buf(b, 0, &e->logits, 0);
        qw_batch_buf(b, 1, &e->cand_h, 0);
        qw_batch_buf(b, 2, &e->cand_h, (size_t)QW_PAR_MAX * 256 * 4);
        qw_batch_bytes(b, 3, a, sizeof a);
        qw_batch_dispatch(b, nb, 1, 1, 1024, 1, 1);
    } else if (sample) {
        const uint32_t a[2] = {nb, (uint32_t)e->V};
        qw_batch_kernel(b, e->k_argmax);
        qw_batch_buf(b, 0, &e->logits, 0);
        qw_batch_buf(b, 1, &e->ids, 0);
        qw_batch_bytes(b, 2, a, sizeof a);
        qw_batch_buf(b, 3, &e->ids_h, 0);
        qw_batch_dispatch(b, nb, 1, 1, 1024, 1, 1);
    }
    {
        qw_batch_kernel(b, sample == 2 ? e->k_adv_feed : e->k_adv);
        qw_batch_buf(b, 0, &e->ctl_d, 128 * 4);
        qw_batch_buf(b, 1, &e->ctl_d, 0);
        qw_batch_buf(b, 2, &e->ids, 0);
        qw_batch_bytes(b, 3, &nb, 4);
        qw_batch_dispatch(b, 1, 1, 1, 64, 1, 1);
    }
}

// validates the rows, reserves pages for `ahead` more tokens, writes the control block; returns max_chunks or 0
uint32_t begin_step(qw_engine *e, const int *sids, const int32_t *toks, int B, int ahead) {
    if (!e) return 0;
    if (!sids || !toks || B < 1 || B > QW_PAR_MAX) return e->fail("par_step: bad arguments"), 0;
    unsigned long long seen = 0;
    int maxpos = 0;
    for (int i = 0; i < B; i++) {
        const int s = sids[i];
        if (s < 0 || s >= (int)e->slots.size() || !e->slots[s].used) return e->fail("par_step: slot %d is not in use", s), 0;
        if (seen >> s & 1) return e->fail("par_step: slot %d appears twice", s), 0;
        seen |= 1ull << s;
        if (toks[i] < 0 || toks[i] >= e->V) return e->fail("par_step: token %d out of range", toks[i]), 0;
        if (e->slots[s].pos + ahead > e->c.max_ctx) return e->fail("par_step: slot %d would exceed max_ctx", s), 0;
        if (!reserve_pages(e, s, e->slots[s].pos + ahead)) return 0;
        maxpos = std::max(maxpos, e->slots[s].pos + ahead);
    }
    // device row order: the caller's, or (slot sharding) grouped by the rank that owns the slot, stable within a rank, so
    // that every rank's rows are one contiguous range -- the same order on every rank
    int lo = 0, hi = B;
    qw_ep_row_order(sids, B, e->slot_shard ? e->c.ep_size : 1, e->slot_shard ? e->c.ep_rank : 0, e->perm, &lo, &hi);
    e->row_lo = (uint32_t)lo;
    e->row_hi = (uint32_t)hi;
    int32_t *ctl = (int32_t *)e->ctl_h.ptr;
    for (int j = 0; j < B; j++) {
        const int i = e->perm[j];
        ctl[j] = toks[i];
        ctl[64 + j] = sids[i];
        ctl[128 + j] = e->slots[sids[i]].pos;
    }
    // chunk count of the attention grid: a multiple of 8 pages so the recorded batch (and its graph) changes rarely
    uint32_t mc = (uint32_t)((maxpos + PAGE - 1) / PAGE);
    mc = std::min<uint32_t>((mc + 7) / 8 * 8, (uint32_t)e->max_pages);
    return mc;
}

void end_step(qw_engine *e, const int *sids, int B, int nsteps, double wall_ms) {
    e->last_sids.assign(sids, sids + B);
    e->lastB = B;
    e->last_ctx = 0;
    e->last_own = 0;
    for (int i = 0; i < B; i++) {
        Slot &s = e->slots[sids[i]];
        s.pos += nsteps;
        s.last_use = ++e->clock;
        // tokens attended by the last of the steps -- under slot sharding only the slots this rank owns are its traffic
        if (!e->slot_shard || sids[i] % e->c.ep_size == e->c.ep_rank) {
            e->last_ctx += s.pos;
            e->last_own++;
        }
    }
    const double per = wall_ms / nsteps;
    e->cost[B] = e->cost[B] == 0 ? per : 0.8 * e->cost[B] + 0.2 * per;
}

// A step whose batch failed (a wait that ran out, a launch error) may have left the expert-FFN kernel's per-item counters
// non-zero; the next step must not find them: they would let down pieces start before their H is complete.
void after_failed_step(qw_engine *e) {
    if (e->ffn_scr.size) qw_buf_zero(e->g, &e->ffn_scr, 0, MOE_FFN_SYNC_BYTES);
}

}  // namespace

extern "C" const float *qw_engine_par_step(qw_engine *e, const int *sids, const int32_t *toks, int B, double *gpu_ms) {
    const double t0 = qw_now();
    const uint32_t mc = begin_step(e, sids, toks, B, 1);
    if (!mc) return nullptr;
    qw_batch *b = qw_batch_begin(e->g, false);
    encode_step(e, b, (uint32_t)B, mc, true, 0);
    const double secs = qw_batch_end(b);
    if (secs < 0) return after_failed_step(e), e->fail("par_step: device batch failed"), nullptr;
    for (int j = 0; j < B; j++)  // device row j is the caller's row perm[j]
        if (!qw_buf_download(e->g, &e->logits, (size_t)j * e->V * 4, (float *)e->logits_h.ptr + (size_t)e->perm[j] * e->V, (size_t)e->V * 4))
            return e->fail("par_step: logits copy failed"), nullptr;
    if (gpu_ms) *gpu_ms = secs * 1e3;
    end_step(e, sids, B, 1, (qw_now() - t0) * 1e3);
    return (const float *)e->logits_h.ptr;
}

extern "C" const int32_t *qw_engine_par_step_greedy(qw_engine *e, const int *sids, const int32_t *toks, int B, double *gpu_ms) {
    const double t0 = qw_now();
    const uint32_t mc = begin_step(e, sids, toks, B, 1);
    if (!mc) return nullptr;
    qw_batch *b = qw_batch_begin(e->g, false);
    encode_step(e, b, (uint32_t)B, mc, true, 1);
    const double secs = qw_batch_end(b);
    if (secs < 0) return after_failed_step(e), e->fail("par_step_greedy: device batch failed"), nullptr;
    if (gpu_ms) *gpu_ms = secs * 1e3;
    end_step(e, sids, B, 1, (qw_now() - t0) * 1e3);
    e->ids_out.resize(QW_PAR_MAX);
    for (int j = 0; j < B; j++) e->ids_out[e->perm[j]] = ((const int32_t *)e->ids_h.ptr)[j];
    return e->ids_out.data();
}

extern "C" int qw_engine_par_decode_greedy(qw_engine *e, const int *sids, const int32_t *toks, int B, int nsteps, int32_t *out_ids, double *gpu_ms) {
    if (!e || nsteps < 1 || !out_ids) return -1;
    const double t0 = qw_now();
    const uint32_t mc = begin_step(e, sids, toks, B, nsteps);
    if (!mc) return -1;
    double total = 0;
    for (int s = 0; s < nsteps; s++) {
        // one batch per step (so identical steps replay one cached graph); submitted back to back, the sampled ids
        // feed the next step on the device
        qw_batch *b = qw_batch_begin(e->g, false);
        encode_step(e, b, (uint32_t)B, mc, s == 0, 2);
        const double secs = qw_batch_end(b);
        if (secs < 0) return after_failed_step(e), e->fail("par_decode_greedy: device batch failed at step %d", s), -1;
        total += secs;
        for (int j = 0; j < B; j++) out_ids[(size_t)s * B + e->perm[j]] = ((const int32_t *)e->ids_h.ptr)[j];
    }
    if (gpu_ms) *gpu_ms = total * 1e3;
    end_step(e, sids, B, nsteps, (qw_now() - t0) * 1e3);
    return nsteps;
}

// ---- sampling on the host from an ordered candidate list: the reference's make_dist + dist_draw (src/engine.c:6094-6143)
// restated for candidates that are already the top ones in its order (value descending, ties by id ascending)
namespace {
uint64_t rng_next(uint64_t *x) {  // splitmix64, src/engine.c:6085-6090
    uint64_t z = (*x += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
int32_t sample_candidates(const int32_t *id, const float *lg, int avail, const qw_sample_params *g, unsigned long long *rng) {
    if (avail < 1) return -1;
    if (g->temperature <= 0) return id[0];
    const int k = g->top_k > 0 && g->top_k < 256 ? g->top_k : 256;
    const int n = std::min(k, avail);
    float p[256];
    const float T = g->temperature, mx = lg[0];
    double sum = 0;
    for (int i = 0; i < n; i++) {
        p[i] = expf((lg[i] - mx) / T);
        sum += p[i];
    }
    double c = 0;
    int keep = n;
    for (int i = 0; i < n; i++) {
        p[i] = (float)(p[i] / sum);
        c += p[i];
        if (g->top_p > 0 && g->top_p < 1 && c >= g->top_p) {
            keep = i + 1;
            break;
        }
    }
    double s2 = 0;
    for (int i = 0; i < keep; i++) s2 += p[i];
    for (int i = 0; i < keep; i++) p[i] = (float)(p[i] / s2);
    double tot = 0;
    for (int i = 0; i < keep; i++) tot += p[i];
    if (tot <= 0) return id[0];
    uint64_t r = *rng;
    double u = (double)(rng_next(&r) >> 11) * (1.0 / 9007199254740992.0) * tot;
    *rng = r;
    for (int i = 0; i < keep; i++) {
        u -= p[i];
        if (u <= 0) return id[i];
    }
    return id[keep - 1];
}
}  // namespace

static int g_sample_vocab = 0;  // the reference compiles its vocabulary size in; here: the engine opened last, or set explicitly
extern "C" void qw_engine_sample_set_vocab(int vocab) { g_sample_vocab = vocab > 0 ? vocab : 0; }
extern "C" int32_t qw_engine_sample(const float *lg, const qw_gen *g, unsigned long long *rng) {
    if (!g || g_sample_vocab < 1) return -1;
    const qw_sample_params sp = {g->temperature, g->top_k, g->top_p};
    return qw_engine_sample_v(lg, g_sample_vocab, &sp, rng);
}

extern "C" int32_t qw_engine_sample_v(const float *lg, int vocab, const qw_sample_params *g, unsigned long long *rng) {
    if (!lg || vocab < 1 || !g || !rng) return -1;
    // the top candidates of the whole row in the reference's order: insertion into a list kept sorted by value, an equal
    // value goes behind the ones already there (they have lower ids)
    const int k = g->temperature <= 0 ? 1 : (g->top_k > 0 && g->top_k < 256 ? g->top_k : 256);
    int32_t id[256];
    float val[256];
    int n = 0;
    for (int v = 0; v < vocab; v++) {
        const float x = lg[v];
        if (n == k && !(x > val[n - 1])) continue;
        int i = n < k ? n++ : n - 1;
        while (i > 0 && val[i - 1] < x) {
            id[i] = id[i - 1];
            val[i] = val[i - 1];
            i--;
        }
        id[i] = v;
        val[i] = x;
    }
    return sample_candidates(id, val, n, g, rng);
}

extern "C" int qw_engine_par_step_sample(qw_engine *e, const int *sids, const int32_t *toks, int B, const qw_sample_params *g, unsigned long long *rng,
                                         int32_t *out_ids, double *gpu_ms) {
    if (!e || !g || !rng || !out_ids) return -1;
    const double t0 = qw_now();
    const uint32_t mc = begin_step(e, sids, toks, B, 1);
    if (!mc) return -1;
    qw_batch *b = qw_batch_begin(e->g, false);
    encode_step(e, b, (uint32_t)B, mc, true, 3);
    const double secs = qw_batch_end(b);
    if (secs < 0) return after_failed_step(e), e->fail("par_step_sample: device batch failed"), -1;
    if (gpu_ms) *gpu_ms = secs * 1e3;
    const int32_t *cid = (const int32_t *)e->cand_h.ptr;
    const float *cval = (const float *)((const char *)e->cand_h.ptr + (size_t)QW_PAR_MAX * 256 * 4);
    const int avail = std::min(256, e->V);
    for (int j = 0; j < B; j++) {  // device row j is the caller's row perm[j]
        const int i = e->perm[j];
        out_ids[i] = sample_candidates(cid + (size_t)j * 256, cval + (size_t)j * 256, avail, &g[i], &rng[i]);
    }
    end_step(e, sids, B, 1, (qw_now() - t0) * 1e3);
    return B;
}

// Prompt processing for one slot (src/engine.h:81) without a prefill kernel family: the prompt is fed through the decode step
// one token at a time (B = 1), from an empty slot -- recurrent and conv state zero, no KV.  It is the decode path's own
// arithmetic, so "prefill then step" equals stepping every token; it costs one step per prompt token and exists so that
// a scheduler can run pick -> prefill -> step -> finish end to end (there is no prefix cache: *cached = 0).
extern "C" const float *qw_engine_par_prefill(qw_engine *e, int sid, const int32_t *prompt, int np, int *cached) {
    if (cached) *cached = 0;
    if (!e || sid < 0 || sid >= (int)e->slots.size() || !prompt || np < 1 || np >= e->c.max_ctx) return e ? (e->fail("par_prefill: bad arguments"), nullptr) : nullptr;
    for (int i = 0; i < np; i++)
        if (prompt[i] < 0 || prompt[i] >= e->V) return e->fail("par_prefill: token %d out of range", prompt[i]), nullptr;
    if (e->slots[sid].used) release_slot(e, sid);
    Slot &s = e->slots[sid];
    if (!reserve_pages(e, sid, np + 1)) return nullptr;
    s.used = true;
    s.pos = 0;
    s.last_use = ++e->clock;
    {   // empty recurrent state
        const size_t sst = (size_t)std::max(1, e->n_gdn) * e->HV * 128 * 128 * 4, cst = (size_t)std::max(1, e->n_gdn) * 3 * e->C * 4;
        qw_batch *b = qw_batch_begin(e->g, false);
        enc_fill(e, b, &e->sstate, (size_t)sid * sst, {0, sst, 0, 0, 0.f, 0.f});
        enc_fill(e, b, &e->cstate, (size_t)sid * cst, {0, cst, 0, 0, 0.f, 0.f});
        if (qw_batch_end(b) < 0) return e->fail("par_prefill: state reset failed"), nullptr;
    }
    const float *lg = nullptr;
    for (int i = 0; i < np; i++) {
        if (i + 1 < np) {  // intermediate positions: the step runs, nothing is copied back
            const double t0 = qw_now();
            const uint32_t mc = begin_step(e, &sid, &prompt[i], 1, 1);
            if (!mc) return nullptr;
            qw_batch *b = qw_batch_begin(e->g, false);
            encode_step(e, b, 1, mc, true, 0);
            if (qw_batch_end(b) < 0) return after_failed_step(e), e->fail("par_prefill: device batch failed at position %d", i), nullptr;
            end_step(e, &sid, 1, 1, (qw_now() - t0) * 1e3);
        } else lg = qw_engine_par_step(e, &sid, &prompt[i], 1, nullptr);
    }
    return lg;
}

extern "C" int qw_engine_set_moe_probe(qw_engine *e, int on) {
    if (!e || !e->k_ffn_probe) return -1;
    e->moe_probe = on != 0;
    return 0;
}

extern "C" double qw_engine_par_cost(qw_engine *e, int B) { return e && B >= 1 && B <= QW_PAR_MAX ? e->cost[B] : 0; }

extern "C" void qw_engine_last_step_bytes(qw_engine *e, qw_step_bytes *o) {
    if (!o) return;
    memset(o, 0, sizeof *o);
    if (!e || e->lastB == 0) return;
    const double gu = (double)e->I * e->rbD;
    int usum = 0;
    for (int l = 0; l < e->L; l++) {
        uint32_t U = 0;
        qw_buf_download(e->g, &e->msel, (size_t)l * e->sel_bytes, &U, 4);
        usum += (int)U;
        const double nexp = (double)U + (e->c.ep_rank == 0 ? 1 : 0);  // the shared expert runs on rank 0
        o->moe += nexp * (e->ffn_iq3x ? (double)(e->x_gus + e->x_dns) : 3 * gu) + (double)(e->E + 1) * e->D * 2;
        o->moe_iq3s += nexp * 3 * gu + (double)(e->E + 1) * e->D * 2;
        const LayerW &w = e->layers[l];
        o->dense += (double)w.n_in * e->rbD + (double)e->D * (w.attn ? e->rbKA : e->rbKG);
    }
    o->unique_experts_sum = usum;
    o->lm_head = (double)e->V * e->rbV;
    o->ctx_tokens = e->last_ctx;
    o->kv = (double)e->last_ctx * 2 * e->KVH * e->HD * 2 * e->n_attn;
    o->gdn_state = (double)e->last_own * e->n_gdn * e->HV * 128 * 128 * 4 * 2;
    o->other = (double)e->lastB * e->V * 4 * 2;
    o->total = o->moe + o->dense + o->lm_head + o->kv + o->gdn_state + o->other;
}

extern "C" size_t qw_engine_tap(qw_engine *e, const char *name, int index, void *dst, size_t cap) {
    if (!e || !name) return 0;
    const qw_buf *b = nullptr;
    size_t n = 0, off = 0;
    const size_t gu = (size_t)e->I * e->rbD, B = (size_t)e->lastB;
    const int ng = std::max(1, e->n_gdn), na = std::max(1, e->n_attn);
    const bool lay = index >= 0 && index < e->L;
    if (!strcmp(name, "h")) { b = &e->h; n = B * e->D * 4; }
    else if (!strcmp(name, "logits")) { b = &e->logits; n = B * e->V * 4; }
    else if (!strcmp(name, "x")) { b = &e->x; n = B * e->D * 2; }
    else if (!strcmp(name, "emb")) { b = &e->emb; n = (size_t)e->V * e->D * 2; }
    else if (!strcmp(name, "lm_head")) { b = &e->lm_head; n = (size_t)e->V * e->rbV; }
    else if (!strcmp(name, "final_norm")) { b = &e->small; off = e->final_norm * 4; n = (size_t)e->D * 4; }
    else if (!strcmp(name, "w_in") && lay) { b = &e->dense; off = e->layers[index].w_in; n = (size_t)e->layers[index].n_in * e->rbD; }
    else if (!strcmp(name, "w_out") && lay) { b = &e->dense; off = e->layers[index].w_out; n = (size_t)e->D * (e->layers[index].attn ? e->rbKA : e->rbKG); }
    else if (!strcmp(name, "small") && lay) { b = &e->small; off = e->layers[index].small * 4; n = e->small_stride * 4; }
    else if (!strcmp(name, "router") && lay) { b = &e->router; off = (size_t)index * (e->E + 1) * e->D * 2; n = (size_t)(e->E + 1) * e->D * 2; }
    else if (!strcmp(name, "exg") && lay) { b = &e->exg; off = (size_t)index * e->EL * gu; n = (size_t)e->EL * gu; }
    else if (!strcmp(name, "exu") && lay) { b = &e->exu; off = (size_t)index * e->EL * gu; n = (size_t)e->EL * gu; }
    else if (!strcmp(name, "exd") && lay) { b = &e->exd; off = (size_t)index * e->EL * gu; n = (size_t)e->EL * gu; }
    else if (!strcmp(name, "shg") && lay) { b = &e->shg; off = (size_t)index * gu; n = gu; }
    else if (!strcmp(name, "shu") && lay) { b = &e->shu; off = (size_t)index * gu; n = gu; }
    else if (!strcmp(name, "shd") && lay) { b = &e->shd; off = (size_t)index * gu; n = gu; }
    else if (!strcmp(name, "sel") && lay) { b = &e->msel; off = (size_t)index * e->sel_bytes; n = qw_moe_sel_bytes(); }
    else if (!strcmp(name, "sstate") && index >= 0 && index < (int)e->slots.size()) { n = (size_t)ng * e->HV * 128 * 128 * 4; b = &e->sstate; off = (size_t)index * n; }
    else if (!strcmp(name, "cstate") && index >= 0 && index < (int)e->slots.size()) { n = (size_t)ng * 3 * e->C * 4; b = &e->cstate; off = (size_t)index * n; }
    else if (!strcmp(name, "kvpage") && index >= 0) { n = (size_t)na * 2 * e->KVH * PAGE * e->HD * 2; b = &e->kvpool; off = (size_t)index * n; }
    else if (!strcmp(name, "pages") && index >= 0 && index < (int)e->slots.size()) {
        n = e->slots[index].pages.size() * 4;
        if (!dst) return n;
        if (n > cap) return 0;
        memcpy(dst, e->slots[index].pages.data(), n);
        return n;
    }
    if (!b) return 0;
    if (!dst) return n;  // size query
    if (n > cap || off + n > b->size) return 0;
    return qw_buf_download(e->g, b, off, dst, n) ? n : 0;
}

extern "C" int qw_ep_comm_init(int rank, int size, const void *id128);

extern "C" int qw_engine_ep_init(qw_engine *e, const void *id128) {
    if (!e) return -1;
    if (e->c.ep_size == 1) return 0;
    if (qw_ep_comm_init(e->c.ep_rank, e->c.ep_size, id128) != 0) {
        e->fail("expert-parallel communicator could not be created");
        return -1;
    }
    e->ep_ready = true;
    return 0;
}

// Fused exchange, step 1: allocate this rank's exchange buffer and export its 64-byte handle.
extern "C" int qw_engine_ep_export(qw_engine *e, void *handle64) {
    if (!e || !handle64) return -1;
    if (e->c.ep_size < 2 || e->c.ep_size > 8) return e->fail("ep_export: needs 2..8 expert-parallel ranks"), -1;
    if (e->L & 1) return e->fail("ep_export: the fused exchange alternates two buffers by layer and needs an even layer count"), -1;
    if (!e->epx.handle) {
        e->pg_bytes = (size_t)QW_PAR_MAX * (e->TOPK + 1) * e->D * 4;
        e->ob_off = 2 * e->pg_bytes + 256;  // [2][Pg] | flags | gathered mixer outputs fp16 [rows][D]
        if (!new_buf(e, &e->epx, e->ob_off + (size_t)QW_PAR_MAX * e->D * 2) || !qw_buf_zero(e->g, &e->epx, 0, e->epx.size)) return -1;
    }
    if (!qw_buf_ipc_export(&e->epx, handle64)) return e->fail(qw_gpu_last_error(e->g)), -1;
    return 0;
}

// Step 2 (after every rank has exported and the handles were gathered in rank order): map the other ranks' buffers and
// switch the step to the fused exchange.  All ranks must have zeroed their buffers (= returned from qw_engine_ep_export)
// before any rank steps; the gather between the two calls orders that.
extern "C" int qw_engine_ep_connect(qw_engine *e, const void *handles, int n) {
    if (!e || !handles || n != e->c.ep_size || !e->epx.handle) return e ? (e->fail("ep_connect: export first, pass one handle per rank"), -1) : -1;
    for (int r = 0; r < n; r++) {
        if (r == e->c.ep_rank) e->ep_peer[r] = e->epx;
        else if (!qw_buf_ipc_import(e->g, (const char *)handles + 64 * r, e->epx.size, &e->ep_peer[r])) return e->fail(qw_gpu_last_error(e->g)), -1;
    }
    std::vector<std::pair<const char *, long>> md = {{"E", e->E}, {"EL", e->EL}, {"D", (long)e->D}, {"I", e->I}, {"TOPK", e->TOPK},
                                                      {"SHARED", e->c.ep_rank == 0 ? 1 : 0}, {"RESID", 0}, {"EPX", n}};
    auto mfx = md;
    mfx.push_back({"IQ3X", e->ffn_iq3x ? 1 : 0});
    if ((e->ffn_fused && !compile(e, "moe_ffn", "moe_ffn_epx", mfx, &e->k_ffn_x)) || !compile(e, "moe_dn", "moe_dn_epx", md, &e->k_dn_x) ||
        !compile(e, "add_rmsnorm", "cmb_add_rmsnorm_epx", {{"CMB", 1}, {"TOPK", e->TOPK}, {"EPX", n}}, &e->k_norm_cmb_x))
        return -1;
    if (!qw_buf_zero(e->g, &e->rcnt, 64, 8)) return -1;
    e->ep_fused = true;
    // slot sharding needs the persistent out-projection kernel (K = 2048 or 4096); QW_SLOT_SHARD=0 keeps every rank on all rows
    const char *ss = getenv("QW_SLOT_SHARD");
    const bool shapes = !e->c.fma && (e->KA == 2048 || e->KA == 4096) && (e->KG == 2048 || e->KG == 4096);
    if (shapes && !(ss && atoi(ss) == 0)) {
        const long NBX = QW_PAR_MAX;
        if (!compile(e, "qmv_mma", "qmv_out_attn_epx", {{"GF", 21}, {"KD", (long)e->KA}, {"NB", NBX}, {"YT_F32", 0}, {"EPX", n}}, &e->k_qmv_o_a_x) ||
            !compile(e, "qmv_mma", "qmv_out_gdn_epx", {{"GF", 21}, {"KD", (long)e->KG}, {"NB", NBX}, {"YT_F32", 0}, {"EPX", n}}, &e->k_qmv_o_g_x) ||
            !compile(e, "add_rmsnorm", "add_rmsnorm_epx", {{"ADD", 1}, {"EPX", n}}, &e->k_norm_x) || !compile(e, "ep_publish", "ep_publish", {{"EPX", n}}, &e->k_pub))
            return -1;
        e->slot_shard = true;
    }
    return 0;
}
