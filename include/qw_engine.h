/* qw_engine.h -- the batched (continuous-batching) decode step as a C ABI: the "par" part of the reference's
 * engine interface (src/engine.h:77-127 in hy-ong/qwental), built only on the device interface of qw_gpu.h.
 *
 * The reference's qw_engine_par_step (src/engine.c:8795) splits more than 8 slots into groups that each re-read
 * all weights; here one step advances up to QW_PAR_MAX slots with a single pass over the weights.
 * Out of scope here (see the reference for them): prefill, speculative decoding, prefix cache, snapshots, the
 * tokenizer and server.  Because prefill is out of scope a slot's context is created by qw_engine_par_seed.
 */
#ifndef QW_ENGINE_H
#define QW_ENGINE_H
#include "qw_gpu.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct qw_engine qw_engine;
enum { QW_PAR_MAX = 64 }; /* src/engine.h:79 */

/* Shape of the model (the reference fixes these in src/model.h:9-24 for its one model). */
typedef struct {
    int hidden;        /* D, 2048 */
    int layers;        /* 48 */
    int attn_every;    /* every attn_every-th layer is gated attention, the others Gated DeltaNet (4) */
    int vocab;         /* 151936 */
    int experts;       /* 512 */
    int topk;          /* 10 */
    int expert_inter;  /* 512 (routed and shared expert) */
    int qh, kvh, hd;   /* 16, 2, 256 */
    int hk, hv;        /* GDN key / value heads 16, 32 (head dims 128) */
    int max_slots;     /* conversation slots to keep state for (<= QW_PAR_MAX) */
    int max_ctx;       /* longest context per slot, tokens */
    int kv_pages;      /* pages of 256 tokens in the KV pool (0: max_slots * max_ctx / 256) */
    int ep_rank, ep_size; /* expert-parallel slice: this process holds experts [rank*E/size, (rank+1)*E/size) */
    int fma;           /* 1: dense matvecs use the fp32 FMA kernels in the oracle's order (qmv_gg); 0: tensor cores */
    unsigned long long seed; /* master seed of the synthetic weights: per-tensor seed = hash(layer, name) */
} qw_model_cfg;

/* Defaults = the Qwen3-Next-80B-A3B shape of the benchmark. */
void qw_model_cfg_default(qw_model_cfg *c);

/* Opens a model with seeded random-init weights generated on the device (no checkpoint is read; role of
 * qw_engine_open, src/engine.c:978-1211, minus the loaders).  NULL on failure (message: qw_engine_error(NULL)). */
qw_engine *qw_engine_open_synth(qw_gpu *g, const qw_model_cfg *cfg);
void qw_engine_close(qw_engine *e);
const char *qw_engine_error(const qw_engine *e);
qw_gpu *qw_engine_gpu(qw_engine *e);                 /* src/engine.h:66 */

int qw_engine_par_slots(qw_engine *e);               /* src/engine.h:78 */
/* src/engine.h:80: a slot whose bit in `busy` is clear, preferring never-used ones, else the least recently
 * used; -1 if none.  (The prompt is not used for prefix matching: the prefix cache is out of scope.) */
int qw_engine_par_pick(qw_engine *e, const int32_t *prompt, int np, unsigned long long busy);
/* Stands in for qw_engine_par_prefill (src/engine.h:81): gives slot sid a context of ctx_len tokens whose KV
 * pages, GDN state and conv state are seeded synthetic values (K, V ~ N(0,1); S ~ N(0, 0.01)).  0 or -1. */
int qw_engine_par_seed(qw_engine *e, int sid, int ctx_len, unsigned long long seed);
/* src/engine.h:81.  Processes a prompt into slot sid (released first if it was in use) and returns the logits of its last
 * position ([vocab], valid until the next step), NULL on failure.  There is no prefill kernel family and no prefix cache in
 * this library: the prompt runs through the decode step one token at a time (*cached = 0). */
const float *qw_engine_par_prefill(qw_engine *e, int sid, const int32_t *prompt, int np, int *cached);
/* src/engine.h:91.  One decode step for B slots (sids distinct, 1 <= B <= QW_PAR_MAX): returns [B][vocab] fp32
 * logits in host-visible memory, valid until the next step; NULL on failure.  *gpu_ms = device time. */
const float *qw_engine_par_step(qw_engine *e, const int *sids, const int32_t *toks, int B, double *gpu_ms);
/* The same step with the arg-max fused on the device (ties -> lowest id, as src/engine.c:6144-6148):
 * returns B token ids in host-visible memory; logits are not copied to the host. */
const int32_t *qw_engine_par_step_greedy(qw_engine *e, const int *sids, const int32_t *toks, int B, double *gpu_ms);
/* Sampling.  qw_gen is the reference's generation request (src/engine.h:39-52), field for field, so that a host compiled
 * against the reference's header passes the same bytes; the sampler reads only temperature (<= 0: greedy), top_k (<= 0 or
 * > 256 means 256) and top_p (>= 1 or <= 0: no nucleus cut).  qw_sample_params = those first three fields.
 *
 * qw_engine_sample is the reference's function of that name with its signature (src/engine.h:125, src/engine.c:9410-9418):
 * candidates = the top_k logits (ties -> lower id first), softmax(logit / T) over them, top-p cut, renormalise, one
 * splitmix64 draw from *rng.  The reference compiles the vocabulary size in; here it is the vocabulary of the engine opened
 * last in this process (or what qw_engine_sample_set_vocab set); -1 if neither happened.  qw_engine_sample_v is the same
 * sampler with the vocabulary size as a parameter.  qw_engine_par_step_sample runs the decode step, selects the 256 best
 * (id, logit) pairs of every row on the device and finishes on the host from those -- the same tokens as qw_engine_sample on
 * the full logits, without copying or scanning the [B][vocab] logits on the host.  g and rng have one entry per row;
 * out_ids [B].  Returns B or -1. */
typedef struct {
    float temperature;
    int top_k;
    float top_p;
    unsigned long long seed;
    int max_tokens;
    const int32_t *stop;
    int nstop;
    bool spec;
    const int *persist;
    int npersist;
    volatile bool *yield;
    bool (*pf_yield)(void *ctx);
} qw_gen;
typedef struct {
    float temperature;
    int top_k;
    float top_p;
} qw_sample_params;
int32_t qw_engine_sample(const float *logits, const qw_gen *g, unsigned long long *rng);
int32_t qw_engine_sample_v(const float *logits, int vocab, const qw_sample_params *g, unsigned long long *rng);
void qw_engine_sample_set_vocab(int vocab);
int qw_engine_par_step_sample(qw_engine *e, const int *sids, const int32_t *toks, int B, const qw_sample_params *g, unsigned long long *rng,
                              int32_t *out_ids, double *gpu_ms);
/* nsteps greedy steps back to back with no host round trip between them (each step's ids feed the next);
 * out_ids [nsteps][B].  Returns nsteps or -1. */
int qw_engine_par_decode_greedy(qw_engine *e, const int *sids, const int32_t *toks, int B, int nsteps, int32_t *out_ids, double *gpu_ms);
void qw_engine_par_finish(qw_engine *e, int sid, const int32_t *gen, int ngen); /* src/engine.h:92: frees the slot */
double qw_engine_par_cost(qw_engine *e, int B);      /* src/engine.h:95: EMA of the wall ms of a B-slot step, 0 = unknown */
size_t qw_engine_par_mem(qw_engine *e);              /* src/engine.h:96: bytes of slot state in use */
int qw_engine_par_pos(qw_engine *e, int sid);        /* tokens in slot sid's context, -1 if unused */

/* Algorithmic bytes one step over these slots must move on THIS rank (weights of the distinct experts the last step chose
 * among the experts held here, the shared expert on rank 0, dense weights, KV of the contexts and GDN state read + write of
 * the slots whose token mixers ran here): the numerator of the HBM roofline. */
typedef struct {
    double moe, dense, lm_head, kv, gdn_state, other, total;
    int unique_experts_sum; /* sum over layers of distinct experts chosen in the last step */
    long long ctx_tokens;   /* sum of context lengths attended in the last step */
    double moe_iq3s;        /* the MoE term counted in IQ3_S bytes (110 per 256 weights): equals `moe` unless the experts run from
                             * their re-coded IQ3X form (136 per 256), in which case `moe` and `total` count the bytes actually read */
} qw_step_bytes;
void qw_engine_last_step_bytes(qw_engine *e, qw_step_bytes *out);

/* Measurement aid (no counterpart in the reference's engine; its benches time pure-read kernels, bench/moe_bw.c:1-3): while
 * on, steps run the copy-only twin of the fused expert FFN kernel -- the same staged copies of the chosen experts' weights,
 * no decode, no output -- so a profiled step shows what the copy pipeline alone sustains.  Steps taken while it is on
 * produce meaningless tokens.  0, or -1 if this engine does not use the fused kernel. */
int qw_engine_set_moe_probe(qw_engine *e, int on);

/* Debug taps for the parity tests (role of the reference's QW_MOE_TEST / QW_DN_TAP dumps, src/engine.c:7942-7999):
 * copy a named internal buffer to the host; dst == NULL returns the size.  Last step: "h" fp32 [B][D],
 * "x" fp16 [B][D], "logits" fp32 [B][V], "sel" (layer index: the MoE selection record).  Weights by layer index:
 * "w_in", "w_out", "small", "router", "exg", "exu", "exd", "shg", "shu", "shd"; "emb", "lm_head", "final_norm".
 * State: "sstate" / "cstate" / "pages" by slot, "kvpage" by page id.  Returns bytes copied, 0 on error. */
size_t qw_engine_tap(qw_engine *e, const char *name, int index, void *dst, size_t cap);

/* Expert-parallel plumbing (no counterpart in the reference, which is single-device): the communicator is
 * created from a 128-byte NCCL unique id that rank 0 obtained from qw_ep_unique_id and shared with the others. */
int qw_ep_unique_id(void *id128);
int qw_engine_ep_init(qw_engine *e, const void *id128);

/* Fused exchange (optional, after or instead of qw_engine_ep_init; ranks on one NVLink/NVSwitch machine, even layer
 * count): the down projection of every rank stores its expert rows directly into every rank's buffer and publishes a
 * sequence number; the next norm kernel waits (bounded) for all ranks' numbers.  No collective call and no zero fill
 * remain on the step.  Every rank calls qw_engine_ep_export, the 64-byte handles are gathered in rank order by any
 * means, then every rank calls qw_engine_ep_connect with the ep_size handles.  All ranks must then step in lockstep
 * with identical inputs.  0 on success, -1 with qw_engine_error set. */
int qw_engine_ep_export(qw_engine *e, void *handle64);
/* The row order the engine uses under slot sharding (host logic only, exposed for schedulers and tests): rows grouped by
 * owning rank (slot mod nranks), stable within a rank; perm[j] = caller's index of device row j; [*lo, *hi) = this rank's
 * rows in that order.  0 or -1. */
int qw_ep_row_order(const int *sids, int B, int nranks, int rank, int *perm, int *lo, int *hi);
int qw_engine_ep_connect(qw_engine *e, const void *handles, int n);

#ifdef __cplusplus
}
#endif
#endif
