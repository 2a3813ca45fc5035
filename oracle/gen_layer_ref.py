#!/usr/bin/env python3
"""Builds oracle/_ref/liblayer_ref.so from the reference's own CPU double-precision checks -- TEST INFRASTRUCTURE.

The reference holds a CPU check for each of the three floating-point layers of the decode path, written inline in
its bench programs (which need Metal and do not build here):
    Gated DeltaNet recurrence   bench/gdn_decode.c:74-84   (helper h2f :20)
    dense softmax . V           bench/qsa.c:184-201        (helper h2f :35-39)
    MoE select + SwiGLU + sum   bench/moe_decode.c:133-177 (helpers f2h, h2f :42-53)
This script cuts exactly those line ranges out of the reference tree into generated C files under oracle/_ref/
(never committed, deleted after the compile) and wraps each in a function: the wrapper only declares the variables
the cut lines use and captures the value they compare with the GPU result (by defining fabs / fmax around the cut,
with the "GPU output" all zeros).  The cut lines are compiled unmodified.

    python oracle/gen_layer_ref.py REF_ROOT        (called by oracle/Makefile; shapes of the MoE check are macros:
                                                    E 32, TOPK 4, D 256, I 256)
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def cut(path, a, b):
    with open(path, encoding="utf-8") as f:
        lines = f.readlines()
    return "".join(lines[a - 1:b])


def main(ref):
    out = os.path.join(HERE, "_ref")
    os.makedirs(out, exist_ok=True)
    gd, qs, mo = (os.path.join(ref, "bench", n) for n in ("gdn_decode.c", "qsa.c", "moe_decode.c"))
    pre = "#include <math.h>\n#include <stdint.h>\n#include <stddef.h>\n#include <stdlib.h>\n#include <string.h>\n"
    units = {}
    # ---- GDN: per v-head, per column: decay, mem = S^T k, delta, S += k delta^T, out = S^T q (state updated in place)
    units["gdn"] = pre + cut(gd, 20, 20) + """
void ref_gdn_core(int HV, int HK, int DK, int DV, const float *pa, const float *pb, const uint16_t *pq, const uint16_t *pk,
                  const uint16_t *pv, double *S0, double *OUT) {
    uint16_t *po = calloc((size_t)HV * DV, 2);
    double eo = 0;
#define fmax(a, b) (b)
#define fabs(x) (OUT[hv * DV + j] = (x))
""" + cut(gd, 74, 84) + """
#undef fabs
#undef fmax
    (void)eo;
    free(po);
}
"""
    # ---- attention: softmax(q . K / sqrt(HD)) . V over the listed tokens, per head
    units["attn"] = pre + cut(qs, 35, 39) + """
enum { QH = 16, KVH = 2, HD = 256, GQA = QH / KVH };
void ref_attn_core(int L, const uint16_t *q, const uint16_t *K, const uint16_t *V, double *OUT) {
    int nt = L, *toks = malloc(sizeof(int) * (size_t)L);
    for (int t = 0; t < L; t++) toks[t] = t;
    uint16_t *out = calloc((size_t)QH * HD, 2);
    double worst = 0;
    double *sv = malloc(sizeof(double) * nt);
#define fmax(a, b) (b)
#define fabs(x) (OUT[h * HD + j] = (x))
""" + cut(qs, 184, 201) + """
#undef fabs
#undef fmax
    (void)worst;
    free(sv); free(toks); free(out);
}
"""
    # ---- MoE: FP64 router, top-k (ties -> lowest id), softmax over the picked logits, H rounded to fp16, weighted sum
    units["moe"] = pre + cut(mo, 42, 53) + """
#define E 32
#define TOPK 4
#define D 256
#define I 256
typedef struct { const float *w; int K; } qm;                  /* a dequantised matrix stands in for the reference's packed one */
static float qm_w(const qm *q, size_t row, int k) { return q->w[row * (size_t)q->K + k]; }
static float bf2f(uint16_t b) { return h2f(b); }               /* the shared-gate row is fp16 here */
static qm Wr, Wg, Wu, Wd, Wsg, Wsu, Wsd;
static struct { const void *ptr; } sel;
void ref_moe_check(const uint16_t *x, const uint16_t *wsg, const float *wr, const float *wg, const float *wu, const float *wd, const float *sg,
                   const float *su, const float *sd, const uint32_t *gpu_ids, int *ids_out, double *OUT) {
    Wr = (qm){wr, D}; Wg = (qm){wg, D}; Wu = (qm){wu, D}; Wd = (qm){wd, I}; Wsg = (qm){sg, D}; Wsu = (qm){su, D}; Wsd = (qm){sd, I};
    sel.ptr = gpu_ids;
""" + cut(mo, 133, 177) + """
    (void)match;
    for (int t = 0; t < TOPK; t++) ids_out[t] = ids[t];
    for (int r = 0; r < D; r++) OUT[r] = ref[r];
}
"""
    objs = []
    for name, src in units.items():
        c = os.path.join(out, "layer_ref_%s_extract.c" % name)
        o = os.path.join(out, "layer_ref_%s.o" % name)
        with open(c, "w", encoding="utf-8") as f:
            f.write(src)
        subprocess.run(["gcc", "-O2", "-fPIC", "-std=c2x", "-ffp-contract=off", "-Wno-unused-variable", "-Wno-unused-but-set-variable", "-c", c, "-o", o], check=True)
        os.remove(c)
        objs.append(o)
    subprocess.run(["gcc", "-shared", "-o", os.path.join(out, "liblayer_ref.so")] + objs + ["-lm"], check=True)
    for o in objs:
        os.remove(o)
    print("built oracle/_ref/liblayer_ref.so from", ref)


if __name__ == "__main__":
    main(sys.argv[1])
