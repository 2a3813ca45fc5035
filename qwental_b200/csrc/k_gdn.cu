// Gated DeltaNet decode step for all slots in one launch, with each slot's fp32 state resident in HBM.
//
//   dn_epi     epilogue of the GDN input projection: depthwise conv-4 + SiLU with the slot's own conv state,
//              a -> log-decay A_neg*softplus(a + dt_bias), b -> beta = sigmoid(b)
//              -- role of dn_epi_rowT, kernels/dn_proj.metal:190-244 (the projection itself is qmv_mma; the
//                 reference rounds the projection to fp16 before this epilogue, :199, so nothing is lost)
//   gdn_fstep  L2-norm of q and k, S <- g*S; mem = S^T k; delta = beta*(v - mem); S += k delta^T; o = S^T q,
//              then the gated RMSNorm o*rsqrt(mean o^2 + eps)*w*sigmoid(z)
//              -- role of gdn_fstep, kernels/gdn_decode.metal:299-418 (q/k norm :281-296)
//
// The reference launches gdn_fstep once per slot (src/engine.c:8992-9007); here the slot is a grid dimension
// and the per-slot state is found through a slot-id table, so the launch count does not grow with the batch.
// A slot's arithmetic never looks at another slot, so batched results equal the slot alone bit for bit.
#include "common.cuh"
#include "qw_kern.h"

using namespace qw;

#define GDN_EPS 1e-6f

// proj row layout (fp16, stride PS): [q: HK*DK | k: HK*DK | v: HV*DV | z: HV*DV | a: HV | b: HV]
struct dn_epi_args {
    uint32_t nb, layer, nlayers, proj_stride;
};

// binds: 0 = proj fp16 [nb][proj_stride], 1 = conv weights fp32 [C][4], 2 = conv state pool fp32
// [slot][nlayers][3][C], 3 = A_neg fp32 [HV], 4 = dt_bias fp32 [HV], 5 = cv out fp16 [nb][C],
// 6 = la fp32 [nb][HV], 7 = beta fp32 [nb][HV], 8 = slot ids int32 [nb], 9 = dn_epi_args.
// grid (ceil((C + 2 HV)/256), nb) x 256
__global__ void __launch_bounds__(256) dn_epi_k(const __half *proj, const float *cw, float *pool, const float *An, const float *dtb, __half *cv,
                                               float *la, float *be, const int32_t *sids, dn_epi_args a, uint32_t C, uint32_t HV, bool early) {
    pdl_launch();
    if (!early) pdl_wait();
    const uint32_t g = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    const __half *pr = proj + (size_t)t * a.proj_stride;
    if (g < C) {
        // early: the conv state (last written by this kernel one step ago), the static weights and the slot table are read before
        // the wait for the projection (see gdn_fstep_k for when that is allowed)
        float *st = pool + ((size_t)sids[t] * a.nlayers + a.layer) * 3 * C;
        const float s0 = st[g], s1 = st[C + g], s2 = st[2 * C + g];
        const float4 w = *(const float4 *)(cw + 4 * (size_t)g);
        if (early) pdl_wait();
        const float s3 = __half2float(pr[g]);
        const float y = w.x * s0 + w.y * s1 + w.z * s2 + w.w * s3;
        cv[(size_t)t * C + g] = __float2half_rn(y / (1.0f + expf(-y)));
        st[g] = s1;
        st[C + g] = s2;
        st[2 * C + g] = s3;
    } else if (g < C + HV) {
        if (early) pdl_wait();
        const uint32_t j = g - C;
        const float xa = __half2float(pr[C + HV * 128 + j]) + dtb[j];
        const float sp = xa > 20.0f ? xa : logf(1.0f + expf(xa));
        la[t * HV + j] = An[j] * sp;
    } else if (g < C + 2 * HV) {
        if (early) pdl_wait();
        const uint32_t j = g - C - HV;
        be[t * HV + j] = 1.0f / (1.0f + expf(-__half2float(pr[C + HV * 128 + HV + j])));
    }
}

static cudaError_t launch_dn_epi(const QwLaunch &L) {
    const uint32_t HK = (uint32_t)L.def("HK", 16), HV = (uint32_t)L.def("HV", 32), DK = (uint32_t)L.def("DK", 128), DV = (uint32_t)L.def("DV", 128);
    const uint32_t C = 2 * HK * DK + HV * DV;
    dn_epi_args a = L.bytes<dn_epi_args>(9);
    QW_CHECK_ARG(DV == 128 && DK == 128 && L.has_bytes(9, 16) && a.nb >= 1 && a.nb <= 64 && a.layer < a.nlayers);
    QW_CHECK_ARG(a.proj_stride >= C + HV * DV + 2 * HV);
    for (int i = 0; i <= 8; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= ((size_t)(a.nb - 1) * a.proj_stride + C + HV * DV + 2 * HV) * 2 && L.avail(1) >= (size_t)C * 16 &&
                 L.avail(5) >= (size_t)a.nb * C * 2 && L.avail(6) >= (size_t)a.nb * HV * 4 && L.avail(7) >= (size_t)a.nb * HV * 4 &&
                 L.avail(8) >= (size_t)a.nb * 4);
    qw_launch(dn_epi_k, dim3((C + 2 * HV + 255) / 256, a.nb), 256, 0, L.stream, L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<float>(3),
                                                                        L.buf<float>(4), L.buf<__half>(5), L.buf<float>(6), L.buf<float>(7),
                                                                        L.buf<int32_t>(8), a, C, HV, L.def("EARLY", 0) != 0);
    return cudaGetLastError();
}
QW_FAMILY(dn_epi, launch_dn_epi, 256)

// ------------------------------------------------------------------------------------------------ recurrent step
struct gdn_args {
    uint32_t nb, layer, nlayers, z_stride;  // z: fp16 rows of stride z_stride (the z part of the projection)
};

// One block per (v-head, slot): 512 threads, thread (rq = tid / 32, c4 = tid % 32) holds rows 8 rq .. 8 rq + 7 of columns
// 4 c4 .. 4 c4 + 3 of the head's [DK][DV] state in registers: every state access is a 16-byte load or store and a warp
// moves one whole 512-byte row per instruction.  The 16 row groups meet in shared memory (summed in group order); q and k
// are normalised by every warp for itself, so the block has three barriers in all.
// binds: 0 = cv fp16 [nb][C], 1 = la [nb][HV], 2 = beta [nb][HV], 3 = state pool fp32 [slot][nlayers][HV][DK][DV],
// 4 = z fp16, 5 = norm weight fp32 [DV], 6 = gy out fp16 [nb][HV*DV], 7 = slot ids, 8 = gdn_args; with O_OUT
// defined 1 also 9 = o out fp16 [nb][HV*DV] (the un-normalised output, for tests).  grid (HV, nb) x 512
template <bool TILED>
__global__ void __launch_bounds__(512, 2) gdn_fstep_k(const __half *cv, const float *la, const float *beta, float *pool, const __half *z,
                                                  const float *nw, __half *gy, const int32_t *sids, __half *oo, gdn_args a, uint32_t HK, uint32_t HV,
                                                  bool early) {
    constexpr int DK = 128, DV = 128;
    __shared__ float red[8];
    __shared__ float4 part[2][16][32];  // [S^T k | S^T q][row group][column quad]
    pdl_launch();
    if (!early) pdl_wait();
    const uint32_t hv = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, c4 = tid & 31, rq = tid >> 5, lane = tid & 31, warp = tid >> 5;
    const uint32_t hk = TILED ? hv % HK : hv / (HV / HK);
    const uint32_t C = 2 * HK * DK + HV * DV;
    const __half *row = cv + (size_t)t * C;
    float4 *S = (float4 *)(pool + (((size_t)sids[t] * a.nlayers + a.layer) * HV + hv) * DK * DV) + c4;

    // State rows into registers: the long-latency part.  With EARLY defined 1 they are requested before the wait for the previous
    // kernel.  The state of this (slot, layer, head) was last written by this kernel one step ago and the slot table at the step's
    // start.  A launch cannot begin before every block of its predecessor has started; the host defines EARLY only when at least two
    // launches that fill every SM (moe_ffn: as many blocks as fit the device) lie between those writers and this launch -- the later
    // one cannot have started all its blocks before the earlier one has left, and that one has waited for everything before it.
    float4 s[8];
#pragma unroll
    for (int i = 0; i < 8; i++) s[i] = S[(size_t)(8 * rq + i) * (DV / 4)];
    if (early) pdl_wait();  // q, k, v, z, the decay and beta are the previous kernels' output

    // q / k L2 normalisation, by every warp for itself (no block barrier): lane l squares elements 4l .. 4l+3, one butterfly
    // gives the head's sum of squares; then the warp's own eight rows 8 rq .. 8 rq + 7 are scaled
    const __half *qh = row + hk * DK, *kh = row + HK * DK + hk * DK;
    float qn[8], kn[8];
    {
        const uint2 q4 = *(const uint2 *)(qh + 4 * lane), k4 = *(const uint2 *)(kh + 4 * lane);
        const float2 qa = __half22float2(*(const __half2 *)&q4.x), qb = __half22float2(*(const __half2 *)&q4.y);
        const float2 ka = __half22float2(*(const __half2 *)&k4.x), kb = __half22float2(*(const __half2 *)&k4.y);
        const float qss = warp_sum(fmaf(qa.x, qa.x, fmaf(qa.y, qa.y, fmaf(qb.x, qb.x, qb.y * qb.y))));
        const float kss = warp_sum(fmaf(ka.x, ka.x, fmaf(ka.y, ka.y, fmaf(kb.x, kb.x, kb.y * kb.y))));
        const float rq_ = rsqrtf(qss / DK + GDN_EPS), rk_ = rsqrtf(kss / DK + GDN_EPS);
        const uint4 qr = *(const uint4 *)(qh + 8 * rq), kr = *(const uint4 *)(kh + 8 * rq);  // the warp's eight rows (same for all lanes)
        const uint32_t qw[4] = {qr.x, qr.y, qr.z, qr.w}, kw[4] = {kr.x, kr.y, kr.z, kr.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 qf = __half22float2(*(const __half2 *)&qw[j]), kf = __half22float2(*(const __half2 *)&kw[j]);
            qn[2 * j] = __half2float(__float2half_rn(qf.x * rq_ / DK));
            qn[2 * j + 1] = __half2float(__float2half_rn(qf.y * rq_ / DK));
            kn[2 * j] = __half2float(__float2half_rn(kf.x * rk_ * rsqrtf((float)DK)));
            kn[2 * j + 1] = __half2float(__float2half_rn(kf.y * rk_ * rsqrtf((float)DK)));
        }
    }

    const float gdec = expf(la[t * HV + hv]), b = beta[t * HV + hv];
    float4 mem = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float kk = kn[i];
        s[i].x *= gdec; s[i].y *= gdec; s[i].z *= gdec; s[i].w *= gdec;
        mem.x = fmaf(s[i].x, kk, mem.x); mem.y = fmaf(s[i].y, kk, mem.y); mem.z = fmaf(s[i].z, kk, mem.z); mem.w = fmaf(s[i].w, kk, mem.w);
    }
    part[0][rq][c4] = mem;
    __syncthreads();
    mem = part[0][0][c4];
#pragma unroll
    for (int r = 1; r < 16; r++) {
        const float4 pv = part[0][r][c4];
        mem.x += pv.x; mem.y += pv.y; mem.z += pv.z; mem.w += pv.w;
    }
    const uint2 vraw = *(const uint2 *)(row + 2 * HK * DK + hv * DV + 4 * c4);
    const float2 v01 = __half22float2(*(const __half2 *)&vraw.x), v23 = __half22float2(*(const __half2 *)&vraw.y);
    const float4 d = make_float4(b * (v01.x - mem.x), b * (v01.y - mem.y), b * (v23.x - mem.z), b * (v23.y - mem.w));
    float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float kk = kn[i], qq = qn[i];
        s[i].x = fmaf(kk, d.x, s[i].x); s[i].y = fmaf(kk, d.y, s[i].y); s[i].z = fmaf(kk, d.z, s[i].z); s[i].w = fmaf(kk, d.w, s[i].w);
        out.x = fmaf(s[i].x, qq, out.x); out.y = fmaf(s[i].y, qq, out.y); out.z = fmaf(s[i].z, qq, out.z); out.w = fmaf(s[i].w, qq, out.w);
    }
    part[1][rq][c4] = out;
#pragma unroll
    for (int i = 0; i < 8; i++) S[(size_t)(8 * rq + i) * (DV / 4)] = s[i];
    __syncthreads();
    float o1 = 0.f;
    const uint32_t c = tid;  // threads 0..127: one output column each
    if (tid < 128) {
        const float *pc = (const float *)&part[1][0][0] + c;
        o1 = pc[0];
#pragma unroll
        for (int r = 1; r < 16; r++) o1 += pc[r * 128];
        const __half oh = __float2half_rn(o1);
        if (oo) oo[(size_t)t * HV * DV + hv * DV + c] = oh;
        const float x = __half2float(oh);  // the norm sees the fp16-rounded output (kernels/gdn_decode.metal:386,408)
        const float p = warp_sum(x * x);
        if (lane == 0) red[warp] = p;
    }
    __syncthreads();
    if (tid < 128) {
        const float r = rsqrtf((((red[0] + red[1]) + red[2]) + red[3]) / DV + GDN_EPS);
        const float x = __half2float(__float2half_rn(o1));
        const float zz = __half2float(z[(size_t)t * a.z_stride + hv * DV + c]);
        gy[(size_t)t * HV * DV + hv * DV + c] = __float2half_rn(x * r * nw[c] * (1.0f / (1.0f + expf(-zz))));
    }
}

static cudaError_t launch_gdn_fstep(const QwLaunch &L) {
    const uint32_t HK = (uint32_t)L.def("HK", 16), HV = (uint32_t)L.def("HV", 32), DK = (uint32_t)L.def("DK", 128), DV = (uint32_t)L.def("DV", 128);
    const bool tiled = L.def("GDN_TILED", 1) != 0;
    const uint32_t C = 2 * HK * DK + HV * DV;
    gdn_args a = L.bytes<gdn_args>(8);
    QW_CHECK_ARG(DK == 128 && DV == 128 && HV % HK == 0 && L.has_bytes(8, 16) && a.nb >= 1 && a.nb <= 64 && a.layer < a.nlayers && a.z_stride >= HV * DV);
    for (int i = 0; i <= 7; i++) QW_CHECK_ARG(L.buf<void>(i) != nullptr);
    QW_CHECK_ARG(L.avail(0) >= (size_t)a.nb * C * 2 && L.avail(1) >= (size_t)a.nb * HV * 4 && L.avail(2) >= (size_t)a.nb * HV * 4 &&
                 L.avail(4) >= ((size_t)(a.nb - 1) * a.z_stride + HV * DV) * 2 && L.avail(5) >= DV * 4 && L.avail(6) >= (size_t)a.nb * HV * DV * 2 &&
                 L.avail(7) >= (size_t)a.nb * 4);
    QW_CHECK_ARG(L.tx == 512);
    const dim3 grid(HV, a.nb);
    const bool early = L.def("EARLY", 0) != 0;
    __half *oo = L.def("O_OUT", 0) ? L.buf<__half>(9) : nullptr;
    if (L.def("O_OUT", 0)) QW_CHECK_ARG(oo && L.avail(9) >= (size_t)a.nb * HV * DV * 2);
    if (tiled)
        qw_launch(gdn_fstep_k<true>, grid, 512, 0, L.stream, L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<float>(3), L.buf<__half>(4),
                                                     L.buf<float>(5), L.buf<__half>(6), L.buf<int32_t>(7), oo, a, HK, HV, early);
    else
        qw_launch(gdn_fstep_k<false>, grid, 512, 0, L.stream, L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<float>(3), L.buf<__half>(4),
                                                      L.buf<float>(5), L.buf<__half>(6), L.buf<int32_t>(7), oo, a, HK, HV, early);
    return cudaGetLastError();
}
QW_FAMILY(gdn_fstep, launch_gdn_fstep, 512)
