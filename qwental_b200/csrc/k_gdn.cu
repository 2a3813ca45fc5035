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
                                               float *la, float *be, const int32_t *sids, dn_epi_args a, uint32_t C, uint32_t HV) {
    pdl_sync();
    const uint32_t g = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
    const __half *pr = proj + (size_t)t * a.proj_stride;
    if (g < C) {
        float *st = pool + ((size_t)sids[t] * a.nlayers + a.layer) * 3 * C;
        const float s0 = st[g], s1 = st[C + g], s2 = st[2 * C + g], s3 = __half2float(pr[g]);
        const float4 w = *(const float4 *)(cw + 4 * (size_t)g);
        const float y = w.x * s0 + w.y * s1 + w.z * s2 + w.w * s3;
        cv[(size_t)t * C + g] = __float2half_rn(y / (1.0f + expf(-y)));
        st[g] = s1;
        st[C + g] = s2;
        st[2 * C + g] = s3;
    } else if (g < C + HV) {
        const uint32_t j = g - C;
        const float xa = __half2float(pr[C + HV * 128 + j]) + dtb[j];
        const float sp = xa > 20.0f ? xa : logf(1.0f + expf(xa));
        la[t * HV + j] = An[j] * sp;
    } else if (g < C + 2 * HV) {
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
                                                                        L.buf<int32_t>(8), a, C, HV);
    return cudaGetLastError();
}
QW_FAMILY(dn_epi, launch_dn_epi, 256)

// ------------------------------------------------------------------------------------------------ recurrent step
struct gdn_args {
    uint32_t nb, layer, nlayers, z_stride;  // z: fp16 rows of stride z_stride (the z part of the projection)
};

// One block per (v-head, slot): 512 threads, thread (qr = tid / 128, c = tid % 128) holds the 32 rows
// 32 qr .. 32 qr + 31 of column c of the head's [DK][DV] state in registers.  Row reads are 512-byte coalesced.
// binds: 0 = cv fp16 [nb][C], 1 = la [nb][HV], 2 = beta [nb][HV], 3 = state pool fp32 [slot][nlayers][HV][DK][DV],
// 4 = z fp16, 5 = norm weight fp32 [DV], 6 = gy out fp16 [nb][HV*DV], 7 = slot ids, 8 = gdn_args; with O_OUT
// defined 1 also 9 = o out fp16 [nb][HV*DV] (the un-normalised output, for tests).  grid (HV, nb) x 512
template <bool TILED>
__global__ void __launch_bounds__(512) gdn_fstep_k(const __half *cv, const float *la, const float *beta, float *pool, const __half *z,
                                                  const float *nw, __half *gy, const int32_t *sids, __half *oo, gdn_args a, uint32_t HK, uint32_t HV) {
    constexpr int DK = 128, DV = 128;
    __shared__ float ks[DK], qs[DK], part[4][DV], red[8];
    pdl_sync();
    const uint32_t hv = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, c = tid & 127, qr = tid >> 7, lane = tid & 31, warp = tid >> 5;
    const uint32_t hk = TILED ? hv % HK : hv / (HV / HK);
    const uint32_t C = 2 * HK * DK + HV * DV;
    const __half *row = cv + (size_t)t * C;
    float *S = pool + (((size_t)sids[t] * a.nlayers + a.layer) * HV + hv) * DK * DV;

    // state column into registers (issued first: the long-latency part)
    float s[32];
#pragma unroll
    for (int i = 0; i < 32; i++) s[i] = S[(size_t)(32 * qr + i) * DV + c];

    // q / k L2 normalisation (threads 0..127 take q, 128..255 take k)
    float xv = 0.f;
    if (tid < 128) xv = __half2float(row[hk * DK + tid]);
    else if (tid < 256) xv = __half2float(row[HK * DK + hk * DK + (tid - 128)]);
    const float ssq = warp_sum(xv * xv);
    if (warp < 8 && lane == 0) red[warp] = ssq;
    __syncthreads();
    if (tid < 128) {
        const float r = rsqrtf((((red[0] + red[1]) + red[2]) + red[3]) / DK + GDN_EPS);
        qs[tid] = __half2float(__float2half_rn(xv * r / DK));
    } else if (tid < 256) {
        const float r = rsqrtf((((red[4] + red[5]) + red[6]) + red[7]) / DK + GDN_EPS);
        ks[tid - 128] = __half2float(__float2half_rn(xv * r * rsqrtf((float)DK)));
    }
    __syncthreads();

    const float gdec = expf(la[t * HV + hv]), b = beta[t * HV + hv];
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        s[i] = s[i] * gdec;
        mem = fmaf(s[i], ks[32 * qr + i], mem);
    }
    part[qr][c] = mem;
    __syncthreads();
    mem = ((part[0][c] + part[1][c]) + part[2][c]) + part[3][c];
    const float d = b * (__half2float(row[2 * HK * DK + hv * DV + c]) - mem);
    __syncthreads();
    float out = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        s[i] = fmaf(ks[32 * qr + i], d, s[i]);
        out = fmaf(s[i], qs[32 * qr + i], out);
    }
    part[qr][c] = out;
#pragma unroll
    for (int i = 0; i < 32; i++) S[(size_t)(32 * qr + i) * DV + c] = s[i];
    __syncthreads();
    if (tid < 128) {
        out = ((part[0][c] + part[1][c]) + part[2][c]) + part[3][c];
        const __half oh = __float2half_rn(out);
        if (oo) oo[(size_t)t * HV * DV + hv * DV + c] = oh;
        const float x = __half2float(oh);  // the norm sees the fp16-rounded output (kernels/gdn_decode.metal:386,408)
        const float p = warp_sum(x * x);
        if (lane == 0) red[warp] = p;
    }
    __syncthreads();
    if (tid < 128) {
        const float r = rsqrtf((((red[0] + red[1]) + red[2]) + red[3]) / DV + GDN_EPS);
        const float x = __half2float(__float2half_rn(out));
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
    __half *oo = L.def("O_OUT", 0) ? L.buf<__half>(9) : nullptr;
    if (L.def("O_OUT", 0)) QW_CHECK_ARG(oo && L.avail(9) >= (size_t)a.nb * HV * DV * 2);
    if (tiled)
        qw_launch(gdn_fstep_k<true>, grid, 512, 0, L.stream, L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<float>(3), L.buf<__half>(4),
                                                     L.buf<float>(5), L.buf<__half>(6), L.buf<int32_t>(7), oo, a, HK, HV);
    else
        qw_launch(gdn_fstep_k<false>, grid, 512, 0, L.stream, L.buf<__half>(0), L.buf<float>(1), L.buf<float>(2), L.buf<float>(3), L.buf<__half>(4),
                                                      L.buf<float>(5), L.buf<__half>(6), L.buf<int32_t>(7), oo, a, HK, HV);
    return cudaGetLastError();
}
QW_FAMILY(gdn_fstep, launch_gdn_fstep, 512)
