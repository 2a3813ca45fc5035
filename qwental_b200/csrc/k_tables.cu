// Lookup tables built once per device at qw_gpu_open -- the role of gg_tab_init in the reference
// (kernels/moe_gg.metal:495-515), here computed on the host and uploaded.
#include "qw_kern.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <vector>

static const uint32_t h_iq3s_grid[512] = {
#include "_gen/iq3s_grid.inc"
};

cudaError_t qw_tables_create(void **out, cudaStream_t s) {
    std::vector<QwTables> hv(1);
    QwTables &t = hv[0];
    for (int e = 0; e < 512; e++) {
        const uint32_t w = h_iq3s_grid[e];
        t.grid_u32[e] = w;
        uint16_t h[4], b[4];
        for (int j = 0; j < 4; j++) {
            const float v = (float)((w >> (8 * j)) & 255);
            const __half hh = __float2half(v);
            const __nv_bfloat16 bb = __float2bfloat16(v);
            memcpy(&h[j], &hh, 2);
            memcpy(&b[j], &bb, 2);
        }
        for (int c = 0; c < 32; c++) t.grid_u32x32[e * 32 + c] = w;
        for (int c = 0; c < 16; c++) {
            t.grid_h4[e * 16 + c] = make_uint2(h[0] | ((uint32_t)h[1] << 16), h[2] | ((uint32_t)h[3] << 16));
            t.grid_b4[e * 16 + c] = make_uint2(b[0] | ((uint32_t)b[1] << 16), b[2] | ((uint32_t)b[3] << 16));
        }
    }
    void *d = nullptr;
    cudaError_t e = cudaMalloc(&d, sizeof(QwTables));
    if (e != cudaSuccess) return e;
    e = cudaMemcpyAsync(d, &t, sizeof(QwTables), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        cudaFree(d);
        return e;
    }
    *out = d;
    return cudaSuccess;
}
