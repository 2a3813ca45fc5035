// Internal interface between the gpu.h backend (gpu_cuda.cu) and the kernel families (k_*.cu).
// A family is a precompiled sm_100a kernel (or small set of template instances) plus a host launcher that
// reads the batch's bind slots the way the reference's MSL kernels read their [[buffer(i)]] arguments.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

struct QwBind {
    void *ptr;      // device address (buffer base + offset) or nullptr
    size_t avail;   // bytes from ptr to the end of the buffer
    uint32_t boff;  // offset of inline bytes in the batch arena
    uint32_t blen;  // length of inline bytes (0 = none)
};

struct QwDefs;  // name -> integer map of the `#define`s given to qw_gpu_compile
long qw_defs_get(const QwDefs *d, const char *name, long dflt);

struct QwLaunch {
    const QwDefs *defs;
    const QwBind *b;        // 32 slots
    const uint8_t *arena;   // inline bytes
    unsigned gx, gy, gz, tx, ty, tz;
    size_t tgmem;
    cudaStream_t stream;
    int sm_count;
    void *tables;           // device lookup tables shared by all kernels of this device (see k_tables.cu)
    unsigned *status;       // device view of a pinned host word: 0, or the code of the first kernel that gave up a wait

    long def(const char *name, long dflt) const { return qw_defs_get(defs, name, dflt); }
    template <class T> T *buf(int i) const { return (T *)b[i].ptr; }
    size_t avail(int i) const { return b[i].avail; }
    bool has_bytes(int i, size_t n) const { return b[i].blen >= n; }
    template <class T> T bytes(int i) const {
        T v;
        memset(&v, 0, sizeof v);
        memcpy(&v, arena + b[i].boff, b[i].blen < sizeof v ? b[i].blen : sizeof v);
        return v;
    }
};

// A launcher returns cudaSuccess, a CUDA error, or cudaErrorInvalidValue for bad bindings / sizes.
typedef cudaError_t (*qw_launch_fn)(const QwLaunch &);

struct QwFamily {
    const char *name;
    qw_launch_fn fn;
    unsigned max_threads;
    QwFamily *next;
};
void qw_register_family(QwFamily *f);

#define QW_FAMILY(NAME, FN, MAXTHR)                                  \
    static QwFamily qw_fam_##NAME = {#NAME, FN, MAXTHR, nullptr};   \
    static int qw_fam_reg_##NAME = (qw_register_family(&qw_fam_##NAME), 0);

// Lookup tables in device memory, built once per device at qw_gpu_open (k_tables.cu).
struct QwTables {
    uint32_t grid_u32[512];          // IQ3_S codebook, 4 unsigned bytes per entry
    uint2 grid_h4[512 * 16];         // the same as 4 fp16 values, 16 interleaved copies (entry e, copy c at e*16+c)
    uint2 grid_b4[512 * 16];         // the same as 4 bf16 values, 16 interleaved copies
    uint32_t grid_u32x32[512 * 32];  // grid_u32 in 32 interleaved copies (entry e, copy c at e*32+c): a warp's 32 lanes read 32 different banks
};
cudaError_t qw_tables_create(void **out, cudaStream_t s);

// Kernel launch used by every family.  With programmatic dependent launch enabled (the default; QW_PDL=0 or qw_set_pdl turn it off) the launch
// carries the programmatic-stream-serialization attribute: the kernel may start while its predecessor in the stream is
// still finishing, runs its data-independent prologue (barrier set-up, lookup tables, staging of weights) and blocks in
// pdl_wait() (common.cuh) until the predecessor's results are complete and visible.  Every kernel of this library
// calls pdl_wait() before it reads or writes anything a predecessor may touch.
bool qw_pdl_enabled();  // for the kernel family being launched (QW_PDL_OFF=name,name excludes families, for debugging)
void qw_set_pdl(bool on);
void qw_pdl_current_family(const char *name);
template <typename... KArgs, typename... Args>
static inline cudaError_t qw_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = qw_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define QW_CHECK_ARG(cond)                         \
    do {                                           \
        if (!(cond)) return cudaErrorInvalidValue; \
    } while (0)
