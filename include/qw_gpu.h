/* qw_gpu.h -- the device interface of the batched decode step, as a C ABI.
 *
 * libqw_gpu_cuda.so exports exactly the functions of the reference's device layer (src/gpu.h:18-83 in
 * hy-ong/qwental) with the same names, argument meaning and error behaviour, so a host written against
 * that header links against this library instead of the Metal backend (src/gpu_metal.m).  Each declaration
 * below cites the reference line it replaces.  Error channels are the reference's: NULL, false, or a
 * negative time from qw_batch_end / qw_batch_wait; nothing throws, nothing sets errno.
 *
 * Differences a host must know (they follow from discrete GPU memory, not from choice):
 *   - qw_buf_new returns CUDA managed memory: `ptr` is valid on host and device, coherent at the
 *     reference's own synchronisation points (after qw_batch_end / qw_batch_wait).
 *   - qw_buf_wrap uploads a private device copy of the region (weights live in HBM); later host writes
 *     to the wrapped region are not seen by kernels.
 *   - qw_gpu_compile cannot consume Metal source.  It reads the `#define` prelude the host prepends
 *     (src/engine.c:298-308) and registers a precompiled sm_100a kernel family under the requested name;
 *     see qw_gpu_compile below.
 */
#ifndef QW_GPU_H
#define QW_GPU_H
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct qw_gpu qw_gpu;       /* src/gpu.h:7 */
typedef struct qw_kernel qw_kernel; /* src/gpu.h:8 */
typedef struct qw_batch qw_batch;   /* src/gpu.h:9 */

/* src/gpu.h:11-15.  handle: backend record; ptr: host-visible address (NULL for device-only buffers made
 * through qw_gpu_ext.h); size: bytes.  The caller owns the struct; qw_buf_free zeroes it. */
typedef struct {
    void *handle;
    void *ptr;
    size_t size;
} qw_buf;

/* ---- device (src/gpu.h:18-21).  One device per process: the device index is read from QW_CUDA_DEVICE,
 * else LOCAL_RANK, else 0.  qw_gpu_open returns NULL on failure. */
qw_gpu *qw_gpu_open(void);
void qw_gpu_close(qw_gpu *g);
const char *qw_gpu_name(const qw_gpu *g);
size_t qw_gpu_max_working_set(const qw_gpu *g); /* total device memory in bytes */

/* ---- kernels.
 * src/gpu.h:25.  `src` is scanned for leading `#define NAME VALUE` lines (blank lines and // comments are
 * skipped, scanning stops at the first other line).  Required: `#define QW_KERNEL <family>` naming a
 * precompiled family (see qw_gpu_ext.h: qw_gpu_family_count/name).  Optional: `#define QW_NAME <entry>`
 * (the name qw_kernel_get will find; default = family), and any integer defines the family reads
 * (GF, KD, NB, ...).  The reference's renaming form `#define <family> <entry>` is accepted too.
 * Returns false and writes a message into err on an unknown family or a malformed prelude.  May be called
 * many times; a later registration of the same entry name replaces the earlier one (src/gpu_metal.m:132). */
bool qw_gpu_compile(qw_gpu *g, const char *src, size_t len, char *err, size_t errlen);
/* src/gpu.h:28-30.  NULL if the name was never registered. */
qw_kernel *qw_kernel_get(qw_gpu *g, const char *name);
unsigned qw_kernel_max_threads(const qw_kernel *k);
unsigned qw_kernel_simd_width(const qw_kernel *k); /* 32 */

/* ---- buffers (src/gpu.h:33-40) */
bool qw_buf_new(qw_gpu *g, size_t size, qw_buf *out);
void qw_buf_free(qw_buf *b);
void *qw_pool_push(void);      /* src/gpu.h:37: no-op off macOS */
void qw_pool_pop(void *pool);  /* src/gpu.h:38 */
bool qw_buf_wrap(qw_gpu *g, void *ptr, size_t len, qw_buf *out);

/* ---- batches (src/gpu.h:45-66).  A batch records dispatches and replays them in order on the CUDA stream
 * selected by qw_gpu_set_stream; bind slots 0..31; qw_batch_bytes holds up to 256 bytes per slot
 * (src/gpu_metal.m:21,63).  Grid sizes are in thread blocks (threadgroups). */
qw_batch *qw_batch_begin(qw_gpu *g, bool concurrent);
void qw_batch_kernel(qw_batch *b, qw_kernel *k);
void qw_batch_buf(qw_batch *b, unsigned index, const qw_buf *buf, size_t offset);
void qw_batch_bytes(qw_batch *b, unsigned index, const void *data, size_t len);
void qw_batch_threadgroup_mem(qw_batch *b, unsigned index, size_t len);
void qw_batch_dispatch(qw_batch *b, unsigned gx, unsigned gy, unsigned gz, unsigned tx, unsigned ty, unsigned tz);
void qw_batch_barrier(qw_batch *b);
void qw_batch_flush(qw_batch *b);
double qw_batch_end(qw_batch *b);   /* submit + wait; GPU seconds, negative on error; frees the batch */
void qw_batch_submit(qw_batch *b);
double qw_batch_wait(qw_batch *b);  /* GPU seconds, negative on error; frees the batch */
bool qw_batch_poll(qw_batch *b);
void qw_gpu_set_stream(qw_gpu *g, int s); /* 0 or 1 */

/* ---- profiling (src/gpu.h:70-72): per-dispatch kernel name and microseconds of the last ended batch */
void qw_profile_enable(qw_gpu *g, bool on);
int qw_profile_count(const qw_gpu *g);
const char *qw_profile_get(const qw_gpu *g, int i, double *us);

/* ---- misc (src/gpu.h:75-83) */
double qw_gpu_empty_commit_latency(qw_gpu *g, qw_kernel *k, int n);
void qw_power_desc(char *out, size_t len);
bool qw_on_battery(void);
double qw_now(void);

#ifdef __cplusplus
}
#endif
#endif
