/* qw_gpu_ext.h -- additions to qw_gpu.h that the reference's unified-memory device layer has no need for.
 * None of these has a counterpart in src/gpu.h; a host that only uses qw_gpu.h still works, it just keeps
 * every buffer in managed memory.
 */
#ifndef QW_GPU_EXT_H
#define QW_GPU_EXT_H
#include "qw_gpu.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Where a buffer lives.  SHARED = what qw_buf_new gives (managed, ptr valid on both sides).
 * DEVICE = HBM only, ptr == NULL: per-slot KV pages, recurrent state, scratch, weights.
 * HOSTIO = pinned host memory mapped into the device: small per-step inputs/outputs (token ids, sampled ids)
 * that the host touches every step. */
enum { QW_BUF_SHARED = 0, QW_BUF_DEVICE = 1, QW_BUF_HOSTIO = 2 };
bool qw_buf_new_kind(qw_gpu *g, size_t size, int kind, qw_buf *out);

/* Copies between host memory and any buffer, ordered after everything already submitted on the current
 * stream; they return when the copy is complete.  false on a range or CUDA error. */
bool qw_buf_upload(qw_gpu *g, const qw_buf *dst, size_t offset, const void *src, size_t len);
bool qw_buf_download(qw_gpu *g, const qw_buf *src, size_t offset, void *dst, size_t len);
bool qw_buf_zero(qw_gpu *g, const qw_buf *dst, size_t offset, size_t len);

/* Sharing a QW_BUF_DEVICE buffer between the processes of one machine (one process per GPU; no counterpart in the
 * single-device reference): the owner exports a 64-byte handle, a peer imports it and gets a buffer that maps the
 * owner's memory through NVLink peer access.  Free an imported buffer with qw_buf_free before the owner frees it. */
bool qw_buf_ipc_export(const qw_buf *b, void *handle64);
bool qw_buf_ipc_import(qw_gpu *g, const void *handle64, size_t size, qw_buf *out);

/* Device address of a buffer (for interop with other CUDA code in the same process). */
void *qw_buf_device_ptr(const qw_buf *b);
/* cudaStream_t of stream s (0 or 1), as an opaque pointer. */
void *qw_gpu_stream_handle(qw_gpu *g, int s);
/* Message of the most recent failure on this device ("" if none). */
const char *qw_gpu_last_error(const qw_gpu *g);
/* Number of kernel launches issued by batches since qw_gpu_open (graph replays count their nodes). */
unsigned long long qw_gpu_launch_count(const qw_gpu *g);
/* Replay identical batches as CUDA graphs (default off; QW_GRAPH=1 in the environment turns it on). */
void qw_gpu_set_graphs(qw_gpu *g, bool on);

/* Programmatic dependent launch for the kernels of later batches (default on; QW_PDL=0 in the environment turns it
 * off): each kernel may start while its predecessor drains and waits on the device for the predecessor's results. */
void qw_gpu_set_pdl(qw_gpu *g, bool on);

/* Attention core + merge with NO allocation anywhere on the path (no counterpart in the reference: its device
 * layer allocates freely from unified memory).  For callers that cannot allocate device memory -- a process whose
 * HBM was fully planned at start-up, or a host thread that may not call cudaMalloc because a stream capture is open.
 * The split-K partials live in a static device array inside the library (8.45 MB per GPU, held until exit), so
 * nb * max_chunks must be <= 512 (e.g. 16 slots of up to 8192 tokens); heads fixed at 16 q / 2 kv / dim 256.
 * Inputs are what qsa_attn + qsa_merge take through a batch: q fp16 [nb][16][256] (already normalised and rotated),
 * the paged KV pool and its size in bytes, the page table int32 [slots][max_pages], pos / slot_ids int32 [nb],
 * qkv fp16 rows (for the output gate), y fp16 [nb][4096] out; `stream` is a cudaStream_t.  All pointers are device
 * pointers; every row must satisfy pos[t] + 1 <= max_chunks * 256 (the entry point cannot read device memory to check:
 * a longer row is attended over its first max_chunks pages only).  The first call on a device looks up the array's
 * address: make it outside any stream capture.  Calls that overlap on the GPU share the array and race: serialise
 * them.  Returns 0, or a negative code with a message in err (-1: bad argument, -2: the request exceeds the static
 * scratch, -3: CUDA error). */
int qw_attn_decode_static(const void *q, const void *kv_pool, size_t kv_pool_bytes, const int32_t *page_table, const int32_t *pos,
                          const int32_t *slot_ids, const void *qkv, void *y, uint32_t nb, uint32_t layer, uint32_t nlayers, uint32_t qkv_stride,
                          uint32_t max_pages, uint32_t max_chunks, void *stream, char *err, size_t errlen);

/* What qw_gpu_compile would make of a source text, without a device: writes "family entry NAME=VALUE ..." (or the
 * error message) into out and returns whether the prelude is valid. */
bool qw_gpu_prelude_describe(const char *src, size_t len, char *out, size_t outlen);

/* Precompiled kernel families that qw_gpu_compile can register. */
int qw_gpu_family_count(void);
const char *qw_gpu_family_name(int i);

#ifdef __cplusplus
}
#endif
#endif
