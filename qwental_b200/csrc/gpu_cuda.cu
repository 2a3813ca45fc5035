// gpu_cuda: the reference's device interface (src/gpu.h in hy-ong/qwental) on one CUDA device.
// Replaces src/gpu_metal.m behaviour for behaviour: named kernels, bind-by-index batches that execute in
// submission order, one wait per step that returns GPU seconds (negative on failure), per-dispatch
// profiling.  The kernels themselves are the precompiled families registered by the k_*.cu files.
#include "../../include/qw_gpu_ext.h"
#include "qw_kern.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <time.h>
#include <unordered_map>
#include <vector>

// ------------------------------------------------------------------------------------------------ launch mode
static int g_pdl = -1;
static const char *g_pdl_family = "";
void qw_pdl_current_family(const char *name) { g_pdl_family = name ? name : ""; }
bool qw_pdl_enabled() {
    if (g_pdl < 0) {
        const char *e = getenv("QW_PDL");
        g_pdl = e ? (atoi(e) != 0) : 1;
    }
    if (!g_pdl) return false;
    static const char *off = getenv("QW_PDL_OFF");  // comma-separated families launched without the attribute
    if (off && *g_pdl_family) {
        const size_t n = strlen(g_pdl_family);
        for (const char *p = off; (p = strstr(p, g_pdl_family)) != nullptr; p += n)
            if ((p == off || p[-1] == ',') && (p[n] == 0 || p[n] == ',')) return false;
    }
    return true;
}
void qw_set_pdl(bool on) { g_pdl = on ? 1 : 0; }
static void graph_cache_clear(qw_gpu *g);
extern "C" void qw_gpu_set_pdl(qw_gpu *g, bool on) {
    if (g) graph_cache_clear(g);  // recorded graphs carry the launch attributes of the mode they were captured in
    qw_set_pdl(on);
}

// ------------------------------------------------------------------------------------------------ registry
static QwFamily *g_families = nullptr;
void qw_register_family(QwFamily *f) {
    f->next = g_families;
    g_families = f;
}
static QwFamily *find_family(const std::string &n) {
    for (QwFamily *f = g_families; f; f = f->next)
        if (n == f->name) return f;
    return nullptr;
}

struct QwDefs {
    std::map<std::string, long> v;
};
long qw_defs_get(const QwDefs *d, const char *name, long dflt) {
    if (!d) return dflt;
    auto it = d->v.find(name);
    return it == d->v.end() ? dflt : it->second;
}

// ------------------------------------------------------------------------------------------------ objects
struct BufRec {
    void *dev;
    void *host;
    size_t size;
    int kind;      // QW_BUF_*; 3 = wrap (device copy, host pointer is the caller's)
    int device;
};

struct qw_kernel {
    std::string name;
    QwFamily *fam;
    QwDefs defs;
};

struct Rec {
    qw_kernel *k;
    QwBind b[32];
    unsigned gx, gy, gz, tx, ty, tz;
    size_t tgmem;
};

struct ProfEnt {
    std::string name;
    double us;
};

struct qw_gpu {
    int dev;
    int sm_count;
    size_t total_mem;
    char name[256];
    cudaStream_t stream[2];
    int cur;
    std::map<std::string, qw_kernel *> kernels;
    bool profile;
    std::vector<ProfEnt> prof;
    std::string err;
    unsigned long long launches;
    bool graphs;
    // CUDA graphs of recorded batches, keyed by a hash of everything a replay depends on (kernel, its specialisation, grid,
    // threadgroup memory, bound addresses, inline bytes, stream, dependent-launch mode); the key bytes are kept and compared
    // on a hit.  Cleared whenever a kernel is re-specialised or the launch mode changes; capped in size.
    struct GraphEnt {
        cudaGraphExec_t exec;
        std::vector<uint8_t> key;
    };
    std::unordered_map<uint64_t, GraphEnt> graph_cache;
    void *tables;
    unsigned *status_host, *status_dev;
};

struct qw_batch {
    qw_gpu *g;
    cudaStream_t stream;
    std::vector<Rec> recs;
    std::vector<uint8_t> arena;
    qw_kernel *cur_k;
    QwBind cur_b[32];
    size_t cur_tg;
    cudaEvent_t e0, e1;
    std::vector<cudaEvent_t> pev;  // profiling: 2 per dispatch
    bool submitted, failed;
};

static void graph_cache_clear(qw_gpu *g) {
    for (auto &kv : g->graph_cache) cudaGraphExecDestroy(kv.second.exec);
    g->graph_cache.clear();
}

static void set_err(qw_gpu *g, const char *what, cudaError_t e) {
    char buf[512];
    snprintf(buf, sizeof buf, "%s: %s", what, e == cudaSuccess ? "invalid argument" : cudaGetErrorString(e));
    g->err = buf;
    if (getenv("QW_GPU_VERBOSE")) fprintf(stderr, "[gpu_cuda] %s\n", buf);
}

// ------------------------------------------------------------------------------------------------ device
extern "C" qw_gpu *qw_gpu_open(void) {
    int dev = 0;
    const char *e = getenv("QW_CUDA_DEVICE");
    if (!e) e = getenv("LOCAL_RANK");
    if (e) dev = atoi(e);
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) return nullptr;
    if (dev < 0 || dev >= n) dev = dev % n;
    if (cudaSetDevice(dev) != cudaSuccess) return nullptr;
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return nullptr;
    qw_gpu *g = new qw_gpu();
    g->dev = dev;
    g->sm_count = p.multiProcessorCount;
    g->total_mem = p.totalGlobalMem;
    snprintf(g->name, sizeof g->name, "%s (sm_%d%d, %d SMs)", p.name, p.major, p.minor, p.multiProcessorCount);
    g->cur = 0;
    g->profile = false;
    g->launches = 0;
    const char *gr = getenv("QW_GRAPH");
    g->graphs = gr && atoi(gr) != 0;
    g->tables = nullptr;
    g->status_host = g->status_dev = nullptr;
    if (cudaHostAlloc((void **)&g->status_host, 64, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer((void **)&g->status_dev, g->status_host, 0) != cudaSuccess) {
        delete g;
        return nullptr;
    }
    memset(g->status_host, 0, 64);
    for (int i = 0; i < 2; i++)
        if (cudaStreamCreateWithFlags(&g->stream[i], cudaStreamNonBlocking) != cudaSuccess) {
            delete g;
            return nullptr;
        }
    if (qw_tables_create(&g->tables, g->stream[0]) != cudaSuccess || cudaStreamSynchronize(g->stream[0]) != cudaSuccess) {
        delete g;
        return nullptr;
    }
    return g;
}

extern "C" void qw_gpu_close(qw_gpu *g) {
    if (!g) return;
    cudaSetDevice(g->dev);
    cudaDeviceSynchronize();
    graph_cache_clear(g);
    for (auto &kv : g->kernels) delete kv.second;
    if (g->tables) cudaFree(g->tables);
    if (g->status_host) cudaFreeHost(g->status_host);
    for (int i = 0; i < 2; i++) cudaStreamDestroy(g->stream[i]);
    delete g;
}

extern "C" const char *qw_gpu_name(const qw_gpu *g) { return g ? g->name : ""; }
extern "C" size_t qw_gpu_max_working_set(const qw_gpu *g) { return g ? g->total_mem : 0; }
extern "C" const char *qw_gpu_last_error(const qw_gpu *g) { return g ? g->err.c_str() : "no device"; }
extern "C" unsigned long long qw_gpu_launch_count(const qw_gpu *g) { return g ? g->launches : 0; }
extern "C" void qw_gpu_set_graphs(qw_gpu *g, bool on) {
    if (g) g->graphs = on;
}
extern "C" void *qw_gpu_stream_handle(qw_gpu *g, int s) { return g ? (void *)g->stream[s ? 1 : 0] : nullptr; }
extern "C" int qw_gpu_family_count(void) {
    int n = 0;
    for (QwFamily *f = g_families; f; f = f->next) n++;
    return n;
}
extern "C" const char *qw_gpu_family_name(int i) {
    for (QwFamily *f = g_families; f; f = f->next)
        if (i-- == 0) return f->name;
    return nullptr;
}

// ------------------------------------------------------------------------------------------------ kernels
static bool is_ident(const std::string &s) {
    if (s.empty() || (!(isalpha((unsigned char)s[0]) || s[0] == '_'))) return false;
    for (char c : s)
        if (!(isalnum((unsigned char)c) || c == '_')) return false;
    return true;
}

// Parses the `#define` prelude of a kernel source (see qw_gpu_compile in qw_gpu.h).  Pure host logic: no device needed.
static bool parse_prelude(const char *src, size_t len, std::string &family, std::string &entry, QwDefs &defs, std::string &msg) {
    std::vector<std::pair<std::string, std::string>> idents;
    size_t i = 0;
    while (i < len) {
        size_t e = i;
        while (e < len && src[e] != '\n') e++;
        std::string line(src + i, e - i);
        i = e + 1;
        size_t a = line.find_first_not_of(" \t\r");
        if (a == std::string::npos) continue;
        if (line.compare(a, 2, "//") == 0) continue;
        if (line.compare(a, 7, "#define") != 0) break;  // end of the prelude
        char nm[128] = {0}, val[256] = {0};
        int got = sscanf(line.c_str() + a + 7, " %127s %255[^\n\r]", nm, val);
        if (got < 1) {
            msg = "qw_gpu_compile: malformed #define: " + line;
            return false;
        }
        std::string v(val);
        size_t c = v.find("//");
        if (c != std::string::npos) v = v.substr(0, c);
        while (!v.empty() && isspace((unsigned char)v.back())) v.pop_back();
        std::string name(nm);
        if (name == "QW_KERNEL") family = v;
        else if (name == "QW_NAME") entry = v;
        else if (got == 2 && !v.empty()) {
            char *endp = nullptr;
            long num = strtol(v.c_str(), &endp, 0);
            if (endp && endp != v.c_str() && (*endp == 0 || *endp == 'u' || *endp == 'U' || *endp == 'l' || *endp == 'L')) defs.v[name] = num;
            else if (name == "YT") defs.v["YT_F32"] = v == "float";  // the reference's output-type define of qmv_gg (kernels/qmv_gg.metal:4-6)
            else if (is_ident(v)) idents.push_back({name, v});
        } else defs.v[name] = 1;
    }
    // the reference's renaming form: #define <family> <entry>
    for (auto &p : idents)
        if (family.empty() && find_family(p.first)) {
            family = p.first;
            if (entry.empty()) entry = p.second;
        }
    if (family.empty()) {
        msg = "qw_gpu_compile: the prelude names no kernel family (#define QW_KERNEL <family>)";
        return false;
    }
    if (!find_family(family)) {
        msg = "qw_gpu_compile: unknown kernel family '" + family + "'";
        return false;
    }
    if (entry.empty()) entry = family;
    if (!is_ident(entry)) {
        msg = "qw_gpu_compile: bad entry name '" + entry + "'";
        return false;
    }
    return true;
}

// Host-logic probe of the prelude parser (no device): writes "family entry NAME=VALUE ..." into out.
extern "C" bool qw_gpu_prelude_describe(const char *src, size_t len, char *out, size_t outlen) {
    std::string family, entry, msg;
    QwDefs defs;
    const bool ok = src && parse_prelude(src, len, family, entry, defs, msg);
    std::string r = ok ? family + " " + entry : msg;
    if (ok)
        for (auto &kv : defs.v) r += " " + kv.first + "=" + std::to_string(kv.second);
    if (out && outlen) snprintf(out, outlen, "%s", r.c_str());
    return ok;
}

extern "C" bool qw_gpu_compile(qw_gpu *g, const char *src, size_t len, char *err, size_t errlen) {
    auto fail = [&](const std::string &m) {
        if (err && errlen) snprintf(err, errlen, "%s", m.c_str());
        if (g) g->err = m;
        return false;
    };
    if (!g || !src) return fail("qw_gpu_compile: null argument");
    std::string family, entry, msg;
    QwDefs defs;
    if (!parse_prelude(src, len, family, entry, defs, msg)) return fail(msg);
    QwFamily *f = find_family(family);
    qw_kernel *k = new qw_kernel();
    k->name = entry;
    k->fam = f;
    k->defs = defs;
    auto it = g->kernels.find(entry);
    if (it != g->kernels.end()) {
        // Replace in place: handles already given out keep working and see the new specialisation; graphs recorded with
        // the old one must not be replayed.
        it->second->fam = f;
        it->second->defs = defs;
        delete k;
        graph_cache_clear(g);
    } else g->kernels[entry] = k;
    if (err && errlen) err[0] = 0;
    return true;
}

extern "C" qw_kernel *qw_kernel_get(qw_gpu *g, const char *name) {
    if (!g || !name) return nullptr;
    auto it = g->kernels.find(name);
    return it == g->kernels.end() ? nullptr : it->second;
}
extern "C" unsigned qw_kernel_max_threads(const qw_kernel *k) { return k ? k->fam->max_threads : 0; }
extern "C" unsigned qw_kernel_simd_width(const qw_kernel *k) { return k ? 32 : 0; }

// ------------------------------------------------------------------------------------------------ buffers
extern "C" bool qw_buf_new_kind(qw_gpu *g, size_t size, int kind, qw_buf *out) {
    if (!g || !out) return false;
    memset(out, 0, sizeof *out);
    if (size == 0) size = 16;
    cudaSetDevice(g->dev);
    // 256 spare bytes at the end: staged bulk copies round row ranges up to 16 bytes.
    const size_t alloc = (size + 255 + 256) & ~(size_t)255;
    BufRec *r = new BufRec{nullptr, nullptr, size, kind, g->dev};
    cudaError_t e;
    if (kind == QW_BUF_DEVICE) {
        e = cudaMalloc(&r->dev, alloc);
    } else if (kind == QW_BUF_HOSTIO) {
        e = cudaHostAlloc(&r->host, alloc, cudaHostAllocMapped | cudaHostAllocPortable);
        if (e == cudaSuccess) e = cudaHostGetDevicePointer(&r->dev, r->host, 0);
        if (e == cudaSuccess) memset(r->host, 0, alloc);
    } else if (kind == QW_BUF_SHARED) {
        e = cudaMallocManaged(&r->dev, alloc, cudaMemAttachGlobal);
        r->host = r->dev;
    } else e = cudaErrorInvalidValue;
    if (e != cudaSuccess) {
        set_err(g, "qw_buf_new", e);
        cudaGetLastError();
        delete r;
        return false;
    }
    out->handle = r;
    out->ptr = r->host;
    out->size = size;
    return true;
}

extern "C" bool qw_buf_new(qw_gpu *g, size_t size, qw_buf *out) { return qw_buf_new_kind(g, size, QW_BUF_SHARED, out); }

extern "C" void qw_buf_free(qw_buf *b) {
    if (!b || !b->handle) return;
    BufRec *r = (BufRec *)b->handle;
    cudaSetDevice(r->device);
    if (r->kind == QW_BUF_HOSTIO) cudaFreeHost(r->host);
    else if (r->kind == 4) cudaIpcCloseMemHandle(r->dev);
    else cudaFree(r->dev);
    delete r;
    memset(b, 0, sizeof *b);
}

extern "C" void *qw_pool_push(void) { return nullptr; }
extern "C" void qw_pool_pop(void *) {}

extern "C" bool qw_buf_wrap(qw_gpu *g, void *ptr, size_t len, qw_buf *out) {
    if (!g || !ptr || !out || len == 0) return false;
    memset(out, 0, sizeof *out);
    cudaSetDevice(g->dev);
    const size_t alloc = (len + 255 + 256) & ~(size_t)255;
    BufRec *r = new BufRec{nullptr, ptr, len, 3, g->dev};
    cudaError_t e = cudaMalloc(&r->dev, alloc);
    if (e == cudaSuccess) e = cudaMemcpy(r->dev, ptr, len, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        set_err(g, "qw_buf_wrap", e);
        cudaGetLastError();
        if (r->dev) cudaFree(r->dev);
        delete r;
        return false;
    }
    out->handle = r;
    out->ptr = ptr;
    out->size = len;
    return true;
}

// ---- sharing a device buffer with the other processes of the same machine (one process per GPU): the owner exports a
// 64-byte handle, a peer imports it and gets a buffer whose device address maps the owner's memory over NVLink.
extern "C" bool qw_buf_ipc_export(const qw_buf *b, void *handle64) {
    if (!b || !b->handle || !handle64) return false;
    BufRec *r = (BufRec *)b->handle;
    if (r->kind != QW_BUF_DEVICE) return false;
    cudaIpcMemHandle_t h;
    cudaSetDevice(r->device);
    if (cudaIpcGetMemHandle(&h, r->dev) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    static_assert(sizeof h == 64, "CUDA IPC handles are 64 bytes");
    memcpy(handle64, &h, 64);
    return true;
}
extern "C" bool qw_buf_ipc_import(qw_gpu *g, const void *handle64, size_t size, qw_buf *out) {
    if (!g || !handle64 || !out) return false;
    memset(out, 0, sizeof *out);
    cudaSetDevice(g->dev);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        set_err(g, "qw_buf_ipc_import", e);
        cudaGetLastError();
        return false;
    }
    BufRec *r = new BufRec{p, nullptr, size, 4 /* imported */, g->dev};
    out->handle = r;
    out->ptr = nullptr;
    out->size = size;
    return true;
}

extern "C" void *qw_buf_device_ptr(const qw_buf *b) { return b && b->handle ? ((BufRec *)b->handle)->dev : nullptr; }

static bool range_ok(const qw_buf *b, size_t off, size_t len) { return b && b->handle && off <= b->size && len <= b->size - off; }

extern "C" bool qw_buf_upload(qw_gpu *g, const qw_buf *dst, size_t offset, const void *src, size_t len) {
    if (!g || !src || !range_ok(dst, offset, len)) return false;
    cudaSetDevice(g->dev);
    cudaStream_t s = g->stream[g->cur];
    cudaError_t e = cudaMemcpyAsync((char *)qw_buf_device_ptr(dst) + offset, src, len, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) set_err(g, "qw_buf_upload", e);
    return e == cudaSuccess;
}
extern "C" bool qw_buf_download(qw_gpu *g, const qw_buf *src, size_t offset, void *dst, size_t len) {
    if (!g || !dst || !range_ok(src, offset, len)) return false;
    cudaSetDevice(g->dev);
    cudaStream_t s = g->stream[g->cur];
    cudaError_t e = cudaMemcpyAsync(dst, (char *)qw_buf_device_ptr(src) + offset, len, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) set_err(g, "qw_buf_download", e);
    return e == cudaSuccess;
}
extern "C" bool qw_buf_zero(qw_gpu *g, const qw_buf *dst, size_t offset, size_t len) {
    if (!g || !range_ok(dst, offset, len)) return false;
    cudaSetDevice(g->dev);
    cudaStream_t s = g->stream[g->cur];
    cudaError_t e = cudaMemsetAsync((char *)qw_buf_device_ptr(dst) + offset, 0, len, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) set_err(g, "qw_buf_zero", e);
    return e == cudaSuccess;
}

// ------------------------------------------------------------------------------------------------ batches
extern "C" qw_batch *qw_batch_begin(qw_gpu *g, bool /*concurrent*/) {
    // Dispatches of a batch always run in order on one stream: a valid execution of both the serial and
    // the concurrent-with-barriers modes of src/gpu.h:42-45.
    if (!g) return nullptr;
    qw_batch *b = new qw_batch();
    b->g = g;
    b->stream = g->stream[g->cur];
    b->cur_k = nullptr;
    memset(b->cur_b, 0, sizeof b->cur_b);
    b->cur_tg = 0;
    b->e0 = b->e1 = nullptr;
    b->submitted = b->failed = false;
    b->recs.reserve(1024);
    return b;
}

extern "C" void qw_batch_kernel(qw_batch *b, qw_kernel *k) {
    if (!b) return;
    if (!k) b->failed = true;
    b->cur_k = k;
}

extern "C" void qw_batch_buf(qw_batch *b, unsigned index, const qw_buf *buf, size_t offset) {
    if (!b || index >= 32) return;
    QwBind &d = b->cur_b[index];
    if (!buf || !buf->handle || offset > buf->size) {
        d = QwBind{nullptr, 0, 0, 0};
        if (buf && buf->handle) b->failed = true;
        return;
    }
    d.ptr = (char *)((BufRec *)buf->handle)->dev + offset;
    d.avail = buf->size - offset;
    d.blen = 0;
}

extern "C" void qw_batch_bytes(qw_batch *b, unsigned index, const void *data, size_t len) {
    if (!b || index >= 32 || !data) return;
    if (len > 256) {
        b->failed = true;
        return;
    }
    QwBind &d = b->cur_b[index];
    d.ptr = nullptr;
    d.avail = 0;
    d.boff = (uint32_t)b->arena.size();
    d.blen = (uint32_t)len;
    b->arena.insert(b->arena.end(), (const uint8_t *)data, (const uint8_t *)data + len);
}

extern "C" void qw_batch_threadgroup_mem(qw_batch *b, unsigned /*index*/, size_t len) {
    if (b) b->cur_tg = len;
}

extern "C" void qw_batch_dispatch(qw_batch *b, unsigned gx, unsigned gy, unsigned gz, unsigned tx, unsigned ty, unsigned tz) {
    if (!b) return;
    if (!b->cur_k) {
        b->failed = true;
        return;
    }
    Rec r;
    r.k = b->cur_k;
    memcpy(r.b, b->cur_b, sizeof r.b);
    r.gx = gx; r.gy = gy; r.gz = gz; r.tx = tx; r.ty = ty; r.tz = tz;
    r.tgmem = b->cur_tg;
    b->recs.push_back(r);
}

extern "C" void qw_batch_barrier(qw_batch *) {}
extern "C" void qw_batch_flush(qw_batch *) {}

static uint64_t hash_bytes(uint64_t h, const void *p, size_t n) {
    const uint8_t *c = (const uint8_t *)p;
    for (size_t i = 0; i < n; i++) h = (h ^ c[i]) * 0x100000001B3ull;
    return h;
}

static cudaError_t launch_one(qw_batch *b, const Rec &r) {
    QwLaunch L;
    L.defs = &r.k->defs;
    L.b = r.b;
    L.arena = b->arena.data();
    L.gx = r.gx; L.gy = r.gy; L.gz = r.gz; L.tx = r.tx; L.ty = r.ty; L.tz = r.tz;
    L.tgmem = r.tgmem;
    L.stream = b->stream;
    L.sm_count = b->g->sm_count;
    L.tables = b->g->tables;
    L.status = b->g->status_dev;
    qw_pdl_current_family(r.k->fam->name);
    cudaError_t e = r.k->fam->fn(L);
    if (e == cudaSuccess) e = cudaPeekAtLastError();
    return e;
}

static void run_records(qw_batch *b) {
    qw_gpu *g = b->g;
    const bool prof = g->profile;
    if (prof) {
        b->pev.resize(2 * b->recs.size());
        for (auto &ev : b->pev) cudaEventCreate(&ev);
    }
    for (size_t i = 0; i < b->recs.size() && !b->failed; i++) {
        if (prof) cudaEventRecord(b->pev[2 * i], b->stream);
        cudaError_t e = launch_one(b, b->recs[i]);
        if (prof) cudaEventRecord(b->pev[2 * i + 1], b->stream);
        if (e != cudaSuccess) {
            set_err(g, (std::string("dispatch of '") + b->recs[i].k->name + "'").c_str(), e);
            cudaGetLastError();
            b->failed = true;
        }
    }
    g->launches += b->recs.size();
}

extern "C" void qw_batch_submit(qw_batch *b) {
    if (!b || b->submitted) return;
    qw_gpu *g = b->g;
    b->submitted = true;
    cudaSetDevice(g->dev);
    cudaEventCreate(&b->e0);
    cudaEventCreate(&b->e1);
    if (b->failed) {
        if (g->err.empty()) g->err = "batch recorded an invalid kernel, buffer or byte argument";
        return;
    }
    cudaEventRecord(b->e0, b->stream);
    if (g->graphs && !g->profile && b->recs.size() > 1) {
        std::vector<uint8_t> key;
        key.reserve(b->recs.size() * 320);
        auto put = [&](const void *p, size_t n) { key.insert(key.end(), (const uint8_t *)p, (const uint8_t *)p + n); };
        for (const Rec &r : b->recs) {
            put(&r.k, sizeof r.k);
            put(&r.k->fam, sizeof r.k->fam);
            for (auto &kv : r.k->defs.v) {
                put(kv.first.data(), kv.first.size());
                put(&kv.second, sizeof kv.second);
            }
            put(&r.gx, 6 * sizeof(unsigned));
            put(&r.tgmem, sizeof r.tgmem);
            for (int i = 0; i < 32; i++) {
                put(&r.b[i].ptr, sizeof(void *));
                put(&r.b[i].blen, 4);
                if (r.b[i].blen) put(b->arena.data() + r.b[i].boff, r.b[i].blen);
            }
            qw_pdl_current_family(r.k->fam->name);
            const uint8_t pdl = qw_pdl_enabled() ? 1 : 0;
            put(&pdl, 1);
        }
        put(&b->stream, sizeof b->stream);
        const uint64_t h = hash_bytes(0xcbf29ce484222325ull, key.data(), key.size());
        auto it = g->graph_cache.find(h);
        if (it != g->graph_cache.end() && it->second.key != key) {  // a hash collision: the stored graph is another batch's
            cudaGraphExecDestroy(it->second.exec);
            g->graph_cache.erase(it);
            it = g->graph_cache.end();
        }
        if (it == g->graph_cache.end()) {
            if (g->graph_cache.size() >= 256) graph_cache_clear(g);  // e.g. one entry per (rows, chunk count) a long run went through
            cudaGraph_t graph = nullptr;
            cudaGraphExec_t exec = nullptr;
            cudaError_t e = cudaStreamBeginCapture(b->stream, cudaStreamCaptureModeThreadLocal);
            if (e == cudaSuccess) {
                for (size_t i = 0; i < b->recs.size() && !b->failed; i++) {
                    cudaError_t le = launch_one(b, b->recs[i]);
                    if (le != cudaSuccess) {
                        set_err(g, (std::string("capture of '") + b->recs[i].k->name + "'").c_str(), le);
                        b->failed = true;
                    }
                }
                e = cudaStreamEndCapture(b->stream, &graph);
            }
            if (e == cudaSuccess && !b->failed) e = cudaGraphInstantiate(&exec, graph, 0);
            if (graph) cudaGraphDestroy(graph);
            if (e != cudaSuccess || b->failed) {
                if (e != cudaSuccess) set_err(g, "graph capture", e);
                cudaGetLastError();
                b->failed = true;
                return;
            }
            it = g->graph_cache.emplace(h, qw_gpu::GraphEnt{exec, std::move(key)}).first;
        }
        cudaError_t e = cudaGraphLaunch(it->second.exec, b->stream);
        if (e != cudaSuccess) {
            set_err(g, "graph launch", e);
            b->failed = true;
        }
        g->launches += b->recs.size();
    } else run_records(b);
    cudaEventRecord(b->e1, b->stream);
}

extern "C" bool qw_batch_poll(qw_batch *b) {
    if (!b || !b->submitted || b->failed) return true;
    return cudaEventQuery(b->e1) != cudaErrorNotReady;
}

extern "C" double qw_batch_wait(qw_batch *b) {
    if (!b) return -1.0;
    if (!b->submitted) qw_batch_submit(b);
    qw_gpu *g = b->g;
    double secs = -1.0;
    if (!b->failed) {
        cudaError_t e = cudaEventSynchronize(b->e1);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e == cudaSuccess) {
            float ms = 0;
            e = cudaEventElapsedTime(&ms, b->e0, b->e1);
            if (e == cudaSuccess) secs = ms * 1e-3;
        }
        if (e != cudaSuccess) set_err(g, "qw_batch_wait", e);
        else if (*(volatile unsigned *)g->status_host != 0) {
            char m[96];
            snprintf(m, sizeof m, "a kernel gave up a bounded wait or rejected its arguments (status 0x%x)", *(volatile unsigned *)g->status_host);
            g->err = m;
            *(volatile unsigned *)g->status_host = 0;
            secs = -1.0;
        }
    }
    if (g->profile) {
        g->prof.clear();
        if (secs >= 0)
            for (size_t i = 0; i < b->recs.size() && 2 * i + 1 < b->pev.size(); i++) {
                float ms = 0;
                cudaEventElapsedTime(&ms, b->pev[2 * i], b->pev[2 * i + 1]);
                g->prof.push_back({b->recs[i].k->name, ms * 1e3});
            }
    }
    for (auto &ev : b->pev) cudaEventDestroy(ev);
    if (b->e0) cudaEventDestroy(b->e0);
    if (b->e1) cudaEventDestroy(b->e1);
    delete b;
    return secs;
}

extern "C" double qw_batch_end(qw_batch *b) {
    if (!b) return -1.0;
    qw_batch_submit(b);
    return qw_batch_wait(b);
}

extern "C" void qw_gpu_set_stream(qw_gpu *g, int s) {
    if (g) g->cur = s ? 1 : 0;
}

// ------------------------------------------------------------------------------------------------ profiling / misc
extern "C" void qw_profile_enable(qw_gpu *g, bool on) {
    if (g) g->profile = on;
}
extern "C" int qw_profile_count(const qw_gpu *g) { return g ? (int)g->prof.size() : 0; }
extern "C" const char *qw_profile_get(const qw_gpu *g, int i, double *us) {
    if (!g || i < 0 || i >= (int)g->prof.size()) return nullptr;
    if (us) *us = g->prof[i].us;
    return g->prof[i].name.c_str();
}

extern "C" double qw_now(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + ts.tv_nsec * 1e-9;
}

extern "C" double qw_gpu_empty_commit_latency(qw_gpu *g, qw_kernel * /*k*/, int n) {
    if (!g || n <= 0) return -1.0;
    cudaSetDevice(g->dev);
    cudaStream_t s = g->stream[g->cur];
    cudaEvent_t ev;
    cudaEventCreate(&ev);
    cudaStreamSynchronize(s);
    const double t0 = qw_now();
    for (int i = 0; i < n; i++) {
        cudaEventRecord(ev, s);
        cudaEventSynchronize(ev);
    }
    const double t1 = qw_now();
    cudaEventDestroy(ev);
    return (t1 - t0) / n;
}

extern "C" void qw_power_desc(char *out, size_t len) {
    if (out && len) snprintf(out, len, "power: mains (datacentre GPU); clocks are not set or reset by this library");
}
extern "C" bool qw_on_battery(void) { return false; }
