// Runtime of libtrainlib_b200: device context, error state, staging arena, memory modes,
// streams mode, timers and the PMSIS stand-in (pi_cl_team_fork & friends).
#include "tl_common.h"
namespace tl { int conv_tc_status(); int *tc_status_word_if_any(); }
#include "../../include/pmsis.h"
#include <cstdarg>
#include <cstring>
#include <cstdlib>
#include <mutex>

namespace tl {

struct Chunk { char *base; size_t cap; size_t off; };

struct Context {
    bool inited = false;
    bool failed = false;
    int device = 0;
    int sms = 148;
    cudaStream_t own_stream = nullptr;
    cudaStream_t cur_stream = nullptr;
    int mem_mode = TL_MEM_AUTO;
    int n_streams = 1;
    int gemm_path = 0;
    long long launches = 0;
    std::vector<Chunk> chunks;     // staging arena; normally exactly one chunk
    int scope_depth = 0;
    bool arena_pinned = false;     // a captured graph holds arena addresses: never free or merge chunks again
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    int err = TL_OK;
    bool cuda_sticky = false;      // the context is lost: TL_ERR_CUDA cannot be cleared
    char err_msg[512] = {0};
};
static Context g;

void set_error(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    char buf[480];
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fprintf(stderr, "[trainlib_b200] %s\n", buf);
    if (g.err == TL_OK || (code == TL_ERR_CUDA && g.err != TL_ERR_CUDA)) {     // first error wins, except that a CUDA failure replaces a softer one
        g.err = code; snprintf(g.err_msg, sizeof g.err_msg, "%s", buf);
    }
}

// Errors that leave the CUDA context unusable (every later call fails too): only these make TL_ERR_CUDA permanent.
static bool cuda_error_is_sticky(cudaError_t e)
{
    switch (e) {
    case cudaErrorIllegalAddress: case cudaErrorLaunchFailure: case cudaErrorIllegalInstruction: case cudaErrorMisalignedAddress:
    case cudaErrorInvalidAddressSpace: case cudaErrorInvalidPc: case cudaErrorHardwareStackError: case cudaErrorAssert:
    case cudaErrorLaunchTimeout: case cudaErrorECCUncorrectable: case cudaErrorDevicesUnavailable: case cudaErrorNoDevice:
    case cudaErrorInsufficientDriver: case cudaErrorCudartUnloading: case cudaErrorContextIsDestroyed:
        return true;
    default:
        return false;
    }
}

bool cuda_ok(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return true;
    cudaGetLastError();                              // a non-sticky error must not resurface at the next launch check
    if (e == cudaErrorMemoryAllocation) {            // recoverable: callers fall back (smaller scratch, other kernel) or report it
        set_error(TL_ERR_NO_MEMORY, "allocation failed (%s) in %s", cudaGetErrorString(e), what);
        return false;
    }
    if (cuda_error_is_sticky(e)) g.cuda_sticky = true;
    set_error(TL_ERR_CUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return false;
}

static int init_device(int device)
{
    if (g.inited) return g.failed ? g.err : TL_OK;
    g.inited = true;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        g.failed = true;
        set_error(TL_ERR_NO_DEVICE, "no CUDA device available (%s); this library has no CPU fallback",
                  e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
        return g.err;
    }
    if (device < 0) {
        const char *env = getenv("TRAINLIB_B200_DEVICE");
        device = env ? atoi(env) : -1;
        if (device < 0) { if (cudaGetDevice(&device) != cudaSuccess) device = 0; }
    }
    if (!TL_CUDA(cudaSetDevice(device))) { g.failed = true; return g.err; }
    g.device = device;
    cudaDeviceProp prop;
    if (TL_CUDA(cudaGetDeviceProperties(&prop, device))) g.sms = prop.multiProcessorCount;
    if (!TL_CUDA(cudaStreamCreateWithFlags(&g.own_stream, cudaStreamNonBlocking))) { g.failed = true; return g.err; }
    g.cur_stream = g.own_stream;
    TL_CUDA(cudaEventCreate(&g.ev0));
    TL_CUDA(cudaEventCreate(&g.ev1));
    return TL_OK;
}

bool ready() { return init_device(-1) == TL_OK && !g.cuda_sticky && g.err != TL_ERR_NO_DEVICE; }
cudaStream_t stream() { return g.cur_stream; }
int streams() { return g.n_streams; }
int sm_count() { return g.sms; }
int gemm_path() { return g.gemm_path; }
void count_launch() { g.launches++; }

// ---------------------------------------------------------------- per-kernel profile
struct ProfEntry { const char *name; long long launches; double ms; double flops; };
struct ProfPending { int entry; cudaEvent_t a, b; };
static bool g_prof_on = false;
static std::vector<ProfEntry> g_prof;
static std::vector<ProfPending> g_prof_pending;
static std::vector<cudaEvent_t> g_prof_free;
static int g_prof_cur = -1;
static int g_prof_last = -1;          // entry of the launch begun last: profile_add_flops credits it
static const size_t PROF_MAX_PENDING = 8192;

bool profiling() { return g_prof_on; }

static void prof_drain()
{
    for (auto &p : g_prof_pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(p.b) == cudaSuccess && cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) g_prof[p.entry].ms += ms;
        g_prof_free.push_back(p.a); g_prof_free.push_back(p.b);
    }
    g_prof_pending.clear();
}

static cudaEvent_t prof_event()
{
    if (!g_prof_free.empty()) { cudaEvent_t e = g_prof_free.back(); g_prof_free.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

void profile_begin(const char *name)
{
    if (g_prof_pending.size() >= PROF_MAX_PENDING) prof_drain();
    int idx = -1;
    for (size_t i = 0; i < g_prof.size(); i++) if (g_prof[i].name == name || strcmp(g_prof[i].name, name) == 0) { idx = (int)i; break; }
    if (idx < 0) { g_prof.push_back({name, 0, 0.0, 0.0}); idx = (int)g_prof.size() - 1; }
    g_prof[idx].launches++;
    g_prof_last = idx;
    ProfPending p; p.entry = idx; p.a = prof_event(); p.b = prof_event();
    cudaEventRecord(p.a, g.cur_stream);
    g_prof_pending.push_back(p);
    g_prof_cur = (int)g_prof_pending.size() - 1;
}

void profile_end()
{
    if (g_prof_cur >= 0) cudaEventRecord(g_prof_pending[g_prof_cur].b, g.cur_stream);
    g_prof_cur = -1;
}

void profile_add_flops(double flops)
{
    if (g_prof_on && g_prof_last >= 0 && g_prof_last < (int)g_prof.size()) g_prof[g_prof_last].flops += flops;
}

bool is_device_pointer(const void *p)
{
    if (p == nullptr) return false;
    if (g.mem_mode == TL_MEM_DEVICE) return true;
    if (g.mem_mode == TL_MEM_HOST) return false;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) { cudaGetLastError(); return false; }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

// ---------------------------------------------------------------- arena
bool arena_pinned() { return g.arena_pinned; }

static size_t arena_mark()
{
    // position encoded as (chunk index << 48) | offset; scopes nest in stack order
    if (g.chunks.empty()) return 0;
    return ((size_t)(g.chunks.size() - 1) << 48) | g.chunks.back().off;
}

static void arena_release(size_t mark)
{
    if (g.chunks.empty()) return;
    size_t idx = mark >> 48, off = mark & (((size_t)1 << 48) - 1);
    if (g.scope_depth == 0) {
        // top level: merge a fragmented arena into one chunk of the total size
        if (g.chunks.size() > 1 && !g.arena_pinned) {
            size_t total = 0;
            cudaStreamSynchronize(g.cur_stream);
            for (auto &c : g.chunks) { total += c.cap; cudaFree(c.base); }
            g.chunks.clear();
            char *base = nullptr;
            if (TL_CUDA(cudaMalloc(&base, total))) g.chunks.push_back({base, total, 0});
        } else {
            for (auto &c : g.chunks) c.off = 0;
        }
        return;
    }
    if (idx < g.chunks.size()) {
        for (size_t i = idx + 1; i < g.chunks.size(); i++) g.chunks[i].off = 0;
        g.chunks[idx].off = off;
    }
}

static void *arena_alloc(size_t bytes)
{
    bytes = (bytes + 255) & ~(size_t)255;
    if (bytes == 0) bytes = 256;
    for (size_t i = g.chunks.empty() ? 0 : g.chunks.size() - 1; i < g.chunks.size(); i++) {
        Chunk &c = g.chunks[i];
        if (c.off + bytes <= c.cap) { void *p = c.base + c.off; c.off += bytes; return p; }
    }
    size_t cap = (size_t)64 << 20;
    if (!g.chunks.empty()) cap = g.chunks.back().cap * 2;
    while (cap < bytes) cap *= 2;
    char *base = nullptr;
    if (!TL_CUDA(cudaMalloc(&base, cap))) return nullptr;
    g.chunks.push_back({base, cap, bytes});
    return base;
}

Scope::Scope() : arena_mark_(0), ok_(true), staged_(false)
{
    ok_ = ready();
    arena_mark_ = arena_mark();
    g.scope_depth++;
}

void *Scope::alloc(size_t bytes)
{
    void *p = arena_alloc(bytes);
    if (!p) ok_ = false;
    return p;
}

void *Scope::map(void *p, size_t bytes, bool copy_in, bool copy_out)
{
    if (p == nullptr || !ok_) return nullptr;
    if (is_device_pointer(p)) return p;
    for (auto &e : entries_) {
        if (e.host == p && e.bytes >= bytes) {
            // same host range again: one mirror.  It was filled only if some earlier mapping asked for it.
            if (copy_in && !e.copied_in) {
                if (!TL_CUDA(cudaMemcpyAsync(e.dev, p, e.bytes, cudaMemcpyHostToDevice, g.cur_stream))) ok_ = false;
                e.copied_in = true;
            }
            e.write_back |= copy_out;
            return e.dev;
        }
        // ranges that overlap without being the same (an in-place operation at an offset, a longer view of the same array)
        // would get two mirrors and the last write-back would win silently: refuse
        const char *a0 = (const char *)e.host, *a1 = a0 + e.bytes, *b0 = (const char *)p, *b1 = b0 + bytes;
        if (b0 < a1 && a0 < b1) {
            set_error(TL_ERR_BAD_ARGS, "host buffers of one call overlap without being identical (%p+%zu and %p+%zu)", e.host, e.bytes, p, bytes);
            ok_ = false;
            return nullptr;
        }
    }
    void *d = arena_alloc(bytes);
    if (!d) { ok_ = false; return nullptr; }
    staged_ = true;
    if (copy_in) {
        if (!TL_CUDA(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, g.cur_stream))) ok_ = false;
    }
    entries_.push_back({p, d, bytes, copy_out, copy_in});
    return d;
}

Scope::~Scope()
{
    if (staged_) {
        for (auto &e : entries_)
            if (e.write_back) TL_CUDA(cudaMemcpyAsync(e.host, e.dev, e.bytes, cudaMemcpyDeviceToHost, g.cur_stream));
        TL_CUDA(cudaStreamSynchronize(g.cur_stream));
    }
    g.scope_depth--;
    arena_release(arena_mark_);
}

} // namespace tl

using namespace tl;

// ==================================================================== public C ABI
#pragma GCC visibility push(default)
extern "C" {

int trainlib_last_error(void) { return g.err; }
const char *trainlib_last_error_string(void) { return g.err_msg; }
void trainlib_clear_error(void) { if (!(g.err == TL_ERR_CUDA && g.cuda_sticky) && g.err != TL_ERR_NO_DEVICE) { g.err = TL_OK; g.err_msg[0] = 0; } }

int trainlib_init(int device) { return init_device(device); }
int trainlib_device(void) { return g.device; }
void trainlib_set_stream(void *s) { if (ready()) { defer_flush(); g.cur_stream = s ? (cudaStream_t)s : g.own_stream; } }
void *trainlib_stream(void) { return ready() ? (void *)g.cur_stream : nullptr; }
static bool g_capturing_now();
// A tensor-core kernel whose bounded wait gave up returns early and records the wait's id in a device word.  Every
// synchronisation point of the API reads that word ON THE LIBRARY'S STREAM (ordered behind the kernels) and latches
// TL_ERR_TIMEOUT, so results of a broken launch cannot be taken for good ones.
static void check_tc_status()
{
    int *dev = tc_status_word_if_any();
    if (!dev || g_capturing_now()) return;
    int h = 0;
    if (cudaMemcpyAsync(&h, dev, sizeof(int), cudaMemcpyDeviceToHost, g.cur_stream) != cudaSuccess) { cudaGetLastError(); return; }
    if (cudaStreamSynchronize(g.cur_stream) != cudaSuccess) { cudaGetLastError(); return; }
    if (h != 0) set_error(TL_ERR_TIMEOUT, "a tensor-core kernel gave up on bounded wait %d and returned early: its output is invalid", h);
}
void trainlib_synchronize(void) { if (!ready()) return; defer_flush(); if (TL_CUDA(cudaStreamSynchronize(g.cur_stream))) check_tc_status(); }

void trainlib_set_memory_mode(int mode) { if (mode >= TL_MEM_AUTO && mode <= TL_MEM_HOST) g.mem_mode = mode; }
int trainlib_memory_mode(void) { return g.mem_mode; }
void *trainlib_malloc(size_t bytes)
{
    if (!ready()) return nullptr;
    void *p = nullptr;
    if (!TL_CUDA(cudaMalloc(&p, bytes ? bytes : 256))) return nullptr;
    return p;
}
void trainlib_free(void *p) { if (p && ready()) { cudaStreamSynchronize(g.cur_stream); TL_CUDA(cudaFree(p)); } }
void *trainlib_malloc_host(size_t bytes)
{
    if (!ready()) return nullptr;
    void *p = nullptr;
    if (!TL_CUDA(cudaMallocHost(&p, bytes ? bytes : 256))) return nullptr;
    return p;
}
void trainlib_free_host(void *p) { if (p && ready()) TL_CUDA(cudaFreeHost(p)); }
int trainlib_memcpy_h2d(void *dev, const void *host, size_t bytes)
{
    if (!ready()) return g.err;
    if (!TL_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, g.cur_stream))) return g.err;
    return TL_CUDA(cudaStreamSynchronize(g.cur_stream)) ? TL_OK : g.err;
}
int trainlib_memcpy_d2h(void *host, const void *dev, size_t bytes)
{
    if (!ready()) return g.err;
    defer_flush();                                  // the bytes read may be a gradient whose sum is still pending
    if (!TL_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, g.cur_stream))) return g.err;
    return TL_CUDA(cudaStreamSynchronize(g.cur_stream)) ? TL_OK : g.err;
}
// Overlapped upload for double-buffered inputs.  The copy runs on a second stream: it first waits until the work
// that last read buffer `slot` (marked with trainlib_mark_consumed) has finished, and the library's stream waits for
// the copy, so kernels queued afterwards see the new data while kernels queued before keep running beside the copy.
static cudaStream_t g_copy_stream = nullptr;
static cudaEvent_t g_consumed[2] = {nullptr, nullptr}, g_uploaded = nullptr;
static bool g_consumed_set[2] = {false, false};
static bool overlap_ready()
{
    if (g_copy_stream) return true;
    if (!TL_CUDA(cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking))) return false;
    for (int i = 0; i < 2; i++) if (!TL_CUDA(cudaEventCreateWithFlags(&g_consumed[i], cudaEventDisableTiming))) return false;
    return TL_CUDA(cudaEventCreateWithFlags(&g_uploaded, cudaEventDisableTiming));
}
int trainlib_memcpy_h2d_overlapped(void *dev, const void *host, size_t bytes, int slot)
{
    if (!ready()) return g.err;
    if (slot < 0 || slot > 1) { set_error(TL_ERR_BAD_ARGS, "trainlib_memcpy_h2d_overlapped: slot %d", slot); return TL_ERR_BAD_ARGS; }
    if (!overlap_ready()) return g.err;
    if (g_consumed_set[slot] && !TL_CUDA(cudaStreamWaitEvent(g_copy_stream, g_consumed[slot], 0))) return g.err;
    if (!TL_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, g_copy_stream))) return g.err;
    if (!TL_CUDA(cudaEventRecord(g_uploaded, g_copy_stream))) return g.err;
    return TL_CUDA(cudaStreamWaitEvent(g.cur_stream, g_uploaded, 0)) ? TL_OK : g.err;
}
int trainlib_mark_consumed(int slot)
{
    if (!ready()) return g.err;
    if (slot < 0 || slot > 1) { set_error(TL_ERR_BAD_ARGS, "trainlib_mark_consumed: slot %d", slot); return TL_ERR_BAD_ARGS; }
    if (!overlap_ready()) return g.err;
    g_consumed_set[slot] = true;
    return TL_CUDA(cudaEventRecord(g_consumed[slot], g.cur_stream)) ? TL_OK : g.err;
}
int trainlib_memset(void *dev, int byte, size_t bytes)
{
    if (!ready()) return g.err;
    return TL_CUDA(cudaMemsetAsync(dev, byte, bytes, g.cur_stream)) ? TL_OK : g.err;
}

void trainlib_set_streams(int n) { g.n_streams = n < 1 ? 1 : n; }
int trainlib_streams(void) { return g.n_streams; }

void trainlib_timer_start(void) { if (ready()) TL_CUDA(cudaEventRecord(g.ev0, g.cur_stream)); }
double trainlib_timer_stop_ms(void)
{
    if (!ready()) return -1.0;
    float ms = 0.f;
    defer_flush();                                  // pending sums belong to the timed work
    if (!TL_CUDA(cudaEventRecord(g.ev1, g.cur_stream))) return -1.0;
    if (!TL_CUDA(cudaEventSynchronize(g.ev1))) return -1.0;
    if (!TL_CUDA(cudaEventElapsedTime(&ms, g.ev0, g.ev1))) return -1.0;
    check_tc_status();
    return (double)ms;
}
long long trainlib_kernel_launches(void) { return g.launches; }

// ---- CUDA graphs: capture the entry-point calls queued between begin and end, replay them with one launch
struct TlGraph { cudaGraphExec_t exec; cudaGraph_t graph; long long kernels; };
static long long g_capture_launches0 = 0;
static bool g_capturing = false;
static bool g_capturing_now() { return g_capturing; }
int trainlib_graph_begin(void)
{
    if (!ready()) return g.err;
    if (g_capturing) { set_error(TL_ERR_BAD_ARGS, "trainlib_graph_begin: a capture is already open"); return TL_ERR_BAD_ARGS; }
    defer_flush();                                  // sums pending from before the capture run now, outside the graph
    if (!TL_CUDA(cudaStreamBeginCapture(g.cur_stream, cudaStreamCaptureModeRelaxed))) return g.err;
    g_capturing = true; g_capture_launches0 = g.launches;
    g.arena_pinned = true;
    return TL_OK;
}
void *trainlib_graph_end(void)
{
    if (!ready() || !g_capturing) return nullptr;
    defer_flush();                                  // sums pending from the captured calls become the graph's last node
    g_capturing = false;
    cudaGraph_t graph = nullptr;
    if (!TL_CUDA(cudaStreamEndCapture(g.cur_stream, &graph)) || !graph) return nullptr;
    cudaGraphExec_t exec = nullptr;
    if (!TL_CUDA(cudaGraphInstantiate(&exec, graph, 0))) { cudaGraphDestroy(graph); return nullptr; }
    TlGraph *t = new TlGraph{exec, graph, g.launches - g_capture_launches0};
    g.launches = g_capture_launches0;        // nothing ran during the capture
    return t;
}
int trainlib_graph_launch(void *handle)
{
    if (!ready()) return g.err;
    TlGraph *t = (TlGraph *)handle;
    if (!t) { set_error(TL_ERR_BAD_ARGS, "trainlib_graph_launch: null graph"); return TL_ERR_BAD_ARGS; }
    if (!TL_CUDA(cudaGraphLaunch(t->exec, g.cur_stream))) return g.err;
    g.launches += t->kernels;
    return TL_OK;
}
void trainlib_graph_destroy(void *handle)
{
    TlGraph *t = (TlGraph *)handle;
    if (!t) return;
    cudaGraphExecDestroy(t->exec); cudaGraphDestroy(t->graph);
    delete t;
}
void trainlib_profile(int on)
{
    if (!ready()) return;
    if (on) { g_prof.clear(); g_prof_last = -1; g_prof_on = true; }
    else { prof_drain(); g_prof_on = false; }
}
int trainlib_profile_entries(void) { prof_drain(); return (int)g_prof.size(); }
const char *trainlib_profile_entry(int i, long long *launches, double *total_ms)
{
    if (i < 0 || i >= (int)g_prof.size()) return nullptr;
    if (launches) *launches = g_prof[i].launches;
    if (total_ms) *total_ms = g_prof[i].ms;
    return g_prof[i].name;
}
double trainlib_profile_entry_flops(int i) { return (i < 0 || i >= (int)g_prof.size()) ? 0.0 : g_prof[i].flops; }
int trainlib_tc_status(void) { return ready() ? conv_tc_status() : -1; }
void trainlib_set_gemm_path(int p) { g.gemm_path = (p >= 0 && p <= 4) ? p : 0; }
int trainlib_gemm_path(void) { return g.gemm_path; }

// -------------------------------------------------------------------- PMSIS stand-in
static thread_local int t_core_id = 0;
int pi_core_id(void) { return t_core_id; }
void pi_cl_team_barrier(void) {}

bool tl_is_library_worker(void (*fn)(void *));   // defined with the entry-point table

void pi_cl_team_fork(int n, void (*fn)(void *), void *arg)
{
    if (fn == nullptr) return;
    if (tl_is_library_worker(fn)) { fn(arg); return; }        // one launch does the whole tensor
    for (int i = 0; i < (n < 1 ? 1 : n); i++) { t_core_id = i; fn(arg); }
    t_core_id = 0;
}

void pi_cl_dma_cmd(uintptr_t ext, uintptr_t loc, int size, int dir, pi_cl_dma_cmd_t *cmd)
{
    (void)cmd;
    if (dir == PI_CL_DMA_DIR_EXT2LOC) memcpy((void *)loc, (const void *)ext, (size_t)size);
    else memcpy((void *)ext, (const void *)loc, (size_t)size);
}
void pi_cl_dma_cmd_2d(uintptr_t ext, uintptr_t loc, int size, int stride, int length, int dir, pi_cl_dma_cmd_t *cmd)
{
    (void)cmd;
    if (length <= 0) return;
    for (int done = 0, row = 0; done < size; done += length, row++) {
        int n = size - done < length ? size - done : length;
        char *e = (char *)ext + (size_t)row * (size_t)stride, *l = (char *)loc + done;
        if (dir == PI_CL_DMA_DIR_EXT2LOC) memcpy(l, e, (size_t)n); else memcpy(e, l, (size_t)n);
    }
}
void pi_cl_dma_cmd_wait(pi_cl_dma_cmd_t *cmd) { (void)cmd; }

static double g_perf_ns = 0.0;
void pi_perf_conf(unsigned events) { (void)events; }
void pi_perf_reset(void) { g_perf_ns = 0.0; }
void pi_perf_start(void) { trainlib_timer_start(); }
void pi_perf_stop(void) { double ms = trainlib_timer_stop_ms(); if (ms > 0) g_perf_ns += ms * 1e6; }
unsigned pi_perf_read(int event)
{
    if (event != PI_PERF_CYCLES && event != PI_PERF_ACTIVE_CYCLES) return 0;      // no such counter on this device
    return g_perf_ns > 4294967295.0 ? 4294967295u : (unsigned)g_perf_ns;
}
// cluster bring-up of the reference's main.c files: open = device initialisation, a task = one call of its entry function
void pi_cluster_conf_init(struct pi_cluster_conf *conf) { if (conf) { conf->id = 0; conf->device_type = 0; } }
void pi_open_from_conf(struct pi_device *device, void *conf) { if (device) { device->config = conf; device->data = nullptr; } }
int pi_cluster_open(struct pi_device *device) { (void)device; return trainlib_init(-1) == TL_OK ? 0 : -1; }
int pi_cluster_close(struct pi_device *device) { (void)device; trainlib_synchronize(); return 0; }
struct pi_cluster_task *pi_cluster_task(struct pi_cluster_task *task, void (*entry)(void *), void *arg)
{
    if (task) { task->entry = entry; task->arg = arg; task->stack_size = 0; task->slave_stack_size = 0; }
    return task;
}
int pi_cluster_send_task_to_cl(struct pi_device *device, struct pi_cluster_task *task)
{
    (void)device;
    if (!task || !task->entry) return -1;
    task->entry(task->arg);
    trainlib_synchronize();
    return 0;
}
void pmsis_exit(int status) { fflush(stdout); exit(status); }
void *pi_l2_malloc(int bytes) { return malloc((size_t)(bytes > 0 ? bytes : 1)); }
void pi_l2_free(void *p, int bytes) { (void)bytes; free(p); }

} // extern "C"
#pragma GCC visibility pop
