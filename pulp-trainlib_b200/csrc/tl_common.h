// Internal header of libtrainlib_b200: runtime context, staging scopes and launch helpers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstddef>
#include <cstdio>
#include <vector>

typedef __half fp16;   // device-side storage type of the ABI's fp16 (IEEE binary16)
#define TRAINLIB_NO_FP16_TYPEDEF
#include "../../include/trainlib_b200_abi.h"
#include "../../include/trainlib_b200.h"

namespace tl {

// ---------------------------------------------------------------- errors
void set_error(int code, const char *fmt, ...);
bool cuda_ok(cudaError_t e, const char *what);
bool ready();                       // lazily initialises the device; false => error latched

#define TL_CUDA(call) ::tl::cuda_ok((call), #call)

// ---------------------------------------------------------------- context
cudaStream_t stream();
int streams();                      // number of independent batch-1 streams (>= 1)
int sm_count();
int gemm_path();
void count_launch();
// Per-kernel timing (off by default): when on, every launch is bracketed by CUDA events on the
// library stream and its duration is added to the entry of its kernel name.
bool profiling();
void profile_begin(const char *kernel_name);
void profile_end();
// Useful floating-point operations of the launch begun last (2 per multiply-add of the operator's definition:
// zeros a kernel multiplies for its own convenience are not work).  No-op unless profiling is on.
void profile_add_flops(double flops);

// Launch a kernel on the library stream, count it, latch launch errors.
#define TL_LAUNCH(kernel, grid, block, smem, ...)                                   \
    do {                                                                            \
        const bool tl_prof_ = ::tl::profiling();                                    \
        if (tl_prof_) ::tl::profile_begin(#kernel);                                 \
        kernel<<<(grid), (block), (smem), ::tl::stream()>>>(__VA_ARGS__);           \
        if (tl_prof_) ::tl::profile_end();                                          \
        ::tl::count_launch();                                                       \
        ::tl::cuda_ok(cudaGetLastError(), #kernel);                                 \
    } while (0)

// ---------------------------------------------------------------- staging
// A Scope maps the pointers of one entry-point call to device addresses.
// Device pointers pass through; host pointers get a mirror in the staging arena that is
// filled before (in / inout) and copied back after (out / inout) the kernels of the call.
class Scope {
public:
    Scope();
    ~Scope();                       // copies outputs back, synchronises if anything was staged
    template <class T> const T *in(const T *p, size_t n) { return (const T *)map((void *)p, n * sizeof(T), true, false); }
    template <class T> T *out(T *p, size_t n) { return (T *)map((void *)p, n * sizeof(T), false, true); }
    template <class T> T *inout(T *p, size_t n) { return (T *)map((void *)p, n * sizeof(T), true, true); }
    template <class T> T *scratch(size_t n) { return (T *)alloc(n * sizeof(T)); }   // device-only temporary
    bool ok() const { return ok_; }
    bool staged() const { return staged_; }   // some buffer of this call lives in host memory (mirrored in the arena)
    // a reduction of this call may be deferred: every buffer is the caller's own device memory and the call does not go
    // on to read the result itself
    bool may_defer() const { return !staged_ && !no_defer_; }
    void no_deferral() { no_defer_ = true; }
private:
    struct Entry { void *host; void *dev; size_t bytes; bool write_back; bool copied_in; };
    void *map(void *p, size_t bytes, bool copy_in, bool copy_out);
    void *alloc(size_t bytes);
    std::vector<Entry> entries_;
    size_t arena_mark_;
    bool ok_;
    bool staged_;
    bool no_defer_ = false;
};

bool is_device_pointer(const void *p);
bool arena_pinned();                // a captured graph holds addresses of library-owned device memory: never move it again

// deferred reductions (tl_defer.cu): partial results kept until one batched launch sums them all
bool defer_enabled();
float *defer_alloc(size_t floats);
void defer_plain(const float *part, float *out, long long n, int groups);
void defer_columns(const float *part, float *out, int rows, int dim, int pairs);
void defer_wgt(const float *part, float *out, int groups, long long group_floats, int Cin, int Cout, int s2, int xg, int cigs, int ncopy);
void defer_flush();

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

} // namespace tl
