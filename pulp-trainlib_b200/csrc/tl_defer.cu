// Deferred reductions (extension, off by default).
//
// A weight gradient or a norm-parameter gradient is first produced as partial results (one per CTA, or one per stream)
// and then summed in a fixed order by a small kernel.  In a network of a few thousand streams there are two dozen such
// sums per backward pass, each a launch of a few microseconds that runs alone on the GPU.  With
// trainlib_set_deferred_reductions(1) the library keeps the partial results of device-resident calls in an arena of its
// own, notes what is to be summed into which gradient, and runs ALL pending sums as one launch
//   - when an entry point that reads gradients is called (pulp_gradient_descent_*), on trainlib_synchronize(),
//     trainlib_memcpy_d2h(), trainlib_graph_end(), trainlib_set_stream(), when the mode is switched off, when the arena or
//     the job table is full, and
//   - on trainlib_flush_reductions(), which a caller must issue before anything outside the library (a collective,
//     its own kernels) reads a gradient.
// Until then the gradient buffers named by the deferred calls do not hold their values: that is the contract of the
// mode, and the reason it is an extension and off unless asked for.  The summation trees are the ones of the kernels
// the sums would otherwise run on (reduce_partials_kernel, wgt_reduce_kernel, column_direct_kernel), so results are
// bit-identical to the immediate mode wherever that mode uses those kernels.
#include "tl_kernels.h"

namespace tl {

static constexpr int DEFER_MAX_JOBS = 48;
enum { DEFER_PLAIN = 0, DEFER_COLUMNS = 1, DEFER_WGT = 2 };

struct DeferJob {
    const float *part; float *out;
    long long n;                     // elements per partial result (columns)
    int groups;                      // partial results (rows)
    int kind, first_cta;
    int a0, a1, a2, a3, a4, a5, a6;  // COLUMNS: a0 = pairs; WGT: Cin, Cout, s2, xg, cigs, ncopy, MB
};
struct DeferBatch { DeferJob job[DEFER_MAX_JOBS]; int count, ctas; };

static struct {
    bool on = false;
    char *base = nullptr;
    size_t cap = 0, off = 0, need = 0;   // bytes; `need` = what this epoch asked for, granted or not
    DeferBatch batch = {};
} d;

// A CTA serves one job.  Weight-gradient partials (PLAIN, WGT): 512 consecutive elements through partial_sums_quad, the
// function the immediate kernels use.  Norm-parameter partials (COLUMNS: few columns, one row per stream): 32 columns x 32
// slices of the rows, thread (slice, column) adds rows slice, slice + 32, ... four at a time, the 32 slice sums are added
// in slice order: the tree of column_direct_kernel up to 1024 rows; above, a lane keeps eight running sums so that more
// loads are in flight (the immediate mode takes two passes there).
__global__ void __launch_bounds__(1024) deferred_reduce_kernel(const __grid_constant__ DeferBatch b)
{
    __shared__ float4 sm4[8][128];
    int j = 0;
    while (j + 1 < b.count && (int)blockIdx.x >= b.job[j + 1].first_cta) j++;
    const float *__restrict__ part = b.job[j].part;
    float *out = b.job[j].out;
    const long long n = b.job[j].n;
    const int groups = b.job[j].groups, kind = b.job[j].kind, cta = (int)blockIdx.x - b.job[j].first_cta;
    if (kind != DEFER_COLUMNS) {
        const int Cin = b.job[j].a0, Cout = b.job[j].a1, s2 = b.job[j].a2, xg = b.job[j].a3, cigs = b.job[j].a4, ncopy = b.job[j].a5;
        const long long i = (long long)cta * PSUM_ELEMS + (threadIdx.x & 127) * 4;
        const bool used = kind == DEFER_PLAIN || (i < n && (int)(i / (ncopy * Cout)) / 8 < 3 * xg);
        float4 t;
        if (!partial_sums_quad(part, n, groups, i, used, t, sm4)) return;
        const float v[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (i + e >= n) break;
            const long long o = kind == DEFER_PLAIN ? i + e : wgt_partial_index(i + e, Cin, Cout, s2, xg, cigs, ncopy);
            if (o >= 0) out[o] = v[e];
        }
        return;
    }
    float (*sm)[33] = reinterpret_cast<float (*)[33]>(sm4);          // 32 x 33 floats of the 16 KB
    const int wx = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const long long i = (long long)cta * 32 + wx;
    float s = 0.f;
    if (i < n) {
        if (groups > 1024) {
            float a[8];
#pragma unroll
            for (int q = 0; q < 8; q++) a[q] = 0.f;
            int r = sl;
            for (; r + 224 < groups; r += 256)
#pragma unroll
                for (int q = 0; q < 8; q++) a[q] += part[(long long)(r + 32 * q) * n + i];
            for (; r < groups; r += 32) a[0] += part[(long long)r * n + i];
            s = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
        } else {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            int r = sl;
            for (; r + 96 < groups; r += 128) {
                s0 += part[(long long)r * n + i]; s1 += part[(long long)(r + 32) * n + i];
                s2 += part[(long long)(r + 64) * n + i]; s3 += part[(long long)(r + 96) * n + i];
            }
            for (; r < groups; r += 32) s0 += part[(long long)r * n + i];
            s = (s0 + s1) + (s2 + s3);
        }
    }
    sm[sl][wx] = s;
    __syncthreads();
    if (sl != 0 || i >= n) return;
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) t += sm[k][wx];
    const int pairs = b.job[j].a0;
    out[pairs > 0 ? (i & 1) * pairs + (i >> 1) : i] = t;
}

bool defer_enabled() { return d.on; }

// all pending sums as one launch; the arena is free again afterwards (stream order: what follows runs after the sums)
void defer_flush()
{
    if (d.batch.count > 0) {
        TL_LAUNCH(deferred_reduce_kernel, d.batch.ctas, 1024, 0, d.batch);
        d.batch.count = 0; d.batch.ctas = 0;
    }
    // grow to what the last epoch asked for, unless a captured graph holds addresses inside the arena
    if (d.need > d.cap && !arena_pinned()) {
        const size_t want = d.need + d.need / 4;
        cudaStreamSynchronize(stream());
        if (d.base) cudaFree(d.base);
        d.base = nullptr; d.cap = 0;
        char *p = nullptr;
        if (cudaMalloc(&p, want) == cudaSuccess) { d.base = p; d.cap = want; }
        else cudaGetLastError();                                    // no arena: every sum runs at once, as without the mode
    }
    d.off = 0; d.need = 0;
}

// room for partial results that a deferred sum will read; nullptr = not now (the caller sums at once from its own scratch)
float *defer_alloc(size_t floats)
{
    if (!d.on) return nullptr;
    const size_t bytes = (floats * sizeof(float) + 255) & ~(size_t)255;
    if (d.batch.count >= DEFER_MAX_JOBS) defer_flush();          // table full: what is pending has been produced already
    d.need += bytes;
    if (d.off + bytes > d.cap) return nullptr;
    float *p = reinterpret_cast<float *>(d.base + d.off);
    d.off += bytes;
    return p;
}

static void defer_push(const DeferJob &job)
{
    DeferJob &J = d.batch.job[d.batch.count++];
    J = job;
    J.first_cta = d.batch.ctas;
    d.batch.ctas += ceil_div(job.n, job.kind == DEFER_COLUMNS ? 32 : PSUM_ELEMS);
}
void defer_plain(const float *part, float *out, long long n, int groups)
{
    DeferJob j = {}; j.part = part; j.out = out; j.n = n; j.groups = groups; j.kind = DEFER_PLAIN;
    defer_push(j);
}
void defer_columns(const float *part, float *out, int rows, int dim, int pairs)
{
    DeferJob j = {}; j.part = part; j.out = out; j.n = dim; j.groups = rows; j.kind = DEFER_COLUMNS; j.a0 = pairs;
    defer_push(j);
}
void defer_wgt(const float *part, float *out, int groups, long long group_floats, int Cin, int Cout, int s2, int xg, int cigs, int ncopy)
{
    DeferJob j = {}; j.part = part; j.out = out; j.n = group_floats; j.groups = groups; j.kind = DEFER_WGT;
    j.a0 = Cin; j.a1 = Cout; j.a2 = s2; j.a3 = xg; j.a4 = cigs; j.a5 = ncopy;
    defer_push(j);
}

void defer_set(bool on)
{
    if (!on && d.on) defer_flush();
    d.on = on;
}

} // namespace tl

extern "C" {
__attribute__((visibility("default"))) void trainlib_set_deferred_reductions(int on) { if (tl::ready()) tl::defer_set(on != 0); }
__attribute__((visibility("default"))) void trainlib_flush_reductions(void) { if (tl::ready()) tl::defer_flush(); }
}
