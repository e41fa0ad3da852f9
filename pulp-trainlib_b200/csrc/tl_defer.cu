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

// One CTA = 32 consecutive elements of one job x 32 slices of its partial results: thread (slice, lane) adds the partials
// slice, slice + 32, ... of element lane, the 32 slice sums of an element are then added in slice order.  That is the
// summation tree of reduce_partials_kernel / wgt_reduce_kernel (PLAIN, WGT) and of column_direct_kernel (COLUMNS, up to
// 1024 rows); above 1024 rows a lane keeps eight running sums instead of four so that more loads are in flight (the
// immediate mode takes two passes there).  (128 elements per CTA with four per thread measured slower: 89 against 70 us
// for the sums of a 4096-stream backward pass.)
static constexpr int DEFER_ELEMS = 32;
__global__ void __launch_bounds__(1024) deferred_reduce_kernel(const __grid_constant__ DeferBatch b)
{
    __shared__ float sm[32][33];
    int j = 0;
    while (j + 1 < b.count && (int)blockIdx.x >= b.job[j + 1].first_cta) j++;
    const float *__restrict__ part = b.job[j].part;
    const long long n = b.job[j].n;
    const int groups = b.job[j].groups, kind = b.job[j].kind;
    const int wx = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const long long i = (long long)((int)blockIdx.x - b.job[j].first_cta) * DEFER_ELEMS + wx;
    float s = 0.f;
    bool used = i < n;
    if (kind == DEFER_WGT && used) used = (int)(i / (b.job[j].a5 * b.job[j].a1)) / 8 < 3 * b.job[j].a3;   // padding rows are never written
    if (used) {
        if (kind == DEFER_COLUMNS && groups > 1024) {
            float a[8];
#pragma unroll
            for (int q = 0; q < 8; q++) a[q] = 0.f;
            int r = sl;
            for (; r + 224 < groups; r += 256)
#pragma unroll
                for (int q = 0; q < 8; q++) a[q] += part[(long long)(r + 32 * q) * n + i];
            for (; r < groups; r += 32) a[0] += part[(long long)r * n + i];
            s = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
        } else if (kind == DEFER_COLUMNS) {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            int r = sl;
            for (; r + 96 < groups; r += 128) {
                s0 += part[(long long)r * n + i]; s1 += part[(long long)(r + 32) * n + i];
                s2 += part[(long long)(r + 64) * n + i]; s3 += part[(long long)(r + 96) * n + i];
            }
            for (; r < groups; r += 32) s0 += part[(long long)r * n + i];
            s = (s0 + s1) + (s2 + s3);
        } else {
            for (int g = sl; g < groups; g += 32) s += part[(long long)g * n + i];
        }
    }
    sm[sl][wx] = s;
    __syncthreads();
    if (sl != 0 || !used) return;
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) t += sm[k][wx];
    float *out = b.job[j].out;
    if (kind == DEFER_PLAIN) { out[i] = t; return; }
    if (kind == DEFER_COLUMNS) { const int pairs = b.job[j].a0; out[pairs > 0 ? (i & 1) * pairs + (i >> 1) : i] = t; return; }
    // DEFER_WGT: the accumulator layout of conv_wgt_kernel -> dW[co][ci][kh][kw] (see wgt_reduce_kernel)
    const int Cin = b.job[j].a0, Cout = b.job[j].a1, s2 = b.job[j].a2, xg = b.job[j].a3, cigs = b.job[j].a4, ncopy = b.job[j].a5;
    const int NBc = ncopy * Cout;
    const int row = (int)(i / NBc), col = (int)(i % NBc);
    const int grp = row / 8, ci8 = row & 7;
    if (grp >= 3 * xg) return;
    const int a = grp / xg, par = (grp % xg) / cigs, ci = (grp % cigs) * 8 + ci8;
    const int bb = col / Cout, co = col % Cout;
    const int kw = !s2 ? bb : (par == 0 ? (bb == 1 ? 1 : -1) : (bb == 1 ? 2 : 0));
    if (kw >= 0) out[((long long)co * Cin + ci) * 9 + a * 3 + kw] = t;
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
    d.batch.ctas += ceil_div(job.n, DEFER_ELEMS);
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
