// C ABI: stage entry points with host buffers, and the device-resident session handle.
// See include/tsnecuda_b200.h for the contract of each function and the reference interface it
// replaces.
#include <string.h>

#include <algorithm>
#include <new>
#include <string>
#include <vector>

#include "../../include/tsnecuda_b200.h"
#include "comm.h"
#include "peer.h"
#include "session.h"

using namespace b200;

struct b200tsne_session {
    Session s;
};

static thread_local KnnStats g_last_knn_stats;

namespace {
int check_device(int device)
{
    int n = 0;
    B200_CUDA(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n) { set_error("no such CUDA device"); return B200TSNE_ERR_CUDA; }
    B200_CUDA(cudaSetDevice(device));
    return 0;
}
struct StreamGuard {
    cudaStream_t st = nullptr;
    int create() { B200_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking)); return 0; }
    ~StreamGuard() { if (st) cudaStreamDestroy(st); }
};
template <class T> int up(DeviceArena &a, T **d, const T *h, size_t n, cudaStream_t st)
{
    B200_TRY(a.alloc((void **)d, sizeof(T) * std::max<size_t>(n, 1)));
    if (n) B200_CUDA(cudaMemcpyAsync(*d, h, sizeof(T) * n, cudaMemcpyHostToDevice, st));
    return 0;
}
template <class T> int down(T *h, const T *d, size_t n, cudaStream_t st)
{
    if (n) B200_CUDA(cudaMemcpyAsync(h, d, sizeof(T) * n, cudaMemcpyDeviceToHost, st));
    return 0;
}
}  // namespace

extern "C" {

const char *b200tsne_last_error(void) { return last_error().c_str(); }
int b200tsne_version(void) { return (0 << 16) | (1 << 8) | 0; }

const char *b200tsne_stage_name(int stage)
{
    static const char *names[kStages] = {"spread", "convolve", "gather", "attractive", "update", "exchange", "knn", "affinities", "order"};
    return (stage >= 0 && stage < kStages) ? names[stage] : "";
}

int b200tsne_knn(const float *X, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo, int64_t db_hi,
                 int32_t *ids, float *d2, int device)
{
    if (!X || !ids || !d2 || N <= 0 || D <= 0 || K <= 0 || q_lo < 0 || q_hi > N || q_lo > q_hi || db_lo < 0 ||
        db_hi > N || db_lo > db_hi || N > 2147483647LL) {
        set_error("b200tsne_knn: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dX = nullptr, *dd = nullptr;
    int32_t *di = nullptr;
    const size_t nq = (size_t)(q_hi - q_lo);
    B200_TRY(up(a, &dX, X, (size_t)N * D, sg.st));
    B200_TRY(a.alloc((void **)&di, sizeof(int32_t) * std::max<size_t>(nq * K, 1)));
    B200_TRY(a.alloc((void **)&dd, sizeof(float) * std::max<size_t>(nq * K, 1)));
    B200_TRY(knn_search(dX, N, D, K, q_lo, q_hi, db_lo, db_hi, di, dd, &g_last_knn_stats, sg.st));
    B200_TRY(launch_knn_finalize(di, dd, (int64_t)nq * K, sg.st));
    B200_TRY(down(ids, di, nq * K, sg.st));
    B200_TRY(down(d2, dd, nq * K, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    return 0;
}

int b200tsne_perplexity(const float *d2, int64_t N, int K, float perplexity, float epsilon, float max_override,
                        float *p, float *betas, float *max_out, int device)
{
    if (!d2 || !p || N <= 0 || K <= 0 || !(perplexity > 0.0f)) {
        set_error("b200tsne_perplexity: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dd = nullptr, *dp = nullptr, *db = nullptr;
    unsigned int *dm = nullptr;
    const size_t n = (size_t)N * K;
    B200_TRY(up(a, &dd, d2, n, sg.st));
    B200_TRY(a.alloc((void **)&dp, sizeof(float) * n));
    B200_TRY(a.alloc((void **)&db, sizeof(float) * N));
    B200_TRY(a.alloc((void **)&dm, sizeof(unsigned int)));
    const unsigned int init = enc_float(max_override > 0.0f ? max_override : 0.0f);
    B200_CUDA(cudaMemcpyAsync(dm, &init, sizeof(init), cudaMemcpyHostToDevice, sg.st));
    if (!(max_override > 0.0f)) B200_TRY(launch_absmax(dd, (int64_t)n, dm, sg.st));
    B200_TRY(launch_perplexity(dd, N, K, perplexity, epsilon, dm, dp, db, sg.st));
    B200_TRY(down(p, dp, n, sg.st));
    if (betas) B200_TRY(down(betas, db, (size_t)N, sg.st));
    unsigned int m = 0;
    B200_TRY(down(&m, dm, 1, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    if (max_out) *max_out = dec_float(m);
    return 0;
}

int b200tsne_symmetrize(const float *p, const int32_t *ids, int64_t N, int K, float *P, int device)
{
    if (!p || !ids || !P || N <= 0 || K <= 0) { set_error("b200tsne_symmetrize: invalid arguments"); return B200TSNE_ERR_INVALID; }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dp = nullptr, *dP = nullptr;
    int32_t *di = nullptr;
    const size_t n = (size_t)N * K;
    B200_TRY(up(a, &dp, p, n, sg.st));
    B200_TRY(up(a, &di, ids, n, sg.st));
    B200_TRY(a.alloc((void **)&dP, sizeof(float) * n));
    B200_TRY(launch_symmetrize(dp, di, N, K, 0, N, dP, sg.st));
    B200_TRY(down(P, dP, n, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    return 0;
}

int b200tsne_attractive(const float *P, const int32_t *ids, const float *Y, int64_t N, int K, int64_t row_lo,
                        int64_t row_hi, float *F, int device)
{
    if (!P || !ids || !Y || !F || N <= 0 || K <= 0 || row_lo < 0 || row_hi > N || row_lo > row_hi) {
        set_error("b200tsne_attractive: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dP = nullptr, *dY = nullptr, *dF = nullptr;
    float2 *dY2 = nullptr, *dF2 = nullptr;
    int32_t *di = nullptr;
    const size_t rows = (size_t)(row_hi - row_lo);
    B200_TRY(up(a, &dP, P + (size_t)row_lo * K, rows * K, sg.st));
    B200_TRY(up(a, &di, ids + (size_t)row_lo * K, rows * K, sg.st));
    B200_TRY(up(a, &dY, Y, (size_t)2 * N, sg.st));
    B200_TRY(a.alloc((void **)&dY2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF, sizeof(float) * 2 * N));
    B200_CUDA(cudaMemsetAsync(dF2, 0, sizeof(float2) * N, sg.st));
    B200_TRY(launch_soa_to_aos(dY, dY2, N, sg.st));
    B200_TRY(launch_attractive(dP, di, dY2, N, K, row_lo, row_hi, dF2, sg.st));
    B200_TRY(launch_aos_to_soa(dF2, dF, N, sg.st));
    B200_TRY(down(F, dF, (size_t)2 * N, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    return 0;
}

int b200tsne_attractive_blocked(const float *P, const int32_t *ids, const float *Y, int64_t N, int K, int64_t row_lo,
                                int64_t row_hi, const float *X, int D, float *F, float *entries_per_group, int device)
{
    if (!P || !ids || !Y || !F || N <= 0 || K <= 0 || row_lo < 0 || row_hi > N || row_lo > row_hi || (X && D <= 0)) {
        set_error("b200tsne_attractive_blocked: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dP = nullptr, *dY = nullptr, *dF = nullptr, *dX = nullptr;
    float2 *dY2 = nullptr, *dF2 = nullptr;
    int32_t *di = nullptr, *perm = nullptr;
    const size_t rows = (size_t)(row_hi - row_lo);
    B200_TRY(up(a, &dP, P + (size_t)row_lo * K, rows * K, sg.st));
    B200_TRY(up(a, &di, ids + (size_t)row_lo * K, rows * K, sg.st));
    B200_TRY(up(a, &dY, Y, (size_t)2 * N, sg.st));
    B200_TRY(a.alloc((void **)&dY2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF, sizeof(float) * 2 * N));
    if (X) {
        B200_TRY(up(a, &dX, X, (size_t)N * D, sg.st));
        B200_TRY(a.alloc((void **)&perm, sizeof(int32_t) * N));
        B200_TRY(order_points_by_cell(dX, N, D, perm, sg.st));
    }
    B200_CUDA(cudaMemsetAsync(dF2, 0, sizeof(float2) * N, sg.st));
    B200_TRY(launch_soa_to_aos(dY, dY2, N, sg.st));
    BlockedAttractive blk;
    B200_TRY(blocked_attractive_build(&blk, a, dP, di, N, K, row_lo, row_hi, perm, nullptr, sg.st));
    if (entries_per_group) *entries_per_group = blk.entries_per_group;
    if (!blk.ready) {
        set_error("b200tsne_attractive_blocked: the blocked copy was not built for this graph (entries per row and tile: " +
                  std::to_string(blk.entries_per_group) + "); use b200tsne_attractive");
        return B200TSNE_ERR_UNSUPPORTED;
    }
    B200_TRY(launch_attractive_blocked(blk, dY2, dF2, sg.st));
    B200_TRY(launch_aos_to_soa(dF2, dF, N, sg.st));
    B200_TRY(down(F, dF, (size_t)2 * N, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    return 0;
}

int b200tsne_attractive_symmetric(const float *p, const int32_t *ids, const float *Y, int64_t N, int K, const float *X, int D, float *F,
                                  float *P_fixed, int64_t *extra_entries, float *extra_sum, int *blocked, int device)
{
    if (!p || !ids || !Y || !F || N <= 0 || K <= 0 || (X && D <= 0)) {
        set_error("b200tsne_attractive_symmetric: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dp = nullptr, *dP = nullptr, *dY = nullptr, *dF = nullptr, *dX = nullptr, *ext_val = nullptr;
    float2 *dY2 = nullptr, *dF2 = nullptr;
    int32_t *di = nullptr, *perm = nullptr, *ext_ids = nullptr;
    int *ptr = nullptr, *cursor = nullptr;
    const size_t nk = (size_t)N * K;
    B200_TRY(up(a, &dp, p, nk, sg.st));
    B200_TRY(up(a, &di, ids, nk, sg.st));
    B200_TRY(up(a, &dY, Y, (size_t)2 * N, sg.st));
    B200_TRY(a.alloc((void **)&dP, sizeof(float) * nk));
    B200_TRY(a.alloc((void **)&dY2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF, sizeof(float) * 2 * N));
    B200_TRY(a.alloc((void **)&ptr, sizeof(int) * (N + 1)));
    B200_TRY(a.alloc((void **)&cursor, sizeof(int) * N));
    B200_TRY(launch_symmetrize(dp, di, N, K, 0, N, dP, sg.st));
    ExtraEntries extra;
    B200_TRY(launch_reverse_only_count(dp, di, N, K, 0, N, ptr, &extra.count, sg.st));
    B200_TRY(a.alloc((void **)&ext_ids, sizeof(int32_t) * std::max<int64_t>(extra.count, 1)));
    B200_TRY(a.alloc((void **)&ext_val, sizeof(float) * std::max<int64_t>(extra.count, 1)));
    B200_TRY(launch_reverse_only_fill(dp, di, N, K, 0, N, ptr, cursor, ext_ids, ext_val, sg.st));
    extra.ptr = ptr; extra.ids = ext_ids; extra.val = ext_val;
    if (X) {
        B200_TRY(up(a, &dX, X, (size_t)N * D, sg.st));
        B200_TRY(a.alloc((void **)&perm, sizeof(int32_t) * N));
        B200_TRY(order_points_by_cell(dX, N, D, perm, sg.st));
    }
    B200_CUDA(cudaMemsetAsync(dF2, 0, sizeof(float2) * N, sg.st));
    B200_TRY(launch_soa_to_aos(dY, dY2, N, sg.st));
    BlockedAttractive blk;
    B200_TRY(blocked_attractive_build(&blk, a, dP, di, N, K, 0, N, perm, extra.count > 0 ? &extra : nullptr, sg.st));
    if (blocked) *blocked = blk.ready ? 1 : 0;
    if (blk.ready) {
        B200_TRY(launch_attractive_blocked(blk, dY2, dF2, sg.st));
    } else {
        B200_TRY(launch_attractive(dP, di, dY2, N, K, 0, N, dF2, sg.st));
        if (extra.count > 0) B200_TRY(launch_attractive_extra(ptr, ext_ids, ext_val, dY2, N, 0, N, dF2, sg.st));
    }
    B200_TRY(launch_aos_to_soa(dF2, dF, N, sg.st));
    B200_TRY(down(F, dF, (size_t)2 * N, sg.st));
    if (P_fixed) B200_TRY(down(P_fixed, dP, nk, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    if (extra_entries) *extra_entries = extra.count;
    if (extra_sum) {
        std::vector<float> v((size_t)extra.count);
        if (extra.count) B200_CUDA(cudaMemcpy(v.data(), ext_val, sizeof(float) * extra.count, cudaMemcpyDeviceToHost));
        double t = 0.0;
        for (float x : v) t += x;
        *extra_sum = (float)t;
    }
    return 0;
}

int b200tsne_session_set_symmetric(b200tsne_session *h, int on)
{
    if (!h) { set_error("session_set_symmetric: null session"); return B200TSNE_ERR_INVALID; }
    h->s.symmetric_p = on != 0;
    return 0;
}

int b200tsne_session_attractive_mode(b200tsne_session *h, float *entries_per_group)
{
    if (!h) return 0;
    if (entries_per_group) *entries_per_group = h->s.blocked.entries_per_group;
    return h->s.blocked.ready ? 1 : 0;
}

int b200tsne_repulsive(const float *Y, int64_t N, float *Frep, float *Z, float *w_out, float *ytilde_out, int device)
{
    if (!Y || !Frep || !Z || N <= 0) { set_error("b200tsne_repulsive: invalid arguments"); return B200TSNE_ERR_INVALID; }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *dY = nullptr, *dF = nullptr;
    float2 *dY2 = nullptr, *dF2 = nullptr;
    float4 *dw = nullptr, *dyt = nullptr;
    void *fmem = nullptr;
    IterState *st = nullptr;
    FftWorkspace ws;
    const size_t gsz = sizeof(float4) * kG * kG;
    B200_TRY(up(a, &dY, Y, (size_t)2 * N, sg.st));
    B200_TRY(a.alloc((void **)&dY2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF2, sizeof(float2) * N));
    B200_TRY(a.alloc((void **)&dF, sizeof(float) * 2 * N));
    B200_TRY(a.alloc((void **)&dw, gsz));
    B200_TRY(a.alloc((void **)&dyt, gsz));
    B200_TRY(a.alloc(&fmem, fft_workspace_bytes()));
    B200_TRY(a.alloc((void **)&st, sizeof(IterState)));
    B200_TRY(fft_workspace_init(&ws, fmem, sg.st));
    B200_CUDA(cudaMemsetAsync(dw, 0, gsz, sg.st));
    B200_TRY(launch_soa_to_aos(dY, dY2, N, sg.st));
    B200_TRY(launch_state_reset(st, sg.st));
    B200_TRY(launch_minmax_init(dY2, N, st, 0, sg.st));
    const InterpConsts ic = make_interp_consts();
    B200_TRY(launch_spread(dY2, 0, N, nullptr, st, 0, ic, dw, sg.st));
    if (w_out) B200_TRY(down(w_out, reinterpret_cast<float *>(dw), (size_t)kG * kG * 4, sg.st));
    B200_TRY(launch_convolve(dw, dyt, st, 0, ws, false, sg.st));
    B200_TRY(launch_gather(dY2, 0, N, st, 0, ic, dyt, dF2, true, sg.st));
    B200_TRY(launch_aos_to_soa(dF2, dF, N, sg.st));
    B200_TRY(down(Frep, dF, (size_t)2 * N, sg.st));
    if (ytilde_out) B200_TRY(down(ytilde_out, reinterpret_cast<float *>(dyt), (size_t)kG * kG * 4, sg.st));
    IterState hs;
    B200_CUDA(cudaMemcpyAsync(&hs, st, sizeof(IterState), cudaMemcpyDeviceToHost, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    *Z = (float)hs.zsum[0] - (float)N;
    // the device keeps each node as (x, y, count, r^2); callers get the reference's (count, x, y, r^2)
    for (float *g : {w_out, ytilde_out}) {
        if (!g) continue;
        for (size_t k = 0; k < (size_t)kG * kG; k++) {
            const float a = g[4 * k], b = g[4 * k + 1], c = g[4 * k + 2];
            g[4 * k] = c; g[4 * k + 1] = a; g[4 * k + 2] = b;
        }
    }
    return 0;
}

int b200tsne_apply_forces(float *Y, float *attr, float *rep, float *gains, float *old_forces, float eta,
                          float normalization, float momentum, float exaggeration, int64_t N, int device)
{
    if (!Y || !attr || !rep || !gains || !old_forces || N <= 0) {
        set_error("b200tsne_apply_forces: invalid arguments");
        return B200TSNE_ERR_INVALID;
    }
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    DeviceArena a;
    a.serve(sg.st);
    float *d[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    float *h[5] = {Y, attr, rep, gains, old_forces};
    for (int k = 0; k < 5; k++) B200_TRY(up(a, &d[k], (const float *)h[k], (size_t)2 * N, sg.st));
    B200_TRY(launch_apply_forces_soa(d[0], d[1], d[2], d[3], d[4], eta, normalization, momentum, exaggeration, N, sg.st));
    for (int k = 0; k < 5; k++) B200_TRY(down(h[k], d[k], (size_t)2 * N, sg.st));
    B200_CUDA(cudaStreamSynchronize(sg.st));
    return 0;
}

int b200tsne_knn_last_stats(int *tensor_core, int *rows_recomputed, float *filter_error_ratio)
{
    if (tensor_core) *tensor_core = g_last_knn_stats.tensor_core;
    if (rows_recomputed) *rows_recomputed = g_last_knn_stats.rows_recomputed;
    if (filter_error_ratio) *filter_error_ratio = g_last_knn_stats.filter_error_ratio;
    return 0;
}

int b200tsne_knn_noalloc(const float *X_device, int64_t N, int D, int K, int32_t *ids_device, float *d2_device,
                         void *cuda_stream)
{
    if (!X_device || !ids_device || !d2_device) { set_error("b200tsne_knn_noalloc: null pointer"); return B200TSNE_ERR_INVALID; }
    if (N > 2147483647LL) { set_error("b200tsne_knn_noalloc: too many points"); return B200TSNE_ERR_UNSUPPORTED; }
    return knn_noalloc(X_device, N, D, K, ids_device, d2_device, static_cast<cudaStream_t>(cuda_stream));
}

int64_t b200tsne_knn_noalloc_max_elements(void) { return knn_noalloc_max_elems(); }

// ---- session -------------------------------------------------------------------------------------
int b200tsne_session_create(b200tsne_session **out, int64_t N, int K, int64_t row_lo, int64_t row_hi, int device)
{
    if (!out) { set_error("session_create: null output"); return B200TSNE_ERR_INVALID; }
    *out = nullptr;
    B200_TRY(check_device(device));
    b200tsne_session *h = new (std::nothrow) b200tsne_session();
    if (!h) { set_error("out of host memory"); return B200TSNE_ERR_INVALID; }
    const int rc = h->s.init(N, K, row_lo, row_hi, device);
    if (rc != 0) { h->s.destroy(); delete h; return rc; }
    *out = h;
    return 0;
}

void b200tsne_session_destroy(b200tsne_session *h)
{
    if (!h) return;
    h->s.destroy();
    delete h;
}

int b200tsne_session_set_affinities(b200tsne_session *h, const float *P_rows, const int32_t *ids_rows)
{
    if (!h || !P_rows || !ids_rows) { set_error("session_set_affinities: invalid arguments"); return B200TSNE_ERR_INVALID; }
    Session &s = h->s;
    B200_CUDA(cudaSetDevice(s.device));
    const size_t n = (size_t)s.rows() * s.K;
    B200_CUDA(cudaMemcpyAsync(s.P, P_rows, sizeof(float) * n, cudaMemcpyHostToDevice, s.stream));
    B200_CUDA(cudaMemcpyAsync(s.ids, ids_rows, sizeof(int32_t) * n, cudaMemcpyHostToDevice, s.stream));
    B200_CUDA(cudaStreamSynchronize(s.stream));
    s.cell_order = nullptr;   // no points to order by: the blocked copy, if the graph suits it, uses the natural order
    return s.build_blocked();
}

int b200tsne_session_get_affinities(b200tsne_session *h, float *P_rows, int32_t *ids_rows)
{
    if (!h) { set_error("session_get_affinities: invalid arguments"); return B200TSNE_ERR_INVALID; }
    Session &s = h->s;
    B200_CUDA(cudaSetDevice(s.device));
    const size_t n = (size_t)s.rows() * s.K;
    if (P_rows) B200_CUDA(cudaMemcpyAsync(P_rows, s.P, sizeof(float) * n, cudaMemcpyDeviceToHost, s.stream));
    if (ids_rows) B200_CUDA(cudaMemcpyAsync(ids_rows, s.ids, sizeof(int32_t) * n, cudaMemcpyDeviceToHost, s.stream));
    B200_CUDA(cudaStreamSynchronize(s.stream));
    return 0;
}

int b200tsne_session_affinities_from_points(b200tsne_session *h, const float *X, int D, float perplexity, float epsilon)
{
    if (!h || !X) { set_error("session_affinities_from_points: invalid arguments"); return B200TSNE_ERR_INVALID; }
    return h->s.affinities_from_points(X, D, perplexity, epsilon);
}

int b200tsne_session_set_embedding(b200tsne_session *h, const float *Y, int reset)
{
    if (!h || !Y) { set_error("session_set_embedding: invalid arguments"); return B200TSNE_ERR_INVALID; }
    return h->s.set_embedding_soa(Y, reset != 0);
}

int b200tsne_session_get_embedding(b200tsne_session *h, float *Y)
{
    if (!h || !Y) { set_error("session_get_embedding: invalid arguments"); return B200TSNE_ERR_INVALID; }
    return h->s.get_embedding_soa(Y);
}

int b200tsne_session_get_state(b200tsne_session *h, float *Y, float *momentum, float *gains, int *step)
{
    if (!h) { set_error("session_get_state: null session"); return B200TSNE_ERR_INVALID; }
    if (Y) B200_TRY(h->s.get_embedding_soa(Y));
    B200_TRY(h->s.get_optimizer_soa(momentum, gains));
    if (step) *step = h->s.step;
    return 0;
}

int b200tsne_session_set_state(b200tsne_session *h, const float *Y, const float *momentum, const float *gains, int step)
{
    if (!h || !Y || step < 0) { set_error("session_set_state: invalid arguments"); return B200TSNE_ERR_INVALID; }
    Session &s = h->s;
    if (s.comm && s.comm->world > 1 && ((step ^ s.step) & 1)) {
        // the exchange buffers alternate with the iteration's parity, alike on all ranks
        set_error("session_set_state: in a sharded session the step must keep the parity of the current step");
        return B200TSNE_ERR_UNSUPPORTED;
    }
    s.step = step;                       // set_embedding prepares the min/max slot of this step
    B200_TRY(s.set_embedding_soa(Y, false));
    return s.set_optimizer_soa(momentum, gains);
}

int b200tsne_session_set_schedule(b200tsne_session *h, float learning_rate, float early_exaggeration,
                                  int force_magnify_iters, float pre_momentum, float post_momentum)
{
    if (!h) { set_error("session_set_schedule: null session"); return B200TSNE_ERR_INVALID; }
    h->s.eta = learning_rate;
    h->s.exaggeration = early_exaggeration;
    h->s.force_magnify_iters = force_magnify_iters;
    h->s.pre_momentum = pre_momentum;
    h->s.post_momentum = post_momentum;
    return 0;
}

int b200tsne_session_run(b200tsne_session *h, int n_iters, float min_gradient_norm, float *elapsed_ms, int *iters_done)
{
    if (!h || n_iters < 0) { set_error("session_run: invalid arguments"); return B200TSNE_ERR_INVALID; }
    return h->s.iterate(n_iters, min_gradient_norm, elapsed_ms, iters_done);
}

int b200tsne_session_stats(b200tsne_session *h, float *Z, float *update_norm, int *step)
{
    if (!h) { set_error("session_stats: null session"); return B200TSNE_ERR_INVALID; }
    if (Z) *Z = h->s.last_Z;
    if (update_norm) *update_norm = h->s.last_unorm;
    if (step) *step = h->s.step;
    return 0;
}

int b200tsne_session_enable_stage_timers(b200tsne_session *h, int enable)
{
    if (!h) { set_error("null session"); return B200TSNE_ERR_INVALID; }
    h->s.stage_timers = enable != 0;
    return 0;
}

int b200tsne_session_stage_times(b200tsne_session *h, float *out_ms, int64_t *out_launches)
{
    if (!h) { set_error("null session"); return B200TSNE_ERR_INVALID; }
    for (int k = 0; k < kStages; k++) {
        if (out_ms) out_ms[k] = h->s.stage_ms[k];
        if (out_launches) out_launches[k] = h->s.stage_launches[k];
    }
    return 0;
}

int64_t b200tsne_session_launch_count(b200tsne_session *h) { return h ? h->s.launches : 0; }

int b200tsne_comm_unique_id(void *id128)
{
    if (!id128) { set_error("null id buffer"); return B200TSNE_ERR_INVALID; }
    return comm_unique_id(id128);
}

int b200tsne_session_attach_comm(b200tsne_session *h, const void *id128, int rank, int world_size)
{
    if (!h || !id128) { set_error("attach_comm: invalid arguments"); return B200TSNE_ERR_INVALID; }
    Session &s = h->s;
    if (world_size > 16) { set_error("attach_comm: at most 16 ranks"); return B200TSNE_ERR_UNSUPPORTED; }
    const int64_t chunk = (s.N + world_size - 1) / world_size;
    const int64_t lo = std::min<int64_t>(s.N, (int64_t)rank * chunk), hi = std::min<int64_t>(s.N, lo + chunk);
    if (s.row_lo != lo || s.row_hi != hi) {
        set_error("attach_comm: the session must own rows [rank*ceil(N/world), ...) for the in-place exchanges");
        return B200TSNE_ERR_INVALID;
    }
    B200_CUDA(cudaSetDevice(s.device));
    B200_TRY(s.set_resident(false));   // a sharded session keeps its state in the natural order
    B200_TRY(comm_acquire(&s.comm, id128, rank, world_size));
    return s.attach_peer_exchange();
}

void b200tsne_comm_release_all(void) { comm_release_all(); }

int b200tsne_release_cached_memory(int device)
{
    B200_CUDA(cudaSetDevice(device));
    return release_cached_memory();
}

int b200tsne_session_exchange_mode(b200tsne_session *h)
{
    if (!h || !h->s.comm || h->s.comm->world < 2) return 0;
    return h->s.px ? 2 : 1;
}

int b200tsne_session_set_peer_timeout_ms(b200tsne_session *h, int timeout_ms)
{
    if (!h || timeout_ms <= 0) { set_error("set_peer_timeout_ms: invalid arguments"); return B200TSNE_ERR_INVALID; }
    if (!h->s.px) return 0;   // nothing to bound: single GPU or collectives
    h->s.px->timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    h->s.drop_graphs();       // the limit is a launch argument frozen into captured iterations
    return 0;
}

int b200tsne_selftest_bounded_waits(int device, int timeout_ms, int *peer_status, float *peer_ms, int *barrier_status,
                                    float *barrier_ms)
{
    B200_TRY(check_device(device));
    StreamGuard sg;
    B200_TRY(sg.create());
    const int ps = peer_wait_selftest(timeout_ms, peer_ms, sg.st);
    if (ps != 0 && ps != B200TSNE_ERR_COMM) return ps;
    const int bs = mbar_wait_selftest(timeout_ms, barrier_ms, sg.st);
    if (bs != 0 && bs != B200TSNE_ERR_COMM) return bs;
    if (peer_status) *peer_status = ps;
    if (barrier_status) *barrier_status = bs;
    return 0;
}

}  // extern "C"
