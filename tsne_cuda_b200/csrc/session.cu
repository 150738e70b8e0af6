// Host orchestration of the device-resident FIt-SNE state: allocation, the set-up pipeline from
// points to affinities, and the gradient loop (reference: the body of tsnecuda::RunTsne,
// src/fit_tsne.cu:84-166 for the set-up and :402-580 for the loop).
//
// One iteration is seven kernels (ten when the spread order is refreshed) and no host synchronisation:
//   stream  : [order x3] -> spread -> FFT rows -> FFT columns -> FFT rows^-1 -> gather --> update
//   stream2 : attractive (gather-bound; overlaps the latency-bound grid pipeline) ------^
// The embedding's min/max and the normalisation sum travel between kernels in device memory
// (IterState), so the two per-iteration host round trips of the reference do not exist.
// A sharded run adds two meetings of the ranks per iteration and exchanges over peer memory
// (peer.h): spread -> meet -> sum of the partial grids -> FFT ... update into every rank -> meet.
#include "session.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>

#include "comm.h"
#include "peer.h"

namespace b200 {

// ---- error plumbing -------------------------------------------------------------------------
static thread_local std::string g_last_error;
void set_error(const std::string &msg) { g_last_error = msg; }
const std::string &last_error() { return g_last_error; }
int cuda_fail(cudaError_t e, const char *what, const char *file, int line)
{
    g_last_error = std::string("CUDA error '") + cudaGetErrorString(e) + "' in " + what + " at " + file + ":" +
                   std::to_string(line);
    return -2;
}

// ---- arena ------------------------------------------------------------------------------------
// Device memory comes from the device's default stream-ordered pool with the release threshold lifted, so
// what one call frees the next call gets back without a trip to the driver (a fit allocates and frees
// about 5 GB at N = 10^6; cudaMalloc/cudaFree of that cost tens of milliseconds per call).  Every arena
// is released only after the streams that used its memory have been synchronised, so the memory may be
// handed to any stream afterwards.  b200tsne_release_cached_memory() returns the pool to the driver.
static int configure_pool()
{
    static bool done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || done[dev]) return 0;
    cudaMemPool_t pool;
    B200_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    unsigned long long keep = ~0ull;
    B200_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    done[dev] = true;
    return 0;
}

int release_cached_memory()
{
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    cudaMemPool_t pool;
    B200_CUDA(cudaDeviceGetDefaultMemPool(&pool, dev));
    B200_CUDA(cudaDeviceSynchronize());
    B200_CUDA(cudaMemPoolTrimTo(pool, 0));
    return 0;
}

DeviceArena::~DeviceArena() { release(); }
int DeviceArena::alloc(void **p, size_t bytes)
{
    *p = nullptr;
    if (bytes == 0) bytes = 16;
    B200_TRY(configure_pool());
    B200_CUDA(cudaMallocAsync(p, bytes, cudaStreamPerThread));
    ptrs.push_back(*p);
    // B200TSNE_POISON=1 fills every new allocation with 0xFF bytes (NaN floats, -1 ints): pooled memory is not
    // zero like fresh device memory often is, and this makes any read of memory the library has not written
    // show up at once (the GPU suite passes with it)
    static const bool poison = getenv("B200TSNE_POISON") && atoi(getenv("B200TSNE_POISON")) != 0;
    if (poison) {
        B200_CUDA(cudaMemsetAsync(*p, 0xff, bytes, cudaStreamPerThread));
        B200_CUDA(cudaStreamSynchronize(cudaStreamPerThread));
    }
    return 0;
}
void DeviceArena::release()
{
    // also on error paths, where kernels queued on a consumer stream may still be running
    if (!ptrs.empty())
        for (cudaStream_t st : consumers) cudaStreamSynchronize(st);
    consumers.clear();
    for (void *p : ptrs) cudaFreeAsync(p, cudaStreamPerThread);
    if (!ptrs.empty()) cudaStreamSynchronize(cudaStreamPerThread);
    ptrs.clear();
}

// ---- session ------------------------------------------------------------------------------------
int Session::init(int64_t N_, int K_, int64_t lo, int64_t hi, int device_)
{
    if (N_ <= 0 || K_ <= 0 || lo < 0 || hi > N_ || lo > hi) { set_error("session: invalid sizes"); return -1; }
    if (N_ >= (int64_t)1 << 31) { set_error("session: more than 2^31-1 points are not supported (int32 ids)"); return -4; }
    N = N_; K = K_; row_lo = lo; row_hi = hi; device = device_;
    B200_CUDA(cudaSetDevice(device));
    // (Stream priorities were measured both ways and change nothing: the attractive kernel and the grid
    // pipeline compete for the same load/store units rather than for block slots.)
    B200_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    B200_CUDA(cudaStreamCreateWithFlags(&stream2, cudaStreamNonBlocking));
    B200_CUDA(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
    B200_CUDA(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
    B200_CUDA(cudaEventCreate(&ev_t0));
    B200_CUDA(cudaEventCreate(&ev_t1));
    arena.serve(stream);
    arena.serve(stream2);
    blocked_arena.serve(stream);
    blocked_arena.serve(stream2);
    // Y2 and the force arrays are padded so that an in-place all-gather over up to 16 ranks fits
    const int64_t npad = N + 16;
    const int64_t r = std::max<int64_t>(rows(), 1);
    B200_TRY(arena.alloc((void **)&P, sizeof(float) * r * K));
    B200_TRY(arena.alloc((void **)&ids, sizeof(int32_t) * r * K));
    B200_TRY(arena.alloc((void **)&order, sizeof(int32_t) * r));
    B200_TRY(arena.alloc((void **)&order_alt, sizeof(int32_t) * r));
    B200_TRY(arena.alloc((void **)&order_keys, sizeof(int32_t) * r));
    B200_TRY(arena.alloc((void **)&box_hist, sizeof(int32_t) * kBoxes * kBoxes));
    B200_TRY(launch_order_identity(order, rows(), stream));
    if (const char *e = getenv("B200TSNE_ORDER_REFRESH")) order_refresh = atoi(e);
    if (const char *e = getenv("B200TSNE_ORDER_REFRESH_EARLY")) order_refresh_early = std::max(1, atoi(e));
    if (const char *e = getenv("B200TSNE_GRAPHS")) use_graphs = atoi(e) != 0;
    B200_TRY(arena.alloc((void **)&Y2, sizeof(float2) * npad));
    B200_TRY(arena.alloc((void **)&Fattr, sizeof(float2) * npad));
    B200_TRY(arena.alloc((void **)&Frep, sizeof(float2) * npad));
    B200_TRY(arena.alloc((void **)&gains, sizeof(float2) * r));
    B200_TRY(arena.alloc((void **)&u, sizeof(float2) * r));
    B200_TRY(arena.alloc((void **)&soa_tmp, sizeof(float) * 2 * N));
    B200_TRY(arena.alloc((void **)&w, sizeof(float4) * kG * kG));
    B200_TRY(arena.alloc((void **)&ytilde, sizeof(float4) * kG * kG));
    B200_TRY(arena.alloc(&fft_mem, fft_workspace_bytes()));
    B200_TRY(arena.alloc((void **)&state, sizeof(IterState)));
    B200_CUDA(cudaMallocHost((void **)&h_state, sizeof(IterState)));
    B200_TRY(fft_workspace_init(&fft, fft_mem, stream));
    Y2_own = Y2;
    w_own = w;
    ic = make_interp_consts();
    B200_CUDA(cudaMemsetAsync(w, 0, sizeof(float4) * kG * kG, stream));
    B200_CUDA(cudaMemsetAsync(Y2, 0, sizeof(float2) * npad, stream));
    B200_CUDA(cudaMemsetAsync(Fattr, 0, sizeof(float2) * npad, stream));
    B200_CUDA(cudaMemsetAsync(Frep, 0, sizeof(float2) * npad, stream));
    B200_TRY(launch_state_reset(state, stream));
    B200_TRY(launch_fill(reinterpret_cast<float *>(gains), 1.0f, 2 * r, stream));
    B200_CUDA(cudaMemsetAsync(u, 0, sizeof(float2) * r, stream));
    B200_CUDA(cudaStreamSynchronize(stream));
    return 0;
}

void Session::destroy()
{
    cudaSetDevice(device);
    if (stream) cudaStreamSynchronize(stream);
    if (stream2) cudaStreamSynchronize(stream2);
    drop_graphs();
    if (px) { peer_exchange_release(px, comm); px = nullptr; }
    comm = nullptr;  // owned by the communicator cache (comm.h)
    blocked.clear();
    blocked_arena.release();
    arena.release();
    if (h_state) cudaFreeHost(h_state);
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
    if (ev_t0) cudaEventDestroy(ev_t0);
    if (ev_t1) cudaEventDestroy(ev_t1);
    if (stream) cudaStreamDestroy(stream);
    if (stream2) cudaStreamDestroy(stream2);
    h_state = nullptr; stream = stream2 = nullptr; ev_fork = ev_join = ev_t0 = ev_t1 = nullptr;
}

int Session::set_embedding_soa(const float *Y_host, bool reset)
{
    B200_CUDA(cudaSetDevice(device));
    B200_CUDA(cudaMemcpyAsync(soa_tmp, Y_host, sizeof(float) * 2 * N, cudaMemcpyHostToDevice, stream));
    B200_TRY(launch_soa_to_aos(soa_tmp, Y2, N, stream, state_order()));
    if (reset) {
        const int64_t r = std::max<int64_t>(rows(), 1);
        B200_TRY(launch_fill(reinterpret_cast<float *>(gains), 1.0f, 2 * r, stream));
        B200_CUDA(cudaMemsetAsync(u, 0, sizeof(float2) * r, stream));
        step = 0;
    }
    B200_TRY(launch_state_reset(state, stream));
    B200_TRY(launch_minmax_init(Y2, N, state, step & 1, stream));
    B200_CUDA(cudaMemsetAsync(w, 0, sizeof(float4) * kG * kG, stream));
    B200_CUDA(cudaStreamSynchronize(stream));
    launches += 4;
    return 0;
}

int Session::get_embedding_soa(float *Y_host)
{
    B200_CUDA(cudaSetDevice(device));
    B200_TRY(launch_aos_to_soa(Y2, soa_tmp, N, stream, state_order()));
    B200_CUDA(cudaMemcpyAsync(Y_host, soa_tmp, sizeof(float) * 2 * N, cudaMemcpyDeviceToHost, stream));
    B200_CUDA(cudaStreamSynchronize(stream));
    launches += 1;
    return 0;
}

int Session::get_optimizer_soa(float *momentum_host, float *gains_host)
{
    B200_CUDA(cudaSetDevice(device));
    const int64_t r = rows();
    if (r == 0) return 0;
    if (momentum_host) {
        B200_TRY(launch_aos_to_soa(u, soa_tmp, r, stream, state_order()));
        B200_CUDA(cudaMemcpyAsync(momentum_host, soa_tmp, sizeof(float) * 2 * r, cudaMemcpyDeviceToHost, stream));
        B200_CUDA(cudaStreamSynchronize(stream));
    }
    if (gains_host) {
        B200_TRY(launch_aos_to_soa(gains, soa_tmp, r, stream, state_order()));
        B200_CUDA(cudaMemcpyAsync(gains_host, soa_tmp, sizeof(float) * 2 * r, cudaMemcpyDeviceToHost, stream));
        B200_CUDA(cudaStreamSynchronize(stream));
    }
    return 0;
}

int Session::set_optimizer_soa(const float *momentum_host, const float *gains_host)
{
    B200_CUDA(cudaSetDevice(device));
    const int64_t r = rows();
    if (r == 0) return 0;
    if (momentum_host) {
        B200_CUDA(cudaMemcpyAsync(soa_tmp, momentum_host, sizeof(float) * 2 * r, cudaMemcpyHostToDevice, stream));
        B200_TRY(launch_soa_to_aos(soa_tmp, u, r, stream, state_order()));
        B200_CUDA(cudaStreamSynchronize(stream));
    }
    if (gains_host) {
        B200_CUDA(cudaMemcpyAsync(soa_tmp, gains_host, sizeof(float) * 2 * r, cudaMemcpyHostToDevice, stream));
        B200_TRY(launch_soa_to_aos(soa_tmp, gains, r, stream, state_order()));
        B200_CUDA(cudaStreamSynchronize(stream));
    }
    return 0;
}

namespace {
// Times the stages of one iteration when stage timers are on (serialised on one stream).
struct StageClock {
    Session *s;
    cudaEvent_t a = nullptr, b = nullptr;
    explicit StageClock(Session *s_) : s(s_)
    {
        if (s->stage_timers) { cudaEventCreate(&a); cudaEventCreate(&b); }
    }
    ~StageClock()
    {
        if (a) cudaEventDestroy(a);
        if (b) cudaEventDestroy(b);
    }
    void begin(cudaStream_t st) { if (a) cudaEventRecord(a, st); }
    void end(cudaStream_t st, int stage, int n_launches)
    {
        s->launches += n_launches;
        if (!a) return;
        s->stage_launches[stage] += n_launches;
        cudaEventRecord(b, st);
        cudaEventSynchronize(b);
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, a, b);
        s->stage_ms[stage] += ms;
    }
};
}  // namespace

int Session::one_iteration(bool want_norm)
{
    const int slot = step & 1;
    const bool late = step >= force_magnify_iters;
    const float momentum = late ? post_momentum : pre_momentum;
    const float exag = late ? 1.0f : exaggeration;
    const bool multi = comm && comm->world > 1;
    const bool p2p = multi && px != nullptr;   // exchanges over peer memory instead of collectives
    StageClock clk(this);
    cudaStream_t sa = stage_timers ? stream : stream2;  // attractive stream
    if (p2p) {
        // the grid buffer of the next iteration: the peers finished reading it before they signalled the
        // update this rank waited for at the end of the previous iteration
        B200_CUDA(cudaMemsetAsync(px->w_local(px->parity ^ 1), 0, sizeof(float4) * kG * kG, stream));
    }

    // The attractive kernel (one block per SM on 8/9 of the SMs) and the grid pipeline run side by side.  Timestamps
    // taken inside the kernels at N = 10^6 (one GPU): the attractive kernel runs 190 us and ends 37 us before the
    // update can start; the pipeline, 90 us when it has the GPU to itself, takes 229 us on the SMs that are left and
    // is what the update waits for.  More SMs for the pipeline slow the attractive kernel by as much as they speed
    // the pipeline up (124, 132 and 140 attractive blocks: 3 940, 3 955, 3 905 iterations/s): the iteration is bound
    // by the SM time of its kernels, not by their overlap.  Neither a higher stream priority for the attractive
    // kernel nor holding the pipeline back until its blocks are resident (they are within 8 us anyway) changed it.
    // Inside the pipeline it is the spread that suffers: 118 us on the 16 spare SMs against 28 alone (scatter 37
    // against 26; FFT and gather as when alone), 60 us when 32 SMs are spared, which costs the attractive kernel more.
    // An L2 evict-first policy on the attractive kernel's stream loads: +0.8 %, not kept.
    if (!stage_timers) {
        B200_CUDA(cudaEventRecord(ev_fork, stream));
        B200_CUDA(cudaStreamWaitEvent(stream2, ev_fork, 0));
        B200_TRY(attractive(sa));
        B200_CUDA(cudaEventRecord(ev_join, stream2));
        launches += attractive_launches();
    }

    // The embedding reshuffles quickly while it is being exaggerated and slowly afterwards: sort every
    // iteration early, every order_refresh iterations later.  (Sorting the rows for iteration t + 1 at the end of
    // iteration t, while waiting for the other ranks, was measured on two GPUs: the next bounding box is only
    // known after that meeting, and boxes taken from the previous one - the embedding grows by more than a box
    // width per exaggerated iteration - break the runs of equal boxes: spread 61 us instead of 15.)
    const bool settling = step < force_magnify_iters + 50;
    const int refresh_every = settling ? order_refresh_early : order_refresh;
    if (order_refresh > 0 && step % refresh_every == 0) {
        clk.begin(stream);
        B200_TRY(launch_order_refresh(Y2, row_lo, row_hi, order, order_alt, order_keys, box_hist, state, slot, stream));
        std::swap(order, order_alt);
        clk.end(stream, kStOrder, 3);
    }
    clk.begin(stream);
    B200_TRY(launch_spread(Y2, row_lo, row_hi, order_refresh > 0 ? order : nullptr, state, slot, ic, w, stream));
    clk.end(stream, kStSpread, 1);
    if (p2p) {
        clk.begin(stream);
        if (grid_two_shot) {
            B200_TRY(launch_peer_grid_allreduce(px, px->parity, stream));
            clk.end(stream, kStExchange, 1);
        } else {
            B200_TRY(launch_peer_barrier(px, kFlagSpread, nullptr, 0, stream));
            B200_TRY(launch_peer_grid_reduce(px, px->parity, w_sum, stream));
            clk.end(stream, kStExchange, 2);
        }
    } else if (multi) {
        clk.begin(stream);
        B200_TRY(comm->all_reduce_sum_f32(reinterpret_cast<float *>(w), (size_t)kG * kG * 4, stream));
        clk.end(stream, kStExchange, 0);
    }
    clk.begin(stream);
    B200_TRY(launch_convolve(p2p ? w_sum : w, ytilde, state, slot, fft, !p2p, stream));
    clk.end(stream, kStConvolve, 3);
    clk.begin(stream);
    B200_TRY(launch_gather(Y2, row_lo, row_hi, state, slot, ic, ytilde, Frep, !p2p, stream));
    clk.end(stream, kStGather, 1);
    if (p2p) {
        // sum of Z_i over ALL points from the summed grid: no exchange
        clk.begin(stream);
        B200_TRY(launch_grid_z(w_sum, ytilde, state, slot, stream));
        clk.end(stream, kStGather, 1);
    } else if (multi) {
        clk.begin(stream);
        B200_TRY(comm->all_reduce_sum_f64(&state->zsum[slot], 1, stream));
        clk.end(stream, kStExchange, 0);
    }
    if (stage_timers) {
        clk.begin(stream);
        B200_TRY(attractive(stream));
        clk.end(stream, kStAttractive, attractive_launches());
    } else {
        B200_CUDA(cudaStreamWaitEvent(stream, ev_join, 0));
    }
    clk.begin(stream);
    UpdateTargets dst;
    dst.n = 1;
    dst.p[0] = Y2;
    if (p2p) {   // the new rows go straight into the next embedding buffer of every rank
        dst.n = comm->world;
        for (int r = 0; r < comm->world; r++) dst.p[r] = px->tab.y[px->parity ^ 1][r];
    }
    B200_TRY(launch_update(Y2, dst, Fattr, Frep, gains, u, N, row_lo, row_hi, state, slot, eta, momentum, exag,
                           want_norm ? 1 : 0, stream));
    clk.end(stream, kStUpdate, 1);
    if (p2p) {
        clk.begin(stream);
        // the update kernel left this rank's min/max in slot^1; the meeting makes them global
        B200_TRY(launch_peer_barrier(px, kFlagUpdate, state, slot ^ 1, stream));
        px->parity ^= 1;
        Y2 = px->y_local(px->parity);
        w = px->w_local(px->parity);
        clk.end(stream, kStExchange, 1);
    } else if (multi) {
        clk.begin(stream);
        const int64_t chunk = (N + comm->world - 1) / comm->world;
        B200_TRY(comm->all_gather_inplace(Y2, sizeof(float2) * (size_t)chunk, stream));
        B200_TRY(launch_minmax_init(Y2, N, state, slot ^ 1, stream));
        clk.end(stream, kStExchange, 2);
    }
    step++;
    return 0;
}

int Session::attractive(cudaStream_t st)
{
    if (blocked.ready) return launch_attractive_blocked(blocked, Y2, Fattr, st, resident);
    B200_TRY(launch_attractive(P, ids, Y2, N, K, row_lo, row_hi, Fattr, st));
    if (extra.count > 0) B200_TRY(launch_attractive_extra(extra.ptr, extra.ids, extra.val, Y2, N, row_lo, row_hi, Fattr, st));
    return 0;
}

int Session::set_resident(bool on)
{
    if (on == resident) return 0;
    if (!blocked.ready || rows() != N) { set_error("session: no point order to keep the state in"); return -1; }
    // Frep is scratch between iterations
    float2 *arrays[3] = {Y2, u, gains};
    for (float2 *a : arrays) {
        B200_TRY(launch_reorder_pairs(a, Frep, N, blocked.perm, /*scatter=*/!on, stream));
        B200_CUDA(cudaMemcpyAsync(a, Frep, sizeof(float2) * (size_t)N, cudaMemcpyDeviceToDevice, stream));
    }
    B200_CUDA(cudaStreamSynchronize(stream));
    resident = on;
    return 0;
}

int Session::build_blocked()
{
    B200_CUDA(cudaStreamSynchronize(stream));
    B200_CUDA(cudaStreamSynchronize(stream2));
    drop_graphs();   // captured iterations hold the pointers of the previous copy
    B200_TRY(set_resident(false));   // back to the natural order while the old copy's order still exists
    blocked.clear();
    blocked_arena.release();
    blocked_arena.serve(stream);
    blocked_arena.serve(stream2);
    B200_TRY(blocked_attractive_build(&blocked, blocked_arena, P, ids, N, K, row_lo, row_hi, cell_order, extra.count > 0 ? &extra : nullptr,
                                      stream));
    const char *e = getenv("B200TSNE_ATTRACTIVE_RESIDENT");
    const bool multi = comm && comm->world > 1;
    if (blocked.ready && !multi && rows() == N && !(e && atoi(e) == 0)) B200_TRY(set_resident(true));
    return 0;
}

void Session::drop_graphs()
{
    for (IterGraph &g : graphs) {
        if (g.exec) cudaGraphExecDestroy(g.exec);
        g = IterGraph();
    }
}

// Which graph covers the iterations from `step` on, and how many of them; 0 when the next iteration has to be
// launched directly (misaligned with the block, a phase boundary inside it, or a feature graphs do not carry).
int Session::graph_block(int remaining, bool want_norm, int *kind) const
{
    // (a sharded run qualifies when it exchanges over peer memory: its meetings are kernels of this library)
    if (!use_graphs || stage_timers || want_norm || (comm && comm->world > 1 && !px) || order_refresh_early != 1) return 0;
    const int settle_end = force_magnify_iters + 50;
    int k, block, limit;
    if (step < force_magnify_iters) { k = 0; block = 2; limit = force_magnify_iters; }
    else if (step < settle_end) { k = 1; block = 2; limit = settle_end; }
    else { k = 2; block = order_refresh > 0 ? 2 * order_refresh : 2; limit = INT_MAX; }
    if (step % block != 0 || remaining < block || (long long)step + block > limit) return 0;
    *kind = k;
    return block;
}

int Session::run_graph_block(int kind, int iters)
{
    IterGraph &g = graphs[kind];
    const bool late = kind > 0;
    const float momentum = late ? post_momentum : pre_momentum, exag = late ? 1.0f : exaggeration;
    const int parity = px ? px->parity : 0;   // which exchange buffers the block starts from
    if (g.exec && (g.iters != iters || g.eta != eta || g.exaggeration != exag || g.momentum != momentum || g.refresh != order_refresh ||
                   g.parity != parity)) {
        cudaGraphExecDestroy(g.exec);
        g = IterGraph();
    }
    if (!g.exec) {
        // capture: the launches are recorded, not run, so the host-side counters are put back afterwards
        const int step0 = step;
        const int64_t launches0 = launches;
        int32_t *const order0 = order;
        cudaGraph_t graph = nullptr;
        B200_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        int rc = 0;
        for (int b = 0; b < iters && rc == 0; b++) rc = one_iteration(false);
        const cudaError_t end = cudaStreamEndCapture(stream, &graph);
        g.launches = launches - launches0;
        step = step0;
        launches = launches0;
        const bool same_order = order == order0 && (!px || px->parity == parity);
        if (order != order0) std::swap(order, order_alt);
        if (px && px->parity != parity) { px->parity = parity; Y2 = px->y_local(parity); w = px->w_local(parity); }
        if (rc != 0 || end != cudaSuccess || !graph || !same_order) {
            if (graph) cudaGraphDestroy(graph);
            (void)cudaGetLastError();
            use_graphs = false;   // the caller falls back to direct launches
            return 1;
        }
        const cudaError_t inst = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (inst != cudaSuccess) {
            (void)cudaGetLastError();
            g = IterGraph();
            use_graphs = false;
            return 1;
        }
        g.iters = iters;
        g.eta = eta; g.exaggeration = exag; g.momentum = momentum; g.refresh = order_refresh; g.parity = parity;
    }
    B200_CUDA(cudaGraphLaunch(g.exec, stream));
    step += iters;
    launches += g.launches;
    return 0;
}

int Session::iterate(int n_iters, float min_gradient_norm, float *elapsed_ms, int *iters_done)
{
    B200_CUDA(cudaSetDevice(device));
    const bool early_stop = min_gradient_norm > 0.0f;
    const bool want_norm = early_stop || force_norm;
    int done = 0;
    B200_CUDA(cudaEventRecord(ev_t0, stream));
    for (int it = 0; it < n_iters; it++) {
        // a meeting of the ranks gave up (the kernel says so in mapped host memory): queue nothing more
        if (px && *px->err_host) break;
        int kind = 0;
        const int block = graph_block(n_iters - it, want_norm, &kind);
        if (block > 0) {
            const int rc = run_graph_block(kind, block);
            if (rc < 0) return rc;
            if (rc == 0) { done += block; it += block - 1; continue; }
        }
        if (want_norm) B200_CUDA(cudaMemsetAsync(&state->unorm2, 0, sizeof(double), stream));
        B200_TRY(one_iteration(want_norm));
        done++;
        if (early_stop) {
            B200_CUDA(cudaMemcpyAsync(h_state, state, sizeof(IterState), cudaMemcpyDeviceToHost, stream));
            B200_CUDA(cudaStreamSynchronize(stream));
            double n2 = h_state->unorm2;
            if (comm && comm->world > 1) {
                // every rank must take the same decision: sum the squared norms
                B200_TRY(comm->all_reduce_sum_f64(&state->unorm2, 1, stream));
                B200_CUDA(cudaMemcpyAsync(h_state, state, sizeof(IterState), cudaMemcpyDeviceToHost, stream));
                B200_CUDA(cudaStreamSynchronize(stream));
                n2 = h_state->unorm2;
            }
            last_unorm = (float)sqrt(n2);
            if (last_unorm < min_gradient_norm) break;
        }
    }
    B200_CUDA(cudaEventRecord(ev_t1, stream));
    B200_CUDA(cudaMemcpyAsync(h_state, state, sizeof(IterState), cudaMemcpyDeviceToHost, stream));
    B200_CUDA(cudaStreamSynchronize(stream));
    B200_CUDA(cudaStreamSynchronize(stream2));
    if (elapsed_ms) B200_CUDA(cudaEventElapsedTime(elapsed_ms, ev_t0, ev_t1));
    if (iters_done) *iters_done = done;
    if (done > 0) last_Z = (float)h_state->zsum[(step - 1) & 1] - (float)N;
    if (want_norm && !early_stop && done > 0) last_unorm = (float)sqrt(h_state->unorm2);
    if (h_state->bad) { set_error("non-finite coordinates in the embedding"); return -3; }
    if (px) {
        int expired = 0;
        B200_CUDA(cudaMemcpy(&expired, px->err, sizeof(int), cudaMemcpyDeviceToHost));
        if (expired || *px->err_host) {
            px->failed = true;
            set_error("peer exchange: a rank did not arrive within " + std::to_string(px->timeout_ns / 1000000ull) + " ms");
            return -5;
        }
    }
    return 0;
}

int Session::attach_peer_exchange()
{
    if (!comm || comm->world < 2 || px) return 0;
    const char *e = getenv("B200TSNE_EXCHANGE");   // "nccl": collectives only (must be set alike on all ranks)
    if (e && strcmp(e, "nccl") == 0) return 0;
    B200_CUDA(cudaSetDevice(device));
    B200_TRY(peer_exchange_acquire(&px, comm, N + 16, stream));
    if (!px) return 0;
    // The grid sum: every rank reads all partial grids ((W - 1) x 2.4 MB over NVLink per rank), or the slice owners
    // form (2 x 2.4 MB x (W - 1) / W and one more flag round trip).  B200TSNE_GRID_SUM = "all" / "slices"; default:
    // slices from eight ranks on.  Measured at N = 10^6: four ranks, slices 3 % slower (6 078 against 6 290
    // iterations/s: the extra round trip costs more than 3.6 MB less traffic saves); eight ranks, slices 12 % faster
    // (7 807 against 6 939: 4.2 MB instead of 16.8 MB per rank and iteration).
    {
        const char *g = getenv("B200TSNE_GRID_SUM");
        grid_two_shot = g ? strcmp(g, "slices") == 0 : comm->world >= 8;
    }
    if (grid_two_shot) w_sum = px->ws_local();
    else B200_TRY(arena.alloc((void **)&w_sum, sizeof(float4) * kG * kG));
    B200_CUDA(cudaMemcpyAsync(px->y_local(px->parity), Y2_own, sizeof(float2) * (size_t)N, cudaMemcpyDeviceToDevice, stream));
    B200_CUDA(cudaStreamSynchronize(stream));
    Y2 = px->y_local(px->parity);
    w = px->w_local(px->parity);
    return 0;
}

// ---- set-up: points -> kNN -> perplexity -> symmetrised fixed-width P ------------------------------
int Session::affinities_from_points(const float *X_host, int D, float perplexity, float eps)
{
    B200_CUDA(cudaSetDevice(device));
    if (D <= 0 || !X_host) { set_error("affinities: invalid points"); return -1; }
    if (K > N) { set_error("affinities: num_neighbors exceeds num_points"); return -1; }
    const bool multi = comm && comm->world > 1;
    DeviceArena tmp;
    tmp.serve(stream);
    float *X = nullptr, *d2 = nullptr, *p_all = nullptr;
    int32_t *ids_all = nullptr;
    unsigned int *max_enc = nullptr;
    const int64_t r = rows();
    const int64_t chunk = multi ? (N + comm->world - 1) / comm->world : N;
    const int64_t npad = multi ? chunk * comm->world : N;

    StageClock clk(this);
    B200_TRY(tmp.alloc((void **)&X, sizeof(float) * N * D));
    B200_CUDA(cudaMemcpyAsync(X, X_host, sizeof(float) * N * D, cudaMemcpyHostToDevice, stream));
    clk.begin(stream);   // the search itself: the points are on their way
    B200_TRY(tmp.alloc((void **)&d2, sizeof(float) * std::max<int64_t>(chunk, 1) * K));
    B200_TRY(tmp.alloc((void **)&max_enc, sizeof(unsigned int)));
    // Every rank holds all the points.  By default the QUERIES are sharded: a rank searches its own
    // rows against the whole database and needs no exchange, and its cost falls as 1/world (the
    // search costs about the same per query whatever the database size).  B200TSNE_KNN_SHARD=database
    // shards the DATABASE instead, as a deployment whose points do not fit one GPU would: every rank
    // searches all queries against its own rows, and the owners of the query rows receive the
    // partial lists (all-to-all) and merge them.  Both give the same lists bit for bit.
    const char *shard_env = getenv("B200TSNE_KNN_SHARD");
    bool db_sharded = multi && shard_env && strcmp(shard_env, "database") == 0;
    if (multi && !shard_env && knn_tc_supported(N, D, K)) {
        // no wish stated: shard the database when the operand images of ALL points and the buffers of this rank's
        // queries would not fit in half of what is free (every rank decides alike: same sizes, and the ranks of a
        // node have the same memory)
        size_t free_b = 0, total_b = 0;
        B200_CUDA(cudaMemGetInfo(&free_b, &total_b));
        const int64_t batch = std::min<int64_t>(std::max<int64_t>(r, 1), 1 << 20);
        if (knn_tc_workspace_bytes(D, K, batch, N) > total_b / 2) db_sharded = true;
    }
    if (!db_sharded) {
        B200_TRY(knn_search(X, N, D, K, row_lo, row_hi, 0, N, ids, d2, &knn_stats, stream));
    } else {
        int32_t *part_i = nullptr, *recv_i = nullptr;
        float *part_d = nullptr, *recv_d = nullptr;
        B200_TRY(tmp.alloc((void **)&part_i, sizeof(int32_t) * npad * K));
        B200_TRY(tmp.alloc((void **)&part_d, sizeof(float) * npad * K));
        B200_TRY(tmp.alloc((void **)&recv_i, sizeof(int32_t) * npad * K));
        B200_TRY(tmp.alloc((void **)&recv_d, sizeof(float) * npad * K));
        B200_CUDA(cudaMemsetAsync(part_i, 0x7f, sizeof(int32_t) * npad * K, stream));
        B200_CUDA(cudaMemsetAsync(part_d, 0x7f, sizeof(float) * npad * K, stream));
        B200_TRY(knn_search(X, N, D, K, 0, N, row_lo, row_hi, part_i, part_d, &knn_stats, stream));
        B200_TRY(comm->all_to_all(part_i, recv_i, sizeof(int32_t) * (size_t)chunk * K, stream));
        B200_TRY(comm->all_to_all(part_d, recv_d, sizeof(float) * (size_t)chunk * K, stream));
        B200_TRY(launch_knn_merge(recv_i, recv_d, comm->world, chunk * K, r, K, ids, d2, stream));
    }
    B200_TRY(launch_knn_finalize(ids, d2, r * K, stream));
    clk.end(stream, kStKnn, 4);

    clk.begin(stream);
    // the order in which the attractive force's blocked copy of P numbers the points (every rank computes the same)
    {
        const char *mode = getenv("B200TSNE_ATTRACTIVE");
        if (!(mode && strcmp(mode, "rows") == 0)) {
            if (!cell_order) B200_TRY(arena.alloc((void **)&cell_order, sizeof(int32_t) * N));
            B200_TRY(order_points_by_cell(X, N, D, cell_order, stream));
        }
    }

    clk.begin(stream);
    const unsigned int zero_enc = enc_float(0.0f);
    B200_CUDA(cudaMemcpyAsync(max_enc, &zero_enc, sizeof(unsigned int), cudaMemcpyHostToDevice, stream));
    B200_TRY(launch_absmax(d2, r * K, max_enc, stream));
    if (multi) B200_TRY(comm->all_reduce_max_u32(max_enc, 1, stream));
    B200_TRY(tmp.alloc((void **)&p_all, sizeof(float) * npad * K));
    float *p_rows = p_all + (multi ? (size_t)comm->rank * chunk * K : 0);
    B200_TRY(launch_perplexity(d2, r, K, perplexity, eps, max_enc, p_rows, nullptr, stream));
    const int32_t *ids_for_sym = ids;
    if (multi) {
        B200_TRY(tmp.alloc((void **)&ids_all, sizeof(int32_t) * npad * K));
        B200_CUDA(cudaMemcpyAsync(ids_all + (size_t)comm->rank * chunk * K, ids, sizeof(int32_t) * r * K,
                                  cudaMemcpyDeviceToDevice, stream));
        B200_TRY(comm->all_gather_inplace(ids_all, sizeof(int32_t) * (size_t)chunk * K, stream));
        B200_TRY(comm->all_gather_inplace(p_all, sizeof(float) * (size_t)chunk * K, stream));
        ids_for_sym = ids_all;
    }
    // one GPU: the rows are taken in the cell order, cluster by cluster (the rows a row looks up are then in L2)
    B200_TRY(launch_symmetrize(p_all, ids_for_sym, N, K, row_lo, row_hi, P, stream, (!multi && cell_order && row_lo == 0 && row_hi == N) ? cell_order : nullptr));
    extra = ExtraEntries();
    if (symmetric_p || (getenv("B200TSNE_SYMMETRIC_P") && atoi(getenv("B200TSNE_SYMMETRIC_P")) != 0)) {
        // the mirror images of the one-directional edges whose target is an owned row (affinities.cu)
        int64_t n_extra = 0;
        int *cursor = nullptr;
        if (!extra_ptr) B200_TRY(arena.alloc((void **)&extra_ptr, sizeof(int) * (r + 1)));
        B200_TRY(launch_reverse_only_count(p_all, ids_for_sym, N, K, row_lo, row_hi, extra_ptr, &n_extra, stream));
        B200_TRY(tmp.alloc((void **)&cursor, sizeof(int) * std::max<int64_t>(r, 1)));
        B200_TRY(arena.alloc((void **)&extra_ids, sizeof(int32_t) * std::max<int64_t>(n_extra, 1)));   // (a second call leaves the first lists to the arena)
        B200_TRY(arena.alloc((void **)&extra_val, sizeof(float) * std::max<int64_t>(n_extra, 1)));
        B200_TRY(launch_reverse_only_fill(p_all, ids_for_sym, N, K, row_lo, row_hi, extra_ptr, cursor, extra_ids, extra_val, stream));
        extra.ptr = extra_ptr; extra.ids = extra_ids; extra.val = extra_val; extra.count = n_extra;
    }
    B200_TRY(build_blocked());
    clk.end(stream, kStAffinities, 3);
    B200_CUDA(cudaStreamSynchronize(stream));
    return 0;
}

}  // namespace b200
