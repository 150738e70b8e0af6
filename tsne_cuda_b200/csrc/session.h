// Device-resident state of one FIt-SNE run on one GPU (one rank of a multi-GPU run).
#pragma once
#include <cuda_runtime.h>

#include <vector>

#include "common.cuh"

namespace b200 {

struct Comm;          // comm.h
struct PeerExchange;  // peer.h

enum Stage { kStSpread = 0, kStConvolve, kStGather, kStAttractive, kStUpdate, kStExchange, kStKnn, kStAffinities, kStOrder };

// RAII holder for device allocations of a session
struct DeviceArena {
    std::vector<void *> ptrs;
    std::vector<cudaStream_t> consumers;   // streams whose work uses this memory: synchronised before anything is freed
    ~DeviceArena();
    void serve(cudaStream_t st) { consumers.push_back(st); }
    int alloc(void **p, size_t bytes);
    void release();
};

struct Session {
    int device = 0;
    int64_t N = 0;           // all points
    int K = 0;
    int64_t row_lo = 0, row_hi = 0;  // owned rows
    cudaStream_t stream = nullptr;
    cudaStream_t stream2 = nullptr;  // attractive force overlaps the grid pipeline
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_t0 = nullptr, ev_t1 = nullptr;
    DeviceArena arena;

    // affinities (owned rows)
    float *P = nullptr;       // [rows][K]
    int32_t *ids = nullptr;   // [rows][K]
    // Column-blocked copy of P for the attractive force (attractive_blocked.cu), built with the affinities when the
    // neighbours of a row fall into few tiles of the cell order; otherwise the row-major kernel reads P / ids.
    BlockedAttractive blocked;
    DeviceArena blocked_arena;
    int32_t *cell_order = nullptr;   // [N] point order by cell (from the points; null = natural order)
    int build_blocked();             // (re)builds `blocked` from P / ids; drops captured iterations
    // One GPU with the blocked copy: the embedding, momentum and gains live in the copy's point order (`resident`),
    // so the attractive stage needs no conversion; the accessors convert where values enter and leave.
    bool resident = false;
    int set_resident(bool on);       // converts the three arrays when the state changes
    const int32_t *state_order() const { return resident ? blocked.perm : nullptr; }
    // Opt-in: P truly symmetric, (p + p^T) / 2N, instead of the reference's fixed-width form that drops the mirror
    // image of one-directional edges.  The extra entries of the owned rows live beside P / ids.
    bool symmetric_p = false;
    ExtraEntries extra;
    int *extra_ptr = nullptr;
    int32_t *extra_ids = nullptr;
    float *extra_val = nullptr;
    // embedding and optimiser state
    float2 *Y2 = nullptr;     // [N] AoS, replicated on every rank
    float2 *Fattr = nullptr;  // [N] (owned rows valid)
    float2 *Frep = nullptr;   // [N] (owned rows valid)
    float2 *gains = nullptr;  // [rows]
    float2 *u = nullptr;      // [rows]
    float *soa_tmp = nullptr; // [2N] staging for SoA <-> AoS conversion
    int32_t *order = nullptr, *order_alt = nullptr, *order_keys = nullptr, *box_hist = nullptr;  // spread order (owned rows)
    int order_refresh_early = 1;  // the same while the embedding is still being exaggerated (and 50 iterations after)
    int order_refresh = 8;    // iterations between two counting sorts of the spread order once the embedding has settled (0 = natural order)
    // grid
    float4 *w = nullptr;      // [G][G]
    float4 *ytilde = nullptr; // [G][G]
    void *fft_mem = nullptr;
    FftWorkspace fft;
    IterState *state = nullptr;
    IterState *h_state = nullptr;  // pinned mirror
    InterpConsts ic;

    // schedule
    float eta = 200.0f, exaggeration = 12.0f, pre_momentum = 0.5f, post_momentum = 0.8f;
    int force_magnify_iters = 250;
    int step = 0;
    float last_Z = 0.0f, last_unorm = 0.0f;

    // instrumentation
    bool stage_timers = false;
    bool force_norm = false;   // maintain the update norm even without an early-stop threshold
    float stage_ms[kStages] = {0};
    int64_t stage_launches[kStages] = {0};
    int64_t launches = 0;

    KnnStats knn_stats;    // of the last affinities_from_points
    Comm *comm = nullptr;  // null on a single GPU
    // Sharded runs exchange over peer memory when every rank could map the others (peer.h); Y2 and w then
    // point into the exchange block and alternate between its two buffers, w_sum holds the reduced grid.
    PeerExchange *px = nullptr;
    float2 *Y2_own = nullptr;   // the session's own allocations, used whenever px is null
    float4 *w_own = nullptr;
    float4 *w_sum = nullptr;
    bool grid_two_shot = false;   // peer-memory exchange: the grid sum as slice owners (peer.h), chosen at attach
    int attach_peer_exchange();   // collective, after comm is set

    // Captured iterations (single GPU or peer-memory exchange, no stage timers, no update norm): at small N the loop is bound by the
    // launch and dependency latency of its ten kernels, so whole blocks of iterations are replayed as CUDA
    // graphs.  One graph per phase of the schedule: [0] exaggerated, [1] the 50 iterations after, [2]
    // settled.  A block holds an even number of iterations (the state slots alternate) and an even number
    // of order refreshes (the two order buffers swap at each).
    struct IterGraph {
        cudaGraphExec_t exec = nullptr;
        int iters = 0;
        int64_t launches = 0;
        float eta = 0, exaggeration = 0, momentum = 0;
        int refresh = 0, parity = 0;
    };
    IterGraph graphs[3];
    bool use_graphs = true;   // B200TSNE_GRAPHS=0 turns them off
    int graph_block(int remaining, bool want_norm, int *kind) const;   // iterations the next graph would cover, 0 = none
    int run_graph_block(int kind, int iters);
    void drop_graphs();

    int64_t rows() const { return row_hi - row_lo; }
    int init(int64_t N, int K, int64_t row_lo, int64_t row_hi, int device);
    void destroy();
    int set_embedding_soa(const float *Y_host, bool reset);
    int get_embedding_soa(float *Y_host);
    // optimiser state of the owned rows (momentum = the reference's old_forces, gains), SoA [2][rows] on the host
    int get_optimizer_soa(float *momentum_host, float *gains_host);
    int set_optimizer_soa(const float *momentum_host, const float *gains_host);
    int iterate(int n_iters, float min_gradient_norm, float *elapsed_ms, int *iters_done);
    int one_iteration(bool want_norm);
    int attractive(cudaStream_t st);   // Fattr of the owned rows from the current embedding
    int attractive_launches() const { return blocked.ready ? (resident ? 1 : 3) + (blocked.extra_C > 0) : 1 + (extra.count > 0); }
    int affinities_from_points(const float *X_host, int D, float perplexity, float eps);
};

}  // namespace b200
