#include "peer.h"

#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <string>
#include <vector>

#include "comm.h"

namespace b200 {

namespace {
constexpr size_t kAlign = 256;
size_t round_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// Flag words of a rank: [kind][writer rank] epochs, then [writer rank][2] the writers' min/max encodings, then one
// abort word that a rank whose wait expired sets in every rank's block.
constexpr int kMinMaxOffset = kFlagKinds * kMaxPeers;
constexpr int kAbortOffset = (kFlagKinds + 2) * kMaxPeers;
constexpr int kFlagWords = (kFlagKinds + 2) * kMaxPeers + 16;
constexpr int kErrWords = 8;

struct Layout {
    size_t w[2], ws, y[2], flags, total;
};
Layout block_layout(int64_t npad)
{
    Layout l;
    size_t o = 0;
    for (int b = 0; b < 2; b++) { l.w[b] = o; o += round_up(sizeof(float4) * (size_t)kG * kG); }
    l.ws = o;
    o += round_up(sizeof(float4) * (size_t)kG * kG);
    for (int b = 0; b < 2; b++) { l.y[b] = o; o += round_up(sizeof(float2) * (size_t)npad); }
    l.flags = o;
    o += round_up(sizeof(unsigned int) * kFlagWords);   // epochs [2][ranks], min/max [ranks][2], abort word
    l.total = o;
    return l;
}

__device__ __forceinline__ unsigned long long peer_global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// One warp, one launch per meeting: lane r publishes `value` in this rank's slot of rank r's flag array, then
// waits until rank r's slot of the local array has reached it; gives up after 2 s.  With `state` the ranks also
// exchange the min/max of the rows they have just updated (IterState slot mm_slot) and leave the global
// min/max there, which replaces a pass over the whole embedding.
__global__ void peer_barrier_kernel(PeerTable tab, int kind, unsigned int *epochs, IterState *state, int mm_slot, int *err,
                                    int *err_host, unsigned long long timeout_ns)
{
    const int lane = threadIdx.x;
    // An earlier meeting of this exchange gave up, here or on a peer (which then set the abort word in every
    // rank's block): publish (a live peer may still wait for it) but do not wait again.
    bool dead = *reinterpret_cast<volatile int *>(err) != 0;
    if (!dead && *reinterpret_cast<volatile unsigned int *>(tab.flags[tab.rank] + kAbortOffset) != 0) {
        dead = true;
        if (lane == 0) { atomicExch(err, 1); *reinterpret_cast<volatile int *>(err_host) = 1; }
    }
    // the meeting's number: a device counter per kind that every rank advances alike (a launch parameter
    // would be frozen into a captured graph)
    unsigned int value = 0;
    if (lane == 0) value = ++epochs[kind];
    value = __shfl_sync(0xffffffffu, value, 0);
    unsigned int my_min = 0, my_max = 0;
    if (state) { my_min = state->min_enc[mm_slot]; my_max = state->max_enc[mm_slot]; }
    __threadfence_system();   // everything this stream wrote before (kernel boundary) is ordered before the flag
    if (lane < tab.world) {
        unsigned int *base = tab.flags[lane];
        if (state) {
            base[kMinMaxOffset + 2 * tab.rank] = my_min;
            base[kMinMaxOffset + 2 * tab.rank + 1] = my_max;
        }
        unsigned int *f = base + kind * kMaxPeers + tab.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(value) : "memory");
    }
    unsigned int mn = 0xffffffffu, mx = 0u;
    if (dead) return;
    if (lane < tab.world) {
        const unsigned int *mine = tab.flags[tab.rank];
        const unsigned int *f = mine + kind * kMaxPeers + lane;
        const unsigned long long t0 = peer_global_ns();
        int spins = 0;
        bool ok = true;
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int)(v - value) >= 0) break;
            if ((++spins & 255) == 0) {
                const bool aborted = *reinterpret_cast<const volatile unsigned int *>(mine + kAbortOffset) != 0;
                if (aborted || peer_global_ns() - t0 > timeout_ns) {
                    atomicExch(err, 1);
                    *reinterpret_cast<volatile int *>(err_host) = 1;
                    // tell every rank: whoever still waits, or meets later, gives up too instead of carrying on
                    // with what this rank computes from now on
                    for (int r = 0; r < tab.world; r++)
                        *reinterpret_cast<volatile unsigned int *>(tab.flags[r] + kAbortOffset) = 1u;
                    ok = false;
                    break;
                }
            }
        }
        if (state && ok) {
            // written by rank `lane` before its release store, read after the acquire load that saw it
            mn = *reinterpret_cast<const volatile unsigned int *>(mine + kMinMaxOffset + 2 * lane);
            mx = *reinterpret_cast<const volatile unsigned int *>(mine + kMinMaxOffset + 2 * lane + 1);
        }
    }
    __syncwarp();
    if (state) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (lane == 0) { state->min_enc[mm_slot] = mn; state->max_enc[mm_slot] = mx; }
    }
    __threadfence_system();
}

struct GridSources {
    const float4 *p[kMaxPeers];
    int world;
};

__global__ void __launch_bounds__(256)
peer_grid_reduce_kernel(GridSources src, float4 *__restrict__ w_sum)
{
    const int n = kG * kG;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float4 v[kMaxPeers];
#pragma unroll
        for (int s = 0; s < kMaxPeers; s++)
            if (s < src.world) v[s] = src.p[s][i];   // all loads first: the peer round trips overlap
        float4 acc = v[0];
#pragma unroll
        for (int s = 1; s < kMaxPeers; s++)
            if (s < src.world) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
        w_sum[i] = acc;
    }
}

// Waits until the `kind` flags of all ranks in this rank's flag array have reached `value`; one thread per rank.
// Returns false (and sets the error words and every rank's abort word) when the limit runs out or a peer has aborted.
__device__ __forceinline__ bool wait_flags(const PeerTable &tab, int kind, unsigned int value, int who, int *err, int *err_host,
                                           unsigned long long timeout_ns)
{
    const unsigned int *mine = tab.flags[tab.rank];
    const unsigned int *f = mine + kind * kMaxPeers + who;
    const unsigned long long t0 = peer_global_ns();
    int spins = 0;
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if ((int)(v - value) >= 0) return true;
        if ((++spins & 255) == 0) {
            const bool aborted = *reinterpret_cast<const volatile unsigned int *>(mine + kAbortOffset) != 0;
            if (aborted || peer_global_ns() - t0 > timeout_ns) {
                atomicExch(err, 1);
                *reinterpret_cast<volatile int *>(err_host) = 1;
                for (int r = 0; r < tab.world; r++) *reinterpret_cast<volatile unsigned int *>(tab.flags[r] + kAbortOffset) = 1u;
                return false;
            }
        }
    }
}

// Grid sum and "all spreads done" meeting in one launch (see peer.h).  Every block publishes nothing but waits for
// the spread flags itself (block 0 publishes this rank's); the block that finishes its share of the slice last
// publishes "slice stored", waits for the other ranks' slices and advances the epoch counters.
constexpr int kAllreduceBlocks = 48;
__global__ void __launch_bounds__(256)
peer_grid_allreduce_kernel(PeerTable tab, int buf, unsigned int *epochs, int *block_counter, int *err, int *err_host,
                           unsigned long long timeout_ns)
{
    __shared__ int s_ok, s_last;
    const unsigned int v_spread = epochs[kFlagSpread] + 1, v_slice = epochs[kFlagSlice] + 1;   // alike in all blocks: written only by the last one
    bool dead = *reinterpret_cast<volatile int *>(err) != 0 ||
                *reinterpret_cast<volatile unsigned int *>(tab.flags[tab.rank] + kAbortOffset) != 0;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < tab.world) {
        __threadfence_system();   // this rank's spread (earlier in the stream) before its flag
        unsigned int *f = tab.flags[threadIdx.x] + kFlagSpread * kMaxPeers + tab.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v_spread) : "memory");
    }
    if (!dead && threadIdx.x < tab.world) {
        if (!wait_flags(tab, kFlagSpread, v_spread, threadIdx.x, err, err_host, timeout_ns)) s_ok = 0;
    }
    __syncthreads();
    if (!dead && s_ok) {
        const int n = kG * kG, slice = (n + tab.world - 1) / tab.world;
        const int lo = tab.rank * slice, hi = min(n, lo + slice);
        for (int i = lo + blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += gridDim.x * blockDim.x) {
            float4 v[kMaxPeers];
#pragma unroll
            for (int s = 0; s < kMaxPeers; s++)
                if (s < tab.world) v[s] = tab.w[buf][s][i];   // all loads first: the peer round trips overlap
            float4 acc = v[0];
#pragma unroll
            for (int s = 1; s < kMaxPeers; s++)
                if (s < tab.world) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
#pragma unroll
            for (int s = 0; s < kMaxPeers; s++)
                if (s < tab.world) tab.ws[s][i] = acc;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(block_counter, 1) == (int)gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();   // the other blocks' stores (each fenced before its count) before this rank's flag
    if (threadIdx.x == 0) *block_counter = 0;
    if (threadIdx.x < tab.world) {
        unsigned int *f = tab.flags[threadIdx.x] + kFlagSlice * kMaxPeers + tab.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(v_slice) : "memory");
        dead = dead || *reinterpret_cast<volatile int *>(err) != 0;
        if (!dead) wait_flags(tab, kFlagSlice, v_slice, threadIdx.x, err, err_host, timeout_ns);
    }
    __syncthreads();
    if (threadIdx.x == 0) { epochs[kFlagSpread] = v_spread; epochs[kFlagSlice] = v_slice; }
    __threadfence_system();
}

// sum_i Z_i with Z_i = (1 + |y_i|^2) phi_count(y_i) - 2 (x_i phi_x(y_i) + y_i phi_y(y_i)) + phi_r2(y_i) and every
// phi interpolated from the node potentials with the weights that spread the charges: summing over the
// points first turns it into  sum_nodes  pot.count * (w.count + w.r2) - 2 (pot.x * w.x + pot.y * w.y) + pot.r2 * w.count.
// Node layout (x, y, count, r^2) for charges and potentials alike.
__global__ void __launch_bounds__(256)
grid_z_kernel(const float4 *__restrict__ w_sum, const float4 *__restrict__ ytilde, IterState *state, int slot)
{
    const int n = kG * kG;
    double z = 0.0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float4 q = w_sum[i], p = ytilde[i];
        z += (double)p.z * ((double)q.z + (double)q.w) - 2.0 * ((double)p.x * (double)q.x + (double)p.y * (double)q.y) +
             (double)p.w * (double)q.z;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    __shared__ double sz[8];
    if ((threadIdx.x & 31) == 0) sz[threadIdx.x >> 5] = z;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int k = 0; k < 8; k++) t += sz[k];
        atomicAdd(&state->zsum[slot], t);
    }
}
}  // namespace

void peer_exchange_release(PeerExchange *px, Comm *comm)
{
    if (!px) return;
    // a block whose meeting gave up keeps its error word and diverged epochs: never cache it
    if (comm && !comm->px_idle && !px->failed && !*px->err_host) comm->px_idle = px;   // every rank releases and acquires in the same order
    else peer_exchange_destroy(px, comm, nullptr);
}

int peer_exchange_acquire(PeerExchange **out, Comm *comm, int64_t npad, cudaStream_t st)
{
    *out = nullptr;
    if (!comm || comm->world < 2 || comm->world > kMaxPeers) return 0;
    if (comm->px_idle) {
        PeerExchange *idle = comm->px_idle;
        comm->px_idle = nullptr;
        if (idle->npad == npad) {
            // the grids must start empty; nobody reads them before this rank's next spread signal
            for (int b = 0; b < 2; b++) B200_CUDA(cudaMemsetAsync(idle->w_local(b), 0, sizeof(float4) * kG * kG, st));
            *out = idle;
            return 0;
        }
        peer_exchange_destroy(idle, comm, st);   // another problem size: all ranks get here together
    }
    const int W = comm->world, me = comm->rank;
    const Layout lay = block_layout(npad);
    PeerExchange *px = new PeerExchange();
    px->npad = npad;
    for (int r = 0; r < kMaxPeers; r++) px->mapped[r] = nullptr;
    struct Fail {
        PeerExchange *px;
        bool armed = true;
        ~Fail()
        {
            if (!armed) return;
            if (px->local) cudaFree(px->local);
            if (px->err) cudaFree(px->err);
            if (px->err_host) cudaFreeHost(const_cast<int *>(px->err_host));
            delete px;
        }
    } fail{px};
    if (const char *e = getenv("B200TSNE_PEER_TIMEOUT_MS")) {
        const long long ms = atoll(e);
        if (ms > 0) px->timeout_ns = (unsigned long long)ms * 1000000ull;
    }
    B200_CUDA(cudaMalloc(&px->local, lay.total));
    B200_CUDA(cudaMalloc((void **)&px->err, sizeof(int) * kErrWords));
    {
        int *h = nullptr;
        B200_CUDA(cudaHostAlloc((void **)&h, sizeof(int), cudaHostAllocMapped));
        *h = 0;
        px->err_host = h;
        B200_CUDA(cudaHostGetDevicePointer((void **)&px->err_host_dev, h, 0));
    }
    B200_CUDA(cudaMemsetAsync(px->local, 0, lay.total, st));
    B200_CUDA(cudaMemsetAsync(px->err, 0, sizeof(int) * kErrWords, st));

    // handles of all ranks, gathered through the communicator
    cudaIpcMemHandle_t mine;
    int local_fail = cudaIpcGetMemHandle(&mine, px->local) == cudaSuccess ? 0 : 1;
    if (local_fail) { (void)cudaGetLastError(); memset(&mine, 0, sizeof(mine)); }
    unsigned char *d_handles = nullptr;
    B200_CUDA(cudaMalloc((void **)&d_handles, sizeof(cudaIpcMemHandle_t) * W + sizeof(unsigned int)));
    struct FreeTmp { void *p; ~FreeTmp() { cudaFree(p); } } free_tmp{d_handles};
    B200_CUDA(cudaMemcpyAsync(d_handles + sizeof(cudaIpcMemHandle_t) * me, &mine, sizeof(mine), cudaMemcpyHostToDevice, st));
    B200_TRY(comm->all_gather_inplace(d_handles, sizeof(cudaIpcMemHandle_t), st));
    std::vector<cudaIpcMemHandle_t> all(W);
    B200_CUDA(cudaMemcpyAsync(all.data(), d_handles, sizeof(cudaIpcMemHandle_t) * W, cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    for (int r = 0; r < W && !local_fail; r++) {
        if (r == me) continue;
        if (cudaIpcOpenMemHandle(&px->mapped[r], all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            px->mapped[r] = nullptr;
            local_fail = 1;
        }
    }
    // all ranks take the same decision
    unsigned int *d_flag = reinterpret_cast<unsigned int *>(d_handles + sizeof(cudaIpcMemHandle_t) * W);
    unsigned int h_flag = (unsigned int)local_fail;
    B200_CUDA(cudaMemcpyAsync(d_flag, &h_flag, sizeof(h_flag), cudaMemcpyHostToDevice, st));
    B200_TRY(comm->all_reduce_max_u32(d_flag, 1, st));
    B200_CUDA(cudaMemcpyAsync(&h_flag, d_flag, sizeof(h_flag), cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    if (h_flag) {
        for (int r = 0; r < W; r++)
            if (px->mapped[r]) cudaIpcCloseMemHandle(px->mapped[r]);
        // nobody may free a block that a slower peer still has mapped: meet once more after closing
        B200_TRY(comm->all_reduce_max_u32(d_flag, 1, st));
        B200_CUDA(cudaStreamSynchronize(st));
        return 0;   // `fail` frees the rest; the caller keeps the collectives
    }
    px->tab.world = W;
    px->tab.rank = me;
    for (int r = 0; r < kMaxPeers; r++) {
        char *base = (r == me) ? static_cast<char *>(px->local) : (r < W ? static_cast<char *>(px->mapped[r]) : nullptr);
        for (int b = 0; b < 2; b++) {
            px->tab.w[b][r] = base ? reinterpret_cast<float4 *>(base + lay.w[b]) : nullptr;
            px->tab.y[b][r] = base ? reinterpret_cast<float2 *>(base + lay.y[b]) : nullptr;
        }
        px->tab.ws[r] = base ? reinterpret_cast<float4 *>(base + lay.ws) : nullptr;
        px->tab.flags[r] = base ? reinterpret_cast<unsigned int *>(base + lay.flags) : nullptr;
    }
    fail.armed = false;
    *out = px;
    return 0;
}

void peer_exchange_destroy(PeerExchange *px, Comm *comm, cudaStream_t st)
{
    if (!px) return;
    cudaStreamSynchronize(st);
    for (int r = 0; r < kMaxPeers; r++)
        if (px->mapped[r]) cudaIpcCloseMemHandle(px->mapped[r]);
    // Nobody may free a block that a peer still has mapped: meet the other ranks first.  The wait is
    // bounded (10 s) so that a rank whose peer has died does not hang; it then leaks its block instead.
    bool met = false;
    if (comm) {
        unsigned int *d = reinterpret_cast<unsigned int *>(px->err) + 1;
        if (comm->all_reduce_max_u32(d, 1, st) == 0) {
            for (int i = 0; i < 10000; i++) {
                const cudaError_t q = cudaStreamQuery(st);
                if (q == cudaSuccess) { met = true; break; }
                if (q != cudaErrorNotReady) break;
                struct timespec ts = {0, 1000000};
                nanosleep(&ts, nullptr);
            }
        }
        (void)cudaGetLastError();
    }
    if (met) {
        cudaFree(px->local);
        cudaFree(px->err);
        if (px->err_host) cudaFreeHost(const_cast<int *>(px->err_host));
    }
    delete px;
}

int launch_peer_barrier(PeerExchange *px, int kind, IterState *state, int mm_slot, cudaStream_t st)
{
    peer_barrier_kernel<<<1, 32, 0, st>>>(px->tab, kind, reinterpret_cast<unsigned int *>(px->err) + 2, state, mm_slot, px->err,
                                          px->err_host_dev, px->timeout_ns);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int peer_wait_selftest(int timeout_ms, float *waited_ms, cudaStream_t st)
{
    if (timeout_ms <= 0 || timeout_ms > 2000) { set_error("peer wait self-test: timeout must be 1..2000 ms"); return -1; }
    // "rank 0" and "rank 1" are two local flag arrays; nothing ever writes rank 1's epoch into rank 0's array
    unsigned int *flags = nullptr;
    int *err = nullptr, *err_host = nullptr, *err_host_dev = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    struct Free {
        unsigned int *&f; int *&e; int *&h; cudaEvent_t &a, &b;
        ~Free() { if (f) cudaFree(f); if (e) cudaFree(e); if (h) cudaFreeHost(h); if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); }
    } guard{flags, err, err_host, a, b};
    const size_t words = kFlagWords;
    B200_CUDA(cudaMalloc((void **)&flags, sizeof(unsigned int) * words * 2));
    B200_CUDA(cudaMalloc((void **)&err, sizeof(int) * kErrWords));
    B200_CUDA(cudaHostAlloc((void **)&err_host, sizeof(int), cudaHostAllocMapped));
    *err_host = 0;
    B200_CUDA(cudaHostGetDevicePointer((void **)&err_host_dev, err_host, 0));
    B200_CUDA(cudaMemsetAsync(flags, 0, sizeof(unsigned int) * words * 2, st));
    B200_CUDA(cudaMemsetAsync(err, 0, sizeof(int) * kErrWords, st));
    B200_CUDA(cudaEventCreate(&a));
    B200_CUDA(cudaEventCreate(&b));
    PeerTable tab;
    memset(&tab, 0, sizeof(tab));
    tab.world = 2;
    tab.rank = 0;
    tab.flags[0] = flags;
    tab.flags[1] = flags + words;
    const unsigned long long ns = (unsigned long long)timeout_ms * 1000000ull;
    B200_CUDA(cudaEventRecord(a, st));
    peer_barrier_kernel<<<1, 32, 0, st>>>(tab, kFlagSpread, reinterpret_cast<unsigned int *>(err) + 2, nullptr, 0, err, err_host_dev, ns);
    B200_CUDA(cudaGetLastError());
    // a second meeting on the failed exchange must return at once (it sees the error word on entry)
    peer_barrier_kernel<<<1, 32, 0, st>>>(tab, kFlagUpdate, reinterpret_cast<unsigned int *>(err) + 2, nullptr, 0, err, err_host_dev, ns);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaEventRecord(b, st));
    B200_CUDA(cudaStreamSynchronize(st));
    float ms = 0.0f;
    B200_CUDA(cudaEventElapsedTime(&ms, a, b));
    if (waited_ms) *waited_ms = ms;
    int d_err = 0;
    B200_CUDA(cudaMemcpy(&d_err, err, sizeof(int), cudaMemcpyDeviceToHost));
    if (d_err && *err_host) { set_error("peer exchange: a rank did not arrive within the limit (self-test)"); return -5; }
    return 0;
}

int launch_peer_grid_reduce(PeerExchange *px, int buf, float4 *w_sum, cudaStream_t st)
{
    GridSources src;
    src.world = px->tab.world;
    for (int r = 0; r < kMaxPeers; r++) src.p[r] = px->tab.w[buf][r];
    peer_grid_reduce_kernel<<<148 * 2, 256, 0, st>>>(src, w_sum);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_peer_grid_allreduce(PeerExchange *px, int buf, cudaStream_t st)
{
    unsigned int *epochs = reinterpret_cast<unsigned int *>(px->err) + 2;
    peer_grid_allreduce_kernel<<<kAllreduceBlocks, 256, 0, st>>>(px->tab, buf, epochs, px->err + 5, px->err, px->err_host_dev, px->timeout_ns);
    B200_CUDA(cudaGetLastError());
    return 0;
}

int launch_grid_z(const float4 *w_sum, const float4 *ytilde, IterState *state, int slot, cudaStream_t st)
{
    grid_z_kernel<<<148, 256, 0, st>>>(w_sum, ytilde, state, slot);
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
