// Per-iteration exchanges of a sharded run over peer memory (NVLink loads and stores issued by this
// library's own kernels) instead of collectives.
//
// Every rank allocates one block with the same layout (two partial grids, two copies of the embedding,
// flag words) and maps the blocks of all other ranks through CUDA IPC.  An iteration then needs
//   * one reduction of the partial grids: each rank reads the W partial grids (its own and W - 1 peers')
//     node by node in rank order and keeps the sum, so all ranks hold bit-identical grids;
//   * no exchange for the normalisation: sum_i Z_i is a bilinear form of the summed grid and the
//     potentials, which every rank evaluates locally;
//   * no all-gather: the update kernel stores each new coordinate pair into the embedding copy of every
//     rank.
// Ranks meet twice per iteration ("all spreads done", "all updates done") through flag words: a one-warp
// kernel stores the iteration's epoch into its slot of every rank's flag array (release, system scope) and
// then polls the local array until all slots carry it (acquire).  The polls are bounded (2 s unless
// B200TSNE_PEER_TIMEOUT_MS or the session says otherwise).  On expiry the kernel sets an error word in device
// memory and a second one in mapped host memory: every later meeting sees the first on entry and returns at
// once instead of waiting again, and the host sees the second without synchronising, stops queueing
// iterations and returns status -5.  An exchange that has failed is never reused.  The second meeting also
// carries the min/max of each rank's new rows, so the bounding box of the next grid needs no pass over the
// embedding.
//
// Buffers are double-buffered by iteration parity so that a fast rank never overwrites what a slow rank
// still reads: grid buffer b is written by the spread of iterations with parity b and read by the peers in
// the same iteration; embedding buffer b is read in iterations with parity b and written, by all ranks,
// in the iteration before.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace b200 {

struct Comm;

constexpr int kMaxPeers = 16;
enum PeerFlag { kFlagSpread = 0, kFlagUpdate = 1, kFlagSlice = 2 };
constexpr int kFlagKinds = 3;

// pointer table handed to kernels by value
struct PeerTable {
    int world, rank;
    float4 *w[2][kMaxPeers];     // [buffer][rank] partial grids
    float4 *ws[kMaxPeers];       // [rank] summed grid of that rank (written by the owners of its slices)
    float2 *y[2][kMaxPeers];     // [buffer][rank] embedding copies
    unsigned int *flags[kMaxPeers];   // [rank] flag words: [kind * kMaxPeers + writer rank], then min/max per writer
};

struct PeerExchange {
    PeerTable tab;
    void *local = nullptr;       // this rank's block
    void *mapped[kMaxPeers];     // peers' blocks as mapped here (null for this rank)
    int *err = nullptr;          // device words: [0] a bounded wait expired, [1] scratch of the closing meeting, [2..4] epoch counters per kind, [5] block counter of the grid sum
    volatile int *err_host = nullptr;   // mapped host word the kernel sets on expiry (read by the host without a sync)
    int *err_host_dev = nullptr;        // the same word as the device addresses it
    unsigned long long timeout_ns = 2000000000ull;   // limit of one meeting
    bool failed = false;         // a wait expired: the block is destroyed, not cached, when it is released
    int parity = 0;              // which of the two buffers holds the current embedding / grid (alike on all ranks)
    int64_t npad = 0;

    float4 *w_local(int b) { return tab.w[b][tab.rank]; }
    float4 *ws_local() { return tab.ws[tab.rank]; }
    float2 *y_local(int b) { return tab.y[b][tab.rank]; }
};

// Collective over the communicator: takes over the communicator's idle block if it has the right size, else
// allocates, exchanges the IPC handles and maps the peers.  *out stays null (and 0 is returned) when any rank
// could not map a peer; the caller then keeps using the collectives.
int peer_exchange_acquire(PeerExchange **out, Comm *comm, int64_t npad, cudaStream_t st);
// Hands the block back to the communicator (local; the mappings stay).
void peer_exchange_release(PeerExchange *px, Comm *comm);
// Collective: unmaps the peers, meets the other ranks, then frees the local block.
void peer_exchange_destroy(PeerExchange *px, Comm *comm, cudaStream_t st);

// All ranks meet: publish the next epoch of `kind` everywhere, wait (bounded) until every rank has.  With `state`, the
// ranks' min/max encodings in IterState slot mm_slot are combined across the ranks on the way.
int launch_peer_barrier(PeerExchange *px, int kind, IterState *state, int mm_slot, cudaStream_t st);
// Exercises the bounded wait on one GPU without a peer: a two-rank table whose second rank is local memory
// that nothing writes.  The meeting must give up after timeout_ms, set both error words and leave the device
// usable; returns -5 when it did, 0 when the wait (wrongly) succeeded.
int peer_wait_selftest(int timeout_ms, float *waited_ms, cudaStream_t st);
// w_sum[node] = sum over ranks (in rank order) of their partial grid `buf`
int launch_peer_grid_reduce(PeerExchange *px, int buf, float4 *w_sum, cudaStream_t st);
// The same sum in one launch that also is the "all spreads done" meeting, with 1/world of the traffic per rank:
// every rank sums the nodes of its own slice from all ranks' partial grids and stores the sums into every
// rank's summed grid (ws), then the ranks meet once more ("all slices stored").  The result is in px->ws_local().
int launch_peer_grid_allreduce(PeerExchange *px, int buf, cudaStream_t st);
// state->zsum[slot] += sum over nodes of the bilinear form of charges w_sum and potentials ytilde
int launch_grid_z(const float4 *w_sum, const float4 *ytilde, IterState *state, int slot, cudaStream_t st);

}  // namespace b200
