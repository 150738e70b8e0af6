// Attractive force from a column-blocked copy of P, with the neighbour coordinates read from shared memory.
//
// The row-major kernel (attractive.cu) fetches one neighbour coordinate pair per stored entry with a fully
// divergent 8-byte global load; the L1 serves about one such load per clock and SM, which makes that kernel
// three times slower than the HBM stream of P and ids it has to read.  Here the gathers leave the L1 path:
//
//   * The points are renumbered once (order_points_by_cell: Voronoi cells around sample points, cells chained
//     so that similar cells are adjacent), and the renumbered embedding is cut into tiles of at most 28,672
//     points = 224 KB of float2, which one block keeps in shared memory.
//   * At set-up every stored entry (row i, column j, value p) is moved into the stream of the tile that
//     holds j, ordered by row.  The entries one row has in one tile form a group; a group is padded to a
//     multiple of four entries so that a lane of a warp (four consecutive entries: one 16-byte load of
//     values, one 8-byte load of 16-bit columns) never straddles two rows.  6 bytes per entry instead of 8.
//   * Rows are not stored: bit 15 of a lane's first column says "this lane starts the next row", and a
//     lane whose first column is 0xffff is a marker that carries an absolute row number (needed where a
//     row has no entry in the tile); each chunk of 128 entries knows the row it starts in.  A warp finds
//     its 32 row numbers with one ballot and a population count.
//   * A block owns a contiguous 1/gridDim of the stream, loads the tile(s) it crosses, and its warps walk
//     chunks: gather from shared memory, evaluate p / (1 + d^2) * (y_i - y_j), reduce the lanes of a row
//     with shuffles, and add the partial force with an 8-byte reduction.  The lanes of a group are cut into
//     runs of at most four (never across a chunk) when the stream is built, and bit 15 of a lane's other
//     three columns says "a run starts here", "add the next lane", "add the lane after": two shuffle steps
//     without any control flow, one reduction per run.
//   * With one block of 32 warps per SM the kernel lives on what the set-up precomputes (about 110 instructions per
//     chunk of 128 entries) and on stream loads that run one chunk ahead in registers.
//
// Arithmetic per entry is that of the reference's ComputePijxQijKernelV3 (src/kernels/attr_forces.cu:129-184);
// only the order of the additions differs (and varies from run to run in the last bits, as the sums of
// a row's tiles meet in floating-point reductions).
//
// The blocked copy pays off when a row's neighbours fall into few tiles.  The builder measures that on a
// sample of rows and declines (the caller keeps the row-major kernel) when a group would hold fewer than
// kMinEntriesPerGroup entries on average, or when there are more than 1,024 tiles.
#include <limits.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>

#include "session.h"

namespace b200 {

namespace {

constexpr int kTileMax = 28672;        // points per tile: 224 KB of float2 (227 KB is the block limit)
constexpr int kChunk = 128;            // entries per warp step (4 per lane)
constexpr int kMaxTiles = 1024;        // one bit per tile in a warp-wide bitmap
constexpr int kBlockedThreads = 1024;
constexpr float kMinEntriesPerGroup = 2.5f;
constexpr int kCells = 64;

// ------------------------------------------------------------------------------------------------
// ordering of the points: nearest of kCells sample points, cells chained greedily by distance
// ------------------------------------------------------------------------------------------------
constexpr int kDimChunk = 32;
constexpr int kAssignThreads = 128;

// centre c = row of X picked from the c-th of `cells` equal stretches at a hashed offset (an even spacing
// would alias with a periodic ordering of the data)
__device__ __forceinline__ long long centre_row(int c, int cells, long long N)
{
    const long long stretch = N / cells;
    const unsigned long long h = ((unsigned long long)(c + 1) * 0x9E3779B97F4A7C15ull) >> 20;
    return (long long)c * stretch + (long long)(h % (unsigned long long)stretch);
}

// cell[i] = nearest centre (ties: lower index).  A block takes 128 points; coordinates go through shared
// memory in chunks of 32 dimensions, every thread keeps its 64 partial distances in registers.
__global__ void __launch_bounds__(kAssignThreads)
cell_assign_kernel(const float *__restrict__ X, long long N, int D, int cells, unsigned char *__restrict__ cell)
{
    __shared__ float s_x[kAssignThreads][kDimChunk + 1];
    __shared__ float s_c[kCells][kDimChunk];
    const long long i0 = (long long)blockIdx.x * kAssignThreads;
    float acc[kCells];
#pragma unroll
    for (int c = 0; c < kCells; c++) acc[c] = 0.0f;
    for (int d0 = 0; d0 < D; d0 += kDimChunk) {
        const int nd = min(kDimChunk, D - d0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < kAssignThreads * kDimChunk; idx += kAssignThreads) {
            const int r = idx / kDimChunk, d = idx % kDimChunk;
            const long long i = i0 + r;
            s_x[r][d] = (i < N && d < nd) ? X[i * D + d0 + d] : 0.0f;
        }
        for (int idx = threadIdx.x; idx < kCells * kDimChunk; idx += kAssignThreads) {
            const int c = idx / kDimChunk, d = idx % kDimChunk;
            s_c[c][d] = (c < cells && d < nd) ? X[centre_row(c, cells, N) * D + d0 + d] : 0.0f;
        }
        __syncthreads();
#pragma unroll 4
        for (int d = 0; d < kDimChunk; d++) {
            const float x = s_x[threadIdx.x][d];
#pragma unroll
            for (int c = 0; c < kCells; c++) {
                const float t = x - s_c[c][d];
                acc[c] = fmaf(t, t, acc[c]);
            }
        }
    }
    const long long i = i0 + threadIdx.x;
    if (i >= N) return;
    float best = INFINITY;
    int bc = 0;
#pragma unroll
    for (int c = 0; c < kCells; c++)
        if (c < cells && acc[c] < best) { best = acc[c]; bc = c; }
    cell[i] = (unsigned char)bc;
}

// rank[c] = position of cell c in a greedy nearest-neighbour chain through the centres (start: cell 0), so
// that cells of one cluster end up next to each other.  One block.
__global__ void __launch_bounds__(kCells)
cell_chain_kernel(const float *__restrict__ X, long long N, int D, int cells, int *__restrict__ rank)
{
    __shared__ float s_d[kCells][kCells + 1];
    const int a = threadIdx.x;
    if (a < cells) {
        const float *xa = X + centre_row(a, cells, N) * D;
        for (int b = 0; b < cells; b++) {
            const float *xb = X + centre_row(b, cells, N) * D;
            float acc = 0.0f;
            for (int d = 0; d < D; d++) {
                const float t = xa[d] - xb[d];
                acc = fmaf(t, t, acc);
            }
            s_d[a][b] = acc;
        }
    }
    __syncthreads();
    if (a != 0) return;
    bool used[kCells];
    for (int c = 0; c < kCells; c++) used[c] = false;
    int cur = 0;
    used[0] = true;
    rank[0] = 0;
    for (int k = 1; k < cells; k++) {
        int best = -1;
        float bd = INFINITY;
        for (int c = 0; c < cells; c++)
            if (!used[c] && (best < 0 || s_d[cur][c] < bd)) { bd = s_d[cur][c]; best = c; }
        used[best] = true;
        rank[best] = k;
        cur = best;
    }
}

// Stable counting sort of the points by rank[cell]: a block takes kSortPerBlock consecutive points, each of
// its warps a contiguous share of them.
constexpr int kSortWarps = 8;
constexpr int kSortPerWarp = 512;
constexpr int kSortPerBlock = kSortWarps * kSortPerWarp;

__global__ void __launch_bounds__(kSortWarps * 32)
cell_hist_kernel(const unsigned char *__restrict__ cell, const int *__restrict__ rank, long long N, int *__restrict__ hist /* [kCells][nblocks] */)
{
    __shared__ int s_h[kCells];
    for (int c = threadIdx.x; c < kCells; c += blockDim.x) s_h[c] = 0;
    __syncthreads();
    const long long lo = (long long)blockIdx.x * kSortPerBlock;
    for (int k = threadIdx.x; k < kSortPerBlock; k += blockDim.x)
        if (lo + k < N) atomicAdd(&s_h[rank[cell[lo + k]]], 1);
    __syncthreads();
    for (int c = threadIdx.x; c < kCells; c += blockDim.x) hist[(size_t)c * gridDim.x + blockIdx.x] = s_h[c];
}

// exclusive scan of n ints in place; one block (the tables it serves are small)
__global__ void __launch_bounds__(1024)
scan_inplace_kernel(int *__restrict__ hist, long long n)
{
    __shared__ int s_w[32];
    __shared__ int s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (long long base = 0; base < n; base += 1024) {
        const long long i = base + threadIdx.x;
        const int v = (i < n) ? hist[i] : 0;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, d);
            if ((threadIdx.x & 31) >= d) incl += t;
        }
        if ((threadIdx.x & 31) == 31) s_w[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            int w = s_w[threadIdx.x];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, d);
                if (threadIdx.x >= d) w += t;
            }
            s_w[threadIdx.x] = w;
        }
        __syncthreads();
        const int carry = s_carry;
        const int wbase = (threadIdx.x >> 5) ? s_w[(threadIdx.x >> 5) - 1] : 0;
        if (i < n) hist[i] = carry + wbase + incl - v;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = carry + wbase + incl;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSortWarps * 32)
cell_scatter_kernel(const unsigned char *__restrict__ cell, const int *__restrict__ rank, long long N, const int *__restrict__ offs,
                    int32_t *__restrict__ perm)
{
    __shared__ int s_cnt[kSortWarps][kCells], s_base[kSortWarps][kCells];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int c = lane; c < kCells; c += 32) s_cnt[w][c] = 0;
    __syncwarp();
    const long long lo = (long long)blockIdx.x * kSortPerBlock + (long long)w * kSortPerWarp;
    for (int k = lane; k < kSortPerWarp; k += 32)
        if (lo + k < N) atomicAdd(&s_cnt[w][rank[cell[lo + k]]], 1);
    __syncthreads();
    // first position of (block, warp, cell) = block offset + counts of the warps before this one
    for (int c = lane; c < kCells; c += 32) {
        int base = offs[(size_t)c * gridDim.x + blockIdx.x];
        for (int v = 0; v < w; v++) base += s_cnt[v][c];
        s_base[w][c] = base;
    }
    __syncwarp();
    for (int k0 = 0; k0 < kSortPerWarp; k0 += 32) {
        const long long i = lo + k0 + lane;
        const bool in = i < N;
        const int r = in ? rank[cell[i]] : -1 - lane;   // lanes out of range never match
        const unsigned m = __match_any_sync(0xffffffffu, r);
        const int before = __popc(m & ((1u << lane) - 1u));
        int base = 0;
        if (in) base = s_base[w][r];
        __syncwarp();
        if (in) {
            perm[base + before] = (int32_t)i;
            if (before == __popc(m) - 1) s_base[w][r] = base + __popc(m);
        }
        __syncwarp();
    }
}

}  // namespace

// perm[q] = the point at position q of the cell order.  X: [N][D] on the device.
int order_points_by_cell(const float *X, int64_t N, int D, int32_t *perm, cudaStream_t st)
{
    if (N <= 0 || D <= 0) { set_error("order_points_by_cell: invalid sizes"); return -1; }
    const int cells = (int)std::min<int64_t>(kCells, N);
    const unsigned nblocks = (unsigned)((N + kSortPerBlock - 1) / kSortPerBlock);
    DeviceArena tmp;
    tmp.serve(st);
    unsigned char *cell = nullptr;
    int *rank = nullptr, *hist = nullptr;
    B200_TRY(tmp.alloc((void **)&cell, (size_t)N));
    B200_TRY(tmp.alloc((void **)&rank, sizeof(int) * kCells));
    B200_TRY(tmp.alloc((void **)&hist, sizeof(int) * (size_t)kCells * nblocks));
    B200_CUDA(cudaMemsetAsync(rank, 0, sizeof(int) * kCells, st));
    cell_assign_kernel<<<(unsigned)((N + kAssignThreads - 1) / kAssignThreads), kAssignThreads, 0, st>>>(X, N, D, cells, cell);
    cell_chain_kernel<<<1, kCells, 0, st>>>(X, N, D, cells, rank);
    cell_hist_kernel<<<nblocks, kSortWarps * 32, 0, st>>>(cell, rank, N, hist);
    scan_inplace_kernel<<<1, 1024, 0, st>>>(hist, (long long)kCells * nblocks);
    cell_scatter_kernel<<<nblocks, kSortWarps * 32, 0, st>>>(cell, rank, N, hist, perm);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaStreamSynchronize(st));
    return 0;
}


// ------------------------------------------------------------------------------------------------
// the blocked stream
// ------------------------------------------------------------------------------------------------
namespace {

struct BlockedStream {   // what the kernels need, by value
    const float *ev;          // [E] values; a marker lane's first value holds the row number's bits
    const uint16_t *ec;       // [E] column inside the tile | 0x8000 on a lane's first entry = "next row starts here"; 0xffff = marker
    const int *chunk_row0;    // [C] row in force before the chunk's first lane
    const int *tile_chunk0;   // [ntiles + 1] first chunk of every tile
    int ntiles, T, C;
};

// inverse of a permutation
__global__ void invert_perm_kernel(const int32_t *__restrict__ perm, long long N, int32_t *__restrict__ pos)
{
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q < N) pos[perm ? perm[q] : q] = (int32_t)q;
}
__global__ void iota_kernel(int32_t *__restrict__ a, long long n)
{
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q < n) a[q] = (int32_t)q;
}

// own rows in permuted order (multi-GPU: a rank owns rows [row_lo, row_hi) of the original numbering):
// stable compaction of perm in three launches
constexpr int kCompactPerBlock = 4096;
__global__ void __launch_bounds__(1024)
own_count_kernel(const int32_t *__restrict__ perm, long long N, long long row_lo, long long row_hi, int *__restrict__ bcount)
{
    const long long lo = (long long)blockIdx.x * kCompactPerBlock;
    int c = 0;
    for (int k = threadIdx.x; k < kCompactPerBlock; k += 1024) {
        const long long q = lo + k;
        if (q < N) { const int i = perm[q]; c += (i >= row_lo && i < row_hi); }
    }
    c = __reduce_add_sync(0xffffffffu, c);
    __shared__ int s[32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x < 32) {
        const int t = __reduce_add_sync(0xffffffffu, s[threadIdx.x]);
        if (threadIdx.x == 0) bcount[blockIdx.x] = t;
    }
}
// one warp per block walks the block's 4096 positions in order (small work; keeps the order without a block scan)
__global__ void __launch_bounds__(32)
own_scatter_kernel(const int32_t *__restrict__ perm, long long N, long long row_lo, long long row_hi, const int *__restrict__ boff,
                   int32_t *__restrict__ own_perm, int32_t *__restrict__ own_pos)
{
    const int lane = threadIdx.x;
    const long long lo = (long long)blockIdx.x * kCompactPerBlock;
    int base = boff[blockIdx.x];
    for (int k0 = 0; k0 < kCompactPerBlock; k0 += 32) {
        const long long q = lo + k0 + lane;
        const int i = (q < N) ? perm[q] : -1;
        const bool own = i >= row_lo && i < row_hi;
        const unsigned m = __ballot_sync(0xffffffffu, own);
        if (own) {
            const int lr = base + __popc(m & ((1u << lane) - 1u));
            own_perm[lr] = i;
            own_pos[i - row_lo] = lr;
        }
        base += __popc(m);
    }
}

// ---- walking the rows of a range: per-warp scratch ----
constexpr int kWalkWarps = 1;
constexpr int kMaxK = 1024;
// MAXT tiles and MAXS slots per segment: the common case (up to 64 tiles, rows of up to 128 slots) has a scratch of
// 3 KB, so that a block's one warp shares its SM with 31 others; the general one (1,024 of each) takes 38 KB and
// five warps fill an SM (the walk is a chain of dependent round trips: 14 ms against 5 at N = 10^6, K = 90).
template <int MAXT, int MAXS>
struct WalkScratchT {
    long long run[MAXT];           // count pass: entries this range adds to the tile; fill pass: next free entry of the tile
    int rowcnt[MAXT];              // entries of the current row per tile
    unsigned slot[MAXS];           // per slot of the current row, see kSlot*; 0xffffffff = unused slot
    unsigned short col[MAXS];      // per slot: column inside the tile
    unsigned bitmap[2][32];        // tiles touched by the previous / the current row
    // fill pass, per tile: bank pairs already taken in the half-warp window (16 lanes) that holds the tile's cursor
    // and in the window after it: bit 16 k + b = "the k-th gather of that window reads bank pair b"
    unsigned long long win[MAXT][2];
    int win_id[MAXT];              // absolute lane / 16 of win[.][0]
};
using WalkScratchSmall = WalkScratchT<64, 128>;
using WalkScratch = WalkScratchT<kMaxTiles, kMaxK>;
// slot word: bits 16..25 tile, bit 30 first slot of its (row, tile) group; low 16 bits: rank inside the group in
// slot order, later the cell (4 x lane of the group + entry) the slot's entry is written to
constexpr unsigned kSlotUnused = 0xffffffffu, kSlotLeader = 1u << 30;
__device__ __forceinline__ int slot_tile(unsigned info) { return (info >> 16) & 0x3ffu; }

// The rows come from one of two sources.  Fixed width (seg_row null): segment g is the row at local permuted
// position g, its K slots at val / ids + (own_perm[g] - row_lo) * K.  Variable width: segment g is seg_len[g] <= kMaxK
// slots at val / ids + seg_base[g] of row seg_row[g] (local permuted position; ascending; a long row is several
// consecutive segments, rows without slots have none).
struct WalkArgs {
    const float *val;
    const int32_t *ids;
    const int32_t *seg_row;
    const long long *seg_base;
    const int *seg_len;
    const int32_t *pos;            // [N] point -> permuted position
    const int32_t *own_perm;       // [rows] local permuted position -> point
    long long N, row_lo, n_seg;
    int K, T, ntiles, range_rows;  // range_rows: segments per range
    long long n_ranges;
    int greedy;                    // place a group's entries by bank pair (place_group) instead of in slot order
    int max_len;                   // the longest segment (K when the width is fixed)
};
struct Segment {
    long long lr, base;
    int len;
    bool force;                    // every group of the segment needs a marker: its row is not the previous segment's row + 1
};
__device__ __forceinline__ Segment get_segment(const WalkArgs &a, long long g)
{
    Segment sg;
    if (!a.seg_row) {
        sg.lr = g;
        sg.base = ((long long)a.own_perm[g] - a.row_lo) * a.K;
        sg.len = a.K;
        sg.force = false;
    } else {
        sg.lr = a.seg_row[g];
        sg.base = a.seg_base[g];
        sg.len = a.seg_len[g];
        sg.force = g == 0 || a.seg_row[g - 1] != sg.lr - 1;
    }
    return sg;
}

// slot table, per-tile counts and the tile bitmap of one row
template <class S>
__device__ __forceinline__ void analyse_row(const WalkArgs &a, const Segment &sg, S &s, unsigned *bitmap, int lane)
{
    for (int k0 = 0; k0 < sg.len; k0 += 32) {
        const int sl = k0 + lane;
        const int j = (sl < sg.len) ? a.ids[sg.base + sl] : -1;
        const bool valid = j >= 0 && (long long)j < a.N;
        int t = -1 - lane, c = 0;
        if (valid) {
            const int q = a.pos[j];
            t = q / a.T;
            c = q - t * a.T;
        }
        const unsigned m = __match_any_sync(0xffffffffu, t);
        const int before = __popc(m & ((1u << lane) - 1u));
        const int base = valid ? s.rowcnt[t] : 0;
        __syncwarp();
        if (valid) {
            if (before == __popc(m) - 1) s.rowcnt[t] = base + __popc(m);
            if (before == 0 && base == 0) atomicOr(&bitmap[t >> 5], 1u << (t & 31));
        }
        __syncwarp();
        if (sl < sg.len) {
            s.slot[sl] = valid ? (((unsigned)t << 16) | (unsigned)(base + before) | ((base + before) == 0 ? kSlotLeader : 0u)) : kSlotUnused;
            s.col[sl] = (unsigned short)c;
        }
    }
    __syncwarp();
}

// Geometry of a group in the stream.  Its lanes (a marker lane first, if any, then ceil(cnt / 4) lanes of entries)
// are cut into runs of at most four lanes that never cross a chunk; the kernel reduces a run with two shuffle
// steps and its first lane adds the sum to the row's force.
struct GroupGeom {
    long long lane0;     // absolute lane (= entry offset / 4) of the group's first lane
    int n_lanes;
    __device__ bool start(int i) const { return (i & 3) == 0 || ((lane0 + i) & 31) == 0; }
    __device__ bool take1(int i) const { return i + 1 < n_lanes && !start(i + 1); }
    __device__ bool take2(int i) const { return i + 2 < n_lanes && !start(i + 1) && !start(i + 2); }
    // bit 15 of entry k of lane i (k = 0 is the row bit, set by the caller)
    __device__ unsigned flag(int i, int k) const { return ((k == 1 && start(i)) || (k == 2 && take1(i)) || (k == 3 && take2(i))) ? 0x8000u : 0u; }
};

// Where the entries of a group go when the caller asks for placement by bank pair (off by default, see
// blocked_attractive_build).  A group's entries may stand in any order.  The kernel's k-th gather of a warp
// reads the k-th entry of all 32 lanes, 16 lanes per shared-memory pass, and a pass costs as many cycles as its
// most loaded pair of banks (a float2 at column c lies in bank pair c mod 16): random columns cost 5.6 cycles
// per gather where 2 would do.  The stream of a tile is written front to back by one warp, so the builder keeps,
// per tile, the bank pairs already taken in each of the four passes of the current half-warp window, and gives
// every entry the first free cell of its group whose pass does not have the entry's bank pair yet (else the
// first free cell).  Groups of more than 32 entries keep the slot order.  Returns the cells taken (bit per cell).
template <class S>
__device__ __forceinline__ unsigned place_group(S &s, int K, int t, int cnt, long long first_lane)
{
    const int n_lanes = (cnt + 3) >> 2;
    const int w0 = (int)(first_lane >> 4);
    if (s.win_id[t] != w0) {       // the cursor moved on: the window after the old one becomes the current one, or both start empty
        s.win[t][0] = (s.win_id[t] + 1 == w0) ? s.win[t][1] : 0ull;
        s.win[t][1] = 0ull;
        s.win_id[t] = w0;
    }
    unsigned long long m0 = s.win[t][0], m1 = s.win[t][1];
    unsigned used = 0u;
    for (int sl = 0; sl < K; sl++) {
        const unsigned info = s.slot[sl];
        if (info == kSlotUnused || slot_tile(info) != t) continue;
        const int b = s.col[sl] & 15;
        int cell = -1;
        for (int l = 0; l < n_lanes && cell < 0; l++) {
            const unsigned long long m = (((first_lane + l) >> 4) == w0) ? m0 : m1;
            for (int k = 0; k < 4; k++) {
                const int c = 4 * l + k;
                if (!((used >> c) & 1u) && !((m >> (16 * k + b)) & 1ull)) { cell = c; break; }
            }
        }
        if (cell < 0) cell = __ffs(~used) - 1;
        used |= 1u << cell;
        const unsigned long long bit = 1ull << (16 * (cell & 3) + b);
        if (((first_lane + (cell >> 2)) >> 4) == w0) m0 |= bit; else m1 |= bit;
        s.slot[sl] = (info & 0xffff0000u) | (unsigned)cell;
    }
    s.win[t][0] = m0;
    s.win[t][1] = m1;
    return used;
}

// FILL = false: add the row's groups to run[] (sizes) and count them.  FILL = true: write the row's entries.
template <bool FILL, class S>
__device__ __forceinline__ void emit_row(const WalkArgs &a, const Segment &sg, S &s, const unsigned *prev, int lane,
                                         float *__restrict__ ev, uint16_t *__restrict__ ec, int *__restrict__ chunk_row0,
                                         unsigned long long &n_groups)
{
    const long long lr = sg.lr;
    const int K = sg.len;
    if (FILL) {
        // every group's first slot places the group's entries and writes what no entry owns
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int sl = k0 + lane;
            const unsigned info = (sl < K) ? s.slot[sl] : kSlotUnused;
            if (info == kSlotUnused || !(info & kSlotLeader)) continue;
            const int t = slot_tile(info);
            const int cnt = s.rowcnt[t];
            const int marker = (!sg.force && ((prev[t >> 5] >> (t & 31)) & 1u)) ? 0 : 1;
            const long long gs = s.run[t];
            GroupGeom g;
            g.lane0 = gs >> 2;
            g.n_lanes = marker + ((cnt + 3) >> 2);
            unsigned used = (cnt >= 32) ? 0xffffffffu : ((1u << cnt) - 1u);      // slot order: the first cnt cells
            if (cnt <= 32 && a.greedy) used = place_group(s, K, t, cnt, g.lane0 + marker);
            if (marker) {
                ev[gs] = __int_as_float((int)lr);
                ec[gs] = 0xffffu;
                for (int kk = 1; kk < 4; kk++) ec[gs + kk] = (uint16_t)g.flag(0, kk);
                atomicOr(reinterpret_cast<unsigned *>(chunk_row0) + gs / kChunk, 0x80000000u);   // "this chunk holds a marker"
            }
            // cells without an entry (value 0, column 0) still carry their lane's flags
            const int n_cells = 4 * ((cnt + 3) >> 2);
            const bool placed = cnt <= 32 && a.greedy;
            for (int c = (placed ? 0 : cnt); c < n_cells; c++) {
                if (placed && ((used >> c) & 1u)) continue;
                const int i = marker + (c >> 2), k = c & 3;
                ec[gs + 4 * marker + c] = (uint16_t)(k == 0 ? ((c == 0 && !marker) ? 0x8000u : 0u) : g.flag(i, k));
            }
            const int size = 4 * g.n_lanes;
            for (long long mm = (gs + kChunk - 1) / kChunk * kChunk; mm < gs + size; mm += kChunk)
                atomicOr(reinterpret_cast<unsigned *>(chunk_row0) + mm / kChunk, (unsigned)((mm == gs && !marker) ? (int)lr - 1 : (int)lr));
        }
        __syncwarp();
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int sl = k0 + lane;
            const unsigned info = (sl < K) ? s.slot[sl] : kSlotUnused;
            if (info == kSlotUnused) continue;
            const int t = slot_tile(info), x = info & 0xffffu;
            const int cnt = s.rowcnt[t];
            const int marker = (!sg.force && ((prev[t >> 5] >> (t & 31)) & 1u)) ? 0 : 1;
            const long long gs = s.run[t];
            GroupGeom g;
            g.lane0 = gs >> 2;
            g.n_lanes = marker + ((cnt + 3) >> 2);
            const int i = marker + (x >> 2), k = x & 3;
            const long long off = gs + 4 * marker + x;
            ev[off] = a.val[sg.base + sl];
            ec[off] = (uint16_t)(s.col[sl] | (k == 0 ? ((x == 0 && !marker) ? 0x8000u : 0u) : g.flag(i, k)));
        }
        __syncwarp();
    }
    // group leaders close the row: advance the tile's cursor, clear the row's count
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int sl = k0 + lane;
        const unsigned info = (sl < K) ? s.slot[sl] : kSlotUnused;
        if (info == kSlotUnused || !(info & kSlotLeader)) continue;
        const int t = slot_tile(info);
        const int marker = (!sg.force && ((prev[t >> 5] >> (t & 31)) & 1u)) ? 0 : 1;
        s.run[t] += ((s.rowcnt[t] + 3) & ~3) + 4 * marker;
        s.rowcnt[t] = 0;
        n_groups++;
    }
    __syncwarp();
}

// A warp walks the rows of one range in order.  Count pass: range_size[t][range] = entries (padding and
// markers included) the range puts into tile t.  Fill pass: starts from tile_start[t] + range_off[t][range].
template <bool FILL, class S>
__global__ void __launch_bounds__(kWalkWarps * 32)
walk_kernel(WalkArgs a, unsigned *__restrict__ range_size, const unsigned *__restrict__ range_off, const long long *__restrict__ tile_start,
            float *__restrict__ ev, uint16_t *__restrict__ ec, int *__restrict__ chunk_row0, unsigned long long *__restrict__ totals)
{
    __shared__ S scratch[kWalkWarps];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    S &s = scratch[w];
    const long long range = (long long)blockIdx.x * kWalkWarps + w;
    if (range >= a.n_ranges) return;
    for (int t = lane; t < a.ntiles; t += 32) {
        s.rowcnt[t] = 0;
        s.run[t] = FILL ? tile_start[t] + (long long)range_off[(size_t)t * a.n_ranges + range] : 0;
        s.win_id[t] = -2;
        s.win[t][0] = s.win[t][1] = 0ull;
    }
    s.bitmap[0][lane] = 0u;
    s.bitmap[1][lane] = 0u;
    __syncwarp();
    const long long g0 = range * a.range_rows, g1 = min(a.n_seg, g0 + (long long)a.range_rows);
    unsigned long long n_groups = 0;
    int cur = 0;
    if (g0 > 0) {   // the tiles of the segment before the range decide the first segment's markers
        const Segment before = get_segment(a, g0 - 1);
        analyse_row(a, before, s, s.bitmap[0], lane);
        for (int k0 = 0; k0 < before.len; k0 += 32) {
            const int sl = k0 + lane;
            const unsigned info = (sl < before.len) ? s.slot[sl] : kSlotUnused;
            if (info != kSlotUnused && (info & kSlotLeader)) s.rowcnt[slot_tile(info)] = 0;
        }
        __syncwarp();
        cur = 1;
    }
    for (long long g = g0; g < g1; g++) {
        const Segment sg = get_segment(a, g);
        s.bitmap[cur][lane] = 0u;
        __syncwarp();
        analyse_row(a, sg, s, s.bitmap[cur], lane);
        emit_row<FILL, S>(a, sg, s, s.bitmap[cur ^ 1], lane, ev, ec, chunk_row0, n_groups);
        cur ^= 1;
    }
    if (!FILL) {
        for (int t = lane; t < a.ntiles; t += 32) range_size[(size_t)t * a.n_ranges + range] = (unsigned)s.run[t];
        n_groups = __reduce_add_sync(0xffffffffu, (unsigned)n_groups);
        if (lane == 0) atomicAdd(&totals[0], n_groups);
    }
}

// distinct tiles and valid entries of a sample of rows: totals[1] += groups, totals[2] += entries
template <class S>
__global__ void __launch_bounds__(kWalkWarps * 32)
sample_kernel(WalkArgs a, long long n_samples, unsigned long long *__restrict__ totals)
{
    __shared__ S scratch[kWalkWarps];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    S &s = scratch[w];
    const long long k = (long long)blockIdx.x * kWalkWarps + w;
    if (k >= n_samples) return;
    for (int t = lane; t < a.ntiles; t += 32) s.rowcnt[t] = 0;
    s.bitmap[0][lane] = 0u;
    __syncwarp();
    const Segment sg = get_segment(a, k * (a.n_seg / n_samples));
    analyse_row(a, sg, s, s.bitmap[0], lane);
    unsigned groups = 0, entries = 0;
    for (int k0 = 0; k0 < sg.len; k0 += 32) {
        const int sl = k0 + lane;
        const unsigned info = (sl < sg.len) ? s.slot[sl] : kSlotUnused;
        if (info == kSlotUnused) continue;
        entries++;
        groups += (info & kSlotLeader) != 0;
    }
    groups = __reduce_add_sync(0xffffffffu, groups);
    entries = __reduce_add_sync(0xffffffffu, entries);
    if (lane == 0) { atomicAdd(&totals[1], (unsigned long long)groups); atomicAdd(&totals[2], (unsigned long long)entries); }
}

// per tile: exclusive scan of the ranges' sizes (in place) and the tile's total; one block per tile
__global__ void __launch_bounds__(1024)
tile_scan_kernel(unsigned *__restrict__ range_size, long long n_ranges, unsigned long long *__restrict__ tile_total)
{
    __shared__ unsigned long long s_w[32];
    __shared__ unsigned long long s_carry;
    unsigned *row = range_size + (size_t)blockIdx.x * n_ranges;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (long long base = 0; base < n_ranges; base += 1024) {
        const long long i = base + threadIdx.x;
        const unsigned long long v = (i < n_ranges) ? row[i] : 0;
        unsigned long long incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, d);
            if ((threadIdx.x & 31) >= d) incl += t;
        }
        if ((threadIdx.x & 31) == 31) s_w[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            unsigned long long wv = s_w[threadIdx.x];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const unsigned long long t = __shfl_up_sync(0xffffffffu, wv, d);
                if (threadIdx.x >= d) wv += t;
            }
            s_w[threadIdx.x] = wv;
        }
        __syncthreads();
        const unsigned long long carry = s_carry;
        const unsigned long long wbase = (threadIdx.x >> 5) ? s_w[(threadIdx.x >> 5) - 1] : 0;
        if (i < n_ranges) row[i] = (unsigned)(carry + wbase + incl - v);
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = carry + wbase + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) tile_total[blockIdx.x] = s_carry;
}

// tile t's entries start at a multiple of the chunk size; totals[3] = all entries, totals[4] = 1 if a tile overflows 32 bits
__global__ void tile_layout_kernel(const unsigned long long *__restrict__ tile_total, int ntiles, long long *__restrict__ tile_start,
                                   int *__restrict__ tile_chunk0, unsigned long long *__restrict__ totals)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    long long e = 0;
    unsigned long long bad = 0;
    for (int t = 0; t < ntiles; t++) {
        tile_start[t] = e;
        tile_chunk0[t] = (int)(e / kChunk);
        if (tile_total[t] >= 0xffffffffull) bad = 1;
        e += (long long)((tile_total[t] + kChunk - 1) / kChunk * kChunk);
    }
    tile_start[ntiles] = e;
    tile_chunk0[ntiles] = (int)(e / kChunk);
    totals[3] = (unsigned long long)e;
    totals[4] = bad;
}

// ---- per iteration ----
// Yp[q] = Y[perm[q]] for all points; Yown[lr] = Y[own_perm[lr]] and Fp[lr] = 0 for the owned rows
__global__ void __launch_bounds__(256)
permute_kernel(const float2 *__restrict__ Y2, const int32_t *__restrict__ perm, long long N, float2 *__restrict__ Yp,
               const int32_t *__restrict__ own_perm, long long rows, float2 *__restrict__ Yown, float2 *__restrict__ Fp)
{
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q < N) Yp[q] = Y2[perm[q]];
    if (q < rows) {
        if (Yown != Yp) Yown[q] = Y2[own_perm[q]];
        Fp[q] = make_float2(0.0f, 0.0f);
    }
}
__global__ void __launch_bounds__(256)
unpermute_kernel(const float2 *__restrict__ Fp, const int32_t *__restrict__ own_pos, long long row_lo, long long rows, float2 *__restrict__ F2)
{
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) F2[row_lo + r] = Fp[own_pos[r]];
}

// A chunk in a warp's registers: the stream loads are issued one round before the chunk is processed; then the
// lane's row is found (it takes the place of row0), the row's own coordinate fetched, and the forces evaluated.
// The kernel is bound by the L1/shared-memory data path (about two thirds busy: per chunk 4 gathers of 5 to 6
// bank-conflict cycles each, 7 cycles of stream loads, the coordinate load, 4 shuffles, the reduction) and by
// latency at one block of 32 warps per SM; more loads in flight make it slower, not faster.  Measured on B200
// at N = 10^6, K = 90 (attractive stage of the iteration, 148 blocks): as below 190 us; without
// L1::no_allocate on the stream 191 us; two register sets in turn instead of the copy 212 us; stream loads two
// rounds ahead 218 us; rows and own coordinates a round ahead as well (three sets) 247 us; the row coordinates
// of a chunk fetched a round ahead as one coalesced load and handed to the lanes by shuffle 244 us; an L2
// prefetch six rounds ahead changes nothing; 768 threads with 79 registers 241 us.
struct ChunkSet {
    float4 p;      // values of the lane's four entries
    uint2 c;       // their 16-bit words: column (15 bits) | flag (bit 15): entry 0 "next row", 1 "run starts", 2, 3 "add lane + 1 / + 2"
    int r;         // the chunk's row0 word (sign bit: the chunk holds a marker lane), then this lane's row
};
// The stream is read once: its loads do not take lines of the (small, beside 224 KB of shared memory) L1.
__device__ __forceinline__ void stage_load(ChunkSet &s, const BlockedStream &b, int cc, int lane)
{
    const float4 *pv = reinterpret_cast<const float4 *>(b.ev) + (size_t)cc * 32 + lane;
    const uint2 *pc = reinterpret_cast<const uint2 *>(b.ec) + (size_t)cc * 32 + lane;
    asm volatile("ld.global.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(s.p.x), "=f"(s.p.y), "=f"(s.p.z), "=f"(s.p.w) : "l"(pv));
    asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(s.c.x), "=r"(s.c.y) : "l"(pc));
    s.r = __ldg(b.chunk_row0 + cc);
}

__device__ __forceinline__ void add_entry(float2 yi, float2 yj, float p, float &ox, float &oy)
{
    const float dx = yi.x - yj.x, dy = yi.y - yj.y;
    const float pq = __fdividef(p, fmaf(dy, dy, fmaf(dx, dx, 1.0f)));
    ox = fmaf(pq, dx, ox);
    oy = fmaf(pq, dy, oy);
}
__device__ __forceinline__ float2 tile_at(const float2 *tile, unsigned byte_offset)
{
    return *reinterpret_cast<const float2 *>(reinterpret_cast<const char *>(tile) + byte_offset);
}

__device__ __forceinline__ void process_chunk(ChunkSet &w, const float2 *__restrict__ tile, const float2 *__restrict__ Yown,
                                              float2 *__restrict__ Fp, int lane)
{
    const bool head = w.c.x & 0x8000u;
    const unsigned hm = __ballot_sync(0xffffffffu, head);
    if (w.r >= 0) {
        w.r += __popc(hm & (0xffffffffu >> (31 - lane)));   // heads up to and including this lane
    } else {
        // a marker lane (first word 0xffff) sets the row to the number its first value holds; rows are then a
        // scan over (row set by a marker, heads since)
        const bool marker = (w.c.x & 0xffffu) == 0xffffu;
        int s = marker ? __float_as_int(w.p.x) : INT_MIN, n = (head && !marker) ? 1 : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int sa = __shfl_up_sync(0xffffffffu, s, d), na = __shfl_up_sync(0xffffffffu, n, d);
            if (lane >= d && s == INT_MIN) { s = sa; n += na; }
        }
        w.r = (s == INT_MIN ? (w.r & 0x7fffffff) : s) + n;
        if (marker) { w.p.x = 0.0f; w.c.x &= 0xffff0000u; }   // from here on an entry of value 0 at column 0
    }
    const float2 yi = __ldg(Yown + w.r);
    // byte offsets of the four columns in the tile
    const float2 yj0 = tile_at(tile, (w.c.x << 3) & 0x3fff8u), yj1 = tile_at(tile, (w.c.x >> 13) & 0x3fff8u);
    const float2 yj2 = tile_at(tile, (w.c.y << 3) & 0x3fff8u), yj3 = tile_at(tile, (w.c.y >> 13) & 0x3fff8u);
    float ox = 0.0f, oy = 0.0f;
    add_entry(yi, yj0, w.p.x, ox, oy);
    add_entry(yi, yj1, w.p.y, ox, oy);
    add_entry(yi, yj2, w.p.z, ox, oy);
    add_entry(yi, yj3, w.p.w, ox, oy);
    // runs of at most four lanes: two steps, the flags say which lanes add
    {
        const float tx = __shfl_down_sync(0xffffffffu, ox, 1), ty = __shfl_down_sync(0xffffffffu, oy, 1);
        if (w.c.y & 0x8000u) { ox += tx; oy += ty; }
    }
    {
        const float tx = __shfl_down_sync(0xffffffffu, ox, 2), ty = __shfl_down_sync(0xffffffffu, oy, 2);
        if (w.c.y & 0x80000000u) { ox += tx; oy += ty; }
    }
    if (w.c.x & 0x80000000u) atomicAdd(Fp + w.r, make_float2(ox, oy));
}

__global__ void __launch_bounds__(kBlockedThreads, 1)
attractive_blocked_kernel(BlockedStream b, const float2 *__restrict__ Yp, const float2 *__restrict__ Yown, long long N,
                          float2 *__restrict__ Fp)
{
    extern __shared__ float2 tile[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int nwarps = kBlockedThreads / 32;
    const int c_lo = (int)((long long)b.C * blockIdx.x / gridDim.x), c_hi = (int)((long long)b.C * (blockIdx.x + 1) / gridDim.x);
    if (c_lo >= c_hi) return;
    int t = 0;
    {
        int lo = 0, hi = b.ntiles;
        while (hi - lo > 1) {
            const int m = (lo + hi) >> 1;
            if (b.tile_chunk0[m] <= c_lo) lo = m; else hi = m;
        }
        t = lo;
    }
    int c = c_lo, cc = c_lo + warp;
    const int last = b.C - 1;
    ChunkSet next;   // the stream of the chunk this warp processes in the next round
    stage_load(next, b, min(cc, last), lane);
    while (c < c_hi) {
        while (b.tile_chunk0[t + 1] <= c) t++;
        const int c_end = min(c_hi, b.tile_chunk0[t + 1]);
        const long long base = (long long)t * b.T;
        const int cnt = (int)min((long long)b.T, N - base);
        __syncthreads();   // every warp is done with the previous tile
        {
            const float4 *src = reinterpret_cast<const float4 *>(Yp + base);   // base is even: 16-byte aligned
            float4 *dst = reinterpret_cast<float4 *>(tile);
            const int n4 = cnt >> 1;
            for (int i = threadIdx.x; i < n4; i += kBlockedThreads) dst[i] = __ldg(src + i);
            if ((cnt & 1) && threadIdx.x == 0) tile[cnt - 1] = Yp[base + cnt - 1];
        }
        __syncthreads();
        for (; cc < c_end; cc += nwarps) {
            ChunkSet cur = next;
            stage_load(next, b, min(cc + nwarps, last), lane);
            process_chunk(cur, tile, Yown, Fp, lane);
        }
        c = c_end;
    }
}

}  // namespace

void BlockedAttractive::clear() { *this = BlockedAttractive(); }

int launch_exclusive_scan_i32(int *data, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    scan_inplace_kernel<<<1, 1024, 0, st>>>(data, (long long)n);
    B200_CUDA(cudaGetLastError());
    return 0;
}

namespace {
// segments of a variable-width source: row at local permuted position lr has ptr[r + 1] - ptr[r] slots (r = own_perm[lr] - row_lo)
__global__ void seg_count_kernel(const int *__restrict__ ptr, const int32_t *__restrict__ own_perm, long long row_lo, long long rows,
                                 int *__restrict__ nseg)
{
    const long long lr = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (lr >= rows) return;
    const long long r = own_perm[lr] - row_lo;
    nseg[lr] = (ptr[r + 1] - ptr[r] + kMaxK - 1) / kMaxK;
}
__global__ void seg_fill_kernel(const int *__restrict__ ptr, const int32_t *__restrict__ own_perm, long long row_lo, long long rows,
                                const int *__restrict__ seg_off, int32_t *__restrict__ seg_row, long long *__restrict__ seg_base,
                                int *__restrict__ seg_len)
{
    const long long lr = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (lr >= rows) return;
    const long long r = own_perm[lr] - row_lo;
    const int lo = ptr[r], hi = ptr[r + 1];
    int g = seg_off[lr];
    for (int o = lo; o < hi; o += kMaxK, g++) {
        seg_row[g] = (int32_t)lr;
        seg_base[g] = o;
        seg_len[g] = min(kMaxK, hi - o);
    }
}

struct StreamOut {
    float *ev = nullptr;
    uint16_t *ec = nullptr;
    int *chunk_row0 = nullptr, *tile_chunk0 = nullptr;
    int C = 0;
    int64_t E = 0, groups = 0;
    float entries_per_group = 0.0f;
    bool built = false;
};

// One stream from the source described in `a` (val / ids / segments, pos, own_perm, N, row_lo, K, T, ntiles filled in).
// min_entries_per_group <= 0: build whatever the sample says.
int build_stream(StreamOut *out, DeviceArena &arena, DeviceArena &tmp, WalkArgs a, float min_entries_per_group, cudaStream_t st)
{
    *out = StreamOut();
    if (a.n_seg <= 0) return 0;
    const int ntiles = a.ntiles;
    // Measured at N = 10^6, K = 90: placing by bank pair takes the attractive stage from 197 to 191 us per iteration
    // and the set-up from 0.190 to 0.217 s (one lane per group walks the group's entries): it pays from 4,500
    // iterations on, so it is off unless B200TSNE_ATTRACTIVE_PLACE=1 asks for it.
    a.greedy = getenv("B200TSNE_ATTRACTIVE_PLACE") ? atoi(getenv("B200TSNE_ATTRACTIVE_PLACE")) : 0;
    a.range_rows = 64;
    while ((a.n_seg + a.range_rows - 1) / a.range_rows * ntiles > (1ll << 24)) a.range_rows *= 2;
    a.n_ranges = (a.n_seg + a.range_rows - 1) / a.range_rows;

    unsigned long long *totals = nullptr, h_tot[5] = {0, 0, 0, 0, 0};
    B200_TRY(tmp.alloc((void **)&totals, sizeof(h_tot)));
    B200_CUDA(cudaMemsetAsync(totals, 0, sizeof(h_tot), st));
    const long long n_samples = std::min<long long>(a.n_seg, 4096);
    // the small scratch when the tiles and the longest segment fit it
    const bool small = ntiles <= 64 && a.max_len <= 128;
    if (small) sample_kernel<WalkScratchSmall><<<(unsigned)((n_samples + kWalkWarps - 1) / kWalkWarps), kWalkWarps * 32, 0, st>>>(a, n_samples, totals);
    else sample_kernel<WalkScratch><<<(unsigned)((n_samples + kWalkWarps - 1) / kWalkWarps), kWalkWarps * 32, 0, st>>>(a, n_samples, totals);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaMemcpyAsync(h_tot, totals, sizeof(h_tot), cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    out->entries_per_group = h_tot[1] ? (float)((double)h_tot[2] / (double)h_tot[1]) : 0.0f;
    if (h_tot[1] == 0 || out->entries_per_group < min_entries_per_group) return 0;

    unsigned *range_size = nullptr;
    unsigned long long *tile_total = nullptr;
    long long *tile_start = nullptr;
    B200_TRY(tmp.alloc((void **)&range_size, sizeof(unsigned) * (size_t)ntiles * a.n_ranges));
    B200_TRY(tmp.alloc((void **)&tile_total, sizeof(unsigned long long) * ntiles));
    B200_TRY(tmp.alloc((void **)&tile_start, sizeof(long long) * (ntiles + 1)));
    B200_TRY(arena.alloc((void **)&out->tile_chunk0, sizeof(int) * (ntiles + 1)));
    const unsigned walk_blocks = (unsigned)((a.n_ranges + kWalkWarps - 1) / kWalkWarps);
    if (small) walk_kernel<false, WalkScratchSmall><<<walk_blocks, kWalkWarps * 32, 0, st>>>(a, range_size, nullptr, nullptr, nullptr, nullptr, nullptr, totals);
    else walk_kernel<false, WalkScratch><<<walk_blocks, kWalkWarps * 32, 0, st>>>(a, range_size, nullptr, nullptr, nullptr, nullptr, nullptr, totals);
    tile_scan_kernel<<<ntiles, 1024, 0, st>>>(range_size, a.n_ranges, tile_total);
    tile_layout_kernel<<<1, 1, 0, st>>>(tile_total, ntiles, tile_start, out->tile_chunk0, totals);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaMemcpyAsync(h_tot, totals, sizeof(h_tot), cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    const long long E = (long long)h_tot[3];
    if (E <= 0 || h_tot[4] || E / kChunk >= INT_MAX) return 0;
    B200_TRY(arena.alloc((void **)&out->ev, sizeof(float) * E));
    B200_TRY(arena.alloc((void **)&out->ec, sizeof(uint16_t) * E));
    B200_TRY(arena.alloc((void **)&out->chunk_row0, sizeof(int) * (E / kChunk)));
    B200_CUDA(cudaMemsetAsync(out->ev, 0, sizeof(float) * E, st));
    B200_CUDA(cudaMemsetAsync(out->ec, 0, sizeof(uint16_t) * E, st));
    B200_CUDA(cudaMemsetAsync(out->chunk_row0, 0, sizeof(int) * (E / kChunk), st));
    if (small) walk_kernel<true, WalkScratchSmall><<<walk_blocks, kWalkWarps * 32, 0, st>>>(a, nullptr, range_size, tile_start, out->ev, out->ec, out->chunk_row0, totals);
    else walk_kernel<true, WalkScratch><<<walk_blocks, kWalkWarps * 32, 0, st>>>(a, nullptr, range_size, tile_start, out->ev, out->ec, out->chunk_row0, totals);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaStreamSynchronize(st));   // the temporaries of the caller may go away
    out->C = (int)(E / kChunk);
    out->E = E;
    out->groups = (int64_t)h_tot[0];
    out->built = true;
    return 0;
}
}  // namespace

// Builds the blocked copy of the owned rows' fixed-width P and, with `extra`, a second stream from a variable-width
// list of further entries of the same rows (the reverse-only edges of a truly symmetric P).  perm (device, [N];
// null = identity) is the order of the points; persistent buffers come from `arena`.  On return b->ready says
// whether the copy was built; it is not when the sampled rows average fewer than kMinEntriesPerGroup entries per
// (row, tile), when there are too many tiles, or when K exceeds 1,024 - none of which is an error.
int blocked_attractive_build(BlockedAttractive *b, DeviceArena &arena, const float *P_rows, const int32_t *ids_rows, int64_t N, int K,
                             int64_t row_lo, int64_t row_hi, const int32_t *perm_in, const ExtraEntries *extra, cudaStream_t st)
{
    b->clear();
    const int64_t rows = row_hi - row_lo;
    if (rows <= 0 || N <= 0 || K <= 0) return 0;
    const char *mode = getenv("B200TSNE_ATTRACTIVE");   // "rows": never build; "blocked": build whatever the sample says
    if (mode && strcmp(mode, "rows") == 0) return 0;
    const bool forced = mode && strcmp(mode, "blocked") == 0;
    int ntiles = (int)((N + kTileMax - 1) / kTileMax);
    if (ntiles > kMaxTiles || K > kMaxK) return 0;
    int T = (int)(((N + ntiles - 1) / ntiles + 31) / 32 * 32);
    ntiles = (int)((N + T - 1) / T);

    DeviceArena tmp;
    tmp.serve(st);
    int32_t *perm = nullptr, *pos = nullptr, *own_perm = nullptr, *own_pos = nullptr;
    B200_TRY(arena.alloc((void **)&perm, sizeof(int32_t) * N));
    B200_TRY(tmp.alloc((void **)&pos, sizeof(int32_t) * N));
    const unsigned gN = (unsigned)((N + 255) / 256);
    if (perm_in) B200_CUDA(cudaMemcpyAsync(perm, perm_in, sizeof(int32_t) * N, cudaMemcpyDeviceToDevice, st));
    else iota_kernel<<<gN, 256, 0, st>>>(perm, N);
    invert_perm_kernel<<<gN, 256, 0, st>>>(perm, N, pos);
    if (rows == N) {
        own_perm = perm;
        B200_TRY(arena.alloc((void **)&own_pos, sizeof(int32_t) * N));
        B200_CUDA(cudaMemcpyAsync(own_pos, pos, sizeof(int32_t) * N, cudaMemcpyDeviceToDevice, st));
    } else {
        B200_TRY(arena.alloc((void **)&own_perm, sizeof(int32_t) * rows));
        B200_TRY(arena.alloc((void **)&own_pos, sizeof(int32_t) * rows));
        const unsigned nb = (unsigned)((N + kCompactPerBlock - 1) / kCompactPerBlock);
        int *bcount = nullptr;
        B200_TRY(tmp.alloc((void **)&bcount, sizeof(int) * nb));
        own_count_kernel<<<nb, 1024, 0, st>>>(perm, N, row_lo, row_hi, bcount);
        scan_inplace_kernel<<<1, 1024, 0, st>>>(bcount, nb);
        own_scatter_kernel<<<nb, 32, 0, st>>>(perm, N, row_lo, row_hi, bcount, own_perm, own_pos);
    }
    B200_CUDA(cudaGetLastError());

    WalkArgs a;
    memset(&a, 0, sizeof(a));
    a.val = P_rows; a.ids = ids_rows; a.pos = pos; a.own_perm = own_perm;
    a.N = N; a.row_lo = row_lo; a.n_seg = rows; a.K = K; a.T = T; a.ntiles = ntiles; a.max_len = K;
    StreamOut main_stream, extra_stream;
    B200_TRY(build_stream(&main_stream, arena, tmp, a, forced ? 0.0f : kMinEntriesPerGroup, st));
    b->entries_per_group = main_stream.entries_per_group;
    if (!main_stream.built) return 0;

    if (extra && extra->count > 0) {
        // segments of at most kMaxK slots, in the order of the rows' local permuted positions
        int *seg_off = nullptr, *seg_len = nullptr, h_last[2] = {0, 0};
        int32_t *seg_row = nullptr;
        long long *seg_base = nullptr;
        const unsigned gR = (unsigned)((rows + 255) / 256);
        B200_TRY(tmp.alloc((void **)&seg_off, sizeof(int) * (rows + 1)));
        B200_CUDA(cudaMemsetAsync(seg_off, 0, sizeof(int) * (rows + 1), st));
        seg_count_kernel<<<gR, 256, 0, st>>>(extra->ptr, own_perm, row_lo, rows, seg_off);
        B200_TRY(launch_exclusive_scan_i32(seg_off, rows + 1, st));
        B200_CUDA(cudaMemcpyAsync(h_last, seg_off + rows, sizeof(int), cudaMemcpyDeviceToHost, st));
        B200_CUDA(cudaStreamSynchronize(st));
        const long long n_seg = h_last[0];
        B200_TRY(tmp.alloc((void **)&seg_row, sizeof(int32_t) * std::max<long long>(n_seg, 1)));
        B200_TRY(tmp.alloc((void **)&seg_base, sizeof(long long) * std::max<long long>(n_seg, 1)));
        B200_TRY(tmp.alloc((void **)&seg_len, sizeof(int) * std::max<long long>(n_seg, 1)));
        seg_fill_kernel<<<gR, 256, 0, st>>>(extra->ptr, own_perm, row_lo, rows, seg_off, seg_row, seg_base, seg_len);
        B200_CUDA(cudaGetLastError());
        WalkArgs e = a;
        e.val = extra->val; e.ids = extra->ids;
        e.seg_row = seg_row; e.seg_base = seg_base; e.seg_len = seg_len; e.n_seg = n_seg; e.max_len = kMaxK;
        B200_TRY(build_stream(&extra_stream, arena, tmp, e, 0.0f, st));
        if (!extra_stream.built) { set_error("attractive: the stream of the reverse-only entries could not be built"); return -4; }
    }

    float2 *Yp = nullptr, *Yown = nullptr, *Fp = nullptr;
    B200_TRY(arena.alloc((void **)&Yp, sizeof(float2) * (size_t)ntiles * T));
    if (rows == N) Yown = Yp;
    else B200_TRY(arena.alloc((void **)&Yown, sizeof(float2) * rows));
    B200_TRY(arena.alloc((void **)&Fp, sizeof(float2) * rows));
    B200_CUDA(cudaMemsetAsync(Yp, 0, sizeof(float2) * (size_t)ntiles * T, st));
    static bool attr_set[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        B200_CUDA(cudaFuncSetAttribute(attractive_blocked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileMax * (int)sizeof(float2)));
        attr_set[dev] = true;
    }
    B200_CUDA(cudaStreamSynchronize(st));   // the temporaries go away with `tmp`

    b->ev = main_stream.ev; b->ec = main_stream.ec; b->chunk_row0 = main_stream.chunk_row0; b->tile_chunk0 = main_stream.tile_chunk0;
    b->C = main_stream.C; b->E = main_stream.E; b->groups = main_stream.groups;
    b->extra_ev = extra_stream.ev; b->extra_ec = extra_stream.ec; b->extra_chunk_row0 = extra_stream.chunk_row0;
    b->extra_tile_chunk0 = extra_stream.tile_chunk0; b->extra_C = extra_stream.C; b->extra_E = extra_stream.E;
    b->perm = perm; b->own_perm = own_perm; b->own_pos = own_pos;
    b->Yp = Yp; b->Yown = Yown; b->Fp = Fp;
    b->ntiles = ntiles; b->T = T;
    b->N = N; b->row_lo = row_lo; b->rows = rows;
    b->ready = true;
    return 0;
}

// F2[row_lo + r] = attractive force of the owned rows on the embedding Y2 (three launches)
// (Reading the force in cell order from the update kernel and letting it keep the cell-ordered embedding current
// instead of these two conversion kernels was measured on one GPU: the update kernel's three scattered 8-byte
// accesses per point cost it 148 us more - 169 instead of 21 - against the 17 us the conversions take.)
int launch_attractive_blocked(const BlockedAttractive &b, const float2 *Y2, float2 *F2, cudaStream_t st, bool in_cell_order)
{
    if (!b.ready) { set_error("attractive: the blocked copy of P was not built"); return -1; }
    if (in_cell_order && b.rows != b.N) { set_error("attractive: the cell order as the caller's order needs all rows"); return -1; }
    // in_cell_order: the caller keeps its points in this copy's order (a session on one GPU does: it converts where
    // embeddings enter and leave), so the kernel reads the embedding and adds to the forces where they are: the two
    // conversions are 18 of the stage's 209 us at N = 10^6
    const float2 *Yp = in_cell_order ? Y2 : b.Yp, *Yown = in_cell_order ? Y2 : b.Yown;
    float2 *Fp = in_cell_order ? F2 : b.Fp;
    const unsigned gN = (unsigned)((std::max(b.N, b.rows) + 255) / 256);
    if (in_cell_order) B200_CUDA(cudaMemsetAsync(F2, 0, sizeof(float2) * (size_t)b.rows, st));
    else permute_kernel<<<gN, 256, 0, st>>>(Y2, b.perm, b.N, b.Yp, b.own_perm, b.rows, b.Yown, b.Fp);
    BlockedStream s;
    s.ev = b.ev; s.ec = b.ec; s.chunk_row0 = b.chunk_row0; s.tile_chunk0 = b.tile_chunk0;
    s.ntiles = b.ntiles; s.T = b.T; s.C = b.C;
    int sms = 148;
    {
        static int cached[64] = {0};
        int dev = 0;
        B200_CUDA(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64) {
            if (!cached[dev]) B200_CUDA(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
            sms = cached[dev];
        }
    }
    // A block fills its SM (1,024 threads, all registers, 224 KB of shared memory), so the grid pipeline that runs
    // beside this kernel on the other stream only gets the SMs this kernel leaves alone.  Measured at N = 10^6,
    // K = 90 on 148 SMs, one GPU: 148 blocks 3,645 iterations/s (attractive stage 175 us), 140: 3,906, 132: 3,962
    // (196 us), 124: 3,936.  A rank of a sharded run has fewer rows for this kernel and the same grid pipeline
    // plus the meetings beside it: two GPUs 132 blocks 5,092 iterations/s, 116: 5,498, 100: 5,413, 92: 5,508, 74:
    // 4,991; four GPUs 132: 6,302, 100: 7,159, 80: 6,935, 64: 6,579, 48: 5,926.  Default: one SM in nine stays free
    // when the copy holds all rows, one in three when it holds a rank's share; B200TSNE_ATTRACTIVE_BLOCKS overrides.
    static const int want_blocks = getenv("B200TSNE_ATTRACTIVE_BLOCKS") ? atoi(getenv("B200TSNE_ATTRACTIVE_BLOCKS")) : 0;
    sms = want_blocks > 0 ? std::min(sms, want_blocks) : (b.rows == b.N ? sms - sms / 9 : sms - sms / 3);
    const int grid = std::max(1, std::min(sms, b.C));
    attractive_blocked_kernel<<<grid, kBlockedThreads, (size_t)b.T * sizeof(float2), st>>>(s, Yp, Yown, b.N, Fp);
    if (b.extra_C > 0) {   // the reverse-only entries of a truly symmetric P add to the same forces
        BlockedStream x = s;
        x.ev = b.extra_ev; x.ec = b.extra_ec; x.chunk_row0 = b.extra_chunk_row0; x.tile_chunk0 = b.extra_tile_chunk0; x.C = b.extra_C;
        attractive_blocked_kernel<<<std::max(1, std::min(sms, b.extra_C)), kBlockedThreads, (size_t)b.T * sizeof(float2), st>>>(x, Yp, Yown, b.N,
                                                                                                                          Fp);
    }
    if (!in_cell_order) unpermute_kernel<<<(unsigned)((b.rows + 255) / 256), 256, 0, st>>>(b.Fp, b.own_pos, b.row_lo, b.rows, F2);
    B200_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace b200
