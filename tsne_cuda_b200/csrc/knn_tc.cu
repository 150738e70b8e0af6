// Exact k-nearest-neighbour search on the tensor cores (tcgen05 + TMEM): a kernel that keeps the whole inner
// dimension in shared memory (D <= 63) and a chunked one for wider points (knn_tc_wide_kernel).
//
// Replaces the reference's FAISS IVF-Flat call (src/util/distance_utils.cu:79-121, approximate).
// The result is the same as the SIMT search of knn.cu: ids ordered by the canonical fp32 distance
// (sequential, unfused) with ties broken by index.  It is obtained in three steps:
//
//  1. Filter.  Ranking keys  key_ij = |x_j|^2 - 2 x_i.x_j  come straight out of the tensor cores: the
//     query operand is [x_i, 1], the database operand [-2 x_j, |x_j|^2] (padding columns of the inner
//     dimension carry the norm), each value split in a pair v = hi + lo and multiplied as three products
//     hi.hi + lo.hi + hi.lo accumulated in fp32 in TMEM.  By default the pairs are bf16 (kind::f16, K steps
//     of 16, keys accurate to 3 * 2^-16 of sum_k |x_ik||2 x_jk|; the norm travels in two column pairs);
//     B200TSNE_KNN_FILTER=tf32 selects TF32 pairs (K steps of 8, about 2^-20 of |x_i||x_j|) at nearly twice
//     the tensor-core time.  Either error is covered by the proof of step 3.  A block owns 256 queries (one
//     TMEM lane each per query tile) and
//     walks the database in tiles of 128 points; each epilogue thread compares its row of the
//     accumulator tile with a per-query threshold and appends the rare survivors to the query's
//     candidate buffer with plain stores; the L = K + slack best are kept.  No N x N matrix is written.
//  2. Re-rank.  The canonical distance of the L candidates is evaluated exactly and they are ordered by
//     (distance, id).
//  3. Proof.  Every point that is not a candidate has a key >= T (the largest key in the list), hence a
//     canonical distance >= (|x_i|^2 + T - E)(1 - theta) with E bounding the filter's error and theta the
//     rounding of the canonical sum.  If the K-th candidate distance is strictly below that bound the
//     first K candidates are provably the exact answer; otherwise the row is flagged and recomputed by
//     the SIMT search.  The observed filter error on the candidates is checked against E as well.
//
// Operand staging: the prepared operands live in global memory as ready-made shared-memory images,
// one per 128-row tile: for hi then lo, for every 8-wide K step, the 128 x 8 block in the
// no-swizzle K-major core-matrix order (8 rows x 16 bytes contiguous; the two 16-byte halves of a K
// step 128 bytes apart; 8-row groups 256 bytes apart).  A tile is therefore ONE contiguous bulk
// copy (cp.async.bulk + mbarrier complete_tx) with no tensor map and no swizzle.
//
// Thresholds.  For a small database the threshold is maintained online: the L-th best key at the last
// compaction of the query's buffer (a warp-wide bitonic sort).  That appends about L ln(N/L) candidates per
// query, which is rare per thread but not per warp of 32 queries, and each compaction costs thousands of
// issue slots.  For a large database (>= 512 tiles) the threshold is therefore FIXED per query, in three
// levels, each sizing the candidate set of the next: (A) on the CUDA cores, the key of rank ~10 among a
// few thousand jittered sample points; (B) every 16th tile against tau_A (~300 candidates); (C) all
// tiles against tau_B = the key of rank ~3L/16 of sample B, which about 3L points beat.  Nothing is
// compacted during a fixed-threshold scan; the L best are selected once at the end (by bisection on the
// key bits, not by sorting).  A row whose buffer
// overflows or ends with fewer than L candidates is flagged and recomputed by the SIMT search.
//
// Epilogue: a thread first reduces its 32 keys of a chunk to their minimum (a tree of independent
// min operations); only if that minimum beats the threshold, which becomes rare as the scan
// proceeds, does it locate and append the survivors.
//
// Order of the scan.  Queries and database rows are visited by Voronoi cells around sample points; a block
// skips the database cells none of its queries can reach under their thresholds (triangle inequality, see
// the knn_cells_* kernels), which leaves the result untouched and removes most tile pairs on clustered
// data.  A database image much larger than L2 is scanned in windows, one launch per window.
//
// Warp roles: a block serves QH = 2 query tiles (256 queries; 1 when the operand images are too wide for
// that) against every database tile, so a database image is fetched from L2 once per 256 queries.
// Warps 0 .. 8 QH - 1 are the epilogue, in 2 QH groups of four (TMEM lane quarter = warp % 4), then the
// bulk-copy producer warp and the MMA issuer / TMEM owner warp.  Two database stages and two accumulator
// buffers (of QH tiles each), so the MMAs of tile t+1 overlap the epilogue of tile t.  Measured on the
// full pass at N = 10^6, D = 50: with the epilogue's comparisons removed the kernel takes 89 % of its
// time, i.e. it is bound by the tensor pipe (42 MMAs 128x128x8 per tile pair at ~105 cycles each).
// Every wait has a time limit; on expiry the kernel sets an error flag, drains and frees its TMEM.
#include <limits.h>
#include <stdio.h>
#include <string.h>
#include <stdlib.h>

#include "common.cuh"

#include <cuda_bf16.h>

#include <algorithm>

namespace b200 {
namespace {

constexpr int TM = 128;             // queries per block = accumulator rows = TMEM lanes
constexpr int TN = 128;             // database points per tile = accumulator columns
constexpr int kBStages = 2;
constexpr int kAccBufs = 2;
// A block serves QH query tiles (QH = 2 when two query images and two database stages fit in shared
// memory, else 1): every database tile is multiplied with each of them, so the database image is read
// from L2 once per 128 * QH queries.  8 * QH epilogue warps, then the producer warp and the MMA warp;
// TMEM columns = kAccBufs * QH * TN.
constexpr int tc_threads(int QH) { return (8 * QH + 2) * 32; }

// ------------------------------------------------------------------------------------------------
// PTX helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after 4 s or as soon as another thread of the block has given up.  A waiting
// thread sleeps between polls: the producer and the MMA issuer share their schedulers with epilogue
// warps, and a busy poll would take every other issue slot from them.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned sleep_ns = 128,
                                          unsigned long long limit_ns = 4000000000ull)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(sleep_ns);
        if ((++spins & 63) == 0) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > limit_ns) { *abort_flag = 1; return false; }
        }
    }
    return true;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 128 x 128 x 8, TF32 operands, fp32 accumulation
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 128 x 128 x 16, bf16 operands, fp32 accumulation
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// 32 consecutive accumulator columns of this thread's TMEM lane: asynchronous issue ...
__device__ __forceinline__ void tc_ld32_issue(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32"
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
        " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
// ... and the wait that makes the registers valid (they are listed so that no use is scheduled above it)
__device__ __forceinline__ void tc_ld32_wait(uint32_t (&r)[32])
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                   "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                   "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

// three-input minimum (one instruction on sm_100)
__device__ __forceinline__ float min3(float a, float b, float c)
{
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes, the two
// 16-byte halves of a K step 128 bytes apart (leading offset), 8-row groups 256 bytes apart (stride
// offset); offsets are encoded in 16-byte units; bits 46-47 carry the descriptor version (1).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fff);
    d |= (uint64_t)(128 >> 4) << 16;
    d |= (uint64_t)(256 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// The same for a swizzled K-major image: rows of sw = 32, 64 or 128 bytes, 8-row groups 8 * sw bytes apart, the
// 16-byte pieces of a row exchanged by the XOR pattern of that width (layout type 6, 4 or 2 in bits 61-63; the
// leading offset is not used).  A K step inside a row is reached by adding its byte offset to the start address.
__device__ __forceinline__ uint64_t make_desc_swizzled(uint32_t saddr, uint32_t sw)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8u * sw) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(sw == 128u ? 2u : (sw == 64u ? 4u : 6u)) << 61;
    return d;
}
// Instruction descriptor: fp32 accumulate (bits 4-5 = 1), TF32 A and B (bits 7-9, 10-12 = 2), both
// K-major (bits 15, 16 = 0), N/8 in bits 17-22, M/16 in bits 24-28.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
// the same with bf16 A and B (format 1 of kind::f16); one K step is 32 operand bytes per row in either kind
constexpr uint32_t kInstrDescBf16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);


// ------------------------------------------------------------------------------------------------
// operand preparation
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float to_tf32(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// offset (in floats) of element (row r, dimension k) inside a tile image part (hi or lo)
__device__ __forceinline__ size_t image_offset(int r, int k)
{
    return (size_t)(k >> 3) * 1024 + (size_t)(r >> 3) * 64 + (size_t)((k >> 2) & 1) * 32 + (size_t)(r & 7) * 4 + (k & 3);
}

// Rows of X named by `list` (-1 = padding) -> tile images [tiles][Dp/KC chunks][2 (hi, lo)][KC/8][1024 floats] (the
// narrow path has one chunk, KC = Dp; the wide path chunks of kWideKC inner dimensions) in query form
// [x, 1, 0...] or database form [-2x, |x|^2, 0...]; a padding row is all zeros as a query and carries a huge
// finite norm as a database point, so it never ranks.  norms (queries only): exact squared norms, double.
__global__ void __launch_bounds__(128)
knn_tc_prepare_kernel(const float *__restrict__ X, const int *__restrict__ list, int D, int Dp, int KC, int db_form,
                      float *__restrict__ img, double *__restrict__ norms)
{
    const long long tile = blockIdx.x;
    const int r = threadIdx.x;
    const long long pos = tile * TM + r;
    const int i = list[pos];
    float *im_tile = img + (size_t)tile * 2 * Dp * 128;
    const size_t part = (size_t)KC * 128;
    double n2 = 0.0;
    for (int k = 0; k < D; k++) {
        const float x = (i >= 0) ? X[(long long)i * D + k] : 0.0f;
        n2 += (double)x * (double)x;
    }
    for (int k = 0; k < Dp; k++) {
        float v = 0.0f;
        if (k < D) {
            const float x = (i >= 0) ? X[(long long)i * D + k] : 0.0f;
            v = db_form ? -2.0f * x : x;
        } else if (k == D) {
            v = db_form ? ((i >= 0) ? (float)n2 : 3.0e38f) : ((i >= 0) ? 1.0f : 0.0f);
        }
        const float vh = to_tf32(v);
        float *im = im_tile + (size_t)(k / KC) * 2 * part;
        im[image_offset(r, k % KC)] = vh;
        im[part + image_offset(r, k % KC)] = to_tf32(v - vh);
    }
    if (norms) norms[pos] = n2;
}

// The bf16 form of the images: v = hi + lo + r with hi, lo in bf16 (round to nearest) and |r| <= 2^-16 |v|; the
// same byte geometry as the TF32 images (a K step is 16 values = 32 bytes per row, core matrices of 8 rows x 16
// bytes), so the shared-memory descriptors are the same and an image has half the bytes per inner dimension.
// [tiles][Dp/KC chunks][2 (hi, lo)][KC/16][2048 values].  Two columns carry the norm (its bf16 pair and the pair of
// what that pair leaves over: 32 significant bits), against 1, 1 in the query form.
__device__ __forceinline__ size_t image_offset_bf16(int r, int k)
{
    return (size_t)(k >> 4) * 2048 + (size_t)(r >> 3) * 128 + (size_t)((k >> 3) & 1) * 64 + (size_t)(r & 7) * 8 + (k & 7);
}
// The swizzled form (narrow kernel): rows of sw bytes (sw / 2 values), blocks of 128 rows one after the other along
// the inner dimension; inside a block the 16-byte piece p of row r sits where piece p ^ ((r * sw / 128) mod (sw / 16))
// would (the shared-memory swizzle of that width, which the tensor core undoes when it reads: operands in this
// form are fetched about twice as fast as core matrices without swizzle, measured).  Offset in values.
__device__ __forceinline__ size_t image_offset_bf16_swizzled(int r, int k, int sw)
{
    const int per_row = sw >> 1;
    const int block = k / per_row;
    unsigned off = (unsigned)r * (unsigned)sw + (unsigned)(k % per_row) * 2u;   // bytes inside the block
    off ^= ((off >> 7) & ((unsigned)(sw >> 4) - 1u)) << 4;
    return (size_t)block * 64 * sw + (off >> 1);
}

// What the three products drop is bounded per pair from the actual leftovers: with a, b the data columns of a
// query and a database operand, a = a_hi + a_lo + a_r,  |dropped| <= |a_lo||b_lo| + |a - a_r||b_r| + |a_r||b - b_r|
// + |a_r||b_r| (Cauchy-Schwarz on the leftover vectors).  Queries record |a_lo| and |a_r| (res), the database the
// largest |b_lo|/|b| and |b_r|/|b| over its rows (rho_bits: float bits, raised with atomicMax).
__global__ void __launch_bounds__(128)
knn_tc_prepare_bf16_kernel(const float *__restrict__ X, const int *__restrict__ list, int D, int Dp, int KC, int sw, int db_form,
                           __nv_bfloat16 *__restrict__ img, double *__restrict__ norms, float2 *__restrict__ res,
                           int *__restrict__ rho_bits)
{
    const long long tile = blockIdx.x;
    const int r = threadIdx.x;
    const long long pos = tile * TM + r;
    const int i = list[pos];
    __nv_bfloat16 *im_tile = img + (size_t)tile * 2 * Dp * 128;
    const size_t part = (size_t)KC * 128;
    double n2 = 0.0;
    for (int k = 0; k < D; k++) {
        const float x = (i >= 0) ? X[(long long)i * D + k] : 0.0f;
        n2 += (double)x * (double)x;
    }
    const float nf = (i >= 0) ? (float)n2 : 3.0e38f;
    const float nf_hi = __bfloat162float(__float2bfloat16_rn(nf));
    const float nf_rest = (nf - nf_hi) - __bfloat162float(__float2bfloat16_rn(nf - nf_hi));   // both differences are exact in fp32
    double lo2 = 0.0, r2 = 0.0;   // squared norms of the lo parts and of the leftovers of the data columns
    for (int k = 0; k < Dp; k++) {
        float v = 0.0f;
        if (k < D) {
            const float x = (i >= 0) ? X[(long long)i * D + k] : 0.0f;
            v = db_form ? -2.0f * x : x;
        } else if (k == D) {
            v = db_form ? nf : ((i >= 0) ? 1.0f : 0.0f);
        } else if (k == D + 1) {
            v = db_form ? nf_rest : ((i >= 0) ? 1.0f : 0.0f);
        }
        const __nv_bfloat16 vh = __float2bfloat16_rn(v);
        const float rest = v - __bfloat162float(vh);
        const __nv_bfloat16 vl = __float2bfloat16_rn(rest);
        __nv_bfloat16 *im = im_tile + (size_t)(k / KC) * 2 * part;
        const size_t at = sw ? image_offset_bf16_swizzled(r, k % KC, sw) : image_offset_bf16(r, k % KC);
        im[at] = vh;
        im[part + at] = vl;
        if (k < D) {
            const float left = rest - __bfloat162float(vl);
            lo2 += (double)__bfloat162float(vl) * (double)__bfloat162float(vl);
            r2 += (double)left * (double)left;
        }
    }
    if (norms) norms[pos] = n2;
    if (res) res[pos] = make_float2((float)(sqrt(lo2) * 1.000001), (float)(sqrt(r2) * 1.000001));   // rounded up
    if (rho_bits) {
        float rl = 0.0f, rr = 0.0f;
        if (i >= 0 && n2 > 0.0) {
            rl = (float)(sqrt(lo2 / (4.0 * n2)) * 1.000001);
            rr = (float)(sqrt(r2 / (4.0 * n2)) * 1.000001);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            rl = fmaxf(rl, __shfl_xor_sync(0xffffffffu, rl, o));
            rr = fmaxf(rr, __shfl_xor_sync(0xffffffffu, rr, o));
        }
        if ((threadIdx.x & 31) == 0) {   // non-negative floats: integer order == float order
            atomicMax(rho_bits + 0, __float_as_int(rl));
            atomicMax(rho_bits + 1, __float_as_int(rr));
        }
    }
}

// ------------------------------------------------------------------------------------------------
// cells: a coarse partition of the points that lets a block skip database tiles no query of it can reach
// ------------------------------------------------------------------------------------------------
// Both the database rows and the queries of a search are visited in the order of a partition into at
// most kMaxCells Voronoi cells around sample points ("centres").  Database cells start on tile
// boundaries (padding rows in between), so a cell is a run of whole tiles; for every cell the largest
// distance r_c of a member to its centre is known.  Once a query's threshold is fixed, no point of cell c
// can pass it if  |x_q - centre_c| - r_c  exceeds the threshold distance (triangle inequality), and a block
// skips the cells that none of its queries can reach.  On clustered data most tile pairs disappear; on
// data without structure nothing is lost but the few milliseconds of these kernels.
constexpr int kMaxCells = 64;
constexpr int kCellThreads = 256;

struct CellTable {
    float centre[kMaxCells][64];      // zero beyond D
    unsigned int radius_bits[kMaxCells];   // float bits of r_c (non-negative floats order like unsigned integers)
    int db_count[kMaxCells], q_count[kMaxCells];
    int db_start[kMaxCells + 1];      // first list position of the cell (multiple of TN); [cells] = end
    int q_start[kMaxCells + 1];
    int db_cursor[kMaxCells], q_cursor[kMaxCells];
};

__global__ void knn_cells_init_kernel(const float *__restrict__ X, int D, long long db_lo, long long nd, int cells, CellTable *tab)
{
    // centres = database rows, one from each of `cells` equal stretches of the range at a hashed offset (an
    // even spacing would alias with any periodic ordering of the data and could leave whole clusters
    // without a centre)
    for (int idx = threadIdx.x; idx < cells * 64; idx += blockDim.x) {
        const int c = idx >> 6, d = idx & 63;
        const long long stretch = nd / cells;
        const unsigned long long h = ((unsigned long long)(c + 1) * 0x9E3779B97F4A7C15ull) >> 20;
        const long long row = db_lo + (long long)c * stretch + (long long)(h % (unsigned long long)stretch);
        tab->centre[c][d] = (d < D) ? X[row * D + d] : 0.0f;
    }
    for (int c = threadIdx.x; c < kMaxCells; c += blockDim.x) {
        tab->radius_bits[c] = 0u;
        tab->db_count[c] = tab->q_count[c] = 0;
        tab->db_cursor[c] = tab->q_cursor[c] = 0;
    }
}

// cell[i] = nearest centre of row lo + i; counts the members and (for the database) maintains r_c
__global__ void __launch_bounds__(kCellThreads)
knn_cells_assign_kernel(const float *__restrict__ X, int D, long long lo, long long n, int cells, CellTable *tab, int is_db,
                        unsigned char *__restrict__ cell)
{
    __shared__ float s_c[kMaxCells][65];
    __shared__ int s_cnt[kMaxCells];
    __shared__ unsigned int s_rad[kMaxCells];
    for (int idx = threadIdx.x; idx < cells * 64; idx += kCellThreads) s_c[idx >> 6][idx & 63] = tab->centre[idx >> 6][idx & 63];
    for (int c = threadIdx.x; c < kMaxCells; c += kCellThreads) { s_cnt[c] = 0; s_rad[c] = 0u; }
    __syncthreads();
    const long long i = (long long)blockIdx.x * kCellThreads + threadIdx.x;
    if (i < n) {
        float x[64];
#pragma unroll
        for (int d = 0; d < 64; d++) x[d] = (d < D) ? X[(lo + i) * D + d] : 0.0f;
        float best = INFINITY;
        int bc = 0;
        for (int c = 0; c < cells; c++) {
            float acc = 0.0f;
#pragma unroll
            for (int d = 0; d < 64; d++) {
                const float t = x[d] - s_c[c][d];
                acc = fmaf(t, t, acc);
            }
            if (acc < best) { best = acc; bc = c; }
        }
        cell[i] = (unsigned char)bc;
        atomicAdd(&s_cnt[bc], 1);
        if (is_db) atomicMax(&s_rad[bc], __float_as_uint(sqrtf(best)));
    }
    __syncthreads();
    for (int c = threadIdx.x; c < cells; c += kCellThreads) {
        if (s_cnt[c]) atomicAdd(is_db ? &tab->db_count[c] : &tab->q_count[c], s_cnt[c]);
        if (is_db && s_rad[c]) atomicMax(&tab->radius_bits[c], s_rad[c]);
    }
}

// list positions of the cells: database cells padded to whole tiles, query cells back to back
__global__ void knn_cells_layout_kernel(int cells, CellTable *tab)
{
    if (threadIdx.x != 0) return;
    int db = 0, q = 0;
    for (int c = 0; c < cells; c++) {
        tab->db_start[c] = db;
        tab->q_start[c] = q;
        db += (tab->db_count[c] + TN - 1) / TN * TN;
        q += tab->q_count[c];
    }
    for (int c = cells; c <= kMaxCells; c++) { tab->db_start[c] = db; tab->q_start[c] = q; }
}

// list[start(cell) + rank within the cell] = row; the order inside a cell is arbitrary (it decides which
// points share a tile, never the result)
__global__ void __launch_bounds__(kCellThreads)
knn_cells_scatter_kernel(const unsigned char *__restrict__ cell, long long lo, long long n, int cells, CellTable *tab, int is_db,
                         int *__restrict__ list)
{
    __shared__ int s_cnt[kMaxCells], s_base[kMaxCells];
    for (int c = threadIdx.x; c < kMaxCells; c += kCellThreads) s_cnt[c] = 0;
    __syncthreads();
    const long long i = (long long)blockIdx.x * kCellThreads + threadIdx.x;
    int c = 0, local = 0;
    if (i < n) {
        c = cell[i];
        local = atomicAdd(&s_cnt[c], 1);
    }
    __syncthreads();
    for (int k = threadIdx.x; k < cells; k += kCellThreads)
        if (s_cnt[k]) s_base[k] = atomicAdd(is_db ? &tab->db_cursor[k] : &tab->q_cursor[k], s_cnt[k]);
    __syncthreads();
    if (i < n) list[(is_db ? tab->db_start[c] : tab->q_start[c]) + s_base[c] + local] = (int)(lo + i);
}

__global__ void knn_iota_kernel(int *__restrict__ list, long long lo, long long n)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) list[i] = (int)(lo + i);
}

// ------------------------------------------------------------------------------------------------
// candidate buffers: compaction by a warp-wide bitonic sort, EPL elements per lane (32*EPL = capacity)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool pair_less(float ka, int ia, float kb, int ib) { return ka < kb || (ka == kb && ia < ib); }

// One compare-exchange step between registers r and r + J of the same lane (J < EPL).
template <int EPL, int J>
__device__ __forceinline__ void bitonic_in_lane(float (&k)[EPL], int (&id)[EPL], int lane, int size)
{
#pragma unroll
    for (int r = 0; r < EPL; r++) {
        if ((r & J) == 0) {
            const bool up = ((lane * EPL + r) & size) == 0;
            const bool swap = up ? pair_less(k[r + J], id[r + J], k[r], id[r]) : pair_less(k[r], id[r], k[r + J], id[r + J]);
            if (swap) {
                const float tk = k[r]; k[r] = k[r + J]; k[r + J] = tk;
                const int ti = id[r]; id[r] = id[r + J]; id[r + J] = ti;
            }
        }
    }
}

// Warp-wide bitonic sort of 32*EPL (key, id) pairs, ascending; element index = lane * EPL + r.  The two
// outer loops are real loops (the sort runs rarely and from cold instruction cache: a fully unrolled
// network of ~2500 instructions costs more in instruction fetch than it saves).
template <int EPL>
__device__ __forceinline__ void warp_bitonic_sort(float (&k)[EPL], int (&id)[EPL], int lane)
{
#pragma unroll 1
    for (int size = 2; size <= 32 * EPL; size <<= 1) {
#pragma unroll 1
        for (int j = size >> 1; j > 0; j >>= 1) {
            if (j >= EPL) {
                const int lj = j / EPL;
                const bool lower = ((lane * EPL) & j) == 0;     // same for all registers of the lane: j >= EPL
#pragma unroll
                for (int r = 0; r < EPL; r++) {
                    const float ok = __shfl_xor_sync(0xffffffffu, k[r], lj);
                    const int oi = __shfl_xor_sync(0xffffffffu, id[r], lj);
                    const bool up = ((lane * EPL + r) & size) == 0;      // ascending block
                    const bool keep_min = (lower == up);
                    const bool take = keep_min ? pair_less(ok, oi, k[r], id[r]) : pair_less(k[r], id[r], ok, oi);
                    if (take) { k[r] = ok; id[r] = oi; }
                }
            } else if (j == 1) {
                bitonic_in_lane<EPL, 1>(k, id, lane, size);
            } else if (j == 2) {
                bitonic_in_lane<EPL, 2>(k, id, lane, size);
            } else if (j == 4) {
                bitonic_in_lane<EPL, 4>(k, id, lane, size);
            } else {
                if constexpr (EPL > 8) bitonic_in_lane<EPL, 8>(k, id, lane, size);
            }
        }
    }
}

// Sort the first n entries of one query's buffer (capacity 32*EPL) and keep the L best (L = 16*EPL).
// Whole warp; returns the new threshold (key of the L-th best, +inf while fewer than L entries exist).
template <int EPL>
__device__ __noinline__ float warp_compact(float *bk, int32_t *bi, int n, int lane)
{
    constexpr int L = 16 * EPL;
    float k[EPL];
    int id[EPL];
#pragma unroll
    for (int r = 0; r < EPL; r++) {
        const int idx = lane * EPL + r;
        k[r] = (idx < n) ? __ldcg(bk + idx) : INFINITY;
        id[r] = (idx < n) ? __ldcg(bi + idx) : INT_MAX;
    }
    warp_bitonic_sort<EPL>(k, id, lane);
#pragma unroll
    for (int r = 0; r < EPL; r++) {
        const int idx = lane * EPL + r;
        if (idx < L) { __stcg(bk + idx, k[r]); __stcg(bi + idx, id[r]); }
    }
    return __shfl_sync(0xffffffffu, k[EPL - 1], 15);   // element L-1 sits in lane 15, last register
}

// One block per filter block (qpc = its queries): which cells can hold a point that passes the threshold of
// at least one of its queries?  Their tile ranges, merged where adjacent, are the block's segments.
// Rounding: the fp32 distances carry a relative error below 1e-5 (sums of at most 64 squares), the
// inequality is tested with margins ten times that; a comparison that involves a NaN keeps the cell.
__global__ void __launch_bounds__(kCellThreads)
knn_cells_segments_kernel(const float *__restrict__ X, int D, const int *__restrict__ qlist, long long nq, int qpc,
                          const float *__restrict__ tau, const double *__restrict__ norms_q, int cells,
                          const CellTable *__restrict__ tab, int2 *__restrict__ segs, int *__restrict__ nseg)
{
    __shared__ float s_c[kMaxCells][65];
    __shared__ float s_r[kMaxCells];
    __shared__ int s_keep[kMaxCells];
    for (int idx = threadIdx.x; idx < cells * 64; idx += kCellThreads) s_c[idx >> 6][idx & 63] = tab->centre[idx >> 6][idx & 63];
    for (int c = threadIdx.x; c < kMaxCells; c += kCellThreads) {
        s_r[c] = __uint_as_float(tab->radius_bits[c]) * 1.00001f;
        s_keep[c] = 0;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < qpc; j += kCellThreads) {
        const long long q = (long long)blockIdx.x * qpc + j;
        if (q >= nq) continue;
        const double R2 = norms_q[q] + (double)tau[q];   // a point passes if its squared distance is below this
        if (!(R2 <= 0.0)) {
            const float R = (float)sqrt(R2) * 1.0001f;
            const int i = qlist[q];
            float x[64];
#pragma unroll
            for (int d = 0; d < 64; d++) x[d] = (d < D) ? X[(long long)i * D + d] : 0.0f;
            for (int c = 0; c < cells; c++) {
                float acc = 0.0f;
#pragma unroll
                for (int d = 0; d < 64; d++) {
                    const float t = x[d] - s_c[c][d];
                    acc = fmaf(t, t, acc);
                }
                const float lower = sqrtf(acc) * 0.99999f - s_r[c];
                if (!(lower > R)) s_keep[c] = 1;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int n = 0;
        int2 *out = segs + (size_t)blockIdx.x * kMaxCells;
        for (int c = 0; c < cells; c++) {
            if (!s_keep[c] || tab->db_count[c] == 0) continue;
            const int a = tab->db_start[c] / TN, b = tab->db_start[c + 1] / TN;
            if (n > 0 && out[n - 1].y == a) out[n - 1].y = b;
            else out[n++] = make_int2(a, b);
        }
        nseg[blockIdx.x] = n;
    }
}

__global__ void knn_single_segment_kernel(int2 *segs, int *nseg, int tiles)
{
    segs[0] = make_int2(0, tiles);
    nseg[0] = 1;
}

// The database tiles of a block in scan order: the tiles of its segments that are multiples of `stride` and lie
// in the window [win_lo, win_hi) of the launch.
// The producer, the MMA issuer and the epilogue each walk the same sequence.
struct TileWalk {
    const int2 *segs;
    int nseg, stride, win_lo, win_hi, s, t, end;
    __device__ TileWalk(const int2 *segs_, int nseg_, int stride_, int win_lo_, int win_hi_)
        : segs(segs_), nseg(nseg_), stride(stride_), win_lo(win_lo_), win_hi(win_hi_), s(-1), t(0), end(0) {}
    __device__ bool next(int &tile)
    {
        while (t >= end) {
            if (++s >= nseg) return false;
            const int2 g = segs[s];
            t = (max(g.x, win_lo) + stride - 1) / stride * stride;
            end = min(g.y, win_hi);
        }
        tile = t;
        t += stride;
        return true;
    }
};

// ------------------------------------------------------------------------------------------------
// filter kernel
// ------------------------------------------------------------------------------------------------
struct TcShared {
    uint64_t full_a;
    uint64_t full_b[kBStages];
    uint64_t empty_b[kBStages];
    uint64_t acc_full[kAccBufs];
    uint64_t acc_empty[kAccBufs];
    uint32_t tmem_base;
    int abort_flag;
};

// The MMAs of one accumulator tile: three products over NKS K steps, every descriptor a register plus a register.
// NKS is a template argument so that the loops unroll into independent instruction sequences: one thread issues
// every MMA of the block, and whatever it computes per MMA shows in the kernel's time.
template <bool BF16, int NKS>
__device__ __forceinline__ void tc_issue_products(uint32_t d_tmem, uint64_t a_hi, uint64_t a_lo, uint64_t b_hi, uint64_t b_lo,
                                                  const uint32_t (&off16)[NKS])
{
#pragma unroll
    for (int ks = 0; ks < NKS; ks++) {      // hi . hi
        if (BF16) tc_mma_bf16(d_tmem, a_hi + off16[ks], b_hi + off16[ks], kInstrDescBf16, ks ? 1u : 0u);
        else tc_mma_tf32(d_tmem, a_hi + off16[ks], b_hi + off16[ks], kInstrDesc, ks ? 1u : 0u);
    }
#pragma unroll
    for (int ks = 0; ks < NKS; ks++) {      // lo . hi
        if (BF16) tc_mma_bf16(d_tmem, a_lo + off16[ks], b_hi + off16[ks], kInstrDescBf16, 1u);
        else tc_mma_tf32(d_tmem, a_lo + off16[ks], b_hi + off16[ks], kInstrDesc, 1u);
    }
#pragma unroll
    for (int ks = 0; ks < NKS; ks++) {      // hi . lo
        if (BF16) tc_mma_bf16(d_tmem, a_hi + off16[ks], b_lo + off16[ks], kInstrDescBf16, 1u);
        else tc_mma_tf32(d_tmem, a_hi + off16[ks], b_lo + off16[ks], kInstrDesc, 1u);
    }
}

// The MMA issuer's walk over the block's database tiles (one thread).  a16 / b16 / end16: the block's images in
// 16-byte units of shared memory; span16: what one K step reads beyond its start.  Every tile's descriptors are
// checked against that range before they are used (an MMA that reads outside the block's shared memory is a fault).
template <int QH, bool BF16, int NKS>
__device__ __noinline__ void tc_issue_walk(TcShared *shp, volatile int *abort_flag, TileWalk walk, uint32_t tmem_base, uint64_t no_addr,
                                           uint32_t a16, uint32_t b16, uint32_t image16, uint32_t spr_log, uint32_t block16,
                                           uint32_t in_row16, uint32_t span16, uint32_t end16)
{
    TcShared &sh = *shp;
    const uint32_t part16 = image16 >> 1, spr_mask = (1u << spr_log) - 1u;
    uint32_t off16[NKS];
#pragma unroll
    for (int ks = 0; ks < NKS; ks++) off16[ks] = ((uint32_t)ks >> spr_log) * block16 + ((uint32_t)ks & spr_mask) * in_row16;
    const uint32_t reach16 = off16[NKS - 1] + span16;   // the furthest a part's K steps read
    int tile;
    for (long long t = 0; walk.next(tile); t++) {
        const int s = (int)(t % kBStages), b = (int)(t % kAccBufs);
        const uint32_t ph_s = (uint32_t)((t / kBStages) & 1), ph_b = (uint32_t)((t / kAccBufs) & 1);
        if (!mbar_wait(&sh.acc_empty[b], ph_b ^ 1u, abort_flag)) break;
        if (!mbar_wait(&sh.full_b[s], ph_s, abort_flag)) break;
        tc_fence_after();
        const uint32_t bs16 = b16 + (uint32_t)s * image16;
        if (reach16 > part16 || a16 + QH * image16 > b16 || bs16 + image16 > end16) { *abort_flag = 1; break; }
        const uint64_t b_hi = no_addr + (uint64_t)bs16, b_lo = b_hi + part16;
#pragma unroll
        for (int h = 0; h < QH; h++) {
            const uint64_t a_hi = no_addr + (uint64_t)(a16 + (uint32_t)h * image16), a_lo = a_hi + part16;
            tc_issue_products<BF16, NKS>(tmem_base + (uint32_t)((b * QH + h) * TN), a_hi, a_lo, b_hi, b_lo, off16);
        }
        tc_commit(&sh.empty_b[s]);    // the stage may be refilled once these MMAs have read it
        tc_commit(&sh.acc_full[b]);   // the accumulator tiles are complete
    }
}

// img_q / img_db: tile images of the query list and of the database list.  A block serves the queries
// [blockIdx.x * QH * 128, ...) of the list (nq in all) against the database tiles of its segments
// (segs + blockIdx.x * seg_stride, nseg[blockIdx.x * (seg_stride != 0)] of them; seg_stride = 0: one list shared by
// all blocks), taking every tile_stride-th tile.  Candidate ids are database list positions; positions from
// nd_pos on are padding and never kept.
// cand_key / cand_id: [nq][cap] candidate buffers.  FIXED = false: threshold maintained online, cap = 32*EPL;
// on return the first L = 16*EPL entries of each are the L best keys in ascending order ((+inf, INT_MAX)
// where the database had fewer points).  FIXED = true: threshold tau[query] fixed, two segments of cap/2
// entries per query; counts[2*query + buffer] receives the number of entries appended to each (bit 30 set
// if it overflowed); knn_tc_pick_kernel finishes.
// RANKED (with FIXED = false): no candidate buffers at all; every query thread keeps its 16 smallest keys in
// registers and rank_out[query] receives the one of rank `rank` (0-based, < 16) when the scan ends: the first
// threshold level, a scan of a few thousand sample points.
template <int EPL, bool FIXED, int QH, bool RANKED = false>
__global__ void __launch_bounds__(tc_threads(QH), 1)
knn_tc_filter_kernel(const float *__restrict__ img_q, const float *__restrict__ img_db, int Dp, long long nq, long long nd_pos,
                     const int2 *__restrict__ segs, const int *__restrict__ nseg, int seg_stride, int tile_stride, int win_lo,
                     int win_hi, const float *__restrict__ tau, int cap, float *cand_key, int32_t *cand_id, int *counts,
                     int *error_flag, int bf16, int sw, int nks, int rank = 0, float *__restrict__ rank_out = nullptr)
{
    static_assert(!(RANKED && FIXED), "the ranked scan keeps its own threshold");
    // bf16: the images hold bf16 pairs; sw != 0: in swizzled rows of sw bytes (else core matrices without swizzle);
    // nks: K steps of 32 operand bytes per row to multiply
    constexpr int C = 32 * EPL;   // capacity handled by one compaction
    constexpr int L = 16 * EPL;
    constexpr int kProducerWarp = 8 * QH, kMmaWarp = 8 * QH + 1;
    constexpr uint32_t kTmemCols = kAccBufs * QH * TN;
    extern __shared__ __align__(1024) unsigned char smem[];   // swizzled images want their 8-row groups on 8 * sw bytes
    __shared__ __align__(8) TcShared sh;
    const uint32_t image_bytes = (uint32_t)Dp * (bf16 ? 512u : 1024u);        // hi + lo
    float *sA = reinterpret_cast<float *>(smem);                          // [QH] images
    float *sB = reinterpret_cast<float *>(smem + QH * image_bytes);       // [kBStages] images
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long qt = (long long)blockIdx.x * QH;   // first query tile of the block
    const int2 *my_segs = segs + (size_t)blockIdx.x * seg_stride;
    const int my_nseg = nseg[seg_stride ? blockIdx.x : 0];
    {   // nothing of this block's segments in the window: leave before any barrier or TMEM is set up
        TileWalk probe(my_segs, my_nseg, tile_stride, win_lo, win_hi);
        int first;
        if (!probe.next(first)) return;
    }
    volatile int *abort_flag = &sh.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&sh.full_a, 1);
        for (int s = 0; s < kBStages; s++) { mbar_init(&sh.full_b[s], 1); mbar_init(&sh.empty_b[s], 1); }
        for (int b = 0; b < kAccBufs; b++) { mbar_init(&sh.acc_full[b], 1); mbar_init(&sh.acc_empty[b], (FIXED ? 8 : 4) * QH); }
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_base;

    if (warp == kProducerWarp) {
        // ---------------- producer: one bulk copy per tile image ----------------
        if (lane == 0) {
            // the images of the block's QH query tiles are adjacent (the image array is padded to a
            // multiple of QH tiles)
            mbar_expect_tx(&sh.full_a, QH * image_bytes);
            for (int h = 0; h < QH; h++)
                bulk_load(sA + (size_t)h * (image_bytes / 4), img_q + (size_t)(qt + h) * (image_bytes / 4), image_bytes, &sh.full_a);
            TileWalk walk(my_segs, my_nseg, tile_stride, win_lo, win_hi);
            int tile;
            for (long long t = 0; walk.next(tile); t++) {
                const int s = (int)(t % kBStages);
                const uint32_t ph = (uint32_t)((t / kBStages) & 1);
                if (!mbar_wait(&sh.empty_b[s], ph ^ 1u, abort_flag)) break;
                mbar_expect_tx(&sh.full_b[s], image_bytes);
                bulk_load(sB + (size_t)s * (image_bytes / 4), img_db + (size_t)tile * (image_bytes / 4), image_bytes, &sh.full_b[s]);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer ----------------
        // One thread issues every MMA, and a thread runs its dependent instructions several cycles apart: what it
        // computes per MMA shows in the kernel's time (descriptors built inside the K loop: 170 cycles per MMA
        // measured, with additions only 125).  tc_issue_walk is instantiated per number of K steps, so that the
        // MMAs of a tile are unrolled, independent instruction sequences.
        if (lane == 0 && mbar_wait(&sh.full_a, 0, abort_flag)) {
            // offset of K step ks inside a part, in 16-byte units: 4 KB blocks without swizzle; with it, sw / 32
            // steps side by side in a row (2 units apart) and blocks of 128 rows
            const uint32_t spr_log = sw == 128 ? 2u : (sw == 64 ? 1u : 0u);
            const uint32_t block16 = sw ? (128u * (uint32_t)sw) >> 4 : 256u, in_row16 = sw ? 2u : 0u;
            const uint32_t span16 = sw ? (127u * (uint32_t)sw + 32u) >> 4 : 256u;
            const uint64_t no_addr = sw ? make_desc_swizzled(0u, (uint32_t)sw) : make_desc(0u);
            const uint32_t a16 = smem_u32(sA) >> 4, b16 = smem_u32(sB) >> 4, image16 = image_bytes >> 4;
            const uint32_t end16 = (smem_u32(smem) + (uint32_t)(QH + kBStages) * image_bytes) >> 4;
            const TileWalk walk(my_segs, my_nseg, tile_stride, win_lo, win_hi);
#define B200_ISSUE(NKS_)                                                                                                        \
    case NKS_:                                                                                                                  \
        if (bf16) tc_issue_walk<QH, true, NKS_>(&sh, abort_flag, walk, tmem_base, no_addr, a16, b16, image16, spr_log, block16,  \
                                                in_row16, span16, end16);                                                       \
        else tc_issue_walk<QH, false, NKS_>(&sh, abort_flag, walk, tmem_base, no_addr, a16, b16, image16, spr_log, block16,      \
                                            in_row16, span16, end16);                                                           \
        break;
            switch (nks) {
                B200_ISSUE(1) B200_ISSUE(2) B200_ISSUE(3) B200_ISSUE(4) B200_ISSUE(5) B200_ISSUE(6) B200_ISSUE(7) B200_ISSUE(8)
                default: sh.abort_flag = 1; break;   // more K steps than a narrow image holds
            }
#undef B200_ISSUE
        }
    } else {
        // ---------------- epilogue: one query per thread ----------------
        // 2 * QH groups of four warps; a warp reaches the TMEM lane quarter (warp % 4).  Group g belongs to
        // query tile g % QH of the block.  With a fixed threshold every group works on every database tile: it
        // takes the 64 accumulator columns buf * 64 ... (buf = g / QH) and appends to segment buf of the query's
        // candidate buffer, so the groups share nothing.  (A warp walks its keys as one dependent chain, about
        // 800 cycles per 32 keys: with all sixteen warps on a tile its epilogue takes half as long as with the
        // groups taking whole tiles in turn, and the accumulator goes back to the MMAs that much earlier.)  With
        // the online threshold (per-query state that cannot be shared) only the groups with buf = 0 work, on
        // all columns of every tile.
        const int group = warp >> 2, quarter = warp & 3;
        const int buf = group / QH, half = group % QH;
        const bool active = FIXED || buf == 0;
        const int seg_cap = FIXED ? cap / kAccBufs : cap;
        const int row = quarter * 32 + lane;                    // TMEM lane
        const long long gq = (qt + half) * TM + row;
        const bool serve = gq < nq && active;
        float *bk = cand_key + (serve ? gq : 0) * cap + (FIXED ? buf * seg_cap : 0);
        int32_t *bi = cand_id + (serve ? gq : 0) * cap + (FIXED ? buf * seg_cap : 0);
        float thr = serve ? (FIXED ? tau[gq] : INFINITY) : -INFINITY;
        // a fixed-threshold scan may be split into several launches (windows of the database): a launch
        // continues the buffers where the previous one stopped (counts are zeroed before the first)
        int cnt = 0;
        bool overflow = false;
        if (FIXED && serve) {
            const int c0 = counts[gq * kAccBufs + buf];
            cnt = c0 & 0x3fffffff;
            overflow = (c0 & 0x40000000) != 0;
            if (overflow) thr = -INFINITY;
        }
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * TN);

        // One chunk = 32 accumulator columns = 32 keys of this thread's query.  Fast path: a tree of
        // independent three-input min operations and one comparison.  Only if the minimum beats the
        // threshold (rare once the scan is under way) are the quarters whose minimum does so compared
        // element by element; everything is indexed statically, so the keys never leave the registers.
        float top[RANKED ? 16 : 1];
#pragma unroll
        for (int i = 0; i < (RANKED ? 16 : 1); i++) top[i] = INFINITY;
        auto process_chunk = [&](const uint32_t (&r)[32], long long col0, bool tile_inside) {
            float m4[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float a = min3(__uint_as_float(r[8 * q]), __uint_as_float(r[8 * q + 1]), __uint_as_float(r[8 * q + 2]));
                const float b = min3(__uint_as_float(r[8 * q + 3]), __uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                const float c = fminf(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                m4[q] = min3(a, b, c);
            }
            const float mn = fminf(min3(m4[0], m4[1], m4[2]), m4[3]);
            if (mn < thr) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    if (m4[q] < thr) {
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            const int c = q * 8 + e;
                            const float key = __uint_as_float(r[c]);
                            const long long cid = col0 + c;
                            const bool pass = key < thr && (tile_inside || cid < nd_pos);
                            if constexpr (RANKED) {
                                if (pass) {   // replaces the largest of the 16 and sinks to its place
                                    top[15] = key;
#pragma unroll
                                    for (int i = 15; i > 0; i--) {
                                        const float lo = fminf(top[i - 1], top[i]), hi = fmaxf(top[i - 1], top[i]);
                                        top[i - 1] = lo;
                                        top[i] = hi;
                                    }
                                    thr = top[15];
                                }
                            } else if (pass) {
                                __stcg(bk + cnt, key);
                                __stcg(bi + cnt, (int32_t)cid);
                                cnt++;
                            }
                        }
                    }
                }
            }
            if constexpr (RANKED) {
                // nothing is buffered
            } else if (FIXED) {
                // a chunk appends at most 32 entries: stop a buffer that could overflow in the next one
                if (cnt > seg_cap - 32) { overflow = true; thr = -INFINITY; }
            } else {
                // a chunk appends at most 32 entries: compact every buffer that could overflow in the next one
                unsigned full = __ballot_sync(0xffffffffu, cnt > C - 32);
                while (full) {
                    const int owner = __ffs(full) - 1;
                    full &= full - 1;
                    const long long oq = (qt + half) * TM + quarter * 32 + owner;
                    const int n = __shfl_sync(0xffffffffu, cnt, owner);
                    const float nt = warp_compact<EPL>(cand_key + oq * cap, cand_id + oq * cap, n, lane);
                    if (lane == owner) { thr = nt; cnt = L; }
                }
            }
        };

        TileWalk walk(my_segs, active ? my_nseg : 0, tile_stride, win_lo, win_hi);
        int tile;
        for (long long t = 0; walk.next(tile); t++) {
            const int b = (int)(t % kAccBufs);
            const uint32_t ph_b = (uint32_t)((t / kAccBufs) & 1);
            if (!mbar_wait(&sh.acc_full[b], ph_b, abort_flag, 32)) break;
            tc_fence_after();
            const long long p0 = (long long)tile * TN;
            const bool inside = p0 + TN <= nd_pos;
            const uint32_t tcol = lane_base + (uint32_t)(b * QH * TN);
            // one copy of the chunk code, executed once per 32 columns: small code beats overlapping the TMEM reads
            // (16 keys per read with the next read in flight while these are compared was 4 % slower)
            const int c_lo = FIXED ? buf * (TN / 2) : 0, c_hi = FIXED ? c_lo + TN / 2 : TN;   // this group's columns
#pragma unroll 1
            for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
                uint32_t r[32];
                tc_ld32_issue(tcol + (uint32_t)c0, r);
                tc_ld32_wait(r);
                if (c0 == c_hi - 32) {   // the last read has landed: hand the accumulator buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh.acc_empty[b]);
                }
                process_chunk(r, p0 + c0, inside);
            }
        }
        if (FIXED) {
            // The final selection is a separate kernel (one warp per query, thousands in flight): it is a chain of
            // dependent global round trips, which the warps of this block would walk through one query at a time.
            if (serve) counts[gq * kAccBufs + buf] = cnt | (overflow ? 0x40000000 : 0);
        } else if (RANKED) {
            if (serve) {
                float t = top[0];
#pragma unroll
                for (int i = 1; i < (RANKED ? 16 : 1); i++) t = (i == rank) ? top[i] : t;
                rank_out[gq] = t;
            }
        } else if (active) {
            // online threshold (small databases): one last compaction leaves the L best, sorted, in front
            unsigned m = __ballot_sync(0xffffffffu, serve);
            while (m) {
                const int owner = __ffs(m) - 1;
                m &= m - 1;
                const long long oq = (qt + half) * TM + quarter * 32 + owner;
                const int n = __shfl_sync(0xffffffffu, cnt, owner);
                (void)warp_compact<EPL>(cand_key + oq * cap, cand_id + oq * cap, min(n, C), lane);
            }
        }
    }
    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0 && sh.abort_flag) atomicExch(error_flag, 1);
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// filter kernel for wide points (D + 1 > 64): the inner dimension no longer fits in shared memory at once
// ------------------------------------------------------------------------------------------------
// A block multiplies two query tiles with two database tiles (a "unit" of 256 database rows) at a time,
// walking the inner dimension in chunks of kWideKC: a stage holds the chunk images of the four tiles
// (4 x 24 KB), two stages alternate, the four 128 x 128 accumulators fill the 512 TMEM columns.  Operand
// bytes per MMA are those of the narrow kernel with two query tiles, but the query images are streamed
// again for every unit, so the kernel leans on L2 bandwidth (24 KB per tile pair and chunk).  After the
// last chunk of a unit the sixteen epilogue warps (query tile x database tile x TMEM lane quarter) compare
// the keys with the fixed thresholds exactly as in the narrow kernel; the next unit's MMAs wait until the
// accumulators have been read.  Fixed thresholds only (a small database goes to the SIMT search).
constexpr int kWideKC = 24;                       // inner dimensions per chunk = 3 MMA K steps
constexpr uint32_t kWideChunkBytes = kWideKC * 1024;   // hi + lo of one tile and chunk
constexpr int kWideStages = 2;
constexpr int kWideUnit = 2 * TN;                 // database rows per unit

struct WideShared {
    uint64_t full[kWideStages];
    uint64_t empty[kWideStages];
    uint64_t acc_full;
    uint64_t acc_empty;
    uint32_t tmem_base;
    int abort_flag;
};

// RANKED: the first threshold level (see the narrow kernel): no buffers, the warps of the unit's first database tile
// read both tiles and keep the 16 smallest keys of their queries in registers; positions from n_pos on are padding.
template <int EPL, bool RANKED = false>
__global__ void __launch_bounds__(tc_threads(2), 1)
knn_tc_wide_kernel(const float *__restrict__ img_q, const float *__restrict__ img_db, int n_chunks, long long nq,
                   const int2 *__restrict__ segs, const int *__restrict__ nseg, int seg_stride, int unit_stride, int win_lo,
                   int win_hi, const float *__restrict__ tau, int cap, float *cand_key, int32_t *cand_id, int *counts,
                   int *error_flag, int bf16, int rank = 0, float *__restrict__ rank_out = nullptr, long long n_pos = 0)
{
    constexpr int kProducerWarp = 16, kMmaWarp = 17;
    constexpr uint32_t kTmemCols = 512;
    constexpr int kSteps = kWideKC / 8;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ __align__(8) WideShared sh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long qt = (long long)blockIdx.x * 2;   // first query tile of the block
    const int2 *my_segs = segs + (size_t)blockIdx.x * seg_stride;
    const int my_nseg = nseg[seg_stride ? blockIdx.x : 0];
    {   // nothing of this block's segments in the window
        TileWalk probe(my_segs, my_nseg, unit_stride, win_lo, win_hi);
        int first;
        if (!probe.next(first)) return;
    }
    volatile int *abort_flag = &sh.abort_flag;
    const size_t tile_floats = (size_t)n_chunks * (kWideChunkBytes / 4);   // one tile's image, all chunks
    // stage layout: [A0 chunk][A1 chunk][B0 chunk][B1 chunk], each hi then lo
    auto stage_ptr = [&](int s, int which) { return smem + ((size_t)s * 4 + which) * kWideChunkBytes; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWideStages; s++) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        mbar_init(&sh.acc_full, 1);
        mbar_init(&sh.acc_empty, RANKED ? 8 : 16);
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh.tmem_base;

    if (warp == kProducerWarp) {
        if (lane == 0) {
            TileWalk walk(my_segs, my_nseg, unit_stride, win_lo, win_hi);
            int unit;
            long long it = 0;   // stage counter over (unit, chunk)
            bool ok = true;
            while (ok && walk.next(unit)) {
                for (int c = 0; c < n_chunks; c++, it++) {
                    const int s = (int)(it % kWideStages);
                    const uint32_t ph = (uint32_t)((it / kWideStages) & 1);
                    if (!mbar_wait(&sh.empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(&sh.full[s], 4 * kWideChunkBytes);
                    const size_t coff = (size_t)c * (kWideChunkBytes / 4);
                    bulk_load(stage_ptr(s, 0), img_q + (size_t)qt * tile_floats + coff, kWideChunkBytes, &sh.full[s]);
                    bulk_load(stage_ptr(s, 1), img_q + (size_t)(qt + 1) * tile_floats + coff, kWideChunkBytes, &sh.full[s]);
                    bulk_load(stage_ptr(s, 2), img_db + (size_t)(2 * (long long)unit) * tile_floats + coff, kWideChunkBytes, &sh.full[s]);
                    bulk_load(stage_ptr(s, 3), img_db + (size_t)(2 * (long long)unit + 1) * tile_floats + coff, kWideChunkBytes,
                              &sh.full[s]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            TileWalk walk(my_segs, my_nseg, unit_stride, win_lo, win_hi);
            int unit;
            long long it = 0, n_unit = 0;
            bool ok = true;
            const uint64_t no_addr = make_desc(0u);
            const uint32_t stage16 = smem_u32(smem) >> 4, chunk16 = kWideChunkBytes >> 4;
            while (ok && walk.next(unit)) {
                // the accumulators of the previous unit must have been read
                if (!mbar_wait(&sh.acc_empty, (uint32_t)((n_unit & 1) ^ 1), abort_flag)) break;
                for (int c = 0; c < n_chunks; c++, it++) {
                    const int s = (int)(it % kWideStages);
                    const uint32_t ph = (uint32_t)((it / kWideStages) & 1);
                    if (!mbar_wait(&sh.full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    // descriptors by addition only (see the narrow kernel's issuer); a stage's four chunk images
                    // are kWideChunkBytes apart, lo follows hi after kSteps blocks of 4 KB
                    const uint64_t st0 = no_addr + (uint64_t)(stage16 + (uint32_t)s * 4u * chunk16);
#pragma unroll
                    for (int pair = 0; pair < 4; pair++) {
                        const int h = pair >> 1, g = pair & 1;
                        const uint64_t a_hi = st0 + (uint64_t)((uint32_t)h * chunk16), a_lo = a_hi + kSteps * 256u;
                        const uint64_t b_hi = st0 + (uint64_t)((uint32_t)(2 + g) * chunk16), b_lo = b_hi + kSteps * 256u;
                        const uint32_t d_tmem = tmem_base + (uint32_t)((h * 2 + g) * TN);
                        const uint32_t acc0 = (c > 0) ? 1u : 0u;
                        if (bf16) {
#pragma unroll
                            for (int ks = 0; ks < kSteps; ks++)        // hi . hi
                                tc_mma_bf16(d_tmem, a_hi + ks * 256u, b_hi + ks * 256u, kInstrDescBf16, ks ? 1u : acc0);
#pragma unroll
                            for (int ks = 0; ks < kSteps; ks++)        // lo . hi
                                tc_mma_bf16(d_tmem, a_lo + ks * 256u, b_hi + ks * 256u, kInstrDescBf16, 1u);
#pragma unroll
                            for (int ks = 0; ks < kSteps; ks++)        // hi . lo
                                tc_mma_bf16(d_tmem, a_hi + ks * 256u, b_lo + ks * 256u, kInstrDescBf16, 1u);
                        } else {
#pragma unroll
                            for (int ks = 0; ks < kSteps; ks++)        // hi . hi
                                tc_mma_tf32(d_tmem, a_hi + ks * 256u, b_hi + ks * 256u, kInstrDesc, ks ? 1u : acc0);
#pragma unroll
                            for (int ks = 0; ks < kSteps; ks++)        // lo . hi
                                tc_mma_tf32(d_tmem, a_lo + ks * 256u, b_hi + ks * 256u, kInstrDesc, 1u);
#pragma unroll
                            for (int ks = 0; ks < kSteps; ks++)        // hi . lo
                                tc_mma_tf32(d_tmem, a_hi + ks * 256u, b_lo + ks * 256u, kInstrDesc, 1u);
                        }
                    }
                    tc_commit(&sh.empty[s]);
                }
                if (ok) tc_commit(&sh.acc_full);
                n_unit++;
            }
        }
    } else {
        // ---------------- epilogue: one query per thread, one database tile of the unit per warp group ----------------
        const int quarter = warp & 3, half = (warp >> 2) & 1, g = warp >> 3;
        const int seg_cap = cap / 2;
        const int row = quarter * 32 + lane;
        const long long gq = (qt + half) * TM + row;
        const bool active = !RANKED || g == 0;
        const bool serve = gq < nq && active;
        float *bk = cand_key + (serve ? gq : 0) * cap + g * seg_cap;
        int32_t *bi = cand_id + (serve ? gq : 0) * cap + g * seg_cap;
        float thr = serve ? (RANKED ? INFINITY : tau[gq]) : -INFINITY;
        int cnt = 0;
        bool overflow = false;
        if (!RANKED && serve) {
            const int c0 = counts[gq * 2 + g];
            cnt = c0 & 0x3fffffff;
            overflow = (c0 & 0x40000000) != 0;
            if (overflow) thr = -INFINITY;
        }
        float top[RANKED ? 16 : 1];
#pragma unroll
        for (int i = 0; i < (RANKED ? 16 : 1); i++) top[i] = INFINITY;
        // 32 keys of this thread's query: positions pos0 ...
        auto process_chunk = [&](const uint32_t (&r)[32], long long pos0) {
            float m4[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float a = min3(__uint_as_float(r[8 * q]), __uint_as_float(r[8 * q + 1]), __uint_as_float(r[8 * q + 2]));
                const float b = min3(__uint_as_float(r[8 * q + 3]), __uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                const float c = fminf(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                m4[q] = min3(a, b, c);
            }
            const float mn = fminf(min3(m4[0], m4[1], m4[2]), m4[3]);
            if (mn < thr) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    if (m4[q] < thr) {
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            const int c = q * 8 + e;
                            const float key = __uint_as_float(r[c]);
                            if constexpr (RANKED) {
                                if (key < thr && pos0 + c < n_pos) {   // replaces the largest of the 16 and sinks to its place
                                    top[15] = key;
#pragma unroll
                                    for (int i = 15; i > 0; i--) {
                                        const float lo = fminf(top[i - 1], top[i]), hi = fmaxf(top[i - 1], top[i]);
                                        top[i - 1] = lo;
                                        top[i] = hi;
                                    }
                                    thr = top[15];
                                }
                            } else if (key < thr) {   // padding rows carry a huge norm and never pass a finite threshold
                                __stcg(bk + cnt, key);
                                __stcg(bi + cnt, (int32_t)(pos0 + c));
                                cnt++;
                            }
                        }
                    }
                }
            }
            if (!RANKED && cnt > seg_cap - 32) { overflow = true; thr = -INFINITY; }
        };
        const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        TileWalk walk(my_segs, active ? my_nseg : 0, unit_stride, win_lo, win_hi);
        int unit;
        for (long long n_unit = 0; walk.next(unit); n_unit++) {
            if (!mbar_wait(&sh.acc_full, (uint32_t)(n_unit & 1), abort_flag, 32)) break;
            tc_fence_after();
            // this warp's database tiles of the unit: its own, or both when ranked
#pragma unroll 1
            for (int gg = RANKED ? 0 : g; gg <= (RANKED ? 1 : g); gg++) {
                const uint32_t tcol = tlane + (uint32_t)((half * 2 + gg) * TN);
                const long long p0 = (long long)unit * kWideUnit + (long long)gg * TN;
#pragma unroll 1
                for (int c0 = 0; c0 < TN; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32_issue(tcol + (uint32_t)c0, r);
                    tc_ld32_wait(r);
                    if (c0 == TN - 32 && gg == (RANKED ? 1 : g)) {   // the last read has landed: hand the accumulators back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh.acc_empty);
                    }
                    process_chunk(r, p0 + c0);
                }
            }
        }
        if constexpr (RANKED) {
            if (serve) {
                float t = top[0];
#pragma unroll
                for (int i = 1; i < 16; i++) t = (i == rank) ? top[i] : t;
                rank_out[gq] = t;
            }
        } else {
            if (serve) counts[gq * 2 + g] = cnt | (overflow ? 0x40000000 : 0);
        }
    }
    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0 && sh.abort_flag) atomicExch(error_flag, 1);
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// final selection after a fixed-threshold scan: one warp per query
// ------------------------------------------------------------------------------------------------
// Buffer of query q: two segments of cap/2 entries with counts[2q], counts[2q+1] valid entries (bit 30 of a
// count: the segment overflowed, i.e. keys below tau were lost).
// The k smallest keys of the buffer by selection rather than sorting (a warp-wide bitonic sort of the buffer
// was measured at ~17 000 issue slots per query, this takes ~1 500).  The warp holds the keys in
// registers as order-preserving integers, finds the k-th smallest value v by bisection on the 32 bits (each
// step counts the keys <= mid), keeps every key below v and as many of the keys equal to v as are needed.
// kth[q] (optional) = v, or -inf when the buffer lost keys or holds fewer than k; out_* (optional) receive
// the k kept pairs in buffer order, padded with (+inf, INT_MAX); row_flags[q]: bit 0 = a segment overflowed,
// bit 1 = fewer than k candidates.
template <int SLOTS>
__global__ void __launch_bounds__(128)
knn_tc_pick_kernel(const float *__restrict__ cand_key, const int32_t *__restrict__ cand_id, int cap, const int *__restrict__ counts,
                   long long nq, int k, float *__restrict__ out_key, int32_t *__restrict__ out_id, int out_stride,
                   float *__restrict__ kth, int *__restrict__ row_flags)
{
    const int lane = threadIdx.x & 31;
    const long long q = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (q >= nq) return;
    const int c0 = counts[2 * q], c1 = counts[2 * q + 1];
    const bool ovf = ((c0 | c1) & 0x40000000) != 0;
    const int n0 = c0 & 0x3fffffff, n1 = c1 & 0x3fffffff, n = n0 + n1;
    const int jmax = (n + 31) / 32;
    const float *bk = cand_key + q * cap;
    const int32_t *bi = cand_id + q * cap;
    unsigned int enc[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; j++) {
        const int e = lane + 32 * j;
        enc[j] = 0xffffffffu;
        if (e < n) enc[j] = enc_float(__ldcg(bk + (e < n0 ? e : cap / 2 + (e - n0))));
    }
    unsigned int v = 0xffffffffu;   // with fewer than k keys everything is kept
    if (n > k) {
        // bisection between the smallest and the largest key of the buffer: they share their leading bits, so about
        // half of the 32 steps of a search over all encodings are enough
        unsigned int lo = 0xffffffffu, hi = 0u;
#pragma unroll
        for (int j = 0; j < SLOTS; j++) {
            if (j >= jmax) break;
            if (lane + 32 * j < n) { lo = min(lo, enc[j]); hi = max(hi, enc[j]); }
        }
        lo = __reduce_min_sync(0xffffffffu, lo);
        hi = __reduce_max_sync(0xffffffffu, hi);
#pragma unroll 1
        for (int it = 0; it < 32 && lo < hi; it++) {
            const unsigned int mid = lo + ((hi - lo) >> 1);
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < SLOTS; j++) {
                if (j >= jmax) break;
                cnt += (enc[j] <= mid) ? 1 : 0;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
            if (cnt >= k) hi = mid;
            else lo = mid + 1;
        }
        v = lo;
    }
    const bool short_list = n < k;
    if (kth && lane == 0) kth[q] = (ovf || short_list) ? -INFINITY : dec_float(v);
    if (lane == 0) row_flags[q] = (ovf ? 1 : 0) | (short_list ? 2 : 0);
    if (!out_key) return;
    // keys below v, then as many keys equal to v as fit
    int below = 0;
#pragma unroll
    for (int j = 0; j < SLOTS; j++) {
        if (j >= jmax) break;
        below += (enc[j] < v) ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) below += __shfl_xor_sync(0xffffffffu, below, o);
    int room_eq = min(k, n) - below;     // keys equal to v still to take (n <= k: v is above every key, all are "below")
    int out_pos = 0;
    float *ok = out_key + q * out_stride;
    int32_t *oi = out_id + q * out_stride;
    const unsigned int lt = (1u << lane) - 1u;
#pragma unroll
    for (int j = 0; j < SLOTS; j++) {
        if (j >= jmax) break;
        const int e = lane + 32 * j;
        const bool is_eq = enc[j] == v && e < n;
        const unsigned int eqmask = __ballot_sync(0xffffffffu, is_eq);
        const bool keep = (e < n) && (enc[j] < v || (is_eq && __popc(eqmask & lt) < room_eq));
        const unsigned int keepmask = __ballot_sync(0xffffffffu, keep);
        if (keep) {
            const int slot = e < n0 ? e : cap / 2 + (e - n0);
            ok[out_pos + __popc(keepmask & lt)] = dec_float(enc[j]);
            oi[out_pos + __popc(keepmask & lt)] = __ldcg(bi + slot);
        }
        out_pos += __popc(keepmask);
        room_eq -= min(room_eq, __popc(eqmask));
    }
    for (int e = out_pos + lane; e < k; e += 32) { ok[e] = INFINITY; oi[e] = INT_MAX; }
}

// Xp[pos] = X[list[pos]] (zeros for padding): the database rows in visiting order.  The re-rank reads ~130 candidate
// rows per query; in cell order the candidates of neighbouring queries share a few megabytes that stay in L2,
// in the original order they are 200-byte reads scattered over the whole array.
__global__ void knn_gather_rows_kernel(const float *__restrict__ X, const int *__restrict__ list, int D, long long n_pos,
                                       float *__restrict__ Xp)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_pos * D) return;
    const long long pos = t / D;
    const int i = list[pos];
    Xp[t] = (i >= 0) ? X[(long long)i * D + (t - pos * D)] : 0.0f;
}

// ------------------------------------------------------------------------------------------------
// exact re-rank + proof
// ------------------------------------------------------------------------------------------------
// The canonical distance: differences, squares and the running sum rounded one by one, in the order of the
// dimensions.  Rows are read 16 or 8 bytes at a time where D keeps them aligned (a lane reads a row of its own,
// so wide loads mean fewer sectors touched per instruction); the arithmetic and its order do not change.
__device__ __forceinline__ float canon_step(float acc, float x, float y)
{
    const float t = __fsub_rn(x, y);
    return __fadd_rn(acc, __fmul_rn(t, t));
}
__device__ __forceinline__ float canon_dist(const float *__restrict__ a, const float *__restrict__ b, int D)
{
    float acc = 0.0f;
    const unsigned long long both = (unsigned long long)(size_t)a | (unsigned long long)(size_t)b;
    if ((D & 3) == 0 && (both & 15) == 0) {
        const float4 *a4 = reinterpret_cast<const float4 *>(a), *b4 = reinterpret_cast<const float4 *>(b);
        for (int d = 0; d < (D >> 2); d++) {
            const float4 u = a4[d], v = b4[d];
            acc = canon_step(acc, u.x, v.x);
            acc = canon_step(acc, u.y, v.y);
            acc = canon_step(acc, u.z, v.z);
            acc = canon_step(acc, u.w, v.w);
        }
    } else if ((D & 1) == 0 && (both & 7) == 0) {
        const float2 *a2 = reinterpret_cast<const float2 *>(a), *b2 = reinterpret_cast<const float2 *>(b);
        for (int d = 0; d < (D >> 1); d++) {
            const float2 u = a2[d], v = b2[d];
            acc = canon_step(acc, u.x, v.x);
            acc = canon_step(acc, u.y, v.y);
        }
    } else {
        for (int d = 0; d < D; d++) acc = canon_step(acc, a[d], b[d]);
    }
    return acc;
}

constexpr int kRerankWarps = 4;
constexpr int kMaxL = 256;

// One warp per query of the list (query row qlist[q]; candidate ids are positions in dblist).  Row
// (qlist[q] - out_base) of ids/d2 ([.][K]) receives the K best candidates by (canonical distance, row id);
// failed[q] = 1 when the proof does not close for the query.
__global__ void __launch_bounds__(kRerankWarps * 32)
knn_tc_rerank_kernel(const float *__restrict__ X, int D, const int *__restrict__ qlist, const int *__restrict__ dblist,
                     long long out_base, long long nq, const float *__restrict__ cand_key,
                     const int32_t *__restrict__ cand_id, int L, int C, int K, const double *__restrict__ norms_exact,
                     float err_scale, const float2 *__restrict__ res_q, const float *__restrict__ rho, const int *__restrict__ row_flags,
                     int32_t *__restrict__ ids, float *__restrict__ d2,
                     int *__restrict__ failed,
                     int *__restrict__ n_failed, float *__restrict__ max_err_ratio, const float *__restrict__ Xp)
{
    // Xp (optional): the database rows in list order, Xp[pos] = X[dblist[pos]]
    __shared__ float s_d[kRerankWarps][kMaxL];
    __shared__ int s_i[kRerankWarps][kMaxL];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long q = (long long)blockIdx.x * kRerankWarps + w;
    if (q >= nq) return;
    const long long gq = qlist[q];
    const long long orow = gq - out_base;
    const float *xq = X + gq * D;
    const double ni = norms_exact[q];
    float worst = 0.0f;   // largest observed |filter distance - canonical distance| among the candidates
    float T = -INFINITY;
    int n_valid = 0;
    for (int e = lane; e < L; e += 32) {
        const int pos = cand_id[q * C + e];
        int id = (pos != INT_MAX) ? dblist[pos] : INT_MAX;
        if (id < 0) id = INT_MAX;   // a padding position (never kept by a finite threshold)
        const float key = cand_key[q * C + e];
        float dist = INFINITY;
        if (id != INT_MAX) {
            dist = canon_dist(xq, Xp ? Xp + (long long)pos * D : X + (long long)id * D, D);
            n_valid++;
            T = fmaxf(T, key);
            const double approx = ni + (double)key;
            worst = fmaxf(worst, (float)fabs(approx - (double)dist));
        }
        s_d[w][e] = dist;
        s_i[w][e] = id;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        worst = fmaxf(worst, __shfl_xor_sync(0xffffffffu, worst, o));
        T = fmaxf(T, __shfl_xor_sync(0xffffffffu, T, o));
        n_valid += __shfl_xor_sync(0xffffffffu, n_valid, o);
    }
    __syncwarp();
    // rank by counting (ties by id), scatter the first K
    float dK = INFINITY;
    for (int e = lane; e < L; e += 32) {
        const float de = s_d[w][e];
        const int ie = s_i[w][e];
        int rank = 0;
        for (int u = 0; u < L; u++) {
            const float du = s_d[w][u];
            const int iu = s_i[w][u];
            rank += (du < de || (du == de && iu < ie)) ? 1 : 0;
        }
        if (rank < K) {
            ids[orow * K + rank] = (ie == INT_MAX) ? -1 : ie;
            d2[orow * K + rank] = de;
        }
        if (rank == K - 1) dK = de;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dK = fminf(dK, __shfl_xor_sync(0xffffffffu, dK, o));
    if (lane == 0) {
        bool ok = true;
        // Error bound of the filter's key for this row: it scales with |x_i||x_j|, and a point whose key is
        // near T lies within sqrt(|x_i|^2 + T) of x_i, so |x_i||x_j| <= |x_i|^2 + (|x_i|^2 + T)+ up to a factor 2.
        double E = (double)err_scale * (ni + fmax(0.0, ni + (double)T) + 1.0);
        double dropped = 0.0;
        if (res_q) {
            // bf16 pairs: what the three products drop, bounded from the leftovers of this query and the largest
            // relative leftovers of the database, for every point with |x_j| <= |x_i| + sqrt(|x_i|^2 + T) (a point
            // further out cannot come closer than the threshold whatever the error of its key); the last term is
            // the fp32 rounding of the norm column.  err_scale then covers the accumulation only.
            const double xi = sqrt(ni), xj = xi + sqrt(fmax(0.0, ni + (double)T));
            const float2 rq = res_q[q];
            dropped = 1.001 * 2.0 * xj * ((double)rq.x * (double)rho[0] + xi * (double)rho[1] + (double)rq.y) + 1.2e-7 * xj * xj;
            E += dropped;
        }
        if (n_valid == L) {
            // outsiders: key >= T  =>  canonical distance >= (ni + T - E) * (1 - theta)
            const double theta = (double)(D + 4) * 5.9604644775390625e-08;   // (D+4) * 2^-24
            const double bound = (ni + (double)T - E) * (1.0 - theta);
            ok = (double)dK < bound;
        }
        const float ratio = (float)(fmax(0.0, (double)worst - dropped) / (E - dropped));
        if (ratio > 0.5f) ok = false;   // the filter was less accurate than the bound assumes
        if (row_flags && row_flags[q]) ok = false;   // the fixed threshold kept too few or too many candidates
        failed[q] = ok ? 0 : 1;
        if (!ok) atomicAdd(n_failed, 1);
        atomicMax(reinterpret_cast<int *>(max_err_ratio), __float_as_int(ratio));   // ratio >= 0: int order == float order
    }
}

// First threshold level on the CUDA cores: tau[q] = the key of rank `rank` (0-based, < 16) among m sample
// points X[s_lo + k * s_stride + jitter_k], k = 0..m-1, for each of the nq queries of the list.  Keys are
// plain fp32 FMA sums: this threshold only has to be roughly right (it sizes the candidate set of the
// next level).  One query per thread, held in registers; sample points staged 32 at a time in shared
// memory and read as broadcast float4.
// The sample of the first threshold level as a list of rows: position k < m holds the jittered systematic sample
// point s_lo + k * s_stride + jitter_k (a plain stride would alias with any periodic ordering of the data), the
// positions from m on are padding.
__global__ void knn_sample_list_kernel(int *__restrict__ list, long long n_pos, int m, long long s_lo, long long s_stride)
{
    const long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n_pos) return;
    list[k] = (k < m) ? (int)(s_lo + k * s_stride + (long long)(((unsigned long long)k * 2654435761ull) % (unsigned long long)s_stride)) : -1;
}

constexpr int kTauThreads = 128;
__global__ void __launch_bounds__(kTauThreads)
knn_sample_tau_kernel(const float *__restrict__ X, int D, const int *__restrict__ qlist, long long nq, long long s_lo, long long s_stride,
                      int m, int rank, float *__restrict__ tau)
{
    __shared__ __align__(16) float s_pt[32][64];
    __shared__ float s_nrm[32];
    const long long q = (long long)blockIdx.x * kTauThreads + threadIdx.x;
    const long long qrow = (q < nq) ? qlist[q] : 0;
    float4 qv[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int d = 4 * i + e;
            v[e] = (q < nq && d < D) ? X[qrow * D + d] : 0.0f;
        }
        qv[i] = make_float4(v[0], v[1], v[2], v[3]);
    }
    float top[16];
#pragma unroll
    for (int i = 0; i < 16; i++) top[i] = INFINITY;
    for (int k0 = 0; k0 < m; k0 += 32) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < 32 * 64; idx += kTauThreads) {
            const int p = idx >> 6, d = idx & 63;
            // jittered systematic sample: a plain stride would alias with any periodic ordering of the data
            const long long k = k0 + p;
            const long long j = s_lo + k * s_stride + (long long)(((unsigned long long)k * 2654435761ull) % (unsigned long long)s_stride);
            s_pt[p][d] = (k < m && d < D) ? X[j * D + d] : 0.0f;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            float n2 = 0.0f;
            for (int d = 0; d < 64; d++) n2 += s_pt[threadIdx.x][d] * s_pt[threadIdx.x][d];
            s_nrm[threadIdx.x] = (k0 + threadIdx.x < m) ? n2 : INFINITY;
        }
        __syncthreads();
        for (int p = 0; p < 32; p++) {
            const float4 *sp = reinterpret_cast<const float4 *>(s_pt[p]);
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const float4 a = sp[i];
                dot += qv[i].x * a.x + qv[i].y * a.y + qv[i].z * a.z + qv[i].w * a.w;
            }
            const float key = fmaf(-2.0f, dot, s_nrm[p]);
            if (key < top[15]) {
                top[15] = key;
#pragma unroll
                for (int i = 15; i > 0; i--) {
                    const float lo = fminf(top[i - 1], top[i]), hi = fmaxf(top[i - 1], top[i]);
                    top[i - 1] = lo;
                    top[i] = hi;
                }
            }
        }
    }
    if (q < nq) {
        float t = top[0];
#pragma unroll
        for (int i = 1; i < 16; i++) t = (i == rank) ? top[i] : t;
        tau[q] = t;
    }
}

// The same for points of any width: the inner dimension is walked in chunks of 64, the dot products with
// the 32 staged sample points are kept in registers across the chunks.
__global__ void __launch_bounds__(kTauThreads)
knn_sample_tau_wide_kernel(const float *__restrict__ X, int D, const int *__restrict__ qlist, long long nq, long long s_lo,
                           long long s_stride, int m, int rank, float *__restrict__ tau)
{
    __shared__ float s_pt[32][65];
    __shared__ float s_nrm[32];
    const long long q = (long long)blockIdx.x * kTauThreads + threadIdx.x;
    const long long qrow = (q < nq) ? qlist[q] : 0;
    float top[16];
#pragma unroll
    for (int i = 0; i < 16; i++) top[i] = INFINITY;
    for (int k0 = 0; k0 < m; k0 += 32) {
        float dot[32];
#pragma unroll
        for (int p = 0; p < 32; p++) dot[p] = 0.0f;
        float n2 = 0.0f;
        for (int d0 = 0; d0 < D; d0 += 64) {
            __syncthreads();
            for (int idx = threadIdx.x; idx < 32 * 64; idx += kTauThreads) {
                const int p = idx >> 6, d = idx & 63;
                const long long k = k0 + p;
                const long long j = s_lo + k * s_stride + (long long)(((unsigned long long)k * 2654435761ull) % (unsigned long long)s_stride);
                s_pt[p][d] = (k < m && d0 + d < D) ? X[j * D + d0 + d] : 0.0f;
            }
            __syncthreads();
            float qv[64];
#pragma unroll
            for (int d = 0; d < 64; d++) qv[d] = (q < nq && d0 + d < D) ? X[qrow * D + d0 + d] : 0.0f;
#pragma unroll
            for (int p = 0; p < 32; p++) {   // fully unrolled: dot[] stays in registers
                float acc = 0.0f;
#pragma unroll
                for (int d = 0; d < 64; d++) acc = fmaf(qv[d], s_pt[p][d], acc);
                dot[p] += acc;
            }
            if (threadIdx.x < 32)
                for (int d = 0; d < 64; d++) n2 = fmaf(s_pt[threadIdx.x][d], s_pt[threadIdx.x][d], n2);
        }
        __syncthreads();
        if (threadIdx.x < 32) s_nrm[threadIdx.x] = (k0 + threadIdx.x < m) ? n2 : INFINITY;
        __syncthreads();
#pragma unroll
        for (int p = 0; p < 32; p++) {
            const float key = fmaf(-2.0f, dot[p], s_nrm[p]);
            if (key < top[15]) {
                top[15] = key;
#pragma unroll
                for (int i = 15; i > 0; i--) {
                    const float lo = fminf(top[i - 1], top[i]), hi = fmaxf(top[i - 1], top[i]);
                    top[i - 1] = lo;
                    top[i] = hi;
                }
            }
        }
    }
    if (q < nq) {
        float t = top[0];
#pragma unroll
        for (int i = 1; i < 16; i++) t = (i == rank) ? top[i] : t;
        tau[q] = t;
    }
}

__global__ void knn_tc_collect_failed_kernel(const int *__restrict__ failed, long long nq, const int *__restrict__ qlist, int *__restrict__ list,
                                             int *__restrict__ count)
{
    const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (q < nq && failed[q]) list[atomicAdd(count, 1)] = qlist[q];
}


// Exercises mbar_wait's limit: a barrier that expects one arrival and never gets it.  Every thread of the
// block must come back with `false` after limit_ns and the block must exit normally.
__global__ void mbar_wait_selftest_kernel(int *abort_flag, int *gave_up, unsigned long long limit_ns)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait(&bar, 0, abort_flag, 128, limit_ns);
    if (!ok) atomicAdd(gave_up, 1);
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
}
}  // namespace

// wide points: the inner dimension (D + 1) does not fit the narrow kernel's shared-memory images
static bool tc_wide(int D) { return D + 1 > 64; }
// Operand form of the filter: bf16 pairs (three bf16 products per key, half the tensor-core time of 3xTF32, error
// 3 * 2^-16 of sum |x_ik||2 x_jk|) unless B200TSNE_KNN_FILTER=tf32 asks for the TF32 pairs (error ~2^-20).
static bool tc_bf16()
{
    const char *e = getenv("B200TSNE_KNN_FILTER");
    return !(e && strcmp(e, "tf32") == 0);
}
constexpr long long kWideMinRows = 16384;   // the wide kernel has fixed thresholds only: it needs a database to sample

// nd: database rows the search will scan
bool knn_tc_supported(int64_t nd, int D, int K)
{
    if (K + 32 > kMaxL || D > 8192) return false;
    if (tc_wide(D)) return nd >= kWideMinRows;
    return nd >= 2048;   // below this the SIMT search is faster than the set-up of this one
}

// candidate buffer entries per query in a fixed-threshold pass: 8 L (two halves of 4 L for ~1.5 L expected each)
static int fixed_cap(int K) { return (K + 32 <= 128) ? 1024 : 2048; }
constexpr int kSampleStride = 16;    // the sample pass looks at every 16th database tile
constexpr int kMaxSampleTiles = 128; // first threshold level: at most 16 384 sample points
constexpr long long kTwoPassMinTiles = 512;   // below this many database tiles the online pass alone is used

// Device workspace of launch_knn_tc, carved in this order.
struct TcWorkspace {
    bool wide, bf16;
    size_t image_bytes;        // one tile's image (hi and lo)
    int Dp, cells;
    int sw, nks;               // narrow kernel: bytes of a swizzled image row (0: core matrices without swizzle), K steps
    long long tq, td;          // tiles allocated for the query list / the database list
    float *img_q, *img_db;
    double *norms_q;
    float2 *res_q;             // bf16 form: norms of the lo parts and of the leftovers of every query
    float *img_s;              // images of the sample of the first threshold level (two-pass searches)
    int *slist;
    int *qlist, *dblist;
    float *xp;   // database rows in list order (cells only)
    unsigned char *cell_q, *cell_db;
    CellTable *tab;
    int2 *segs;
    int *nseg;
    float *cand_key, *fix_key, *tau;
    int32_t *cand_id, *fix_id;
    int *row_flags, *counts, *failed, *flist, *counters;
    size_t bytes;
};

static TcWorkspace tc_carve(void *base, int D, int K, long long nq, long long nd)
{
    TcWorkspace w;
    w.wide = tc_wide(D);
    w.bf16 = tc_bf16();
    // one extra inner column carries the norm (two in bf16); wide points are chunked along the inner dimension
    w.sw = 0;
    if (w.bf16 && !w.wide) {
        // swizzled rows of 32, 64 or 128 bytes (16, 32 or 64 values); more inner dimensions: blocks of 128-byte rows
        const int need = D + 2;
        w.sw = need <= 16 ? 32 : (need <= 32 ? 64 : 128);
        w.Dp = (need + w.sw / 2 - 1) / (w.sw / 2) * (w.sw / 2);
        w.nks = (need + 15) / 16;
    } else if (w.bf16) {
        w.Dp = (D + 2 + 2 * kWideKC - 1) / (2 * kWideKC) * (2 * kWideKC);
        w.nks = w.Dp / 16;
    } else {
        w.Dp = w.wide ? (D + 1 + kWideKC - 1) / kWideKC * kWideKC : (D + 1 + 7) / 8 * 8;
        w.nks = w.Dp / 8;
    }
    w.image_bytes = (size_t)w.Dp * (w.bf16 ? 512 : 1024);
    const bool two_pass = nd >= (w.wide ? kWideMinRows : kTwoPassMinTiles * TN);
    // cells of at least 16384 points: the padding between them stays below 1 % of the database
    // (wide points are not visited by cells: the cell kernels keep a point in registers)
    w.cells = (two_pass && !w.wide) ? (int)std::min<long long>(kMaxCells, std::max<long long>(1, nd / 16384)) : 1;
    w.tq = (nq + TM - 1) / TM + 1;                 // one padding tile: a block may hold two query tiles
    w.td = (nd + TN - 1) / TN + w.cells;           // every cell may end in a partly filled tile
    if (w.wide) w.td = (w.td + 1) / 2 * 2;         // the wide kernel takes the database two tiles at a time
    const int C = (K + 32 <= 128) ? 256 : 512;
    char *p = static_cast<char *>(base);
    auto take = [&](size_t bytes) { char *r = p; p += (bytes + 255) / 256 * 256; return r; };
    w.img_q = reinterpret_cast<float *>(take((size_t)w.tq * w.image_bytes));
    w.img_db = reinterpret_cast<float *>(take((size_t)w.td * w.image_bytes));
    w.norms_q = reinterpret_cast<double *>(take(sizeof(double) * (size_t)w.tq * TM));
    w.res_q = reinterpret_cast<float2 *>(take(sizeof(float2) * (size_t)w.tq * TM));
    w.qlist = reinterpret_cast<int *>(take(sizeof(int) * (size_t)w.tq * TM));
    w.dblist = reinterpret_cast<int *>(take(sizeof(int) * (size_t)w.td * TN));
    w.xp = (w.cells > 1) ? reinterpret_cast<float *>(take(sizeof(float) * (size_t)w.td * TN * D)) : nullptr;
    w.img_s = nullptr; w.slist = nullptr;
    if (two_pass) {
        w.img_s = reinterpret_cast<float *>(take((size_t)kMaxSampleTiles * w.image_bytes));
        w.slist = reinterpret_cast<int *>(take(sizeof(int) * (size_t)kMaxSampleTiles * TN));
    }
    w.cell_q = reinterpret_cast<unsigned char *>(take((size_t)nq));
    w.cell_db = reinterpret_cast<unsigned char *>(take((size_t)nd));
    w.tab = reinterpret_cast<CellTable *>(take(sizeof(CellTable)));
    w.segs = reinterpret_cast<int2 *>(take(sizeof(int2) * (size_t)w.tq * kMaxCells));
    w.nseg = reinterpret_cast<int *>(take(sizeof(int) * (size_t)w.tq));
    w.cand_key = reinterpret_cast<float *>(take(sizeof(float) * (size_t)nq * C));
    w.cand_id = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * (size_t)nq * C));
    w.fix_key = nullptr; w.fix_id = nullptr; w.tau = nullptr; w.row_flags = nullptr; w.counts = nullptr;
    if (two_pass) {
        w.fix_key = reinterpret_cast<float *>(take(sizeof(float) * (size_t)nq * fixed_cap(K)));
        w.fix_id = reinterpret_cast<int32_t *>(take(sizeof(int32_t) * (size_t)nq * fixed_cap(K)));
        w.tau = reinterpret_cast<float *>(take(sizeof(float) * (size_t)nq));
        w.row_flags = reinterpret_cast<int *>(take(sizeof(int) * (size_t)nq));
        w.counts = reinterpret_cast<int *>(take(sizeof(int) * (size_t)nq * 2));
    }
    w.failed = reinterpret_cast<int *>(take(sizeof(int) * (size_t)nq));
    w.flist = reinterpret_cast<int *>(take(sizeof(int) * (size_t)nq));
    w.counters = reinterpret_cast<int *>(take(sizeof(int) * 16));   // [0] wait time-out flag, [1] failed rows, [2] listed rows, [3] max error ratio (float bits), [4], [5] largest relative lo part / leftover of a database row (float bits)
    w.bytes = (size_t)(p - static_cast<char *>(base));
    return w;
}

// B200TSNE_KNN_TIMERS=1: device time of the phases of one search (CUDA events on the launching stream, printed to
// stderr when the search ends; the marks synchronise nothing, the print waits for the stream).
struct PhaseTimer {
    static constexpr int kMax = 12;
    bool on = false;
    cudaStream_t st = nullptr;
    cudaEvent_t ev[kMax] = {};
    const char *name[kMax] = {};
    int n = 0;
    explicit PhaseTimer(cudaStream_t s) : st(s)
    {
        const char *e = getenv("B200TSNE_KNN_TIMERS");
        on = e && atoi(e) != 0;
    }
    void mark(const char *what)
    {
        if (!on || n >= kMax) return;
        if (cudaEventCreate(&ev[n]) != cudaSuccess) { on = false; return; }
        cudaEventRecord(ev[n], st);
        name[n++] = what;
    }
    ~PhaseTimer()
    {
        if (n > 1 && cudaEventSynchronize(ev[n - 1]) == cudaSuccess) {
            fprintf(stderr, "knn phases (ms):");
            for (int i = 1; i < n; i++) {
                float ms = 0.0f;
                cudaEventElapsedTime(&ms, ev[i - 1], ev[i]);
                fprintf(stderr, " %s %.2f", name[i], ms);
            }
            fprintf(stderr, "\n");
        }
        for (int i = 0; i < n; i++) cudaEventDestroy(ev[i]);
    }
};

// Workspace (device, 256-byte aligned) needed by launch_knn_tc for nq queries against nd database rows.
size_t knn_tc_workspace_bytes(int D, int K, int64_t nq, int64_t nd) { return tc_carve(nullptr, D, K, nq, nd).bytes; }

// X: [N][D] row-major (device).  ids/d2: [(q_hi-q_lo)][K].  n_failed_host receives the number of rows
// whose proof did not close; their global row indices are in failed_list (device, first n entries) and
// the caller recomputes them with the SIMT search.  Returns after the kernels are queued, except for
// the small synchronous read of the counters.
int launch_knn_tc(const float *X, int64_t N, int D, int K, int64_t q_lo, int64_t q_hi, int64_t db_lo, int64_t db_hi,
                  int32_t *ids, float *d2, void *workspace, int **failed_list, int *n_failed_host, float *err_ratio_host,
                  cudaStream_t st)
{
    (void)N;
    const long long nq = q_hi - q_lo, nd = db_hi - db_lo;
    *n_failed_host = 0;
    if (nq <= 0) return 0;
    TcWorkspace w = tc_carve(workspace, D, K, nq, nd);
    const int Dp = w.Dp, cells = w.cells;
    const bool wide = w.wide;
    const int bf16 = w.bf16 ? 1 : 0;
    const int KC = wide ? (bf16 ? 2 * kWideKC : kWideKC) : Dp;   // inner dimensions per image chunk
    const int EPL = (K + 32 <= 128) ? 8 : 16, C = 32 * EPL, L = 16 * EPL;
    const int kFixedCap = fixed_cap(K);
    const bool two_pass = w.fix_key != nullptr;
    float *cand_key = w.cand_key, *fix_key = w.fix_key, *tau = w.tau;
    int32_t *cand_id = w.cand_id, *fix_id = w.fix_id;
    int *row_flags = w.row_flags, *counts = w.counts, *failed = w.failed, *flist = w.flist, *counters = w.counters;
    B200_CUDA(cudaMemsetAsync(counters, 0, sizeof(int) * 16, st));
    PhaseTimer phases(st);
    phases.mark("start");

    // ---- visiting order of the queries and of the database, operand images ----
    B200_CUDA(cudaMemsetAsync(w.qlist, 0xff, sizeof(int) * (size_t)w.tq * TM, st));    // -1 = padding
    B200_CUDA(cudaMemsetAsync(w.dblist, 0xff, sizeof(int) * (size_t)w.td * TN, st));
    long long nd_pos = nd;   // database list positions in use (an upper bound when the cells are padded)
    if (cells > 1) {
        const unsigned gq = (unsigned)((nq + kCellThreads - 1) / kCellThreads), gd = (unsigned)((nd + kCellThreads - 1) / kCellThreads);
        knn_cells_init_kernel<<<1, 256, 0, st>>>(X, D, db_lo, nd, cells, w.tab);
        knn_cells_assign_kernel<<<gd, kCellThreads, 0, st>>>(X, D, db_lo, nd, cells, w.tab, 1, w.cell_db);
        knn_cells_assign_kernel<<<gq, kCellThreads, 0, st>>>(X, D, q_lo, nq, cells, w.tab, 0, w.cell_q);
        knn_cells_layout_kernel<<<1, 32, 0, st>>>(cells, w.tab);
        knn_cells_scatter_kernel<<<gd, kCellThreads, 0, st>>>(w.cell_db, db_lo, nd, cells, w.tab, 1, w.dblist);
        knn_cells_scatter_kernel<<<gq, kCellThreads, 0, st>>>(w.cell_q, q_lo, nq, cells, w.tab, 0, w.qlist);
        nd_pos = w.td * TN;
        knn_gather_rows_kernel<<<(unsigned)((nd_pos * D + 255) / 256), 256, 0, st>>>(X, w.dblist, D, nd_pos, w.xp);
    } else {
        knn_iota_kernel<<<(unsigned)((nd + 255) / 256), 256, 0, st>>>(w.dblist, db_lo, nd);
        knn_iota_kernel<<<(unsigned)((nq + 255) / 256), 256, 0, st>>>(w.qlist, q_lo, nq);
    }
    B200_CUDA(cudaGetLastError());
    if (bf16) {
        knn_tc_prepare_bf16_kernel<<<(unsigned)w.tq, 128, 0, st>>>(X, w.qlist, D, Dp, KC, w.sw, 0, reinterpret_cast<__nv_bfloat16 *>(w.img_q),
                                                                   w.norms_q, w.res_q, nullptr);
        knn_tc_prepare_bf16_kernel<<<(unsigned)w.td, 128, 0, st>>>(X, w.dblist, D, Dp, KC, w.sw, 1, reinterpret_cast<__nv_bfloat16 *>(w.img_db),
                                                                   nullptr, nullptr, counters + 4);
    } else {
        knn_tc_prepare_kernel<<<(unsigned)w.tq, 128, 0, st>>>(X, w.qlist, D, Dp, KC, 0, w.img_q, w.norms_q);
        knn_tc_prepare_kernel<<<(unsigned)w.td, 128, 0, st>>>(X, w.dblist, D, Dp, KC, 1, w.img_db, nullptr);
    }
    B200_CUDA(cudaGetLastError());

    phases.mark("cells+images");
    // two query tiles per block when their images and the database stages fit in shared memory
    // (one query tile per block, two blocks per SM: 3 % faster at N = 10^6, D = 50, for twice the L2 traffic; not used)
    const int QH = ((size_t)(2 + kBStages) * w.image_bytes + 1024 <= 227 * 1024) ? 2 : 1;
    const long long q_tiles = (nq + TM - 1) / TM;
    // Segments of the blocks: all database tiles (one shared list) unless the cells prune (per block).
    // The blocks of an online pass hold one query tile, those of a fixed-threshold pass QH.
    knn_single_segment_kernel<<<1, 1, 0, st>>>(w.segs, w.nseg, wide ? (int)(w.td / 2) : (int)((nd + TN - 1) / TN));
    B200_CUDA(cudaGetLastError());
    int seg_stride = 0;
    auto prune = [&]() -> int {   // segments from the current thresholds
        if (cells <= 1) return 0;
        knn_cells_segments_kernel<<<(unsigned)((q_tiles + QH - 1) / QH), kCellThreads, 0, st>>>(X, D, w.qlist, nq, QH * TM, tau, w.norms_q,
                                                                                              cells, w.tab, w.segs, w.nseg);
        B200_CUDA(cudaGetLastError());
        seg_stride = kMaxCells;
        return 0;
    };
    // A database image much larger than L2 is scanned in windows of tiles, one launch per window: the blocks
    // that run at the same time then read the same ~60 MB, which stays in L2.  In one launch the blocks
    // drift apart until each streams its own copy from HBM with only one 56 KB stage in flight, and the
    // scan becomes latency-bound (measured at 10^7 rows: 3.85 s per 2^20 queries against 1.3 s of MMAs).
    const long long db_image_bytes = (long long)w.td * (long long)w.image_bytes;
    int window_tiles = db_image_bytes > (512ll << 20) ? (int)((60ll << 20) / (long long)w.image_bytes) : INT_MAX;
    if (const char *e = getenv("B200TSNE_KNN_WINDOW_TILES")) window_tiles = std::max(1, atoi(e));   // for tests
#define B200_KNN_FILTER_V(EPL_, FIXED_, QH_, stride_, tau_, cap_, key_, id_, counts_)                                           \
    do {                                                                                                                        \
        const size_t smem_ = (size_t)(QH_ + kBStages) * w.image_bytes;                                                          \
        B200_CUDA(cudaFuncSetAttribute(knn_tc_filter_kernel<EPL_, FIXED_, QH_>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                       (int)smem_));                                                                            \
        if (FIXED_) B200_CUDA(cudaMemsetAsync(counts_, 0, sizeof(int) * (size_t)nq * kAccBufs, st));                            \
        const long long win_ = FIXED_ ? (long long)window_tiles * (stride_) : (long long)INT_MAX;                               \
        for (long long lo_ = 0; lo_ < w.td; lo_ += win_) {                                                                      \
            const int hi_ = (int)std::min<long long>(w.td, lo_ + win_);                                                         \
            knn_tc_filter_kernel<EPL_, FIXED_, QH_><<<(unsigned)((q_tiles + QH_ - 1) / QH_), tc_threads(QH_), smem_, st>>>(      \
                w.img_q, w.img_db, Dp, nq, nd_pos, w.segs, w.nseg, seg_stride, stride_, (int)lo_, hi_, tau_, cap_, key_, id_,   \
                counts_, counters + 0, bf16, w.sw, w.nks);                                                                      \
            B200_CUDA(cudaGetLastError());                                                                                      \
        }                                                                                                                       \
    } while (0)
    // wide points: the same scan by the chunked kernel, in units of two database tiles
#define B200_KNN_FILTER_WIDE(EPL_, stride_, tau_, cap_, key_, id_, counts_)                                                      \
    do {                                                                                                                        \
        const size_t smem_ = (size_t)kWideStages * 4 * kWideChunkBytes;                                                         \
        B200_CUDA(cudaFuncSetAttribute(knn_tc_wide_kernel<EPL_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_));      \
        B200_CUDA(cudaMemsetAsync(counts_, 0, sizeof(int) * (size_t)nq * 2, st));                                               \
        const long long units_ = w.td / 2;                                                                                      \
        const long long win_ = (long long)std::max(1, window_tiles / 2) * (stride_);                                            \
        for (long long lo_ = 0; lo_ < units_; lo_ += win_) {                                                                    \
            const int hi_ = (int)std::min<long long>(units_, lo_ + win_);                                                       \
            knn_tc_wide_kernel<EPL_><<<(unsigned)((q_tiles + 1) / 2), tc_threads(2), smem_, st>>>(                               \
                w.img_q, w.img_db, Dp / KC, nq, w.segs, w.nseg, seg_stride, stride_, (int)lo_, hi_, tau_, cap_, key_, id_,       \
                counts_, counters + 0, bf16);                                                                                   \
            B200_CUDA(cudaGetLastError());                                                                                      \
        }                                                                                                                       \
    } while (0)
    // the online threshold keeps one group per query busy: one query tile per block is enough there
#define B200_KNN_FILTER(EPL_, FIXED_, stride_, tau_, cap_, key_, id_, counts_)                                                   \
    do {                                                                                                                        \
        if (FIXED_ && wide) B200_KNN_FILTER_WIDE(EPL_, stride_, tau_, cap_, key_, id_, counts_);                                 \
        else if (!FIXED_ || QH == 1) B200_KNN_FILTER_V(EPL_, FIXED_, 1, stride_, tau_, cap_, key_, id_, counts_);                \
        else B200_KNN_FILTER_V(EPL_, FIXED_, (FIXED_ ? 2 : 1), stride_, tau_, cap_, key_, id_, counts_);                         \
    } while (0)
    const float *final_key = cand_key;
    const int32_t *final_id = cand_id;
    int final_stride = C;
    if (!two_pass) {
        if (EPL == 8) B200_KNN_FILTER(8, false, 1, nullptr, C, cand_key, cand_id, nullptr);
        else B200_KNN_FILTER(16, false, 1, nullptr, C, cand_key, cand_id, nullptr);
    } else {
        // Three levels, each fixing the threshold of the next:
        //  A  (CUDA cores) rank ~10 of a few thousand sample points spread over the database -> tau_A,
        //     chosen so that ~300 points of sample B beat it;
        //  B  every kSampleStride-th tile against tau_A;
        //  C  everything against tau_B = the key of rank ~3L/kSampleStride in sample B: ~3L points beat it.
        // Before each scan the cells are tested against the thresholds it will use; a skipped cell holds no
        // point below them, so the candidate sets (and the sample statistics) are those of a full scan.
        // (the wide kernel strides over units of two tiles: the same 1/kSampleStride of the database)
        const long long n_db_tiles = (nd + TN - 1) / TN;
        const double b_points = wide ? (double)((n_db_tiles / 2 + kSampleStride - 1) / kSampleStride) * kWideUnit
                                     : (double)((n_db_tiles + kSampleStride - 1) / kSampleStride) * TN;
        const long long db_n = nd;
        // Up to ~400k points the sample of level A is large enough (16 N / 3L points, rank ~16) to fix the
        // threshold of level C directly; beyond that level B refines it.
        const bool direct = db_n <= 393216;
        const int m_a = direct ? (int)std::min<long long>(16384, std::max<long long>(256, 16 * db_n / (3 * L)))
                               : (int)std::min<long long>(16384, std::max<long long>(2048, (long long)(b_points / 32)));
        const long long a_stride = std::max<long long>(1, db_n / m_a);
        const double a_target = direct ? 3.0 * L * m_a / (double)db_n : 300.0 * m_a / b_points;
        const int rank_a = std::min(16, std::max(4, (int)(a_target + 0.5))) - 1;
        const int rank_b = std::max(4, (3 * L + kSampleStride - 1) / kSampleStride) - 1;
        if (getenv("B200TSNE_KNN_LEVEL_A") && strcmp(getenv("B200TSNE_KNN_LEVEL_A"), "simt") == 0) {
            if (wide)
                knn_sample_tau_wide_kernel<<<(unsigned)((nq + kTauThreads - 1) / kTauThreads), kTauThreads, 0, st>>>(X, D, w.qlist, nq, db_lo,
                                                                                                             a_stride, m_a, rank_a, tau);
            else
                knn_sample_tau_kernel<<<(unsigned)((nq + kTauThreads - 1) / kTauThreads), kTauThreads, 0, st>>>(X, D, w.qlist, nq, db_lo,
                                                                                                        a_stride, m_a, rank_a, tau);
        } else {
            // the same sample on the tensor cores: its points as a few tile images, every query thread keeping its
            // 16 smallest keys in registers (the keys differ from the fp32 sums of the CUDA-core kernels by the
            // filter's error only, and this threshold has to be roughly right, no more)
            const int ts = wide ? (m_a + kWideUnit - 1) / kWideUnit * 2 : (m_a + TN - 1) / TN;
            knn_sample_list_kernel<<<(unsigned)((ts * TN + 255) / 256), 256, 0, st>>>(w.slist, (long long)ts * TN, m_a, db_lo, a_stride);
            if (bf16)
                knn_tc_prepare_bf16_kernel<<<(unsigned)ts, 128, 0, st>>>(X, w.slist, D, Dp, KC, w.sw, 1, reinterpret_cast<__nv_bfloat16 *>(w.img_s),
                                                                         nullptr, nullptr, nullptr);
            else
                knn_tc_prepare_kernel<<<(unsigned)ts, 128, 0, st>>>(X, w.slist, D, Dp, KC, 1, w.img_s, nullptr);
            knn_single_segment_kernel<<<1, 1, 0, st>>>(w.segs, w.nseg, wide ? ts / 2 : ts);
            B200_CUDA(cudaGetLastError());
            if (wide) {
                const size_t smem_a = (size_t)kWideStages * 4 * kWideChunkBytes;
                B200_CUDA(cudaFuncSetAttribute(knn_tc_wide_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a));
                knn_tc_wide_kernel<8, true><<<(unsigned)((q_tiles + 1) / 2), tc_threads(2), smem_a, st>>>(
                    w.img_q, w.img_s, Dp / KC, nq, w.segs, w.nseg, 0, 1, 0, ts / 2, nullptr, 0, nullptr, nullptr, nullptr, counters + 0, bf16,
                    rank_a, tau, (long long)m_a);
            } else {
                const size_t smem_a = (size_t)(1 + kBStages) * w.image_bytes;
                B200_CUDA(cudaFuncSetAttribute(knn_tc_filter_kernel<8, false, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a));
                knn_tc_filter_kernel<8, false, 1, true><<<(unsigned)q_tiles, tc_threads(1), smem_a, st>>>(
                    w.img_q, w.img_s, Dp, nq, (long long)m_a, w.segs, w.nseg, 0, 1, 0, ts, nullptr, 0, nullptr, nullptr, nullptr, counters + 0,
                    bf16, w.sw, w.nks, rank_a, tau);
            }
            B200_CUDA(cudaGetLastError());
            // back to all database tiles
            knn_single_segment_kernel<<<1, 1, 0, st>>>(w.segs, w.nseg, wide ? (int)(w.td / 2) : (int)((nd + TN - 1) / TN));
        }
        B200_CUDA(cudaGetLastError());
        phases.mark("level_A");
        B200_TRY(prune());
        const unsigned sel_grid = (unsigned)((nq + 3) / 4);
        if (!direct) {
            // level B: only the key of rank rank_b among the sample's candidates is needed
            if (EPL == 8) {
                B200_KNN_FILTER(8, true, kSampleStride, tau, kFixedCap, fix_key, fix_id, counts);
                knn_tc_pick_kernel<32><<<sel_grid, 128, 0, st>>>(fix_key, fix_id, kFixedCap, counts, nq, rank_b + 1, nullptr, nullptr, 0, tau,
                                                                 row_flags);
            } else {
                B200_KNN_FILTER(16, true, kSampleStride, tau, kFixedCap, fix_key, fix_id, counts);
                knn_tc_pick_kernel<64><<<sel_grid, 128, 0, st>>>(fix_key, fix_id, kFixedCap, counts, nq, rank_b + 1, nullptr, nullptr, 0, tau,
                                                                 row_flags);
            }
            B200_CUDA(cudaGetLastError());
            phases.mark("level_B+pick");
            B200_TRY(prune());
        }
        // level C: the L best go to the (otherwise unused) online buffers, in no particular order
        if (EPL == 8) {
            B200_KNN_FILTER(8, true, 1, tau, kFixedCap, fix_key, fix_id, counts);
            phases.mark("level_C");
            knn_tc_pick_kernel<32><<<sel_grid, 128, 0, st>>>(fix_key, fix_id, kFixedCap, counts, nq, L, cand_key, cand_id, C, nullptr, row_flags);
        } else {
            B200_KNN_FILTER(16, true, 1, tau, kFixedCap, fix_key, fix_id, counts);
            phases.mark("level_C");
            knn_tc_pick_kernel<64><<<sel_grid, 128, 0, st>>>(fix_key, fix_id, kFixedCap, counts, nq, L, cand_key, cand_id, C, nullptr, row_flags);
        }
        phases.mark("pick");
        B200_CUDA(cudaGetLastError());
        final_key = cand_key;
        final_id = cand_id;
        final_stride = C;
    }
#undef B200_KNN_FILTER
#undef B200_KNN_FILTER_V
#undef B200_KNN_FILTER_WIDE
    // Error bound of the filter relative to (|x_i|^2 + d^2 + 1): 3xTF32 drops terms of order 2^-22 |x_i||x_j|,
    // and the fp32 accumulation of D products (not IEEE in the tensor core: take two units in the last place
    // per addition) adds up to 2 D 2^-24 |x_i||x_j| in the worst case.  2^-14 covers both with a wide margin
    // up to D = 256; beyond, the bound grows with D.  The re-rank checks the observed error of every
    // candidate against half of it.
    // bf16 pairs: what the products drop is bounded row by row in the re-rank (see knn_tc_prepare_bf16_kernel), so
    // the scale covers the accumulation only.
    const float err_scale = bf16 ? std::max(1.52587890625e-05f, (float)(D + 8) * 2.384185791015625e-07f)      // max(2^-16, (D + 8) 2^-22)
                                 : std::max(6.103515625e-05f, (float)(D + 8) * 2.384185791015625e-07f);   // max(2^-14, (D + 8) 2^-22)
    knn_tc_rerank_kernel<<<(unsigned)((nq + kRerankWarps - 1) / kRerankWarps), kRerankWarps * 32, 0, st>>>(
        X, D, w.qlist, w.dblist, q_lo, nq, final_key, final_id, L, final_stride, K, w.norms_q, err_scale, bf16 ? w.res_q : nullptr,
        reinterpret_cast<const float *>(counters + 4), two_pass ? row_flags : nullptr, ids, d2,
        failed, counters + 1, reinterpret_cast<float *>(counters + 3), w.xp);
    B200_CUDA(cudaGetLastError());
    knn_tc_collect_failed_kernel<<<(unsigned)((nq + 255) / 256), 256, 0, st>>>(failed, nq, w.qlist, flist, counters + 2);
    B200_CUDA(cudaGetLastError());
    phases.mark("rerank");
    int h[4] = {0, 0, 0, 0};
    B200_CUDA(cudaMemcpyAsync(h, counters, sizeof(h), cudaMemcpyDeviceToHost, st));
    B200_CUDA(cudaStreamSynchronize(st));
    if (h[0]) { set_error("tensor-core kNN: a wait inside the kernel ran out of time"); return -2; }
    *n_failed_host = h[2];
    *failed_list = flist;
    if (err_ratio_host) memcpy(err_ratio_host, &h[3], sizeof(float));
    return 0;
}


// Runs mbar_wait_selftest_kernel: returns -5 when all 64 threads gave up within the limit (the expected
// outcome), 0 if any of them (wrongly) got through.
int mbar_wait_selftest(int timeout_ms, float *waited_ms, cudaStream_t st)
{
    if (timeout_ms <= 0 || timeout_ms > 2000) { set_error("mbarrier wait self-test: timeout must be 1..2000 ms"); return -1; }
    int *d = nullptr;
    cudaEvent_t a = nullptr, b = nullptr;
    struct Free { int *&d; cudaEvent_t &a, &b; ~Free() { if (d) cudaFree(d); if (a) cudaEventDestroy(a); if (b) cudaEventDestroy(b); } } guard{d, a, b};
    B200_CUDA(cudaMalloc((void **)&d, sizeof(int) * 2));
    B200_CUDA(cudaMemsetAsync(d, 0, sizeof(int) * 2, st));
    B200_CUDA(cudaEventCreate(&a));
    B200_CUDA(cudaEventCreate(&b));
    B200_CUDA(cudaEventRecord(a, st));
    mbar_wait_selftest_kernel<<<1, 64, 0, st>>>(d, d + 1, (unsigned long long)timeout_ms * 1000000ull);
    B200_CUDA(cudaGetLastError());
    B200_CUDA(cudaEventRecord(b, st));
    B200_CUDA(cudaStreamSynchronize(st));
    float ms = 0.0f;
    B200_CUDA(cudaEventElapsedTime(&ms, a, b));
    if (waited_ms) *waited_ms = ms;
    int h[2] = {0, 0};
    B200_CUDA(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
    if (h[0] == 1 && h[1] == 64) { set_error("kNN pipeline: a barrier wait ran out (self-test)"); return -5; }
    return 0;
}

}  // namespace b200
