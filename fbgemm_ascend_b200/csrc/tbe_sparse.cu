// Producers of the lookup's inputs on B200 (sm_100a): lengths -> offsets, and the reordering of a
// jagged request (lengths / values / weights) by table.
//
//   complete cumsum     out[0] = 0, out[i + 1] = in[0] + ... + in[i]            (int32 / int64)
//       replaces aclnnAsynchronousCompleteCumsum
//       (reference: src/sparse_ops/asynchronous_complete_cumsum/asynchronous_complete_cumsum.cpp:14-54)
//   permute 2D sparse   out_lengths[i, :] = lengths[permute[i], :]; out_values = the value segments of the
//       tables permute[0], permute[1], ... one after the other; weights alike
//       replaces aclnnPermute2dSparseData
//       (reference: src/sparse_ops/permute2d_sparse_data/permute2d_sparse_data.cpp:45-150, permute1d_sparse_data.cpp:81-165)
//
// Both are streaming integer work bounded by HBM bandwidth.  Both need a little global memory beyond
// their inputs and outputs (per-tile sums; per-table segment lengths and offsets): the caller passes it.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "tbe_common.cuh"

namespace tbe {

namespace {

constexpr int kScanThreads = 256;
constexpr int kScanPerThread = 8;
constexpr int kScanTile = kScanThreads * kScanPerThread;   // elements per block

__device__ __forceinline__ int64_t warp_sum(int64_t v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Sum over the block; every thread gets the result.  `red` holds one value per warp.
__device__ __forceinline__ int64_t block_sum(int64_t v, int64_t* red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();   // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    int64_t t = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    return t;
}

// ---- complete cumsum in three kernels: tile sums, their running sums (one block), then every tile scans itself
// behind its carry.  Needs 8 bytes per tile and nothing cleared: the form behind the entry point with built-in scratch.

template <typename T>
__global__ void __launch_bounds__(kScanThreads) tile_sums_kernel(const T* __restrict__ in, int64_t n, int64_t* __restrict__ tile_sums)
{
    __shared__ int64_t red[kScanThreads / 32];
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile;
    int64_t s = 0;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        const int64_t i = base + j * kScanThreads + threadIdx.x;
        if (i < n) s += static_cast<int64_t>(in[i]);
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = s;
}

// One block turns the tile sums into the sums of everything BEFORE each tile, in place: pieces of 1024 x 4 values, a
// running carry from piece to piece.  Every tile then reads a single value instead of adding up all the tiles before it.
constexpr int kCarryThreads = 1024;
constexpr int kCarryPerThread = 4;
__global__ void __launch_bounds__(kCarryThreads) exclusive_tile_sums_kernel(int64_t* __restrict__ tile_sums, int64_t tiles)
{
    __shared__ int64_t warp_tot[kCarryThreads / 32];
    __shared__ int64_t piece_total;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t carry = 0;
    for (int64_t base = 0; base < tiles; base += kCarryThreads * kCarryPerThread) {
        const int64_t first = base + static_cast<int64_t>(threadIdx.x) * kCarryPerThread;
        int64_t v[kCarryPerThread];
        int64_t mine = 0;
#pragma unroll
        for (int j = 0; j < kCarryPerThread; ++j) {
            v[j] = (first + j < tiles) ? tile_sums[first + j] : 0;
            mine += v[j];
        }
        int64_t incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        __syncthreads();               // the previous piece's totals have been read
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int64_t run = carry + (incl - mine);
        for (int w = 0; w < warp; ++w) run += warp_tot[w];
        if (threadIdx.x == kCarryThreads - 1) piece_total = run + mine - carry;
#pragma unroll
        for (int j = 0; j < kCarryPerThread; ++j) {
            if (first + j < tiles) tile_sums[first + j] = run;
            run += v[j];
        }
        __syncthreads();
        carry += piece_total;
    }
}

// Every warp owns 256 consecutive elements of the tile, as 8 rows of 32: loads and stores are whole coalesced lines
// (thread-contiguous pieces, 64 bytes apart from lane to lane, measured at less than half the copy bandwidth), the
// scan inside a row of 32 runs over shuffles.
template <typename T>
__global__ void __launch_bounds__(kScanThreads) scan_tiles_kernel(const T* __restrict__ in, int64_t n, const int64_t* __restrict__ tiles_before,
                                                                   T* __restrict__ out)
{
    __shared__ int64_t warp_tot[kScanThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // everything before this tile (a single tile has nothing before it and no scratch)
    const int64_t before = (gridDim.x > 1) ? tiles_before[blockIdx.x] : 0;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kScanTile + static_cast<int64_t>(warp) * (32 * kScanPerThread) + lane;
    int64_t v[kScanPerThread];
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) v[j] = (first + j * 32 < n) ? static_cast<int64_t>(in[first + j * 32]) : 0;
    // inclusive scan of every row of 32, then the rows chained: v[j] becomes the sum of the warp's elements up to this one
    int64_t carry = 0;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        int64_t incl = v[j];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        v[j] = carry + incl;
        carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) warp_tot[warp] = carry;
    __syncthreads();
    int64_t base = before;
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
    if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = 0;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j)
        if (first + j * 32 < n) out[first + j * 32 + 1] = static_cast<T>(base + v[j]);
}

// ---- complete cumsum in one pass: every tile publishes its sum, then looks back over its predecessors ------
//
// The three kernels above read the input twice.  Here a block stages a tile of 64 KB (8192 int64 or 16384 int32
// elements) in shared memory with asynchronous copies, adds it up, publishes the tile's sum (state 1), and while its
// eight worker warps turn the tile into its local running sums in place, a ninth warp collects what lies before the
// tile from the descriptors of the tiles in front -- stopping at the nearest one that already knows its own prefix
// (state 2) -- and publishes the tile's inclusive sum.  The copy-out adds the prefix on the way to global memory.
//
// One block per tile, handed out by the hardware in block order, so the tiles a block waits for started before it did.
// The poll loop is bounded all the same: a tile whose wait runs out adds up the input in front of it by itself (slow,
// correct), so no error word is needed and nothing can spin for ever.
//
// A descriptor is one aligned 16-byte word {sum, state}, written and read by single 16-byte accesses, so a reader
// that sees the state sees the sum that belongs to it.  One poll fetches 14 x 32 descriptors, more than the 444 tiles
// that are resident at once on 148 SMs: a tile never waits for another tile's look-back, only for the sums of the
// tiles in front of it, and normally finishes with its first or second poll.
//
// Measured, 16 M int64 (128 MB in, 128 MB out; L2 flushed; the operator with its memset and allocations): 79 us;
// 64 M: 271 us = 3.96 TB/s.  A copy of the same bytes: 49 / 173 us; a library scan: 87 / 314 us; this kernel without
// the look-back (wrong sums, for the experiment): 71 / 239 us.  What bounds it is on-chip capacity: a tile occupies
// its shared memory for load + look-back (two to three L2 round trips under load) + copy-out, about 14 us, and
// 3 x 64 KB per SM held that long is 4 TB/s.  Variants measured: 4096-element tiles in registers, 32 descriptors per
// poll 165 us, 128 per poll 91 us (both bound by the chain of look-backs); 32 KB tiles, 6 blocks per SM, 256 per poll
// 83 us; persistent blocks striding over the tiles 79-89 us; one block per SM walking its tiles through three buffers
// (tile i + 1 arriving, tile i scanned, tile i - 1 written out behind the prefix found for it meanwhile, so that neither
// the load nor the look-back holds the block up) 87 us / 312 us at 64 M: the blocks then run in lockstep, and every
// round waits for the slowest block's sum.
constexpr int kBigWorkers = 256;                          // threads that move and scan data
constexpr int kBigThreads = kBigWorkers + 32;             // + one warp that only looks back
constexpr int kBigChunks = 4096;                          // 16-byte chunks per tile
constexpr int kBigChunksPerThread = kBigChunks / kBigWorkers;
constexpr int kBigSmemBytes = (kBigChunks + kBigChunks / 16) * 16;   // one chunk of padding after every 16
constexpr int kBigBlocksPerSM = 3;
constexpr int kChainLook = 14;             // windows of 32 descriptors fetched per poll
constexpr int kChainPolls = 1 << 20;      // L2 round trips before a tile gives up: the better part of a second

struct __align__(16) TileState {
    int64_t sum;
    int64_t state;     // 0 nothing yet, 1 sum of the tile, 2 sum of everything up to and including the tile
};

__device__ __forceinline__ TileState load_state(const TileState* p)
{
    TileState d;
    asm volatile("ld.relaxed.gpu.global.v2.s64 {%0, %1}, [%2];" : "=l"(d.sum), "=l"(d.state) : "l"(p) : "memory");
    return d;
}
__device__ __forceinline__ void store_state(TileState* p, int64_t sum, int64_t state)
{
    asm volatile("st.relaxed.gpu.global.v2.s64 [%0], {%1, %2};" ::"l"(p), "l"(sum), "l"(state) : "memory");
}

// Asynchronous global -> shared copy of BYTES (4, 8 or 16) bytes, of which the first `valid` come from memory and the
// rest are zeros.
template <int BYTES>
__device__ __forceinline__ void stage_async(void* smem_dst, const void* gsrc, int valid)
{
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(d), "l"(gsrc), "n"(BYTES), "r"(valid) : "memory");
}

// Byte offset of chunk c in the padded tile: a thread's 16 consecutive chunks and 32 lanes' same-numbered chunks both
// fall on distinct banks.
__device__ __forceinline__ int big_chunk_offset(int c) { return (c + (c >> 4)) << 4; }

// Sixteen bytes of shared memory as elements.
template <typename U>
union Chunk {
    uint4 raw;
    U v[16 / sizeof(U)];
};

// What warp 8 does for a tile: sum of all tiles in front of `tile`; false if the wait ran out.
__device__ __forceinline__ bool look_back(const TileState* __restrict__ states, int64_t tile, int lane, int max_polls, int64_t* prefix)
{
    int64_t acc = 0;
    int64_t nearest = tile - 1;          // lane l looks at the tiles nearest - l - 32 * w, w = 0 .. kChainLook - 1
    int polls = 0;
    bool done = false;
    while (!done) {
        TileState d[kChainLook];
#pragma unroll
        for (int w = 0; w < kChainLook; ++w) {
            const int64_t t = nearest - lane - 32 * w;
            if (t >= 0) {
                d[w] = load_state(&states[t]);
            } else {                      // in front of tile 0: "everything up to here is 0"
                d[w].sum = 0;
                d[w].state = 2;
            }
        }
        // Walk the windows from the nearest one outwards; stop at a gap (poll again from the window that has it) or at
        // the nearest tile that knows its prefix.
        int consumed = 0;
#pragma unroll
        for (int w = 0; w < kChainLook; ++w) {
            if (done || consumed != w) continue;
            if (!__all_sync(0xffffffffu, d[w].state != 0)) continue;
            const unsigned known = __ballot_sync(0xffffffffu, d[w].state == 2);
            if (known) {
                const int stop = __ffs(known) - 1;
                acc += warp_sum(lane <= stop ? d[w].sum : 0);
                done = true;
            } else {
                acc += warp_sum(d[w].sum);
                consumed = w + 1;
            }
        }
        nearest -= 32 * consumed;
        if (!done && consumed == 0 && ++polls > max_polls) return false;
    }
    *prefix = acc;
    return true;
}

template <typename T, typename U, bool ALIGNED>
__global__ void __launch_bounds__(kBigThreads, kBigBlocksPerSM) big_tile_scan_kernel(const T* __restrict__ in, int64_t n, T* __restrict__ out,
                                                                                     TileState* __restrict__ states, int64_t tiles, int max_polls)
{
    constexpr int EPC = 16 / static_cast<int>(sizeof(T));   // elements per chunk
    constexpr int E = kBigChunks * EPC;                     // elements per tile
    extern __shared__ __align__(16) unsigned char tile_smem[];
    __shared__ U warp_tot[kBigWorkers / 32];
    __shared__ int64_t red[kBigThreads / 32];
    __shared__ int64_t s_prefix;
    __shared__ int s_alone;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool worker = warp < kBigWorkers / 32;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t e0 = tile * E;
        const int64_t left = n - e0;
        const bool full = left >= E;                      // block-uniform
        if (worker) {
            if (full) {
                // chunk q * 256 + tid: 4096 bytes further in global memory, 17 x 256 bytes further in the padded tile
                const unsigned char* g = reinterpret_cast<const unsigned char*>(in + e0) + tid * 16;
                unsigned char* d = tile_smem + ((tid + (tid >> 4)) << 4);
#pragma unroll
                for (int q = 0; q < kBigChunksPerThread; ++q) {
                    if (ALIGNED) {
                        stage_async<16>(d + q * (kBigWorkers * 17), g + q * (kBigWorkers * 16), 16);
                    } else {
#pragma unroll
                        for (int k = 0; k < EPC; ++k)
                            stage_async<static_cast<int>(sizeof(T))>(d + q * (kBigWorkers * 17) + k * sizeof(T), g + q * (kBigWorkers * 16) + k * sizeof(T),
                                                                     static_cast<int>(sizeof(T)));
                    }
                }
            } else {
#pragma unroll 1
                for (int q = 0; q < kBigChunksPerThread; ++q) {
                    const int c = q * kBigWorkers + tid;
                    const int64_t have = left - static_cast<int64_t>(c) * EPC;           // elements of this chunk that exist
                    unsigned char* dst = tile_smem + big_chunk_offset(c);
                    if (ALIGNED) {
                        const int valid = have >= EPC ? 16 : (have > 0 ? static_cast<int>(have) * static_cast<int>(sizeof(T)) : 0);
                        stage_async<16>(dst, valid ? static_cast<const void*>(in + e0 + static_cast<int64_t>(c) * EPC) : static_cast<const void*>(in), valid);
                    } else {
#pragma unroll
                        for (int k = 0; k < EPC; ++k)
                            stage_async<static_cast<int>(sizeof(T))>(dst + k * sizeof(T), k < have ? in + e0 + static_cast<int64_t>(c) * EPC + k : in,
                                                                     k < have ? static_cast<int>(sizeof(T)) : 0);
                    }
                }
            }
            asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
        }
        if (tid == 0) s_alone = 0;
        __syncthreads();
        // pass 1: every worker adds up its 16 consecutive chunks; the running sums of those totals across the block
        U mine = 0;
        unsigned char* own = tile_smem + tid * (kBigChunksPerThread * 17);     // this worker's 16 chunks: 16 x 16 bytes + padding
        if (worker) {
#pragma unroll
            for (int q = 0; q < kBigChunksPerThread; ++q) {
                Chunk<U> w;
                w.raw = *reinterpret_cast<const uint4*>(own + q * 16);
#pragma unroll
                for (int k = 0; k < EPC; ++k) mine += w.v[k];
            }
        }
        U incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const U up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += up;
        }
        if (worker && lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        U before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kBigWorkers / 32; ++w) {
            const U t = warp_tot[w];
            if (w < warp) before += t;
            total += t;
        }
        if (!worker) {
            // the look-back warp: publish, collect, publish again
            int64_t prefix = 0;
            bool ok = true;
            if (tiles > 1) {
                if (tile == 0) {
                    if (lane == 0) store_state(&states[0], static_cast<int64_t>(total), 2);
                } else {
                    if (lane == 0) store_state(&states[tile], static_cast<int64_t>(total), 1);
                    ok = look_back(states, tile, lane, max_polls, &prefix);
                    if (ok && lane == 0) store_state(&states[tile], static_cast<int64_t>(static_cast<U>(prefix) + total), 2);
                }
            }
            if (lane == 0) {
                s_prefix = prefix;
                if (!ok) s_alone = 1;
            }
        } else {
            // pass 2: the tile's own running sums, in place
            U run = before + incl - mine;
#pragma unroll
            for (int q = 0; q < kBigChunksPerThread; ++q) {
                Chunk<U> w;
                w.raw = *reinterpret_cast<const uint4*>(own + q * 16);
#pragma unroll
                for (int k = 0; k < EPC; ++k) {
                    run += w.v[k];
                    w.v[k] = run;
                }
                *reinterpret_cast<uint4*>(own + q * 16) = w.raw;
            }
        }
        __syncthreads();
        U prefix = static_cast<U>(s_prefix);
        if (s_alone) {       // block-uniform: the wait ran out, add up everything in front of this tile here
            int64_t part = 0;
            for (int64_t i = tid; i < e0; i += kBigThreads) part += static_cast<int64_t>(static_cast<U>(in[i]));
            part = warp_sum(part);
            if (lane == 0) red[warp] = part;
            __syncthreads();
            int64_t all = 0;
            for (int w = 0; w < kBigThreads / 32; ++w) all += red[w];
            prefix = static_cast<U>(all);
            if (tid == 0) store_state(&states[tile], static_cast<int64_t>(prefix + total), 2);
        }
        // copy-out: consecutive threads take consecutive elements
        if (worker) {
            if (tile == 0 && tid == 0) out[0] = 0;
            if (full) {
                // element r * 256 + tid: 256 / EPC chunks, i.e. 17 x 256 / EPC bytes, further in the padded tile per step
                const unsigned char* src = tile_smem + (((tid / EPC) + ((tid / EPC) >> 4)) << 4) + (tid % EPC) * sizeof(T);
                T* dst = out + e0 + 1 + tid;
#pragma unroll 16
                for (int r = 0; r < E / kBigWorkers; ++r)
                    dst[r * kBigWorkers] = static_cast<T>(*reinterpret_cast<const U*>(src + r * (kBigWorkers / EPC * 17)) + prefix);
            } else {
#pragma unroll 1
                for (int r = 0; r < E / kBigWorkers; ++r) {
                    const int e = r * kBigWorkers + tid;
                    if (e < left) {
                        const U x = *reinterpret_cast<const U*>(tile_smem + big_chunk_offset(e / EPC) + (e % EPC) * sizeof(T));
                        out[e0 + e + 1] = static_cast<T>(x + prefix);
                    }
                }
            }
        }
        __syncthreads();     // the tile's shared memory is staged anew on the next round
    }
}

// ---- permute 2D sparse data ----------------------------------------------------------------------------

// seg_len[t] += sum of a slice of lengths[t, :]  (seg_len cleared beforehand)
template <typename T>
__global__ void __launch_bounds__(256) segment_lengths_kernel(const T* __restrict__ lengths, int64_t B, int64_t* __restrict__ seg_len)
{
    __shared__ int64_t red[8];
    const int64_t t = blockIdx.y;
    const T* row = lengths + t * B;
    int64_t s = 0;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < B; b += static_cast<int64_t>(gridDim.x) * blockDim.x)
        s += static_cast<int64_t>(row[b]);
    s = block_sum(s, red);
    if (threadIdx.x == 0 && s != 0) atomicAdd(reinterpret_cast<unsigned long long*>(seg_len + t), static_cast<unsigned long long>(s));
}

// One block: in_off = exclusive sums of seg_len over the input tables; out_off = exclusive sums of
// seg_len[permute[i]] over the output tables.  An entry of `permute` outside [0, T_in) counts as an empty table
// and sets the error flag.
__global__ void __launch_bounds__(kScanThreads) segment_offsets_kernel(const int64_t* __restrict__ seg_len, int64_t T_in,
                                                                        const int32_t* __restrict__ permute, int64_t T_out,
                                                                        int64_t* __restrict__ in_off, int64_t* __restrict__ out_off,
                                                                        int32_t* error_flag)
{
    __shared__ int64_t warp_base[kScanThreads / 32];
    __shared__ int64_t carry;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int pass = 0; pass < 2; ++pass) {
        const int64_t count = pass == 0 ? T_in : T_out;
        int64_t* off = pass == 0 ? in_off : out_off;
        if (threadIdx.x == 0) {
            carry = 0;
            off[0] = 0;
        }
        __syncthreads();
        for (int64_t base = 0; base < count; base += kScanThreads) {
            const int64_t i = base + threadIdx.x;
            int64_t v = 0;
            if (i < count) {
                if (pass == 0) {
                    v = seg_len[i];
                } else {
                    const int64_t p = permute[i];
                    if (p >= 0 && p < T_in) v = seg_len[p];
                    else if (error_flag) atomicOr(error_flag, 1);
                }
            }
            int64_t incl = v;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int64_t up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            if (lane == 31) warp_base[warp] = incl;
            __syncthreads();
            int64_t run = carry + incl;
            for (int w = 0; w < warp; ++w) run += warp_base[w];
            if (i < count) off[i + 1] = run;
            __syncthreads();
            if (threadIdx.x == kScanThreads - 1) carry = run;
            __syncthreads();
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) permute_lengths_kernel(const T* __restrict__ lengths, int64_t T_in, int64_t B,
                                                              const int32_t* __restrict__ permute, T* __restrict__ out)
{
    const int64_t i = blockIdx.y;
    const int64_t p = permute[i];
    const bool ok = p >= 0 && p < T_in;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; b < B; b += static_cast<int64_t>(gridDim.x) * blockDim.x)
        out[i * B + b] = ok ? lengths[p * B + b] : static_cast<T>(0);
}

// Output position o lies in output table i with out_off[i] <= o < out_off[i + 1]; its source is
// in_off[permute[i]] + (o - out_off[i]).  A thread finds the table of its first position by binary search
// and walks forward from there.  VT is the unit copied per position (the element, or 16 bytes of a wide row).
template <typename VT, bool ONE_UNIT>
__global__ void __launch_bounds__(256) permute_segments_kernel(const VT* __restrict__ src, VT* __restrict__ dst, int64_t units_per_pos,
                                                               int64_t capacity /* positions */, const int32_t* __restrict__ permute,
                                                               int64_t T_in, int64_t T_out, const int64_t* __restrict__ in_off,
                                                               const int64_t* __restrict__ out_off)
{
    const int64_t total = min(capacity, out_off[T_out]) * units_per_pos;
    constexpr int kPerThread = 8;
    const int64_t chunk = 256 * kPerThread;   // consecutive units of one block and step: a table changes rarely inside
    int64_t i = -1;                            // current output table
    int64_t seg_hi = 0, delta = 0;
    for (int64_t c0 = static_cast<int64_t>(blockIdx.x) * chunk; c0 < total; c0 += static_cast<int64_t>(gridDim.x) * chunk) {
#pragma unroll 4
        for (int j = 0; j < kPerThread; ++j) {
            const int64_t u = c0 + j * 256 + threadIdx.x;
            if (u >= total) break;
            const int64_t o = ONE_UNIT ? u : u / units_per_pos;   // a position is one unit for plain values
            if (i < 0 || o >= seg_hi) {
                // largest i with out_off[i] <= o; positions only grow, so the search starts at the current table
                int64_t lo = (i < 0) ? 0 : i, hi = T_out;
                while (hi - lo > 1) {
                    const int64_t mid = (lo + hi) >> 1;
                    if (out_off[mid] <= o) lo = mid; else hi = mid;
                }
                i = lo;
                seg_hi = out_off[i + 1];
                const int64_t p = permute[i];
                delta = ((p >= 0 && p < T_in) ? in_off[p] : 0) - out_off[i];
            }
            dst[u] = src[u + (ONE_UNIT ? delta : delta * units_per_pos)];
        }
    }
}

// The same walk, but the output tables go to several buffers: output table i belongs to destination i / tables_per_dest
// and lands at (its position within that destination's group of tables) in dest_bases[destination] -- which may be a
// peer GPU's memory: plain stores over NVLink, the exchange of an all-to-all folded into the permute.  A destination
// takes at most dest_capacity positions; what does not fit is dropped and reported.
template <typename VT>
__global__ void __launch_bounds__(256) permute_segments_to_dests_kernel(const VT* __restrict__ src, const int64_t* __restrict__ dest_bases,
                                                                        int64_t tables_per_dest, int64_t dest_capacity, int64_t units_per_pos,
                                                                        const int32_t* __restrict__ permute, int64_t T_in, int64_t T_out,
                                                                        const int64_t* __restrict__ in_off, const int64_t* __restrict__ out_off,
                                                                        int32_t* __restrict__ error_flag)
{
    const int64_t total = out_off[T_out] * units_per_pos;
    constexpr int kPerThread = 8;
    const int64_t chunk = 256 * kPerThread;
    int64_t i = -1;
    int64_t seg_hi = 0, delta = 0, group_lo = 0, group_hi = 0;
    VT* dst = nullptr;
    for (int64_t c0 = static_cast<int64_t>(blockIdx.x) * chunk; c0 < total; c0 += static_cast<int64_t>(gridDim.x) * chunk) {
#pragma unroll 4
        for (int j = 0; j < kPerThread; ++j) {
            const int64_t u = c0 + j * 256 + threadIdx.x;
            if (u >= total) break;
            const int64_t o = u / units_per_pos;
            if (i < 0 || o >= seg_hi) {
                int64_t lo = (i < 0) ? 0 : i, hi = T_out;
                while (hi - lo > 1) {
                    const int64_t mid = (lo + hi) >> 1;
                    if (out_off[mid] <= o) lo = mid; else hi = mid;
                }
                i = lo;
                seg_hi = out_off[i + 1];
                const int64_t p = permute[i];
                delta = (((p >= 0 && p < T_in) ? in_off[p] : 0) - out_off[i]) * units_per_pos;
                const int64_t g = i / tables_per_dest;
                group_lo = out_off[g * tables_per_dest] * units_per_pos;
                group_hi = group_lo + dest_capacity * units_per_pos;
                dst = reinterpret_cast<VT*>(dest_bases[g]);
            }
            if (u < group_hi) dst[u - group_lo] = src[u + delta];
            else if (error_flag) atomicOr(error_flag, 2);
        }
    }
}

// The same for plain 4- and 8-byte values, two at a time: a thread takes a PAIR of consecutive positions of a
// destination, counted from the destination's start, so that its store is one aligned 8- or 16-byte piece whatever the
// parity of the segment starts (remote stores of twice the width load NVLink half as often); the two values are
// fetched separately, since their sources need not be adjacent (a pair may straddle two tables) nor aligned.
constexpr int kMaxPairDests = 64;
template <typename VT, typename VT2>
__global__ void __launch_bounds__(256) permute_pairs_to_dests_kernel(const VT* __restrict__ src, const int64_t* __restrict__ dest_bases,
                                                                     int64_t tables_per_dest, int64_t dest_capacity, int n_dest,
                                                                     const int32_t* __restrict__ permute, int64_t T_in, int64_t T_out,
                                                                     const int64_t* __restrict__ in_off, const int64_t* __restrict__ out_off,
                                                                     int32_t* __restrict__ error_flag)
{
    __shared__ int64_t pair_start[kMaxPairDests + 1];   // pairs in front of every destination
    __shared__ int64_t group_lo[kMaxPairDests];          // first output position of every destination
    __shared__ int64_t group_n[kMaxPairDests];           // positions it takes (at most dest_capacity)
    if (threadIdx.x == 0) {
        int64_t pairs = 0;
        for (int g = 0; g < n_dest; ++g) {
            const int64_t lo = out_off[g * tables_per_dest];
            int64_t cnt = out_off[(g + 1) * tables_per_dest] - lo;
            if (cnt > dest_capacity) {
                cnt = dest_capacity;
                if (error_flag && blockIdx.x == 0) atomicOr(error_flag, 2);
            }
            group_lo[g] = lo;
            group_n[g] = cnt;
            pair_start[g] = pairs;
            pairs += (cnt + 1) >> 1;
        }
        pair_start[n_dest] = pairs;
    }
    __syncthreads();
    const int64_t total_pairs = pair_start[n_dest];
    constexpr int kPerThread = 4;
    const int64_t chunk = 256 * kPerThread;
    int g = 0;
    int64_t i = -1, seg_hi = 0, delta = 0;
    auto find_table = [&](int64_t o) {
        // largest i with out_off[i] <= o; positions only grow, so the search starts at the current table
        int64_t lo = (i < 0) ? 0 : i, hi = T_out;
        while (hi - lo > 1) {
            const int64_t mid = (lo + hi) >> 1;
            if (out_off[mid] <= o) lo = mid; else hi = mid;
        }
        i = lo;
        seg_hi = out_off[i + 1];
        const int64_t p = permute[i];
        delta = ((p >= 0 && p < T_in) ? in_off[p] : 0) - out_off[i];
    };
    for (int64_t c0 = static_cast<int64_t>(blockIdx.x) * chunk; c0 < total_pairs; c0 += static_cast<int64_t>(gridDim.x) * chunk) {
#pragma unroll 2
        for (int j = 0; j < kPerThread; ++j) {
            const int64_t P = c0 + j * 256 + threadIdx.x;
            if (P >= total_pairs) break;
            while (P >= pair_start[g + 1]) ++g;
            const int64_t rel = (P - pair_start[g]) << 1;
            const int64_t u = group_lo[g] + rel;
            if (i < 0 || u >= seg_hi) find_table(u);
            const VT v0 = src[u + delta];
            VT* dst = reinterpret_cast<VT*>(dest_bases[g]) + rel;
            if (rel + 1 < group_n[g]) {
                if (u + 1 >= seg_hi) find_table(u + 1);
                VT2 both;
                both.x = v0;
                both.y = src[u + 1 + delta];
                *reinterpret_cast<VT2*>(dst) = both;
            } else {
                *dst = v0;
            }
        }
    }
}

template <typename VT>
int launch_segments(const void* src, void* dst, int64_t units_per_pos, int64_t capacity, const int32_t* permute, int64_t T_in,
                    int64_t T_out, const int64_t* in_off, const int64_t* out_off, cudaStream_t s)
{
    const int64_t units = capacity * units_per_pos;
    if (units <= 0) return TBE_B200_OK;
    const int64_t want = (units + 256 * 8 - 1) / (256 * 8);   // eight units per thread and step
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
    if (units_per_pos == 1)
        permute_segments_kernel<VT, true><<<blocks, 256, 0, s>>>(static_cast<const VT*>(src), static_cast<VT*>(dst), 1, capacity, permute, T_in,
                                                                 T_out, in_off, out_off);
    else
        permute_segments_kernel<VT, false><<<blocks, 256, 0, s>>>(static_cast<const VT*>(src), static_cast<VT*>(dst), units_per_pos, capacity,
                                                                  permute, T_in, T_out, in_off, out_off);
    return check_launch("permute_segments_kernel");
}

int copy_segments(const void* src, void* dst, int64_t row_bytes, int64_t capacity, const int32_t* permute, int64_t T_in, int64_t T_out,
                  const int64_t* in_off, const int64_t* out_off, cudaStream_t s)
{
    const uintptr_t both = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst);
    if (row_bytes % 16 == 0 && both % 16 == 0)
        return launch_segments<uint4>(src, dst, row_bytes / 16, capacity, permute, T_in, T_out, in_off, out_off, s);
    if (row_bytes % 8 == 0 && both % 8 == 0)
        return launch_segments<uint64_t>(src, dst, row_bytes / 8, capacity, permute, T_in, T_out, in_off, out_off, s);
    if (row_bytes % 4 == 0 && both % 4 == 0)
        return launch_segments<uint32_t>(src, dst, row_bytes / 4, capacity, permute, T_in, T_out, in_off, out_off, s);
    if (row_bytes % 2 == 0 && both % 2 == 0)
        return launch_segments<uint16_t>(src, dst, row_bytes / 2, capacity, permute, T_in, T_out, in_off, out_off, s);
    return launch_segments<uint8_t>(src, dst, row_bytes, capacity, permute, T_in, T_out, in_off, out_off, s);
}

}  // namespace

// Shared by the entry point that takes the caller's scratch and by any that brings its own.
int complete_cumsum_launch(const void* in, int64_t n, int index_bits, void* out, int64_t* tile_sums, cudaStream_t s)
{
    const int64_t tiles = (n + kScanTile - 1) / kScanTile;
    if (index_bits == 32) {
        if (tiles > 1) {
            tile_sums_kernel<int32_t><<<static_cast<unsigned>(tiles), kScanThreads, 0, s>>>(static_cast<const int32_t*>(in), n, tile_sums);
            exclusive_tile_sums_kernel<<<1, kCarryThreads, 0, s>>>(tile_sums, tiles);
        }
        scan_tiles_kernel<int32_t><<<static_cast<unsigned>(tiles), kScanThreads, 0, s>>>(static_cast<const int32_t*>(in), n, tile_sums,
                                                                                        static_cast<int32_t*>(out));
    } else {
        if (tiles > 1) {
            tile_sums_kernel<int64_t><<<static_cast<unsigned>(tiles), kScanThreads, 0, s>>>(static_cast<const int64_t*>(in), n, tile_sums);
            exclusive_tile_sums_kernel<<<1, kCarryThreads, 0, s>>>(tile_sums, tiles);
        }
        scan_tiles_kernel<int64_t><<<static_cast<unsigned>(tiles), kScanThreads, 0, s>>>(static_cast<const int64_t*>(in), n, tile_sums,
                                                                                        static_cast<int64_t*>(out));
    }
    return check_launch("complete_cumsum");
}

int64_t complete_cumsum_tiles(int64_t n) { return (n + kScanTile - 1) / kScanTile; }

// One-pass form.  Scratch: one 16-byte descriptor per 64 KB tile (sized for 8-byte elements, the smaller tile) plus
// 16 bytes to align the first one; cleared on the stream in front of the kernel.
int64_t chained_tiles(int64_t n, int index_bits) { return (n + kBigChunks * (128 / index_bits) - 1) / (kBigChunks * (128 / index_bits)); }
int64_t chained_scratch_bytes(int64_t n)
{
    const int64_t tiles = chained_tiles(n, 64);
    return tiles > 1 ? 16 + tiles * 16 : 0;
}
int chained_polls()
{
    const char* v = getenv("TBE_B200_SCAN_POLLS");     // 0 makes every tile add up its own prefix (tests)
    static const int polls = (v && *v) ? atoi(v) : kChainPolls;
    return polls;
}

template <typename T, typename U, bool ALIGNED>
int big_tile_scan_launch(const void* in, int64_t n, void* out, TileState* states, int64_t tiles, int variant, cudaStream_t s)
{
    constexpr int kMaxDev = 64;
    static std::atomic<int> prepared[kMaxDev][4];          // the kernel's shared-memory limit is raised once per device
    auto kernel = big_tile_scan_kernel<T, U, ALIGNED>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(TBE_B200_ERR_CUDA, "complete_cumsum: no current device");
    if (dev < 0 || dev >= kMaxDev || prepared[dev][variant].load(std::memory_order_acquire) == 0) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBigSmemBytes) != cudaSuccess)
            return fail(TBE_B200_ERR_CUDA, "complete_cumsum: %d bytes of shared memory per block are not available", kBigSmemBytes);
        if (dev >= 0 && dev < kMaxDev) prepared[dev][variant].store(1, std::memory_order_release);
    }
    // One block per tile, in block order (blocks beyond 2^31 - 1 tiles take several); the hardware hands blocks out in
    // order, so the tiles a block waits for started before it did.
    const unsigned grid = static_cast<unsigned>(tiles < 0x7fffffffll ? tiles : 0x7fffffffll);
    kernel<<<grid, kBigThreads, kBigSmemBytes, s>>>(static_cast<const T*>(in), n, static_cast<T*>(out), states, tiles, chained_polls());
    return check_launch("complete_cumsum");
}

int complete_cumsum_chained_launch(const void* in, int64_t n, int index_bits, void* out, void* scratch, cudaStream_t s)
{
    const int64_t tiles = chained_tiles(n, index_bits);
    TileState* states = nullptr;
    if (tiles > 1) {
        const uintptr_t a = (reinterpret_cast<uintptr_t>(scratch) + 15) & ~static_cast<uintptr_t>(15);
        states = reinterpret_cast<TileState*>(a);
        if (cudaMemsetAsync(states, 0, static_cast<size_t>(tiles) * sizeof(TileState), s) != cudaSuccess)
            return fail(TBE_B200_ERR_CUDA, "complete_cumsum: memset failed");
    }
    const bool aligned = (reinterpret_cast<uintptr_t>(in) & 15) == 0;
    if (index_bits == 32)
        return aligned ? big_tile_scan_launch<int32_t, uint32_t, true>(in, n, out, states, tiles, 0, s)
                       : big_tile_scan_launch<int32_t, uint32_t, false>(in, n, out, states, tiles, 1, s);
    return aligned ? big_tile_scan_launch<int64_t, unsigned long long, true>(in, n, out, states, tiles, 2, s)
                   : big_tile_scan_launch<int64_t, unsigned long long, false>(in, n, out, states, tiles, 3, s);
}

}  // namespace tbe

extern "C" int64_t tbe_b200_complete_cumsum_scratch_bytes(int64_t n)
{
    return tbe::chained_scratch_bytes(n < 0 ? 0 : n);
}

extern "C" int tbe_b200_complete_cumsum(const void* in, int64_t n, int index_bits, void* out, void* scratch, int64_t scratch_bytes,
                                        tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (n < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum: n must be non-negative");
    if (index_bits != 32 && index_bits != 64)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum: index_bits must be 32 or 64, got %d", index_bits);
    if (!out || (n > 0 && !in)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum: a required pointer is NULL");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (n == 0) {
        if (cudaMemsetAsync(out, 0, index_bits / 8, s) != cudaSuccess) return fail(TBE_B200_ERR_CUDA, "complete_cumsum: memset failed");
        return TBE_B200_OK;
    }
    const int64_t need = tbe_b200_complete_cumsum_scratch_bytes(n);
    if (need > 0 && (!scratch || scratch_bytes < need))
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum: %lld bytes of scratch are needed, got %lld", static_cast<long long>(need),
                    static_cast<long long>(scratch ? scratch_bytes : 0));
    return complete_cumsum_chained_launch(in, n, index_bits, out, scratch, s);
}

extern "C" int64_t tbe_b200_permute_2d_sparse_scratch_bytes(int64_t T_in, int64_t T_out)
{
    if (T_in < 0 || T_out < 0) return 0;
    return (T_in + (T_in + 1) + (T_out + 1)) * 8;
}

// Scratch layout: seg_len[T_in], in_off[T_in + 1], out_off[T_out + 1], all int64.
extern "C" int tbe_b200_permute_2d_sparse_offsets(const int32_t* permute, int64_t T_out, const void* lengths, int lengths_bits, int64_t T_in,
                                                  int64_t B, void* out_lengths, void* scratch, int64_t scratch_bytes, int32_t* error_flag,
                                                  tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (T_in <= 0 || T_out <= 0 || B <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: T_in, T_out and B must be positive");
    if (lengths_bits != 32 && lengths_bits != 64)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: lengths must be int32 or int64, got %d bits", lengths_bits);
    if (!permute || !lengths || !out_lengths || !scratch) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: a required pointer is NULL");
    if (scratch_bytes < tbe_b200_permute_2d_sparse_scratch_bytes(T_in, T_out))
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: %lld bytes of scratch are needed, got %lld",
                    static_cast<long long>(tbe_b200_permute_2d_sparse_scratch_bytes(T_in, T_out)), static_cast<long long>(scratch_bytes));
    if (T_in > 65535 || T_out > 65535) return fail(TBE_B200_ERR_UNSUPPORTED, "permute_2d_sparse: at most 65535 tables");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    int64_t* seg_len = static_cast<int64_t*>(scratch);
    int64_t* in_off = seg_len + T_in;
    int64_t* out_off = in_off + T_in + 1;
    if (cudaMemsetAsync(seg_len, 0, static_cast<size_t>(T_in) * 8, s) != cudaSuccess)
        return fail(TBE_B200_ERR_CUDA, "permute_2d_sparse: memset failed");
    const int64_t per_row = (B + 256 * 8 - 1) / (256 * 8);
    const unsigned gx = static_cast<unsigned>(per_row < 64 ? per_row : 64);
    if (lengths_bits == 32) {
        segment_lengths_kernel<int32_t><<<dim3(gx, static_cast<unsigned>(T_in)), 256, 0, s>>>(static_cast<const int32_t*>(lengths), B, seg_len);
    } else {
        segment_lengths_kernel<int64_t><<<dim3(gx, static_cast<unsigned>(T_in)), 256, 0, s>>>(static_cast<const int64_t*>(lengths), B, seg_len);
    }
    segment_offsets_kernel<<<1, kScanThreads, 0, s>>>(seg_len, T_in, permute, T_out, in_off, out_off, error_flag);
    if (lengths_bits == 32) {
        permute_lengths_kernel<int32_t><<<dim3(gx, static_cast<unsigned>(T_out)), 256, 0, s>>>(static_cast<const int32_t*>(lengths), T_in, B, permute,
                                                                                                static_cast<int32_t*>(out_lengths));
    } else {
        permute_lengths_kernel<int64_t><<<dim3(gx, static_cast<unsigned>(T_out)), 256, 0, s>>>(static_cast<const int64_t*>(lengths), T_in, B, permute,
                                                                                                static_cast<int64_t*>(out_lengths));
    }
    return check_launch("permute_2d_sparse_offsets");
}

extern "C" int tbe_b200_permute_2d_sparse_copy(const int32_t* permute, int64_t T_out, int64_t T_in, const void* values, int64_t value_bytes,
                                               const void* weights, int64_t weight_row_bytes, void* out_values, void* out_weights,
                                               int64_t out_capacity, const void* scratch, tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (T_in <= 0 || T_out <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: T_in and T_out must be positive");
    if (out_capacity < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: out_capacity must be non-negative");
    if (!permute || !scratch) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: a required pointer is NULL");
    if (out_capacity == 0) return TBE_B200_OK;
    if (!values || !out_values || value_bytes <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: values are missing");
    if (weights && (!out_weights || weight_row_bytes <= 0)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse: weights output is missing");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int64_t* seg_len = static_cast<const int64_t*>(scratch);
    const int64_t* in_off = seg_len + T_in;
    const int64_t* out_off = in_off + T_in + 1;
    int rc = copy_segments(values, out_values, value_bytes, out_capacity, permute, T_in, T_out, in_off, out_off, s);
    if (rc != TBE_B200_OK) return rc;
    if (weights) rc = copy_segments(weights, out_weights, weight_row_bytes, out_capacity, permute, T_in, T_out, in_off, out_off, s);
    return rc;
}

extern "C" int tbe_b200_permute_2d_sparse_copy_to_dests(const int32_t* permute, int64_t T_out, int64_t T_in, const void* values,
                                                        int64_t value_bytes, const int64_t* dest_bases, int64_t tables_per_dest,
                                                        int64_t dest_capacity, int64_t total_hint, const void* scratch, int32_t* error_flag,
                                                        tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (T_in <= 0 || T_out <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse_copy_to_dests: T_in and T_out must be positive");
    if (tables_per_dest <= 0 || T_out % tables_per_dest != 0)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse_copy_to_dests: T_out (%lld) must be a multiple of tables_per_dest (%lld)",
                    static_cast<long long>(T_out), static_cast<long long>(tables_per_dest));
    if (dest_capacity < 0 || total_hint < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse_copy_to_dests: negative size");
    if (!permute || !scratch || !dest_bases) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse_copy_to_dests: a required pointer is NULL");
    if (total_hint == 0) return TBE_B200_OK;
    if (!values || value_bytes <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "permute_2d_sparse_copy_to_dests: values are missing");
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int64_t* seg_len = static_cast<const int64_t*>(scratch);
    const int64_t* in_off = seg_len + T_in;
    const int64_t* out_off = in_off + T_in + 1;
    // unit of the copy: the widest that divides a value and the source address (destinations are 16-byte aligned)
    const uintptr_t a = reinterpret_cast<uintptr_t>(values);
    int unit = 16;
    while (unit > 1 && (value_bytes % unit != 0 || a % unit != 0)) unit >>= 1;
    const int64_t upp = value_bytes / unit;
    const int64_t units = total_hint * upp;
    const int64_t want = (units + 256 * 8 - 1) / (256 * 8);
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const unsigned blocks = static_cast<unsigned>(want < cap ? want : cap);
    const int64_t n_dest = T_out / tables_per_dest;
    if ((value_bytes == 8 || value_bytes == 4) && a % value_bytes == 0 && n_dest <= kMaxPairDests) {
        const int64_t pairs = (total_hint + 1) / 2 + n_dest;
        const int64_t want2 = (pairs + 256 * 4 - 1) / (256 * 4);
        const unsigned blocks2 = static_cast<unsigned>(want2 < cap ? want2 : cap);
        if (value_bytes == 8)
            permute_pairs_to_dests_kernel<unsigned long long, ulonglong2><<<blocks2, 256, 0, s>>>(
                static_cast<const unsigned long long*>(values), dest_bases, tables_per_dest, dest_capacity, static_cast<int>(n_dest), permute, T_in,
                T_out, in_off, out_off, error_flag);
        else
            permute_pairs_to_dests_kernel<uint32_t, uint2><<<blocks2, 256, 0, s>>>(static_cast<const uint32_t*>(values), dest_bases, tables_per_dest,
                                                                                 dest_capacity, static_cast<int>(n_dest), permute, T_in, T_out, in_off,
                                                                                 out_off, error_flag);
        return check_launch("permute_pairs_to_dests_kernel");
    }
#define TBE_TO_DESTS(VT)                                                                                                                      \
    permute_segments_to_dests_kernel<VT><<<blocks, 256, 0, s>>>(static_cast<const VT*>(values), dest_bases, tables_per_dest, dest_capacity, upp, \
                                                                permute, T_in, T_out, in_off, out_off, error_flag)
    switch (unit) {
        case 16: TBE_TO_DESTS(uint4); break;
        case 8: TBE_TO_DESTS(uint64_t); break;
        case 4: TBE_TO_DESTS(uint32_t); break;
        case 2: TBE_TO_DESTS(uint16_t); break;
        default: TBE_TO_DESTS(uint8_t); break;
    }
#undef TBE_TO_DESTS
    return check_launch("permute_segments_to_dests_kernel");
}

// ---- complete cumsum for callers that must not allocate ---------------------------------------
//
// The tile sums live in a fixed array inside the library image instead of caller-provided scratch.
// Every GPU that loads the library carries these 64 KB until the process ends.

namespace tbe {
namespace {

constexpr int64_t kStaticTiles = 8192;                               // 8192 tile sums = 64 KB
constexpr int64_t kStaticMaxElements = kStaticTiles * kScanTile;     // 16 777 216 input elements
constexpr int kCachedDevices = 64;

static __device__ __align__(256) int64_t g_static_tile_sums[kStaticTiles];

// Device address of the array on the current device.  In host code `g_static_tile_sums` is only a handle
// for the runtime, never a pointer a kernel may use; the address is looked up once per device and kept.
int static_tile_sums(int64_t** out)
{
    static std::mutex lock;
    static int64_t* cached[kCachedDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(TBE_B200_ERR_CUDA, "complete_cumsum_static: no current device");
    std::lock_guard<std::mutex> g(lock);
    if (dev >= 0 && dev < kCachedDevices && cached[dev]) {
        *out = cached[dev];
        return TBE_B200_OK;
    }
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_tile_sums);
    if (e != cudaSuccess || !p)
        return fail(TBE_B200_ERR_CUDA, "complete_cumsum_static: the scratch array has no address on device %d (%s)", dev, cudaGetErrorString(e));
    if (dev >= 0 && dev < kCachedDevices) cached[dev] = static_cast<int64_t*>(p);
    *out = static_cast<int64_t*>(p);
    return TBE_B200_OK;
}

}  // namespace
}  // namespace tbe

extern "C" int64_t tbe_b200_complete_cumsum_static_max_elements(void) { return tbe::kStaticMaxElements; }

extern "C" int tbe_b200_complete_cumsum_static(const void* in, int64_t n, int index_bits, void* out, tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (n < 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum_static: n must be non-negative");
    if (index_bits != 32 && index_bits != 64)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum_static: index_bits must be 32 or 64, got %d", index_bits);
    if (!out || (n > 0 && !in)) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "complete_cumsum_static: a required pointer is NULL");
    if (n > kStaticMaxElements)
        return fail(TBE_B200_ERR_UNSUPPORTED,
                    "complete_cumsum_static: %lld elements exceed the built-in scratch (at most %lld); use tbe_b200_complete_cumsum "
                    "with caller-provided scratch",
                    static_cast<long long>(n), static_cast<long long>(kStaticMaxElements));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (n == 0) {
        if (cudaMemsetAsync(out, 0, index_bits / 8, s) != cudaSuccess) return fail(TBE_B200_ERR_CUDA, "complete_cumsum_static: memset failed");
        return TBE_B200_OK;
    }
    int64_t* tile_sums = nullptr;
    const int rc = static_tile_sums(&tile_sums);
    if (rc != TBE_B200_OK) return rc;
    // Every tile sum the scan reads is written by the first kernel of this call, so nothing has to be cleared.
    return complete_cumsum_launch(in, n, index_bits, out, tile_sums, s);
}
