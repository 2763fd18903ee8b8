// Row-gather ceiling probe for B200 (sm_100a): how many table rows per second can be fetched at all
// under a given index distribution, with no dequantisation or pooling behind the fetch?
//
// The pooled lookup reads rows of `stride` bytes (144 for INT8 D=128, 80 for INT4 D=128) scattered over
// tables far larger than L2, so the copy bandwidth of the device is not its ceiling: every row touches
// two or three 64-byte DRAM atoms and one or two 128-byte lines whatever its payload, and very large
// tables also run out of TLB reach.  This program measures that ceiling directly, with the lookup
// kernel's two fetch methods, so that the kernel's rows/s can be judged against what the memory
// system delivers for the same access pattern:
//   ldg   8 lanes x 16 bytes per row plus the 4-byte tail word, 4 passes (16 rows) in flight per warp
//   bulk  one cp.async.bulk per row (one row per lane, 32 rows per warp in flight) into shared memory,
//         completion on an mbarrier, rows read back with 16-byte shared loads
// Row ids are drawn once into a device array (uniform, or bounded Zipf scattered by a multiplicative
// permutation, per table; samples are table-major like the lookup's bags) and streamed by the gather
// kernels, as the lookup streams `indices`.
//
// Usage: tbe_b200_row_gather_probe [max_gib]      (tables larger than max_gib GiB are skipped; default 120)
// Output: one line per (distribution, stride, method): rows/s and the bytes/s they stand for.
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include <cuda_runtime.h>

#define CK(x)                                                                              \
    do {                                                                                   \
        cudaError_t e_ = (x);                                                              \
        if (e_ != cudaSuccess) {                                                           \
            printf("cuda error: %s (line %d)\n", cudaGetErrorString(e_), __LINE__);        \
            exit(1);                                                                       \
        }                                                                                  \
    } while (0)

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kBlocksPerSM = 8;
constexpr int kWaitTries = 1 << 22;

__device__ __forceinline__ uint32_t hash32(uint32_t x)
{
    x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
    return x;
}

// Row id of sample s: table = s * T / n; rank ~ bounded Zipf(alpha) over N rows (alpha == 0: uniform);
// rank -> row by an odd multiplier modulo N, so hot rows are scattered.
__global__ void draw_rows(uint32_t* rows, uint64_t n, uint32_t T, uint32_t N, float alpha, float c /* N^(1-alpha) - 1 */)
{
    const uint64_t s = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (s >= n) return;
    const uint32_t h = hash32(static_cast<uint32_t>(s) * 2654435761u + 12345u);
    // Table-major, like the lookup's bag order: the warps that run at the same time work on the same one or
    // two tables, so the live footprint is a table, not the whole shard.
    const uint32_t t = static_cast<uint32_t>(s * T / n);
    uint32_t r;
    if (alpha == 0.0f) {
        r = static_cast<uint32_t>((static_cast<uint64_t>(h) * N) >> 32);
    } else {
        const double u = (static_cast<double>(h) + 0.5) / 4294967296.0;
        const double rank = pow(1.0 + u * static_cast<double>(c), 1.0 / (1.0 - static_cast<double>(alpha)));   // in [1, N]
        uint64_t k = static_cast<uint64_t>(rank) - 1;
        if (k >= N) k = N - 1;
        r = static_cast<uint32_t>((k * 2654435761ull) % N);
    }
    rows[s] = t * N + r;   // T * N < 2^32 in every configuration below
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32) gather_ldg(const uint8_t* table, const uint32_t* rows, uint32_t stride,
                                                                   uint32_t chunks, uint32_t rows_per_warp, uint32_t* sink)
{
    constexpr int UNR = 4;
    const int lane = threadIdx.x & 31, k = lane & 7, g = lane >> 3;
    const uint64_t gw = static_cast<uint64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    // Round r of every warp reads one contiguous stretch of the sample array, so all warps move through the
    // tables together, as the blocks of the lookup kernel do.
    const uint64_t round_pitch = static_cast<uint64_t>(gridDim.x) * kWarpsPerBlock * 32;
    const uint32_t* mine = rows + gw * 32;
    uint32_t acc = 0;
    for (uint32_t r = 0; r < rows_per_warp; r += 32) {
        const uint32_t my_row = __ldg(mine + (r / 32) * round_pitch + lane);
        for (int u0 = 0; u0 < 8; u0 += UNR) {
            uint4 v[UNR];
            uint32_t t[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t row = __shfl_sync(0xffffffffu, my_row, (u0 + u) * 4 + g);
                const uint8_t* p = table + static_cast<uint64_t>(row) * stride;
                v[u] = make_uint4(0, 0, 0, 0);
                t[u] = 0;
                if (k < chunks) v[u] = __ldg(reinterpret_cast<const uint4*>(p + k * 16));
                if (k == 0) t[u] = __ldg(reinterpret_cast<const uint32_t*>(p + chunks * 16));
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w ^ t[u];
        }
    }
    if (acc == 0x12345678u) sink[0] = acc;
}

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// Every wait is bounded; a wait that runs out sets *err and ends the warp.
__global__ void __launch_bounds__(kWarpsPerBlock * 32) gather_bulk(const uint8_t* table, const uint32_t* rows, uint32_t stride,
                                                                    uint32_t chunks, uint32_t rows_per_warp, uint32_t* sink,
                                                                    uint32_t* err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[kWarpsPerBlock];
    const int lane = threadIdx.x & 31, k = lane & 7, g = lane >> 3, warp = threadIdx.x >> 5;
    const uint64_t gw = static_cast<uint64_t>(blockIdx.x) * kWarpsPerBlock + warp;
    const uint64_t round_pitch = static_cast<uint64_t>(gridDim.x) * kWarpsPerBlock * 32;
    const uint32_t* mine = rows + gw * 32;
    const uint32_t bar = s32(&bars[warp]);
    const uint32_t base = s32(smem) + warp * 32 * stride;
    if (lane == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(32));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t acc = 0, parity = 0;
    for (uint32_t r = 0; r < rows_per_warp; r += 32) {
        const uint8_t* src = table + static_cast<uint64_t>(__ldg(mine + (r / 32) * round_pitch + lane)) * stride;
        __syncwarp();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stride) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(base + lane * stride),
                     "l"(src), "r"(stride), "r"(bar)
                     : "memory");
        uint32_t done = 0;
        for (int spin = 0; spin < kWaitTries && !done; ++spin)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done)
                         : "r"(bar), "r"(parity)
                         : "memory");
        if (!done) {
            if (lane == 0) atomicOr(err, 1u);
            return;
        }
        parity ^= 1u;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t a = base + (u * 4 + g) * stride;
            uint4 v = make_uint4(0, 0, 0, 0);
            uint32_t h, t = 0;
            if (k < chunks) asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a + k * 16));
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(h) : "r"(a));
            if (k == 0) asm volatile("ld.shared.b32 %0, [%1];" : "=r"(t) : "r"(a + chunks * 16));
            acc ^= v.x ^ v.y ^ v.z ^ v.w ^ h ^ t;
        }
    }
    if (acc == 0x12345678u) sink[0] = acc;
}

struct Dist {
    const char* name;
    uint32_t T, N;
    float alpha;
};

}  // namespace

int main(int argc, char** argv)
{
    const double max_gib = argc > 1 ? atof(argv[1]) : 120.0;
    int dev = 0, sms = 0;
    CK(cudaGetDevice(&dev));
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    uint32_t *sink, *err;
    CK(cudaMalloc(&sink, 4));
    CK(cudaMalloc(&err, 4));
    CK(cudaMemset(err, 0, 4));
    const Dist dists[] = {{"uniform, 26 tables x 1M rows", 26, 1000000, 0.0f},
                          {"zipf 1.05, 26 tables x 1M rows", 26, 1000000, 1.05f},
                          {"zipf 1.05, 64 tables x 600k rows", 64, 600000, 1.05f},
                          {"zipf 1.05, 64 tables x 12M rows", 64, 12000000, 1.05f},
                          {"uniform, 64 tables x 12M rows", 64, 12000000, 0.0f}};
    struct Shape { uint32_t stride, chunks; const char* what; } shapes[] = {{144, 8, "INT8 D=128"}, {80, 4, "INT4 D=128"}};
    const int blocks = sms * kBlocksPerSM;
    const uint64_t total = 32ull << 20;   // rows per launch
    const uint32_t rpw = static_cast<uint32_t>(total / (static_cast<uint64_t>(blocks) * kWarpsPerBlock) / 32 * 32);
    const uint64_t n = static_cast<uint64_t>(rpw) * blocks * kWarpsPerBlock;
    uint32_t* rows;
    CK(cudaMalloc(&rows, n * 4));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    CK(cudaFuncSetAttribute(gather_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, kWarpsPerBlock * 32 * 144));
    printf("row-gather ceiling probe: %d SMs, %d warps per SM, %llu rows per launch\n", sms, kBlocksPerSM * kWarpsPerBlock,
           static_cast<unsigned long long>(n));
    for (const Shape& sh : shapes) {
        for (const Dist& d : dists) {
            const size_t bytes = static_cast<size_t>(d.T) * d.N * sh.stride;
            if (static_cast<double>(bytes) > max_gib * 1073741824.0) {
                printf("%-34s %-10s skipped (%.1f GiB)\n", d.name, sh.what, bytes / 1073741824.0);
                continue;
            }
            uint8_t* table;
            CK(cudaMalloc(&table, bytes));
            CK(cudaMemset(table, 1, bytes));
            const float c = d.alpha == 0.0f ? 0.0f : powf(static_cast<float>(d.N), 1.0f - d.alpha) - 1.0f;
            draw_rows<<<static_cast<unsigned>((n + 255) / 256), 256>>>(rows, n, d.T, d.N, d.alpha, c);
            CK(cudaGetLastError());
            for (int method = 0; method < 2; ++method) {
                float best = 1e30f;
                for (int it = 0; it < 4; ++it) {
                    CK(cudaEventRecord(e0));
                    if (method == 0)
                        gather_ldg<<<blocks, kWarpsPerBlock * 32>>>(table, rows, sh.stride, sh.chunks, rpw, sink);
                    else
                        gather_bulk<<<blocks, kWarpsPerBlock * 32, kWarpsPerBlock * 32 * sh.stride>>>(table, rows, sh.stride, sh.chunks,
                                                                                                     rpw, sink, err);
                    CK(cudaEventRecord(e1));
                    CK(cudaEventSynchronize(e1));
                    CK(cudaGetLastError());
                    float ms;
                    CK(cudaEventElapsedTime(&ms, e0, e1));
                    if (it > 0 && ms < best) best = ms;
                }
                printf("%-34s %-10s %-4s %7.3f ms  %6.2f G rows/s  %5.0f GB/s of %u-byte rows\n", d.name, sh.what,
                       method == 0 ? "ldg" : "bulk", best, n / best / 1e6, static_cast<double>(n) * sh.stride / best / 1e6, sh.stride);
            }
            CK(cudaFree(table));
        }
    }
    uint32_t herr = 0;
    CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
    printf("waits that ran out: %u\n", herr);
    return herr ? 2 : 0;
}
