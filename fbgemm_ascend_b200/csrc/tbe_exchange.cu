// Step flags between the ranks of a table-wise sharded lookup (one process per GPU, peer-mapped memory).
//
// After its lookup kernel has stored pooled rows into the other ranks' output buffers, a rank raises a flag in every
// peer's memory; before a rank hands its output on, it waits until every peer's flag for that step is up.  The
// reference has no multi-device code, so there is no counterpart to cite.  The wait is bounded: after max_polls
// polls the kernel records bit 16 in the error word and returns, so a rank that died between steps cannot leave
// the others' GPUs spinning.  Plain peer stores and loads only (no multicast, no multimem).
#include "tbe_common.cuh"

namespace tbe {
namespace {

__global__ void signal_peers_kernel(int64_t* const* peer_flags, int world, int my_rank, int64_t value)
{
    for (int r = threadIdx.x; r < world; r += blockDim.x) {
        int64_t* dst = peer_flags[r] + my_rank;
        // Everything this GPU wrote before this kernel (the lookup's peer stores among it) is ordered before the flag.
        __threadfence_system();
        asm volatile("st.release.sys.global.b64 [%0], %1;" ::"l"(dst), "l"(value) : "memory");
    }
}

__global__ void wait_flags_kernel(const int64_t* flags, int world, int64_t value, int64_t max_polls, int32_t* error_flag)
{
    for (int r = threadIdx.x; r < world; r += blockDim.x) {
        const int64_t* src = flags + r;
        bool up = false;
        for (int64_t t = 0; t < max_polls; ++t) {
            int64_t v;
            asm volatile("ld.acquire.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(src) : "memory");
            if (v >= value) {
                up = true;
                break;
            }
            __nanosleep(t < 64 ? 100 : 1000);
        }
        if (!up && error_flag) atomicOr(error_flag, 16);
    }
}

}  // namespace
}  // namespace tbe

extern "C" int tbe_b200_signal_peers(int64_t* const* peer_flags, int32_t world, int32_t my_rank, int64_t value,
                                     tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (!peer_flags || world <= 0 || my_rank < 0 || my_rank >= world)
        return fail(TBE_B200_ERR_INVALID_ARGUMENT, "signal_peers: need peer_flags and 0 <= my_rank < world, got rank %d of %d", my_rank, world);
    signal_peers_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(peer_flags, world, my_rank, value);
    return check_launch("signal_peers_kernel");
}

extern "C" int tbe_b200_wait_flags(const int64_t* flags, int32_t world, int64_t value, int64_t max_polls, int32_t* error_flag,
                                   tbe_b200_stream_t stream)
{
    using namespace tbe;
    if (!flags || world <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "wait_flags: need flags and world > 0");
    if (max_polls <= 0) return fail(TBE_B200_ERR_INVALID_ARGUMENT, "wait_flags: max_polls must be positive (the wait is always bounded)");
    wait_flags_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flags, world, value, max_polls, error_flag);
    return check_launch("wait_flags_kernel");
}
