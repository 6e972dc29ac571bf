// A barrier between the ranks of one NVLink box, run as a one-block kernel on the caller's stream: every rank stores
// its epoch into its slot of every peer's flag buffer (peer-mapped memory, plain stores over NVLink) and waits until
// every slot of its own buffer has reached that epoch.  It replaces the one-float ncclAllReduce that ordered the ranks
// after the fused peer-store steps (about 20 us per barrier at eight GPUs against about 5 us here).
//
// Each rank runs on its own GPU, so the kernels that wait on one another never share a device.  The wait is bounded:
// after `limit_cycles` SM clock cycles the kernel records status 301 and returns, and the context stays usable.
// Ordering: the kernel before this one on the stream has completed (its peer stores are performed), a system-scope
// fence precedes the flag stores, and the waiting loads are acquire loads at system scope, so whatever a peer wrote
// before its barrier is visible to the kernel after this one.
//
// Flag buffer of a rank: 32 words, zero-filled once by the caller before first use: [0, 8) arrival slots, one per
// sending rank; [16] the rank's own epoch, advanced by every barrier.  Every rank must run the same sequence of barriers.

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/baracuda_kernels_q.h"
#include "launch.h"

namespace bq {

namespace {

__device__ int g_peer_barrier_device_status = 0;

struct PeerFlags {
    uint32_t* f[BARACUDA_Q_MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(32) peer_flag_barrier_kernel(PeerFlags flags, int rank, int world, long long limit_cycles) {
    uint32_t* mine = flags.f[rank];
    const int t = threadIdx.x;
    const uint32_t epoch = mine[16] + 1u;  // only this kernel writes it, one launch at a time on the stream
    __syncwarp();
    if (t < world) {
        __threadfence_system();
        st_release_sys(flags.f[t] + rank, epoch);
        const long long t0 = clock64();
        // wrap-safe comparison: the slot has reached the epoch when the signed difference is not negative
        while (static_cast<int32_t>(ld_acquire_sys(mine + t) - epoch) < 0) {
            if (clock64() - t0 > limit_cycles) {
                atomicCAS(&g_peer_barrier_device_status, 0, 301);
                break;
            }
            __nanosleep(64);
        }
    }
    __syncwarp();
    if (t == 0) mine[16] = epoch;
}

}  // namespace

int32_t launch_peer_flag_barrier(void* const* peer_flags, int32_t rank, int32_t world, long long limit_cycles,
                                 cudaStream_t stream) {
    if (!peer_flags || world < 1 || world > BARACUDA_Q_MAX_PEERS || rank < 0 || rank >= world) return BQ_STATUS_INVALID_PROBLEM;
    PeerFlags f;
    for (int i = 0; i < BARACUDA_Q_MAX_PEERS; ++i) {
        f.f[i] = i < world ? static_cast<uint32_t*>(peer_flags[i]) : nullptr;
        if (i < world && (!peer_flags[i] || (reinterpret_cast<uintptr_t>(peer_flags[i]) & 3u) != 0)) return BQ_STATUS_INVALID_PROBLEM;
    }
    if (limit_cycles <= 0 || limit_cycles > (1LL << 31)) limit_cycles = 1LL << 31;  // about a second
    peer_flag_barrier_kernel<<<1, 32, 0, stream>>>(f, rank, world, limit_cycles);
    return cudaPeekAtLastError() == cudaSuccess ? BQ_STATUS_OK : BQ_STATUS_LAUNCH_FAILURE;
}

int32_t read_and_clear_peer_barrier_device_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_barrier_device_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        int zero = 0;
        (void)cudaMemcpyToSymbol(g_peer_barrier_device_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace bq
