// All-gather of the per-rank attention outputs over peer memory (NVLink / NVSwitch).
//
// Heads are sharded over the GPUs of a node, so the only data that ever crosses NVLink is the
// [batch, heads/N, head_dim] output of a step -- tens of kilobytes.  For a message that small a
// collective library's launch and protocol cost is several times the wire time, so every rank
// PUSHES its slice straight into each peer's buffer with 16-byte stores, raises one flag per
// peer, and waits (bounded) for the flags of the slices it receives.  The destination is laid
// out [batch, N * heads/N, head_dim], so the gathered tensor needs no permutation afterwards.
//
// One CTA per peer.  Sending never waits, so no rank can block another; a wait that runs out
// sets the time-out bit of the status word and the kernel returns normally.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ffa_device_common.cuh"
#include "ffa_internal.h"

using namespace ffa_dev;

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int kGatherPushThreads = 256;

__global__ void __launch_bounds__(kGatherPushThreads) ffa_peer_gather_kernel(const FfaPeerGatherParams G)
{
    const int r = blockIdx.x, tid = threadIdx.x;   // this CTA talks to rank r
    if (G.phases & 1) {
        // slice of batch row b goes to bytes [(b * world + rank) * row_bytes, +row_bytes) of the destination
        const int vec_per_row = G.row_bytes >> 4;
        const long long total = (long long)G.B * vec_per_row;
        const uint4* src = static_cast<const uint4*>(G.out_local);
        unsigned char* dst = static_cast<unsigned char*>(G.peer_half[r]);
        for (long long i = tid; i < total; i += kGatherPushThreads) {
            const long long b = i / vec_per_row;
            const int x = (int)(i - b * vec_per_row);
            *reinterpret_cast<uint4*>(dst + ((size_t)b * G.world + G.rank) * G.row_bytes + (size_t)x * 16) = src[i];
        }
        if (r != G.rank) {
            __threadfence_system();   // every thread's stores are performed at the peer before the flag
            __syncthreads();
            if (tid == 0) st_release_sys(G.peer_flags[r] + G.rank, G.seq);
        }
    }
    if ((G.phases & 2) && r != G.rank && tid == 0) {
        // rank r's slice of this step has landed once its flag has reached this step's number
        const unsigned long long t0 = global_timer_ns();
        bool ok = false;
        for (;;) {
            if ((int32_t)(ld_acquire_sys(G.local_flags + r) - G.seq) >= 0) {
                ok = true;
                break;
            }
            if (global_timer_ns() - t0 > G.wait_limit_ns) break;
            __nanosleep(200);
        }
        if (!ok) atomicOr(G.status, kStatusWaitTimeout);
    }
}

}  // namespace

int ffa_k_peer_gather(const FfaPeerGatherParams& G, cudaStream_t stream)
{
    ffa_peer_gather_kernel<<<G.world, kGatherPushThreads, 0, stream>>>(G);
    return (int)cudaGetLastError();
}
