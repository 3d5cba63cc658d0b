// All-gather of the per-rank attention outputs over peer memory (NVLink / NVSwitch).
//
// Heads are sharded over the GPUs of a node, so the only data that ever crosses NVLink is the
// [batch, heads/N, head_dim] output of a step -- tens of kilobytes.  For a message that small a
// collective library's launch and protocol cost is several times the wire time, so every rank
// PUSHES its slice straight into a staging buffer of each peer with 16-byte stores, raises one
// flag per peer, waits (bounded) for the flag of the slice it receives from that peer, and
// copies the slice to its place in the caller's [batch, N * heads/N, head_dim] result -- no
// permutation afterwards.
//
// Staging buffer of a rank: half 0 | half 1 | flags[8], step counter, tickets (256 bytes).  A half is
// [batch][N][heads/N * head_dim]; the two halves alternate by step so that a peer already in
// step s+1 never overwrites what this rank still reads for step s (a peer cannot be two steps
// ahead: its wait of step s+1 needs this rank's flag of step s+1).  Flags hold step numbers and
// only grow.  The step number lives in the rank's own buffer and is advanced by the kernel
// (last CTA out, through the ticket), so every launch argument is the same for every step.
//
// A few CTAs per peer (one per 16 KB of slice).  Sending never waits, so no rank can block another; a wait that runs out
// sets the time-out bit of the status word and the kernel returns normally.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ffa_device_common.cuh"
#include "ffa_internal.h"

using namespace ffa_dev;

namespace {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

constexpr int kGatherPushThreads = 256;
constexpr int kVecPerThread = 4;      // 16-byte vectors a thread moves per phase, all loads before the first store
constexpr int kMaxSlices = 16;        // CTAs per peer

constexpr int kTailFlags = kPeerTailFlags, kTailCounter = kPeerTailCounter, kTailTicket = kPeerTailTicket,
              kTailPushTickets = kPeerTailPushTickets;

// Moves vectors [lo, hi) of a [B][row_bytes] slice: `from` and `to` map a vector index to its address.
template <typename From, typename To>
__device__ __forceinline__ void move_vectors(long long lo, long long hi, int tid, From from, To to)
{
    for (long long base = lo + tid; base < hi; base += (long long)kGatherPushThreads * kVecPerThread) {
        uint4 v[kVecPerThread];
#pragma unroll
        for (int k = 0; k < kVecPerThread; ++k) {
            const long long i = base + (long long)k * kGatherPushThreads;
            if (i < hi) v[k] = from(i);
        }
#pragma unroll
        for (int k = 0; k < kVecPerThread; ++k) {
            const long long i = base + (long long)k * kGatherPushThreads;
            if (i < hi) *to(i) = v[k];
        }
    }
}

// grid = world * slices: CTA (r, sl) moves slice sl of what this rank exchanges with rank r.
__global__ void __launch_bounds__(kGatherPushThreads) ffa_peer_gather_kernel(const FfaPeerGatherParams G)
{
    const int r = blockIdx.x / G.slices, sl = blockIdx.x - r * G.slices, tid = threadIdx.x;
    const bool push = (G.phases & 1) != 0, wait = (G.phases & 2) != 0;
    unsigned char* own = static_cast<unsigned char*>(G.peer_base[G.rank]);
    uint32_t* own_tail = reinterpret_cast<uint32_t*>(own + 2 * G.half_bytes);
    volatile uint32_t* counter = own_tail + kTailCounter;
    // a push opens step counter + 1; a lone wait refers to the latest push
    const uint32_t seq = *counter + (push ? 1u : 0u);
    const size_t half_off = (size_t)(seq & 1u) * G.half_bytes;
    const int vec_per_row = G.row_bytes >> 4;
    const long long total = (long long)G.B * vec_per_row;
    const long long per = (total + G.slices - 1) / G.slices;
    const long long lo = min(total, (long long)sl * per), hi = min(total, lo + per);
    // the slice of batch row b sits at bytes [(b * world + rank) * row_bytes, +row_bytes)
    auto slot = [&](long long i, int rank) -> size_t {
        const long long b = i / vec_per_row;
        return ((size_t)b * G.world + rank) * G.row_bytes + (size_t)(i - b * vec_per_row) * 16;
    };

    if (push) {
        const uint4* src = static_cast<const uint4*>(G.out_local);
        if (r == G.rank) {   // the own slice goes straight to the result
            unsigned char* dst = static_cast<unsigned char*>(G.gathered);
            move_vectors(lo, hi, tid, [&](long long i) { return src[i]; },
                         [&](long long i) { return reinterpret_cast<uint4*>(dst + slot(i, G.rank)); });
        } else {
            unsigned char* peer = static_cast<unsigned char*>(G.peer_base[r]);
            unsigned char* dst = peer + half_off;
            move_vectors(lo, hi, tid, [&](long long i) { return src[i]; },
                         [&](long long i) { return reinterpret_cast<uint4*>(dst + slot(i, G.rank)); });
            __threadfence_system();   // every thread's stores are performed at the peer before the flag
            __syncthreads();
            if (tid == 0) {
                // the CTA that finishes last raises the flag, after everybody's stores
                uint32_t* ticket = own_tail + kTailPushTickets + r;
                if (atomicAdd(ticket, 1u) == (uint32_t)G.slices - 1u) {
                    *ticket = 0;
                    __threadfence_system();
                    st_release_sys(reinterpret_cast<uint32_t*>(peer + 2 * G.half_bytes) + kTailFlags + G.rank, seq);
                }
            }
        }
    }
    if (wait && r != G.rank) {
        // rank r's slice of this step has landed once its flag has reached this step's number
        if (tid == 0) {
            const unsigned long long t0 = global_timer_ns();
            bool ok = false;
            for (;;) {
                if ((int32_t)(ld_acquire_sys(own_tail + kTailFlags + r) - seq) >= 0) {
                    ok = true;
                    break;
                }
                if (global_timer_ns() - t0 > G.wait_limit_ns) break;
                __nanosleep(200);
            }
            if (!ok) atomicOr(G.status, kStatusWaitTimeout);
        }
        __syncthreads();
        const unsigned char* src = own + half_off;
        unsigned char* dst = static_cast<unsigned char*>(G.gathered);
        move_vectors(lo, hi, tid, [&](long long i) { return __ldcg(reinterpret_cast<const uint4*>(src + slot(i, r))); },   // written by a peer: read at L2
                     [&](long long i) { return reinterpret_cast<uint4*>(dst + slot(i, r)); });
    }
    if (push) {
        // every CTA has read the counter by now; the last one out advances it
        __syncthreads();
        if (tid == 0) {
            uint32_t* ticket = own_tail + kTailTicket;
            if (atomicAdd(ticket, 1u) == (uint32_t)(G.world * G.slices) - 1u) {
                *ticket = 0;
                *counter = seq;
            }
        }
    }
}

}  // namespace

int ffa_k_peer_gather(FfaPeerGatherParams G, cudaStream_t stream)
{
    const long long vectors = (long long)G.B * (G.row_bytes >> 4);
    long long slices = (vectors + kGatherPushThreads * kVecPerThread - 1) / (kGatherPushThreads * kVecPerThread);
    G.slices = (int)(slices < 1 ? 1 : slices > kMaxSlices ? kMaxSlices : slices);
    ffa_peer_gather_kernel<<<G.world * G.slices, kGatherPushThreads, 0, stream>>>(G);
    return (int)cudaGetLastError();
}
