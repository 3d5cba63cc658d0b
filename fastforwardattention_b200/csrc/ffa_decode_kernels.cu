// Decode masked multi-head attention for sm_100a: launch glue for the kernels in
// ffa_stream_kernel.cuh and ffa_prune_kernels.cuh, the cache-build kernel and a diagnostic.
//
// Replaces mmha::masked_multihead_attention_kernel_optimized (attention.cu:698-1295) and the
// two cache-init kernels (attention.cu:1556-1609) of the reference.  The reference runs one
// CTA per (batch, head) that walks the whole sequence serially and stages every score in
// shared memory; here the flat list of (batch*head, row-tile) units is cut into contiguous
// runs, one per CTA of a persistent grid, so all SMs stream from HBM whatever the batch*head
// count and the sequence length is bounded by memory only.
//
//   ffa_stream_kernel<T, DH>              p == 0: K and V tiles through a bulk-copy ring,
//                                         online softmax, cross-CTA merge by the CTA that
//                                         arrives last (no waiting), k/v append fused
//   ffa_prune_stream_kernel<T, DH>        p > 0 on large steps, one persistent launch: K tiles
//                                         through the ring, fp32 scores to scratch, global max
//                                         and sum; gather warps test every cached row with the
//                                         reference's pruning rule (attention.cu:1184-1191,
//                                         461-469) and load only the V rows that survive, while
//                                         the next pairs' K rows keep streaming
//   ffa_prune_cluster_kernel<T, DH>       p > 0 on small and mid-size steps, and the torch-rounding
//                                         mode: a thread-block cluster per (batch, head), scores in
//                                         shared memory, statistics and partial outputs over
//                                         distributed shared memory; surviving V rows gathered, or
//                                         the V tiles streamed where little or nothing is pruned
//   ffa_cache_init_kernel                 prompt K/V -> rows [0, prompt) of the caches
//
// One query row per head is a matrix-vector product (2 flops per cache element read), so the
// arithmetic runs on the CUDA cores in fp32 and the kernels are bound by HBM bandwidth.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstring>
#include <type_traits>

#include "ffa_internal.h"
#include "ffa_device_common.cuh"
#include "ffa_prune_kernels.cuh"
#include "ffa_prune_stream_kernel.cuh"
#include "ffa_stream_kernel.cuh"

using namespace ffa_dev;

namespace {

// ------------------------------------------------------------------------------------------
// Cache build: rows [0, Lp) of [BH, Lsrc, Dh] -> rows [0, Lp) of [BH, Lmax, Dh], K and V in one launch
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ffa_cache_init_kernel(const uint4* __restrict__ k_src, const uint4* __restrict__ v_src,
                                                              uint4* __restrict__ k_dst, uint4* __restrict__ v_dst,
                                                              long long copy_vecs_per_bh, long long src_vecs_per_bh,
                                                              long long dst_vecs_per_bh, long long total_vecs)
{
    // copies the first copy_vecs_per_bh vectors of every (batch, head) from a source whose pairs
    // are src_vecs_per_bh apart to a destination whose pairs are dst_vecs_per_bh apart
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs; i += stride) {
        const long long bh = i / copy_vecs_per_bh, r = i - bh * copy_vecs_per_bh;
        const long long o = bh * dst_vecs_per_bh + r, si = bh * src_vecs_per_bh + r;
        const uint4 kk = __ldcs(k_src + si), vv = __ldcs(v_src + si);
        k_dst[o] = kk;
        v_dst[o] = vv;
    }
}

// ------------------------------------------------------------------------------------------
// Diagnostic: the bounded wait on a barrier that nothing ever completes
// ------------------------------------------------------------------------------------------
// One warp waits, with the given limit, for a copy barrier no copy was issued against.  The
// wait must run out, raise the flag and let the kernel return normally with the time-out bit
// in the status word -- the behaviour the streaming kernels rely on if a copy never lands.
__global__ void __launch_bounds__(32) ffa_wait_selftest_kernel(int* status, unsigned long long limit_ns, unsigned long long* waited_ns)
{
    __shared__ __align__(8) uint64_t bar;
    __shared__ int dead;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const unsigned long long t0 = global_timer_ns();
    const bool ok = mbar_wait_bounded(smem_u32(&bar), 0, &dead, limit_ns);
    __syncwarp();
    if (threadIdx.x == 0) {
        if (!ok || dead) atomicOr(status, kStatusWaitTimeout);
        if (waited_ns != nullptr) *waited_ns = global_timer_ns() - t0;
    }
}

// ------------------------------------------------------------------------------------------
// Host-side dispatch
// ------------------------------------------------------------------------------------------
template <typename F>
int dispatch(int dtype, int head_dim, F&& f)
{
#define FFA_DH_SWITCH(T)                                        \
    switch (head_dim) {                                         \
        case 64: return f(T{}, std::integral_constant<int, 64>{});   \
        case 80: return f(T{}, std::integral_constant<int, 80>{});   \
        case 128: return f(T{}, std::integral_constant<int, 128>{}); \
        case 256: return f(T{}, std::integral_constant<int, 256>{}); \
        default: return (int)cudaErrorInvalidValue;             \
    }
    switch (dtype) {
        case 0: FFA_DH_SWITCH(float)
        case 1: FFA_DH_SWITCH(__half)
        case 2: FFA_DH_SWITCH(__nv_bfloat16)
        default: return (int)cudaErrorInvalidValue;
    }
#undef FFA_DH_SWITCH
}

int elem_size(int dtype) { return dtype == 0 ? 4 : 2; }
// lanes per row group, as RowGeom computes it
int lanes_per_row(int rowb)
{
    const int vpr = rowb / 16;
    return vpr % 5 == 0 ? vpr / 5 : (vpr >= 32 ? 32 : vpr);
}

}  // namespace

int ffa_k_smem_bytes(int dtype, int head_dim, int tile_rows, int stages, int consumer_warps, int tensors_per_stage)
{
    const int rowb = head_dim * elem_size(dtype);
    const int lpr = lanes_per_row(rowb);
    const int ng = consumer_warps * 32 / lpr;
    if (tensors_per_stage == 1) {
        // the streaming pruning kernel: K ring, scorer groups' (max, sum), survivor lists, gather partials,
        // job slots, barriers, flags
        return stages * tile_rows * rowb + kPsGatherWarps * kPsStageBytes + 2 * ng * 4 * 8 + kPsGatherWarps * kPsListCap * 8 + kPsJobs * kPsStreams * head_dim * 4 +
               (int)sizeof(PsJob) * kPsJobs + 2 * kPsJobs * 4 + (2 * stages + 2 * kPsJobs) * 8 + 16;
    }
    // ring, group reduction area, barriers, flags, the slots that receive a cluster's partials
    return stages * tensors_per_stage * tile_rows * rowb + ng * (head_dim + 4) * 4 + 2 * stages * 8 + 16 + kMaxClusterCtas * (head_dim + 2) * 4;
}

int ffa_k_prune_stream_threads(int scorer_warps) { return 32 * (1 + scorer_warps + kPsGatherWarps); }

int ffa_k_fused_smem_bytes(int dtype, int head_dim, int tile_rows, int stages, int chunk_rows, int cluster)
{
    const int rowb = head_dim * elem_size(dtype);
    const int lpr = lanes_per_row(rowb);
    const int ng = 128 / lpr;
    return stages * tile_rows * rowb + chunk_rows * 4 + kFusedListCap * 4 + kFusedListCap / 32 * 4 + ng * (head_dim + 4) * 4 + cluster * head_dim * 4 + 2 * kMaxClusterCtas * 4 +
           2 * stages * 8 + 16;
}

int ffa_k_prepare(int dtype, int head_dim, int max_smem_bytes)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        // the opt-in limit covers static + dynamic shared memory of a kernel
        auto raise_limit = [&](const void* fn) -> cudaError_t {
            cudaFuncAttributes a;
            cudaError_t err = cudaFuncGetAttributes(&a, fn);
            if (err != cudaSuccess) return err;
            return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_bytes - (int)a.sharedSizeBytes);
        };
        cudaError_t e = raise_limit(reinterpret_cast<const void*>(ffa_stream_kernel<T, DH>));
        if (e != cudaSuccess) return (int)e;
        e = raise_limit(reinterpret_cast<const void*>(ffa_prune_stream_kernel<T, DH>));
        if (e != cudaSuccess) return (int)e;
        e = raise_limit(reinterpret_cast<const void*>(ffa_prune_cluster_kernel<T, DH>));
        return (int)e;
    });
}

int ffa_k_cache_init(int dtype, int BH, int prompt_len, int src_len, int max_len, int head_dim, const void* k_src,
                     const void* v_src, void* k_cache, void* v_cache, int sms, cudaStream_t stream)
{
    const long long rowv = (long long)head_dim * elem_size(dtype) / 16;
    const long long copy_per = rowv * prompt_len, src_per = rowv * src_len, dst_per = rowv * max_len, total = copy_per * BH;
    if (total == 0) return 0;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sms * 16;
    if (blocks > cap) blocks = cap;
    ffa_cache_init_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint4*>(k_src), static_cast<const uint4*>(v_src),
                                                                static_cast<uint4*>(k_cache), static_cast<uint4*>(v_cache),
                                                                copy_per, src_per, dst_per, total);
    return (int)cudaGetLastError();
}

int ffa_k_wait_selftest(int* status, unsigned long long limit_ns, unsigned long long* waited_ns, cudaStream_t stream)
{
    ffa_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, limit_ns, waited_ns);
    return (int)cudaGetLastError();
}

// Steps that stream less than this get the programmatic-serialisation attribute: their launch latency and prologue
// are a visible share of the step (bf16 x 128, 1024 pairs: 512 tokens 44.0 vs 44.9 us, fp32 x 64 batch 1: 8.8 vs
// 9.2 us with it); above, an early start of the next grid's CTAs costs more than it hides (2 K tokens 161.8 vs 156.0 us,
// 8 K 605.8 vs 593.6 us)
constexpr double kPdlBelowBytes = 512e6;

// Launch -- when `overlap`, with the programmatic-serialisation attribute: the kernel may start while the previous
// kernel of the stream drains and waits at pdl_wait() before touching global memory -- and, when cluster > 1, as
// thread-block clusters of that many CTAs.
template <typename K>
cudaError_t launch_pdl(K kernel, int grid, int threads, int smem, int cluster, bool overlap, cudaStream_t stream, const FfaStepParams& P)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (overlap) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster, attr[n].val.clusterDim.y = 1, attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr, cfg.numAttrs = (unsigned)n;
    return cudaLaunchKernelEx(&cfg, kernel, P);
}

int ffa_k_decode_onepass(int dtype, int head_dim, const FfaStepParams& P, int threads, int smem, cudaStream_t stream)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        // rows the step streams: at most t of every pair (per-sample lengths: t is their bound)
        const bool overlap = 2.0 * P.B * P.H * P.t * DH * sizeof(T) < kPdlBelowBytes;
        if (P.cluster > 1) {   // the CTAs that share a (batch, head) as one thread-block cluster
            if (launch_pdl(ffa_stream_kernel<T, DH>, P.grid, threads, smem, P.cluster, overlap, stream, P) == cudaSuccess) return 0;
            // a cluster shape this device cannot co-schedule: the same cut runs without clusters,
            // the parts merging through global memory
            (void)cudaGetLastError();
        }
        FfaStepParams Q = P;
        Q.cluster = 0;
        return (int)launch_pdl(ffa_stream_kernel<T, DH>, Q.grid, threads, smem, 0, overlap, stream, Q);
    });
}

int ffa_k_max_active_clusters(int dtype, int head_dim, int threads, int smem, int cluster, int* clusters)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)cluster, 1, 1);
        cfg.blockDim = dim3((unsigned)threads, 1, 1);
        cfg.dynamicSmemBytes = (size_t)smem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = (unsigned)cluster, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
        cfg.attrs = &attr, cfg.numAttrs = 1;
        return (int)cudaOccupancyMaxActiveClusters(clusters, ffa_stream_kernel<T, DH>, &cfg);
    });
}

int ffa_k_decode_fused_prune(int dtype, int head_dim, const FfaStepParams& P, int smem, cudaStream_t stream)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        // cluster = 1 is a plain launch: the kernel's cluster barriers and shared-memory mappings degenerate to the CTA's own
        const bool overlap = 1.0 * P.B * P.H * P.t * DH * sizeof(T) < kPdlBelowBytes;
        return (int)launch_pdl(ffa_prune_cluster_kernel<T, DH>, P.grid, kFusedThreads, smem, P.cluster, overlap, stream, P);
    });
}

int ffa_k_decode_prune_stream(int dtype, int head_dim, const FfaStepParams& P, int scorer_warps, int smem, cudaStream_t stream)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        if (scorer_warps < 1 || scorer_warps > ps_max_scorer_warps(DH)) return (int)cudaErrorInvalidConfiguration;
        const bool overlap = 1.0 * P.B * P.H * P.t * DH * sizeof(T) < kPdlBelowBytes;
        return (int)launch_pdl(ffa_prune_stream_kernel<T, DH>, P.grid, ffa_k_prune_stream_threads(scorer_warps), smem, 0, overlap, stream, P);
    });
}
