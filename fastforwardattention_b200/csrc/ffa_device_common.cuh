// Device-side building blocks shared by the decode kernels: mbarrier / bulk-copy PTX wrappers
// with time-bounded waits, element traits (16-byte vectors <-> fp32), the lane-group geometry of
// a cache row, per-sample ranges, cache addressing (contiguous or paged) and the work partition.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstring>
#include <type_traits>

#include "ffa_internal.h"

namespace ffa_dev {


constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // bounded barrier wait: 2 s, then give up
constexpr uint32_t kDrainPolls = 1u << 20;
constexpr int kMaxClusterCtas = 8;   // portable thread-block cluster size
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusBadLength = 2;

// ------------------------------------------------------------------------------------------
// PTX wrappers: mbarrier + 1-D bulk copy global -> this CTA's shared memory
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Cache hints: ask for the 128-byte line at p to be brought into L2 (into L1 as well); nothing waits for them.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// same, but the hardware may park the thread for up to `hint_ns` before answering
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for the phase with the given parity.  Never spins for ever: after kWaitLimitNs of wall
// time (or as soon as another thread of the CTA gave up) it raises the CTA's `dead` flag and
// returns false; callers then skip the data but keep walking the same control flow so every
// CTA-level barrier is still reached by everyone.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* dead,
                                                  unsigned long long limit_ns = kWaitLimitNs)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait_parked(bar, parity, 4000u)) return true;
        if (*dead) return false;
        if (global_timer_ns() - t0 > limit_ns) break;
    }
    *dead = 1;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// 16 bytes global -> this thread's slot in shared memory, asynchronously (bypassing L1); the issuing thread
// may read the slot after cp_async_wait_all()
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all()
{
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// L2 eviction policy for data that is read exactly once (cache rows streaming through): such lines are
// the first to go, so that small, re-read data (scores in scratch, partials, inputs) stays in L2
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_copy_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t pol)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ void cp_async_16_hint(uint32_t dst, const void* src, uint64_t pol)
{
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "l"(pol) : "memory");
}
// Programmatic dependent launch.  pdl_release(): the next kernel in the stream (if it was launched with the
// programmatic-serialisation attribute) may start its CTAs as soon as every CTA of this grid has got this far;
// pdl_wait(): blocks until every grid this one depends on has completed and its memory is visible.  A kernel
// does only what needs no global memory (barrier and shared-memory set-up) before pdl_wait(), so its launch
// latency and prologue overlap the previous kernel's last tiles.  Both are no-ops in a plain launch.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The 128-byte line at `p` (128-byte aligned) will not be read again before it is rewritten: L2 may drop it
// without writing it back to HBM
__device__ __forceinline__ void l2_discard_line(const void* p) { asm volatile("discard.global.L2 [%0], 128;" ::"l"(p) : "memory"); }
__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// thread-block clusters: rank, barrier over all threads of all CTAs, a float of a peer CTA's shared memory
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The two halves of a cluster barrier, for a CTA that has other work between "I am here" and "are the others".
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Stores v at the same shared-memory offset in CTA peer_rank of the cluster; visible there after the next cluster barrier.
__device__ __forceinline__ void st_peer_smem_f32(void* own_smem_ptr, uint32_t peer_rank, float v)
{
    uint32_t peer;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(smem_u32(own_smem_ptr)), "r"(peer_rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_peer_smem_f32(const void* own_smem_ptr, uint32_t peer_rank)
{
    uint32_t peer;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(smem_u32(own_smem_ptr)), "r"(peer_rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
    return v;
}

// ------------------------------------------------------------------------------------------
// Element traits: a 16-byte vector holds EPV elements; unpack to fp32, round from fp32
// ------------------------------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static constexpr int EPV = 4;
    static __device__ __forceinline__ void unpack(const uint4& r, float* f)
    {
        f[0] = __uint_as_float(r.x), f[1] = __uint_as_float(r.y), f[2] = __uint_as_float(r.z),
        f[3] = __uint_as_float(r.w);
    }
    static __device__ __forceinline__ void unpack2(const uint4& r, float2* f)
    {
        f[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
        f[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
    }
    static __device__ __forceinline__ float round(float x) { return x; }
    static __device__ __forceinline__ uint32_t bits(float x) { return __float_as_uint(x); }
    static __device__ __forceinline__ float from_bits(uint32_t b) { return __uint_as_float(b); }
    static __device__ __forceinline__ float to_float(float x) { return x; }
    static __device__ __forceinline__ void store(float* p, float x) { *p = x; }
    // attention.cu:461-464
    static __device__ __forceinline__ bool leq(float a, float b) { return a <= b; }
};
template <>
struct Elem<__half> {
    static constexpr int EPV = 8;
    static __device__ __forceinline__ void unpack(const uint4& r, float* f)
    {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = t.x, f[2 * i + 1] = t.y;
        }
    }
    static __device__ __forceinline__ void unpack2(const uint4& r, float2* f)
    {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    }
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    // the 16 bits of a value that round() produced, and back
    static __device__ __forceinline__ uint32_t bits(float x) { return __half_as_ushort(__float2half_rn(x)); }
    static __device__ __forceinline__ float from_bits(uint32_t b) { return __half2float(__ushort_as_half((unsigned short)b)); }
    static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
    static __device__ __forceinline__ void store(__half* p, float x) { *p = __float2half_rn(x); }
    // attention.cu:466-469 hands two raw bit patterns to __hle; the unsigned short -> __half
    // conversion there is the NUMERIC one, so the patterns themselves are rounded to 11
    // significant bits and compared.  Reproduced literally.
    static __device__ __forceinline__ bool leq(float a, float b)
    {
        const unsigned short ba = __half_as_ushort(__float2half_rn(a));
        const unsigned short bb = __half_as_ushort(__float2half_rn(b));
        return __hle(__ushort2half_rn(ba), __ushort2half_rn(bb));
    }
};
template <>
struct Elem<__nv_bfloat16> {
    static constexpr int EPV = 8;
    static __device__ __forceinline__ void unpack(const uint4& r, float* f)
    {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void unpack2(const uint4& r, float2* f)
    {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ uint32_t bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ float from_bits(uint32_t b) { return __bfloat162float(__ushort_as_bfloat16((unsigned short)b)); }
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
    // the reference has no bf16; plain value comparison
    static __device__ __forceinline__ bool leq(float a, float b) { return a <= b; }
};

// Geometry of one cache row of DH elements of T, and of the lane group that owns a row.
template <typename T, int DH>
struct RowGeom {
    static constexpr int EPV = Elem<T>::EPV;
    static constexpr int ROWB = DH * (int)sizeof(T);   // bytes per row, multiple of 16
    static constexpr int VPR = ROWB / 16;               // 16-byte vectors per row
    // Lanes per row group and vectors per lane.  Power-of-two rows: one vector per lane up to a
    // full warp, two per lane for 1024-byte rows.  head_dim 80 (10 or 20 vectors): five vectors
    // per lane and 2 or 4 lanes per row, so that no lane idles.
    static constexpr bool kFiveWide = (VPR % 5) == 0;
    static constexpr int LPR = kFiveWide ? VPR / 5 : (VPR >= 32 ? 32 : VPR);
    static constexpr int VPL = kFiveWide ? 5 : (VPR + 31) / 32;
    static constexpr int RB = VPL >= 4 ? 2 : 4;          // rows per lane group and batch (register budget)
    static_assert(LPR * VPL == VPR && (LPR & (LPR - 1)) == 0, "every lane of a power-of-two group owns VPL vectors");
    static_assert(ROWB % 16 == 0, "rows must be 16-byte multiples");
};

// Per-sample view of the cache for this step (attention.cu:805-817).  `row` is where the new
// token goes and the number of cached rows attended; keys below `first` are masked.  With
// per-sample lengths P.t is the host's upper bound on every length: the work list covers rows
// 0..P.t only, so a longer sample is refused (and reported), never silently cut short.
struct SampleRange {
    int first, row;
    bool ok;
};
__device__ __forceinline__ SampleRange sample_range(const FfaStepParams& P, int b)
{
    SampleRange r;
    r.first = 0, r.row = P.t;
    if (P.seq_lengths != nullptr) {
        const int s = P.seq_lengths[b];
        if (P.right_or_no_padding) r.row = s;
        else r.first = s;
    }
    r.ok = r.row >= 0 && r.row < P.Lmax && r.row <= P.t;
    if (!r.ok) r.row = 0;
    r.first = min(max(r.first, 0), r.row);
    return r;
}

// Byte offset of cache row `row` of pair bh from the start of the cache (or page pool).
// Contiguous slabs: [B*H, Lmax, Dh].  Paged: the pool is [pages, H, page_rows, Dh] and
// page_table[b][row / page_rows] names the page; rows of one (pair, page) are contiguous, and
// the streaming kernel's tiles never straddle pages because tile_rows divides page_rows (the
// fused pruning kernel splits a tile's copy at page boundaries instead).
__device__ __forceinline__ size_t cache_row_offset(const FfaStepParams& P, int bh, int row, int rowb)
{
    if (P.page_table == nullptr) return ((size_t)bh * P.Lmax + row) * rowb;
    const int b = bh / P.H, h = bh - b * P.H;
    const int page = P.page_table[(size_t)b * P.max_pages + row / P.page_rows];
    return (((size_t)page * P.H + h) * P.page_rows + row % P.page_rows) * rowb;
}

// Work decomposition.  Every (batch, head) is cut into `parts_per_bh` parts of whole tiles
// (part p of a pair covers its units [p*upb/C, (p+1)*upb/C)); the flat list of B*H*C parts is
// cut into `grid` equal contiguous runs, one per CTA.  With C = units per pair this is a plain
// even cut of the unit list (large problems: perfect balance); with a small C and grid = B*H*C
// or B*H/k every CTA boundary falls on a part boundary, so a CTA owns exactly one segment and
// a pair is merged from exactly C partials (small problems: the serial per-segment latency
// and the merge traffic are what cost).  Requires C <= upb and grid <= B*H*C.
struct Partition {
    long long parts_total;
    int upb, C, G;
    __device__ __forceinline__ long long unit_of_part(long long p) const
    {
        const long long bh = p / C;
        return bh * upb + ((p - bh * C) * upb) / C;
    }
    __device__ __forceinline__ long long first_unit(long long cta) const { return unit_of_part(cta * parts_total / G); }
    // the CTA that owns part p
    __device__ __forceinline__ int cta_of_part(long long p) const { return (int)(((p + 1) * G + parts_total - 1) / parts_total - 1); }
    __device__ __forceinline__ int first_cta_of(int bh) const { return cta_of_part((long long)bh * C); }
    __device__ __forceinline__ int last_cta_of(int bh) const { return cta_of_part((long long)(bh + 1) * C - 1); }
};
__device__ __forceinline__ Partition make_partition(const FfaStepParams& P)
{
    Partition q;
    q.upb = P.units_per_bh, q.C = P.parts_per_bh, q.G = P.grid;
    q.parts_total = (long long)P.B * P.H * P.parts_per_bh;
    return q;
}

template <typename T, int DH>
__device__ __forceinline__ void load_row_f32(const unsigned char* row, int li, float (&f)[RowGeom<T, DH>::VPL][RowGeom<T, DH>::EPV])
{
    using G = RowGeom<T, DH>;
#pragma unroll
    for (int x = 0; x < G::VPL; ++x) {
        const int vec = li + x * G::LPR;
        if (vec < G::VPR) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + vec * 16);
            Elem<T>::unpack(raw, f[x]);
        } else {
#pragma unroll
            for (int e = 0; e < G::EPV; ++e) f[x][e] = 0.f;
        }
    }
}

// Sums RB per-lane partials over the LPR lanes of a group and leaves ONE of the RB totals in every lane:
// the first log2(RB) butterfly levels exchange halves of the value set instead of adding everything
// everywhere (5 shuffles for 4 values over 16 lanes, where four full butterflies take 16).  Lane `li`
// of the group ends up with the total of value transposed_row<LPR, RB>(li), replicated over LPR / RB lanes.
template <int LPR, int RB>
__device__ __forceinline__ int transposed_row(int li)
{
    static_assert((RB == 4 && LPR >= 4) || (RB == 2 && LPR >= 2), "RB values over at least RB lanes");
    if constexpr (RB == 4) return ((li / (LPR / 2)) & 1) * 2 + ((li / (LPR / 4)) & 1);
    else return (li / (LPR / 2)) & 1;
}
template <int LPR, int RB>
__device__ __forceinline__ float transposed_group_sum(const float (&v)[RB], int li)
{
    float c;
    if constexpr (RB == 4) {
        const bool hi = (li / (LPR / 2)) & 1;            // keeps values {2, 3}, hands {0, 1} to its partner
        float a = hi ? v[2] : v[0], b = hi ? v[3] : v[1];
        a += __shfl_xor_sync(0xffffffffu, hi ? v[0] : v[2], LPR / 2);
        b += __shfl_xor_sync(0xffffffffu, hi ? v[1] : v[3], LPR / 2);
        const bool odd = (li / (LPR / 4)) & 1;           // keeps the odd one of its pair
        c = (odd ? b : a) + __shfl_xor_sync(0xffffffffu, odd ? a : b, LPR / 4);
#pragma unroll
        for (int off = LPR / 8; off >= 1; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
    } else {
        const bool hi = (li / (LPR / 2)) & 1;
        c = (hi ? v[1] : v[0]) + __shfl_xor_sync(0xffffffffu, hi ? v[0] : v[1], LPR / 2);
#pragma unroll
        for (int off = LPR / 4; off >= 1; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
    }
    return c;
}

// ------------------------------------------------------------------------------------------
// Output push over peer memory (see FfaStepParams::push_*)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t* push_tail(const FfaStepParams& P, int rank)
{
    return reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(P.push_peer[rank]) + 2 * P.push_half_bytes);
}
// the step this launch pushes: one past the counter in this rank's own buffer (nobody advances it before every pair is out)
__device__ __forceinline__ uint32_t push_step(const FfaStepParams& P)
{
    return *reinterpret_cast<volatile uint32_t*>(push_tail(P, P.push_rank) + kPeerTailCounter) + 1u;
}
// element d of out[bh, :] -> this rank's slot in the own result and in every peer's staging half of step `seq`.
// Consecutive threads hold consecutive d, so a warp's stores to one peer are one contiguous run.
template <typename T, int DH>
__device__ __forceinline__ void push_store(const FfaStepParams& P, uint32_t seq, int bh, int d, T v)
{
    const int b = bh / P.H, h = bh - b * P.H;
    const size_t at = ((size_t)(b * P.push_world + P.push_rank) * P.H + h) * DH + d;
    static_cast<T*>(P.push_gathered)[at] = v;
    const size_t half = (size_t)(seq & 1u) * P.push_half_bytes;
    for (int r = 0; r < P.push_world; ++r)
        if (r != P.push_rank) reinterpret_cast<T*>(static_cast<unsigned char*>(P.push_peer[r]) + half)[at] = v;
}
// One thread per finished pair, after every thread that pushed the pair has fenced (system scope) and met at a barrier:
// counts the pair; the one that counts the step's last pair raises this rank's flag at every peer and advances the step.
__device__ __forceinline__ void push_pair_done(const FfaStepParams& P, uint32_t seq)
{
    uint32_t* own = push_tail(P, P.push_rank);
    if (atomicAdd(own + kPeerTailPairsDone, 1u) == (uint32_t)(P.B * P.H) - 1u) {
        own[kPeerTailPairsDone] = 0;
        __threadfence_system();   // every CTA's rows (fenced before its count) are at the peers before the flags
        for (int r = 0; r < P.push_world; ++r)
            if (r != P.push_rank) st_release_sys(push_tail(P, r) + kPeerTailFlags + P.push_rank, seq);
        *reinterpret_cast<volatile uint32_t*>(own + kPeerTailCounter) = seq;
    }
}

template <int LPR>
__device__ __forceinline__ float group_sum(float x)
{
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    return x;
}

}  // namespace ffa_dev
