// Decode masked multi-head attention for sm_100a: streaming split-KV kernels.
//
// Replaces mmha::masked_multihead_attention_kernel_optimized (attention.cu:698-1295) and the
// two cache-init kernels (attention.cu:1556-1609) of the reference.  The reference runs one
// CTA per (batch, head) that walks the whole sequence serially and stages every score in
// shared memory; here the flat list of (batch*head, row-tile) units is cut into equal
// contiguous runs, one per CTA of a persistent grid, so all SMs stream from HBM whatever the
// batch*head count and the sequence length is bounded by memory only.
//
//   ffa_stream_kernel<T, DH, PASS_ONE>    p == 0: K and V tiles through a bulk-copy ring,
//                                         online softmax, cross-CTA merge by the CTA that
//                                         arrives last (no waiting), k/v append fused
//   ffa_stream_kernel<T, DH, PASS_SCORE>  first half of the two-pass modes: K tiles only,
//                                         fp32 scores to scratch, global max and sum
//   ffa_value_gather_kernel<T, DH>        second half: tests every cached row with the
//                                         reference's pruning rule (attention.cu:1184-1191,
//                                         461-469) and loads only the V rows that survive
//   ffa_prune_cluster_kernel<T, DH>       both halves in one launch: a thread-block cluster per
//                                         (batch, head), scores in shared memory, statistics
//                                         and partial outputs over distributed shared memory
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

namespace {

constexpr int kPassOne = 0;
constexpr int kPassScore = 1;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // bounded barrier wait: 2 s, then give up
constexpr uint32_t kDrainPolls = 1u << 20;
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusBadLength = 2;
constexpr int kGatherThreads = 256;

// ------------------------------------------------------------------------------------------
// PTX wrappers: mbarrier + 1-D bulk copy global -> this CTA's shared memory
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

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
// token goes and the number of cached rows attended; keys below `first` are masked.
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
    r.ok = r.row >= 0 && r.row < P.Lmax;
    if (!r.ok) r.row = 0;
    r.first = min(max(r.first, 0), r.row);
    return r;
}

// Byte offset of cache row `row` of pair bh from the start of the cache (or page pool).
// Contiguous slabs: [B*H, Lmax, Dh].  Paged: the pool is [pages, H, page_rows, Dh] and
// page_table[b][row / page_rows] names the page; rows of one (pair, page) are contiguous, and
// tiles never straddle pages because tile_rows divides page_rows.
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

template <int LPR>
__device__ __forceinline__ float group_sum(float x)
{
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    return x;
}

// ------------------------------------------------------------------------------------------
// Streaming kernel (one-pass attention, or the score pass of the two-pass modes)
// ------------------------------------------------------------------------------------------
// Shared memory: [stages][K tile | V tile] ring (score pass: K tile only), then the group
// reduction area [NG][DH + 4] (rows 16-byte aligned; max and sum in the tail), then
// full/empty barriers, then two flags.
// Warp 0 issues the copies (one elected lane); warps 1.. compute.  A lane group of LPR lanes
// owns a row: 16-byte shared-memory reads, fp32 FMAs, butterfly sum.  Each group keeps its
// own online-softmax state, so the row loop has no CTA-level synchronisation at all.
template <typename T, int DH, int PASS>
// Register budget: 4 resident CTAs of 160 threads (or 2 of 288) need <= 96 registers per thread;
// head_dim 80 keeps five vectors per lane in flight and is compiled for 2 CTAs of 160 threads.
__global__ void __launch_bounds__(DH == 80 ? 288 : 320, DH == 80 ? 1 : 2) ffa_stream_kernel(const FfaStepParams P)
{
    using G = RowGeom<T, DH>;
    constexpr int EPV = G::EPV, ROWB = G::ROWB, VPR = G::VPR, LPR = G::LPR, VPL = G::VPL, RB = G::RB;
    constexpr bool kPrecise = sizeof(T) == 4 || PASS == kPassScore;  // natural-log domain, full-precision exp
    constexpr int TENSORS = PASS == kPassOne ? 2 : 1;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr int RS = DH + 4;  // row stride of the group reduction area, in floats

    extern __shared__ __align__(128) unsigned char smem[];
    const int R = P.tile_rows, S = P.stages;
    const int ncw = (blockDim.x >> 5) - 1;   // consumer warps
    const int nct = ncw * 32;                // consumer threads
    const int NG = nct / LPR;                // row groups
    const uint32_t tile_bytes = (uint32_t)R * ROWB;
    const uint32_t stage_bytes = tile_bytes * TENSORS;
    float* red = reinterpret_cast<float*>(smem + (size_t)S * stage_bytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + NG * RS);
    volatile int* flags = reinterpret_cast<volatile int*>(bars + 2 * S);  // [0] dead, [1] last-arriver
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + S);
    const uint32_t ring = smem_u32(smem);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, ncw);
        }
        flags[0] = 0, flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int upb = P.units_per_bh;
    const Partition cut = make_partition(P);
    const long long u0 = cut.first_unit(blockIdx.x), u1 = cut.first_unit(blockIdx.x + 1);
    const unsigned char* kc = static_cast<const unsigned char*>(P.k_cache);
    const unsigned char* vc = static_cast<const unsigned char*>(P.v_cache);

    if (threadIdx.x < 32) {
        // ---------------- producer ----------------
        if (threadIdx.x == 0) {
            uint32_t issued = 0, stage = 0, use = 0;  // ring position: buffer index and how often it was used
            int cur_b = -1;
            SampleRange sr{0, 0, false};
            long long u = u0;
            int bh = (int)(u0 / upb), j = (int)(u0 - (long long)bh * upb);
            for (; u < u1; ++u, ++j) {
                if (j == upb) j = 0, ++bh;
                const int b = bh / P.H;
                if (b != cur_b) sr = sample_range(P, b), cur_b = b;
                if (!sr.ok) continue;
                const int lo = max(j * R, sr.first), hi = min((j + 1) * R, sr.row);
                if (hi <= lo) continue;
                if (use > 0 && !mbar_wait_bounded(bar_empty + 8 * stage, (use - 1) & 1, flags)) break;
                const uint32_t bytes = (uint32_t)(hi - lo) * ROWB;
                const size_t off = cache_row_offset(P, bh, lo, ROWB);
                mbar_expect_tx(bar_full + 8 * stage, bytes * TENSORS);
                bulk_copy_g2s(ring + stage * stage_bytes, kc + off, bytes, bar_full + 8 * stage);
                if (TENSORS == 2) bulk_copy_g2s(ring + stage * stage_bytes + tile_bytes, vc + off, bytes, bar_full + 8 * stage);
                ++issued;
                if (++stage == (uint32_t)S) stage = 0, ++use;
            }
            if (flags[0]) {
                // gave up: let the copies already issued land before the CTA releases its
                // shared memory (bounded again)
                const uint32_t pending = issued < (uint32_t)S ? issued : (uint32_t)S;
                for (uint32_t k = 0; k < pending; ++k) {
                    const uint32_t id = issued - 1 - k, st = id % S, us = id / S;
                    for (uint32_t n = 0; n < kDrainPolls && !mbar_try_wait(bar_full + 8 * st, us & 1); ++n) __nanosleep(256);
                }
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int ctid = threadIdx.x - 32;
        const int lane = ctid & 31;
        const int g = ctid / LPR, li = ctid % LPR;
        constexpr int E2 = EPV / 2;
        constexpr bool kAllLanes = (VPR == LPR * VPL);  // every lane of a group owns VPL vectors
        uint32_t stage = 0, phase = 0;
        long long u = u0;
        // q of the first (batch, head) of this CTA's run; the next one is fetched while the
        // current one is being processed, so its global-memory latency is never exposed
        const unsigned char* qbase = static_cast<const unsigned char*>(P.q);
        uint4 qraw[VPL];
#pragma unroll
        for (int x = 0; x < VPL; ++x) {
            qraw[x] = make_uint4(0, 0, 0, 0);
            if (u0 < u1 && li + x * LPR < VPR)
                qraw[x] = *reinterpret_cast<const uint4*>(qbase + (size_t)(u0 / upb) * ROWB + (li + x * LPR) * 16);
        }
        while (u < u1) {
            const int bh = (int)(u / upb), j0 = (int)(u - (long long)bh * upb);
            const int j1 = (int)min((long long)upb, j0 + (u1 - u));
            const int b = bh / P.H;
            const SampleRange sr = sample_range(P, b);
            const int jt = sr.row / R;  // the unit that also owns the new token

            // q for this (batch, head), pre-multiplied so that scores come out of the FMAs
            // ready for the exponential (exact mode: scale only, natural-log domain)
            float qf[VPL][EPV];
#pragma unroll
            for (int x = 0; x < VPL; ++x) Elem<T>::unpack(qraw[x], qf[x]);
            if (u + (j1 - j0) < u1) {   // this CTA goes on with the next (batch, head)
#pragma unroll
                for (int x = 0; x < VPL; ++x)
                    if (li + x * LPR < VPR)
                        qraw[x] = *reinterpret_cast<const uint4*>(qbase + (size_t)(bh + 1) * ROWB + (li + x * LPR) * 16);
            }
            // the new token's k and v are needed only at the end of the segment: fetch them now
            const bool owns_new = sr.ok && j0 <= jt && jt < j1;
            uint4 knew[VPL], vnew[VPL];
#pragma unroll
            for (int x = 0; x < VPL; ++x) {
                knew[x] = vnew[x] = make_uint4(0, 0, 0, 0);
                if (owns_new && li + x * LPR < VPR) {
                    const size_t src = (size_t)bh * ROWB + (li + x * LPR) * 16;
                    knew[x] = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.k) + src);
                    if (PASS == kPassOne) vnew[x] = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.v) + src);
                }
            }
            const float qmul = kPrecise ? 1.f : P.scale * kLog2e;
            float2 q2[VPL][E2];
#pragma unroll
            for (int x = 0; x < VPL; ++x)
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    qf[x][e] *= qmul;
                    if (e & 1) q2[x][e >> 1] = make_float2(qf[x][e - 1], qf[x][e]);
                }

            float m = -CUDART_INF_F, l = 0.f;
            float2 acc2[VPL][E2];
#pragma unroll
            for (int x = 0; x < VPL; ++x)
#pragma unroll
                for (int e = 0; e < E2; ++e) acc2[x][e] = make_float2(0.f, 0.f);

            auto score_of = [&](float dot) -> float {
                if (!kPrecise) return dot;
                if (PASS == kPassScore && P.round_like_torch) return Elem<T>::round(Elem<T>::round(dot) * P.scale);
                return dot * P.scale;
            };
            // the score pass only feeds the softmax denominator: __expf, like the reference (attention.cu:1113)
            auto expo = [&](float x) -> float { return PASS == kPassScore ? __expf(x) : (kPrecise ? expf(x) : fast_exp2(x)); };

            // RB (four; two for head_dim 80) rows per lane group at a time: all shared-memory loads first, then the
            // packed fp32 FMAs (fma.rn.f32x2), four interleaved butterfly sums, one softmax
            // update.  FULL: every row of the batch exists (no predicates, no clamping).
            auto batch = [&](auto full_tag, const unsigned char* ks, const unsigned char* vs, int base, int nrows, int row0) {
                constexpr bool FULL = decltype(full_tag)::value;
                int rc[RB];
                uint4 kraw[RB][VPL];
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    const int r = base + uu * NG + g;
                    rc[uu] = FULL ? r : min(r, nrows - 1);
#pragma unroll
                    for (int x = 0; x < VPL; ++x)
                        if (kAllLanes || li + x * LPR < VPR)
                            kraw[uu][x] = *reinterpret_cast<const uint4*>(ks + (size_t)rc[uu] * ROWB + (li + x * LPR) * 16);
                }
                float sc[RB];
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    float2 a = make_float2(0.f, 0.f);
#pragma unroll
                    for (int x = 0; x < VPL; ++x)
                        if (kAllLanes || li + x * LPR < VPR) {
                            float2 k2[E2];
                            Elem<T>::unpack2(kraw[uu][x], k2);
#pragma unroll
                            for (int e = 0; e < E2; ++e) a = __ffma2_rn(q2[x][e], k2[e], a);
                        }
                    sc[uu] = a.x + a.y;
                }
#pragma unroll
                for (int off = LPR / 2; off >= 1; off >>= 1)
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu) sc[uu] += __shfl_xor_sync(0xffffffffu, sc[uu], off);
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) sc[uu] = (FULL || base + uu * NG + g < nrows) ? score_of(sc[uu]) : -CUDART_INF_F;
                float m_new = m;
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) m_new = fmaxf(m_new, sc[uu]);
                if (!FULL && m_new == -CUDART_INF_F) return;  // this group has no row in this batch
                const float corr = expo(m - m_new);
                m = m_new;
                float pr[RB];
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) pr[uu] = expo(sc[uu] - m);
                float psum = 0.f;
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) psum += pr[uu];
                l = fmaf(l, corr, psum);
                if (PASS == kPassOne) {
                    uint4 vraw[RB][VPL];
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu)
#pragma unroll
                        for (int x = 0; x < VPL; ++x)
                            if (kAllLanes || li + x * LPR < VPR)
                                vraw[uu][x] = *reinterpret_cast<const uint4*>(vs + (size_t)rc[uu] * ROWB + (li + x * LPR) * 16);
                    const float2 c2 = make_float2(corr, corr);
#pragma unroll
                    for (int x = 0; x < VPL; ++x)
#pragma unroll
                        for (int e = 0; e < E2; ++e) acc2[x][e] = __fmul2_rn(acc2[x][e], c2);
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu) {
                        const float2 p2 = make_float2(pr[uu], pr[uu]);
#pragma unroll
                        for (int x = 0; x < VPL; ++x)
                            if (kAllLanes || li + x * LPR < VPR) {
                                float2 v2[E2];
                                Elem<T>::unpack2(vraw[uu][x], v2);
#pragma unroll
                                for (int e = 0; e < E2; ++e) acc2[x][e] = __ffma2_rn(p2, v2[e], acc2[x][e]);
                            }
                    }
                } else if (li == 0) {
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu)
                        if (FULL || base + uu * NG + g < nrows) P.scores[(size_t)bh * P.Lmax + row0 + base + uu * NG + g] = sc[uu];
                }
            };

            if (sr.ok) {
                for (int j = j0; j < j1; ++j) {
                    const int lo = max(j * R, sr.first), hi = min((j + 1) * R, sr.row);
                    if (hi <= lo) continue;
                    const int nrows = hi - lo;
                    const bool ready = mbar_wait_bounded(bar_full + 8 * stage, phase, flags);
                    const unsigned char* ks = smem + (size_t)stage * stage_bytes;
                    const unsigned char* vs = ks + tile_bytes;
                    if (ready) {
                        int base = 0;
                        for (; base + RB * NG <= nrows; base += RB * NG) batch(std::true_type{}, ks, vs, base, nrows, lo);
                        if (base < nrows) batch(std::false_type{}, ks, vs, base, nrows, lo);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
                    if (++stage == (uint32_t)S) stage = 0, phase ^= 1;
                }
            }

            // ---- the new token: score against k, append k (and v) at row sr.row ----
            if (owns_new) {
                float dot = 0.f;
#pragma unroll
                for (int x = 0; x < VPL; ++x) {
                    float kf[EPV];
                    Elem<T>::unpack(knew[x], kf);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) dot = fmaf(qf[x][e], kf[e], dot);
                }
                dot = group_sum<LPR>(dot);  // every group computes it; group 0 uses it
                if (g == 0) {
                    const float st = score_of(dot);
                    const float m_new = fmaxf(m, st);
                    const float corr = expo(m - m_new), pr = expo(st - m_new);
                    m = m_new;
                    l = l * corr + pr;
                    const size_t row_off = cache_row_offset(P, bh, sr.row, ROWB);
#pragma unroll
                    for (int x = 0; x < VPL; ++x) {
                        const int vec = li + x * LPR;
                        if (vec < VPR) {
                            *reinterpret_cast<uint4*>(static_cast<unsigned char*>(P.k_cache) + row_off + vec * 16) = knew[x];
                            if (PASS == kPassOne) {
                                *reinterpret_cast<uint4*>(static_cast<unsigned char*>(P.v_cache) + row_off + vec * 16) = vnew[x];
                                float2 v2[E2];
                                Elem<T>::unpack2(vnew[x], v2);
#pragma unroll
                                for (int e = 0; e < E2; ++e) {
                                    acc2[x][e].x = fmaf(pr, v2[e].x, acc2[x][e].x * corr);
                                    acc2[x][e].y = fmaf(pr, v2[e].y, acc2[x][e].y * corr);
                                }
                            }
                        }
                    }
                    if (PASS == kPassScore && li == 0) P.scores[(size_t)bh * P.Lmax + sr.row] = st;
                }
            }

            // ---- merge the groups of this CTA ----
            float* mine = red + g * RS;
            if (PASS == kPassOne) {
#pragma unroll
                for (int x = 0; x < VPL; ++x) {
                    const int vec = li + x * LPR;
                    if (vec < VPR) {
#pragma unroll
                        for (int e = 0; e < E2; e += 2)
                            *reinterpret_cast<float4*>(mine + vec * EPV + 2 * e) =
                                make_float4(acc2[x][e].x, acc2[x][e].y, acc2[x][e + 1].x, acc2[x][e + 1].y);
                    }
                }
            }
            if (li == 0) mine[DH] = m, mine[DH + 1] = l;
            named_bar_sync(1, nct);
            float M = -CUDART_INF_F;
            for (int gg = 0; gg < NG; ++gg) M = fmaxf(M, red[gg * RS + DH]);
            const bool whole = (j0 == 0 && j1 == upb);
            const int slot = blockIdx.x + bh;
            float* part = P.partials + (size_t)slot * (DH + 2);
            T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
            const int nd = PASS == kPassOne ? DH : 1;
            for (int d = ctid; d < nd; d += nct) {
                float A = 0.f, L = 0.f;
                for (int gg = 0; gg < NG; ++gg) {
                    const float mg = red[gg * RS + DH];
                    const float w = mg == -CUDART_INF_F ? 0.f : expo(mg - M);
                    if (PASS == kPassOne) A = fmaf(w, red[gg * RS + d], A);
                    L = fmaf(w, red[gg * RS + DH + 1], L);
                }
                if (whole) {
                    if (PASS == kPassOne) Elem<T>::store(outp + d, L > 0.f ? A / L : 0.f);
                    else P.stats[2 * bh] = M, P.stats[2 * bh + 1] = L;
                } else {
                    if (PASS == kPassOne) part[d] = A;
                    if (d == 0) part[DH] = M, part[DH + 1] = L;
                }
            }
            if (!whole) {
                // cross-CTA merge without waiting: whoever arrives last does it
                __threadfence();
                named_bar_sync(1, nct);
                const int c_first = cut.first_cta_of(bh), c_last = cut.last_cta_of(bh);
                const int count = c_last - c_first + 1;
                if (ctid == 0) {
                    const int old = atomicAdd(P.tickets + bh, 1);
                    flags[1] = (old == count - 1);
                }
                named_bar_sync(1, nct);
                if (flags[1]) {
                    __threadfence();
                    const float* pbase = P.partials + (size_t)(c_first + bh) * (DH + 2);
                    float MM = -CUDART_INF_F;
                    for (int k = 0; k < count; ++k) MM = fmaxf(MM, __ldcg(pbase + (size_t)k * (DH + 2) + DH));
                    for (int d = ctid; d < nd; d += nct) {
                        float A = 0.f, L = 0.f;
                        for (int k = 0; k < count; ++k) {
                            const float* pk = pbase + (size_t)k * (DH + 2);
                            const float mk = __ldcg(pk + DH);
                            const float w = mk == -CUDART_INF_F ? 0.f : expo(mk - MM);
                            if (PASS == kPassOne) A = fmaf(w, __ldcg(pk + d), A);
                            L = fmaf(w, __ldcg(pk + DH + 1), L);
                        }
                        if (PASS == kPassOne) Elem<T>::store(outp + d, L > 0.f ? A / L : 0.f);
                        else P.stats[2 * bh] = MM, P.stats[2 * bh + 1] = L;
                    }
                    if (ctid == 0) P.tickets[bh] = 0;  // ready for the next launch on this stream
                }
            }
            named_bar_sync(1, nct);  // `red` and the flag are reused by the next segment
            if (!sr.ok && ctid == 0) atomicOr(P.status, kStatusBadLength);
            u += j1 - j0;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && flags[0]) atomicOr(P.status, kStatusWaitTimeout);
}

// ------------------------------------------------------------------------------------------
// Value pass of the two-pass modes: prune test on every cached row, gather the survivors
// ------------------------------------------------------------------------------------------
// Shared memory: kept-row list (index + probability) for one unit of tile_rows rows, then the
// group reduction area [NG][DH].  All 8 warps compute; rows that survive are fetched with
// 16-byte global loads, four rows in flight per lane group.
template <typename T, int DH>
__global__ void __launch_bounds__(kGatherThreads) ffa_value_gather_kernel(const FfaStepParams P)
{
    using G = RowGeom<T, DH>;
    constexpr int EPV = G::EPV, ROWB = G::ROWB, VPR = G::VPR, LPR = G::LPR, VPL = G::VPL, RB = G::RB;
    constexpr int NT = kGatherThreads, NG = NT / LPR;

    extern __shared__ __align__(128) unsigned char smem[];
    const int R = P.tile_rows;  // multiple of 32
    int* list_idx = reinterpret_cast<int*>(smem);
    float* list_p = reinterpret_cast<float*>(list_idx + R);
    float* red = list_p + R;  // [NG][DH]
    __shared__ int s_n, s_last;
    __shared__ unsigned s_words[16];   // one ballot per 32 rows of a 512-row unit

    const int upb = P.units_per_bh;
    const Partition cut = make_partition(P);
    const long long u0 = cut.first_unit(blockIdx.x), u1 = cut.first_unit(blockIdx.x + 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = tid / LPR, li = tid % LPR;
    const bool prune = P.p > 0.f;
    const unsigned char* vc = static_cast<const unsigned char*>(P.v_cache);

    long long u = u0;
    while (u < u1) {
        const int bh = (int)(u / upb), j0 = (int)(u - (long long)bh * upb);
        const int j1 = (int)min((long long)upb, j0 + (u1 - u));
        const SampleRange sr = sample_range(P, bh / P.H);
        const int jt = sr.row / R;
        const float M = P.stats[2 * bh], Lsum = P.stats[2 * bh + 1];
        // pruning follows the reference kernel's arithmetic (attention.cu:1113, 1122, 1125,
        // 1185); the torch-rounding mode divides exactly like torch's softmax does
        const float inv = prune ? __fdividef(1.f, Lsum + 1.e-6f) : 1.f / Lsum;
        const float theta = Elem<T>::round(P.p * inv);
        const float* sc = P.scores + (size_t)bh * P.Lmax;
        auto prob_of = [&](float s) -> float {
            if (prune) return Elem<T>::round(__expf(s - M) * inv);
            return Elem<T>::round(expf(s - M) / Lsum);
        };

        float acc[VPL][EPV];
#pragma unroll
        for (int x = 0; x < VPL; ++x)
#pragma unroll
            for (int e = 0; e < EPV; ++e) acc[x][e] = 0.f;

        for (int j = j0; j < j1 && sr.ok; ++j) {
            const int lo = j * R, hi = min((j + 1) * R, sr.row + 1);  // includes the new token's bit
            if (hi <= lo) break;
            // survivors are listed in row order: ballots first, then a prefix over the words
            __syncthreads();
            float my_p[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int base = lo + (warp + 8 * k) * 32;
                my_p[k] = -1.f;
                if (base >= hi) continue;   // warp-uniform
                const int i = base + lane;
                const bool cached = i < sr.row && i >= sr.first;
                float pr = 0.f;
                bool keep = false;
                if (cached) {
                    pr = prob_of(sc[i]);
                    keep = prune ? !Elem<T>::leq(pr, theta) : true;
                }
                const unsigned bal = __ballot_sync(0xffffffffu, keep);
                if (P.kept_mask != nullptr && lane == 0)
                    P.kept_mask[(size_t)bh * P.mask_words + (base >> 5)] =
                        bal | ((sr.row >= base && sr.row < base + 32) ? (1u << (sr.row - base)) : 0u);
                if (lane == 0) s_words[warp + 8 * k] = bal;
                if (keep) my_p[k] = pr;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                if (my_p[k] >= 0.f) {
                    const int w = warp + 8 * k;
                    int pos = __popc(s_words[w] & ((1u << lane) - 1u));
                    for (int ww = 0; ww < w; ++ww) pos += __popc(s_words[ww]);
                    list_idx[pos] = lo + w * 32 + lane, list_p[pos] = my_p[k];
                }
            }
            if (tid == 0) {
                int tot = 0;
                for (int w = 0; w < ((hi - lo + 31) >> 5); ++w) tot += __popc(s_words[w]);
                s_n = tot;
            }
            __syncthreads();
            const int n = s_n;
            for (int base = 0; base < n; base += RB * NG) {
                uint4 raw[RB][VPL];
                float pr[RB];
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    const int idx = base + uu * NG + g;
                    const bool okr = idx < n;
                    pr[uu] = okr ? list_p[idx] : 0.f;
                    const int row = okr ? list_idx[idx] : 0;
#pragma unroll
                    for (int x = 0; x < VPL; ++x) {
                        const int vec = li + x * LPR;
                        raw[uu][x] = make_uint4(0, 0, 0, 0);
                        if (okr && vec < VPR)
                            raw[uu][x] = __ldg(reinterpret_cast<const uint4*>(vc + ((size_t)bh * P.Lmax + row) * ROWB + vec * 16));
                    }
                }
#pragma unroll
                for (int uu = 0; uu < RB; ++uu)
#pragma unroll
                    for (int x = 0; x < VPL; ++x) {
                        float vf[EPV];
                        Elem<T>::unpack(raw[uu][x], vf);
#pragma unroll
                        for (int e = 0; e < EPV; ++e) acc[x][e] = fmaf(pr[uu], vf[e], acc[x][e]);
                    }
            }
        }

        // the new token is never pruned (attention.cu:1227-1256): append v, add P_t * v
        if (sr.ok && j0 <= jt && jt < j1 && g == 0) {
            const float pt = prob_of(sc[sr.row]);
            const size_t row_off = ((size_t)bh * P.Lmax + sr.row) * ROWB;
#pragma unroll
            for (int x = 0; x < VPL; ++x) {
                const int vec = li + x * LPR;
                if (vec < VPR) {
                    const uint4 vraw = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.v) + (size_t)bh * ROWB + vec * 16);
                    *reinterpret_cast<uint4*>(static_cast<unsigned char*>(P.v_cache) + row_off + vec * 16) = vraw;
                    float vf[EPV];
                    Elem<T>::unpack(vraw, vf);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) acc[x][e] = fmaf(pt, vf[e], acc[x][e]);
                }
            }
        }

        // ---- sum the groups, then the CTAs ----
        __syncthreads();
#pragma unroll
        for (int x = 0; x < VPL; ++x) {
            const int vec = li + x * LPR;
            if (vec < VPR) {
#pragma unroll
                for (int e = 0; e < EPV; e += 4)
                    *reinterpret_cast<float4*>(red + g * DH + vec * EPV + e) =
                        make_float4(acc[x][e], acc[x][e + 1], acc[x][e + 2], acc[x][e + 3]);
            }
        }
        __syncthreads();
        const bool whole = (j0 == 0 && j1 == upb);
        T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
        float* part = P.partials + (size_t)(blockIdx.x + bh) * (DH + 2);
        for (int d = tid; d < DH; d += NT) {
            float A = 0.f;
            for (int gg = 0; gg < NG; ++gg) A += red[gg * DH + d];
            if (whole) Elem<T>::store(outp + d, A);
            else part[d] = A;
        }
        if (!whole) {
            __threadfence();
            __syncthreads();
            const int c_first = cut.first_cta_of(bh), c_last = cut.last_cta_of(bh);
            const int count = c_last - c_first + 1;
            if (tid == 0) s_last = (atomicAdd(P.tickets + bh, 1) == count - 1);
            __syncthreads();
            if (s_last) {
                __threadfence();
                const float* pbase = P.partials + (size_t)(c_first + bh) * (DH + 2);
                for (int d = tid; d < DH; d += NT) {
                    float A = 0.f;
                    for (int k = 0; k < count; ++k) A += __ldcg(pbase + (size_t)k * (DH + 2) + d);
                    Elem<T>::store(outp + d, A);
                }
                if (tid == 0) P.tickets[bh] = 0;
            }
        }
        if (!sr.ok && tid == 0) atomicOr(P.status, kStatusBadLength);
        u += j1 - j0;
    }
}

// ------------------------------------------------------------------------------------------
// Fused pruning step: one thread-block cluster per (batch, head), scores never leave the SMs
// ------------------------------------------------------------------------------------------
// The pruning rule needs the global max and sum of a (batch, head) before any V row may be
// touched (attention.cu:1184-1191), so the score pass and the value pass cannot be one
// streaming sweep.  Here both live in one kernel: a cluster of C CTAs owns a (batch, head);
// CTA r scores its slice of rows from a K-only bulk-copy ring into its OWN shared memory,
// the C pairs (max, sum) are exchanged through distributed shared memory behind a cluster
// barrier, every CTA prunes and gathers the V rows of its slice, and CTA 0 adds the C partial
// outputs (again through distributed shared memory).  No score scratch in HBM, no second
// launch, no arrival counters.  Used when a slice's scores fit in shared memory; the two
// kernels above remain for everything else.
//
// Shared memory: [stages][K tile] ring | scores[chunk_rows] | kept list (index, probability)
// | ballot words | group reduction area [NG][DH + 4] | partial output [DH] | (max, sum) | barriers | flags.
constexpr int kFusedThreads = 160;   // 1 copy warp + 4 compute warps
constexpr int kFusedListCap = 512;   // rows pruned and gathered per round (multiple of 32)

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
__device__ __forceinline__ float ld_peer_smem_f32(const void* own_smem_ptr, uint32_t peer_rank)
{
    uint32_t peer;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(smem_u32(own_smem_ptr)), "r"(peer_rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
    return v;
}

template <typename T, int DH>
__global__ void __launch_bounds__(kFusedThreads) ffa_prune_cluster_kernel(const FfaStepParams P)
{
    using G = RowGeom<T, DH>;
    constexpr int EPV = G::EPV, ROWB = G::ROWB, VPR = G::VPR, LPR = G::LPR, VPL = G::VPL, RB = G::RB;
    constexpr int NCW = 4, NCT = NCW * 32, NG = NCT / LPR, RS = DH + 4, E2 = EPV / 2;
    constexpr bool kAllLanes = (VPR == LPR * VPL);

    extern __shared__ __align__(128) unsigned char smem[];
    const int R = P.tile_rows, S = P.stages, C = P.cluster, chunk = P.chunk_rows;
    const uint32_t tile_bytes = (uint32_t)R * ROWB;
    float* sc = reinterpret_cast<float*>(smem + (size_t)S * tile_bytes);
    int* list_idx = reinterpret_cast<int*>(sc + chunk);
    float* list_p = reinterpret_cast<float*>(list_idx + kFusedListCap);
    unsigned* words = reinterpret_cast<unsigned*>(list_p + kFusedListCap);   // one ballot per 32 rows of a round
    float* red = reinterpret_cast<float*>(words + kFusedListCap / 32);
    float* accs = red + NG * RS;
    float* stat = accs + DH;                       // [0] max, [1] sum of this CTA's slice
    uint64_t* bars = reinterpret_cast<uint64_t*>(stat + 4);
    volatile int* flags = reinterpret_cast<volatile int*>(bars + 2 * S);  // [0] dead, [1] list length
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + S), ring = smem_u32(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t rank = cluster_rank();
    const int bh = blockIdx.x / C;
    const SampleRange sr = sample_range(P, bh / P.H);
    const int c0 = (int)rank * chunk;                                   // first absolute row of this slice
    const int lo = sr.ok ? max(c0, sr.first) : 0;
    const int hi = sr.ok ? min(c0 + chunk, sr.row) : 0;                 // cached rows [lo, hi)
    const bool owns_new = sr.ok && sr.row >= c0 && sr.row < c0 + chunk; // the new token's row is in this slice
    const int nrows = max(hi - lo, 0), ntiles = (nrows + R - 1) / R;
    const bool prune = P.p > 0.f;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, NCW);
        }
        flags[0] = 0, flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int ctid = tid - 32, g = ctid / LPR, li = ctid % LPR;   // meaningful for compute warps only
    float2 q2[VPL][E2];
    float qf[VPL][EPV];
    float m = -CUDART_INF_F, l = 0.f;

    auto score_of = [&](float dot) -> float {
        if (P.round_like_torch) return Elem<T>::round(Elem<T>::round(dot) * P.scale);
        return dot * P.scale;
    };

    // ---------------- phase 1: scores of this slice into shared memory ----------------
    if (warp == 0) {
        if (tid == 0) {
            const unsigned char* kc = static_cast<const unsigned char*>(P.k_cache) + ((size_t)bh * P.Lmax + lo) * ROWB;
            uint32_t stage = 0, use = 0;
            for (int j = 0; j < ntiles; ++j) {
                if (use > 0 && !mbar_wait_bounded(bar_empty + 8 * stage, (use - 1) & 1, flags)) break;
                const uint32_t bytes = (uint32_t)min(R, nrows - j * R) * ROWB;
                mbar_expect_tx(bar_full + 8 * stage, bytes);
                bulk_copy_g2s(ring + stage * tile_bytes, kc + (size_t)j * tile_bytes, bytes, bar_full + 8 * stage);
                if (++stage == (uint32_t)S) stage = 0, ++use;
            }
        }
    } else {
        load_row_f32<T, DH>(static_cast<const unsigned char*>(P.q) + (size_t)bh * ROWB, li, qf);
#pragma unroll
        for (int x = 0; x < VPL; ++x)
#pragma unroll
            for (int e = 1; e < EPV; e += 2) q2[x][e >> 1] = make_float2(qf[x][e - 1], qf[x][e]);

        uint32_t stage = 0, phase = 0;
        for (int j = 0; j < ntiles; ++j) {
            const int n = min(R, nrows - j * R);
            const bool ready = mbar_wait_bounded(bar_full + 8 * stage, phase, flags);
            const unsigned char* ks = smem + (size_t)stage * tile_bytes;
            float* sc_tile = sc + (lo - c0) + j * R;
            if (ready) {
                // RB rows per lane group at a time, loads first; FULL: every row of the batch exists
                auto batch = [&](auto full_tag, int base) {
                    constexpr bool FULL = decltype(full_tag)::value;
                    uint4 kraw[RB][VPL];
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu) {
                        const int r = base + uu * NG + g;
                        const int rc = FULL ? r : min(r, n - 1);
#pragma unroll
                        for (int x = 0; x < VPL; ++x)
                            kraw[uu][x] = *reinterpret_cast<const uint4*>(ks + (size_t)rc * ROWB + (li + x * LPR) * 16);
                    }
                    float s4[RB];
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu) {
                        float2 a = make_float2(0.f, 0.f);
#pragma unroll
                        for (int x = 0; x < VPL; ++x) {
                            float2 k2[E2];
                            Elem<T>::unpack2(kraw[uu][x], k2);
#pragma unroll
                            for (int e = 0; e < E2; ++e) a = __ffma2_rn(q2[x][e], k2[e], a);
                        }
                        s4[uu] = a.x + a.y;
                    }
#pragma unroll
                    for (int off = LPR / 2; off >= 1; off >>= 1)
#pragma unroll
                        for (int uu = 0; uu < RB; ++uu) s4[uu] += __shfl_xor_sync(0xffffffffu, s4[uu], off);
                    float m_new = m;
#pragma unroll
                    for (int uu = 0; uu < RB; ++uu) {
                        const int r = base + uu * NG + g;
                        const bool okr = FULL || r < n;
                        s4[uu] = okr ? score_of(s4[uu]) : -CUDART_INF_F;
                        if (okr && li == 0) sc_tile[r] = s4[uu];
                        m_new = fmaxf(m_new, s4[uu]);
                    }
                    if (FULL || m_new != -CUDART_INF_F) {
                        float psum = 0.f;
#pragma unroll
                        for (int uu = 0; uu < RB; ++uu) psum += __expf(s4[uu] - m_new);   // as attention.cu:1113
                        l = l * __expf(m - m_new) + psum;
                        m = m_new;
                    }
                };
                int base = 0;
                for (; base + RB * NG <= n; base += RB * NG) batch(std::true_type{}, base);
                if (base < n) batch(std::false_type{}, base);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
            if (++stage == (uint32_t)S) stage = 0, phase ^= 1;
        }
        // the new token: score against k, append k at row sr.row (attention.cu:900-958)
        if (owns_new) {
            float kf[VPL][EPV];
            load_row_f32<T, DH>(static_cast<const unsigned char*>(P.k) + (size_t)bh * ROWB, li, kf);
            float dot = 0.f;
#pragma unroll
            for (int x = 0; x < VPL; ++x)
#pragma unroll
                for (int e = 0; e < EPV; ++e) dot = fmaf(qf[x][e], kf[x][e], dot);
            dot = group_sum<LPR>(dot);
            if (g == 0) {
                const float st = score_of(dot);
                const float m_new = fmaxf(m, st);
                l = l * __expf(m - m_new) + __expf(st - m_new);
                m = m_new;
                if (li == 0) sc[sr.row - c0] = st;
                const size_t row_off = ((size_t)bh * P.Lmax + sr.row) * ROWB;
#pragma unroll
                for (int x = 0; x < VPL; ++x) {
                    const int vec = li + x * LPR;
                    if (vec < VPR)
                        *reinterpret_cast<uint4*>(static_cast<unsigned char*>(P.k_cache) + row_off + vec * 16) =
                            *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.k) + (size_t)bh * ROWB + vec * 16);
                }
            }
        }
        if (li == 0) red[g * RS] = m, red[g * RS + 1] = l;
    }
    __syncthreads();
    if (tid == 0) {
        float Mc = -CUDART_INF_F, Lc = 0.f;
        for (int gg = 0; gg < NG; ++gg) Mc = fmaxf(Mc, red[gg * RS]);
        for (int gg = 0; gg < NG; ++gg)
            if (red[gg * RS] != -CUDART_INF_F) Lc += red[gg * RS + 1] * __expf(red[gg * RS] - Mc);
        stat[0] = Mc, stat[1] = Lc;
    }
    cluster_sync_all();   // every slice's (max, sum) is visible cluster-wide; also a CTA barrier

    // ---------------- global statistics of the (batch, head) ----------------
    float M = -CUDART_INF_F, Lsum = 0.f;
    for (int c = 0; c < C; ++c) M = fmaxf(M, ld_peer_smem_f32(stat, c));
    for (int c = 0; c < C; ++c) {
        const float mc = ld_peer_smem_f32(stat, c);
        if (mc != -CUDART_INF_F) Lsum += ld_peer_smem_f32(stat + 1, c) * __expf(mc - M);
    }
    // pruning follows the reference kernel's arithmetic (attention.cu:1113, 1122, 1125, 1185);
    // the torch-rounding mode divides exactly like torch's softmax does
    const float inv = prune ? __fdividef(1.f, Lsum + 1.e-6f) : 1.f / Lsum;
    const float theta = Elem<T>::round(P.p * inv);
    auto prob_of = [&](float s) -> float {
        if (prune) return Elem<T>::round(__expf(s - M) * inv);
        return Elem<T>::round(expf(s - M) / Lsum);
    };

    // ---------------- phase 2: prune, gather the surviving V rows ----------------
    float2 acc2[VPL][E2];
#pragma unroll
    for (int x = 0; x < VPL; ++x)
#pragma unroll
        for (int e = 0; e < E2; ++e) acc2[x][e] = make_float2(0.f, 0.f);
    const unsigned char* vc = static_cast<const unsigned char*>(P.v_cache) + (size_t)bh * P.Lmax * ROWB;
    const int hi_mask = sr.ok ? min(c0 + chunk, sr.row + 1) : c0;   // rows whose mask bit this slice writes
    for (int sub = c0; sub < hi_mask; sub += kFusedListCap) {
        // Survivors are listed in row order (ballots first, then a prefix over the 32-row
        // words), so the order of the floating-point sums below never depends on timing.
        __syncthreads();
        const int sub_hi = min(sub + kFusedListCap, hi_mask);
        constexpr int kMine = (kFusedListCap / 32 + 4) / 5;   // 32-row words per warp and round
        float my_p[kMine];
#pragma unroll
        for (int k = 0; k < kMine; ++k) {
            const int base = sub + (warp + 5 * k) * 32;
            my_p[k] = -1.f;
            if (base >= sub_hi) continue;   // warp-uniform
            const int i = base + lane;
            const bool cached = i >= lo && i < hi;
            float pr = 0.f;
            bool keep = false;
            if (cached) {
                pr = prob_of(sc[i - c0]);
                keep = prune ? !Elem<T>::leq(pr, theta) : true;
            }
            const unsigned bal = __ballot_sync(0xffffffffu, keep);
            if (P.kept_mask != nullptr && lane == 0)
                P.kept_mask[(size_t)bh * P.mask_words + (base >> 5)] =
                    bal | ((sr.row >= base && sr.row < base + 32) ? (1u << (sr.row - base)) : 0u);
            if (lane == 0) words[warp + 5 * k] = bal;
            if (keep) my_p[k] = pr;
        }
        __syncthreads();
        const int nwords = (sub_hi - sub + 31) >> 5;
#pragma unroll
        for (int k = 0; k < kMine; ++k) {
            if (my_p[k] >= 0.f) {
                const int w = warp + 5 * k;
                int pos = __popc(words[w] & ((1u << lane) - 1u));
                for (int ww = 0; ww < w; ++ww) pos += __popc(words[ww]);
                list_idx[pos] = sub + w * 32 + lane, list_p[pos] = my_p[k];
            }
        }
        if (tid == 0) {
            int tot = 0;
            for (int w = 0; w < nwords; ++w) tot += __popc(words[w]);
            flags[1] = tot;
        }
        __syncthreads();
        const int n = flags[1];
        if (warp > 0) {
            for (int base = 0; base < n; base += RB * NG) {
                uint4 raw[RB][VPL];
                float pr[RB];
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    const int idx = base + uu * NG + g;
                    const bool okr = idx < n;
                    pr[uu] = okr ? list_p[idx] : 0.f;
                    const int row = okr ? list_idx[idx] : lo;
#pragma unroll
                    for (int x = 0; x < VPL; ++x) {
                        raw[uu][x] = make_uint4(0, 0, 0, 0);
                        if (okr && (kAllLanes || li + x * LPR < VPR))
                            raw[uu][x] = __ldg(reinterpret_cast<const uint4*>(vc + (size_t)row * ROWB + (li + x * LPR) * 16));
                    }
                }
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    const float2 p2 = make_float2(pr[uu], pr[uu]);
#pragma unroll
                    for (int x = 0; x < VPL; ++x) {
                        float2 v2[E2];
                        Elem<T>::unpack2(raw[uu][x], v2);
#pragma unroll
                        for (int e = 0; e < E2; ++e) acc2[x][e] = __ffma2_rn(p2, v2[e], acc2[x][e]);
                    }
                }
            }
        }
    }
    // the new token is never pruned (attention.cu:1227-1256): append v, add P_t * v
    if (warp > 0) {
        if (owns_new && g == 0) {
            const float pt = prob_of(sc[sr.row - c0]);
            const size_t row_off = ((size_t)bh * P.Lmax + sr.row) * ROWB;
#pragma unroll
            for (int x = 0; x < VPL; ++x) {
                const int vec = li + x * LPR;
                if (vec < VPR) {
                    const uint4 vraw = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.v) + (size_t)bh * ROWB + vec * 16);
                    *reinterpret_cast<uint4*>(static_cast<unsigned char*>(P.v_cache) + row_off + vec * 16) = vraw;
                    float2 v2[E2];
                    Elem<T>::unpack2(vraw, v2);
#pragma unroll
                    for (int e = 0; e < E2; ++e) {
                        acc2[x][e].x = fmaf(pt, v2[e].x, acc2[x][e].x);
                        acc2[x][e].y = fmaf(pt, v2[e].y, acc2[x][e].y);
                    }
                }
            }
        }
#pragma unroll
        for (int x = 0; x < VPL; ++x) {
            const int vec = li + x * LPR;
            if (vec < VPR) {
#pragma unroll
                for (int e = 0; e < E2; e += 2)
                    *reinterpret_cast<float4*>(red + g * RS + vec * EPV + 2 * e) =
                        make_float4(acc2[x][e].x, acc2[x][e].y, acc2[x][e + 1].x, acc2[x][e + 1].y);
            }
        }
    }
    __syncthreads();
    for (int d = tid; d < DH; d += kFusedThreads) {
        float A = 0.f;
        for (int gg = 0; gg < NG; ++gg) A += red[gg * RS + d];
        accs[d] = A;
    }
    cluster_sync_all();   // every slice's partial output is visible cluster-wide
    if (rank == 0) {
        T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
        for (int d = tid; d < DH; d += kFusedThreads) {
            float A = 0.f;
            for (int c = 0; c < C; ++c) A += ld_peer_smem_f32(accs + d, c);   // slice order: deterministic
            Elem<T>::store(outp + d, sr.ok ? A : 0.f);
        }
    }
    cluster_sync_all();   // peers keep their shared memory alive until CTA 0 has read it
    if (tid == 0) {
        if (flags[0]) atomicOr(P.status, kStatusWaitTimeout);
        if (!sr.ok && rank == 0) atomicOr(P.status, kStatusBadLength);
    }
}

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
    return stages * tensors_per_stage * tile_rows * rowb + ng * (head_dim + 4) * 4 + 2 * stages * 8 + 16;
}

int ffa_k_gather_smem_bytes(int dtype, int head_dim, int tile_rows)
{
    const int rowb = head_dim * elem_size(dtype);
    const int lpr = lanes_per_row(rowb);
    return tile_rows * 8 + (kGatherThreads / lpr) * head_dim * 4;
}

int ffa_k_fused_smem_bytes(int dtype, int head_dim, int tile_rows, int stages, int chunk_rows)
{
    const int rowb = head_dim * elem_size(dtype);
    const int lpr = lanes_per_row(rowb);
    const int ng = 128 / lpr;
    return stages * tile_rows * rowb + chunk_rows * 4 + kFusedListCap * 8 + kFusedListCap / 32 * 4 + ng * (head_dim + 4) * 4 + head_dim * 4 + 16 +
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
        cudaError_t e = raise_limit(reinterpret_cast<const void*>(ffa_stream_kernel<T, DH, kPassOne>));
        if (e != cudaSuccess) return (int)e;
        e = raise_limit(reinterpret_cast<const void*>(ffa_stream_kernel<T, DH, kPassScore>));
        if (e != cudaSuccess) return (int)e;
        e = raise_limit(reinterpret_cast<const void*>(ffa_value_gather_kernel<T, DH>));
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

int ffa_k_decode_onepass(int dtype, int head_dim, const FfaStepParams& P, int threads, int smem, cudaStream_t stream)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        ffa_stream_kernel<T, DH, kPassOne><<<P.grid, threads, smem, stream>>>(P);
        return (int)cudaGetLastError();
    });
}

int ffa_k_decode_fused_prune(int dtype, int head_dim, const FfaStepParams& P, int smem, cudaStream_t stream)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)P.grid, 1, 1);
        cfg.blockDim = dim3(kFusedThreads, 1, 1);
        cfg.dynamicSmemBytes = (size_t)smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)P.cluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        return (int)cudaLaunchKernelEx(&cfg, ffa_prune_cluster_kernel<T, DH>, P);
    });
}

int ffa_k_decode_twopass(int dtype, int head_dim, const FfaStepParams& Pk, const FfaStepParams& Pv, int threads,
                         int smem_k, int smem_v, cudaStream_t stream)
{
    return dispatch(dtype, head_dim, [&](auto t, auto dh) -> int {
        using T = decltype(t);
        constexpr int DH = decltype(dh)::value;
        ffa_stream_kernel<T, DH, kPassScore><<<Pk.grid, threads, smem_k, stream>>>(Pk);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
        ffa_value_gather_kernel<T, DH><<<Pv.grid, kGatherThreads, smem_v, stream>>>(Pv);
        return (int)cudaGetLastError();
    });
}
