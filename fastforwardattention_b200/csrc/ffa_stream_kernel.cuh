// The streaming split-KV kernel: exact one-pass attention.
#pragma once
#include "ffa_device_common.cuh"

namespace ffa_dev {

// Combines `count` partials (weighted sum [DH], running max, running sum; stride DH + 2 floats)
// that other CTAs left in global memory, in slot order, and writes the normalised output (and pushes it to the
// peers when the heads are sharded, see FfaStepParams::push_*).  Called by all `nthreads` threads of the CTA that
// arrived last.
template <typename T, int DH, bool kPrecise>
__device__ __forceinline__ void merge_partials(const FfaStepParams& P, uint32_t push_seq, int bh, const float* pbase, int count,
                                               T* outp, int tid, int nthreads)
{
    auto expo = [&](float x) -> float { return kPrecise ? expf(x) : fast_exp2(x); };
    constexpr int kAtOnce = 4;   // partials whose loads are all issued before the first is used (a split pair rarely has more)
    float MM = -CUDART_INF_F;
    if (count > kAtOnce)
        for (int k = 0; k < count; ++k) MM = fmaxf(MM, __ldcg(pbase + (size_t)k * (DH + 2) + DH));
    for (int d = tid; d < DH; d += nthreads) {
        float A = 0.f, L = 0.f;
        if (count <= kAtOnce) {
            // one trip to L2 instead of two: every partial's max, sum and element d are requested together
            float mk[kAtOnce], lk[kAtOnce], ak[kAtOnce];
#pragma unroll
            for (int k = 0; k < kAtOnce; ++k) {
                mk[k] = -CUDART_INF_F, lk[k] = 0.f, ak[k] = 0.f;
                if (k < count) {
                    const float* pk = pbase + (size_t)k * (DH + 2);
                    mk[k] = __ldcg(pk + DH), lk[k] = __ldcg(pk + DH + 1), ak[k] = __ldcg(pk + d);
                }
            }
#pragma unroll
            for (int k = 0; k < kAtOnce; ++k) MM = fmaxf(MM, mk[k]);
#pragma unroll
            for (int k = 0; k < kAtOnce; ++k) {   // slot order, as in the loop below
                if (k < count) {
                    const float w = mk[k] == -CUDART_INF_F ? 0.f : expo(mk[k] - MM);
                    A = fmaf(w, ak[k], A);
                    L = fmaf(w, lk[k], L);
                }
            }
        } else {
            for (int k = 0; k < count; ++k) {
                const float* pk = pbase + (size_t)k * (DH + 2);
                const float mk = __ldcg(pk + DH);
                const float w = mk == -CUDART_INF_F ? 0.f : expo(mk - MM);
                A = fmaf(w, __ldcg(pk + d), A);
                L = fmaf(w, __ldcg(pk + DH + 1), L);
            }
        }
        T o;
        Elem<T>::store(&o, L > 0.f ? A / L : 0.f);
        outp[d] = o;
        if (P.push_world > 1) push_store<T, DH>(P, push_seq, bh, d, o);
    }
}

// ------------------------------------------------------------------------------------------
// Streaming kernel (one-pass attention)
// ------------------------------------------------------------------------------------------
// Shared memory: [stages][K tile | V tile] ring, then the group
// reduction area [NG][DH + 4] (rows 16-byte aligned; max and sum in the tail), then
// full/empty barriers, then two flags, then [8][DH + 2] slots in which CTA 0 of a thread-block
// cluster receives the partial results of the cluster's CTAs.
// Warp 0 issues the copies (one elected lane); warps 1.. compute.  A lane group of LPR lanes
// owns a row: 16-byte shared-memory reads, fp32 FMAs, butterfly sum.  Each group keeps its
// own online-softmax state, so the row loop has no CTA-level synchronisation at all.
template <typename T, int DH>
// Register budget: 4 resident CTAs of 160 threads (or 2 of 288) need <= 96 registers per thread;
// head_dim 80 keeps five vectors per lane in flight and is compiled for 2 CTAs of 160 threads.
__global__ void __launch_bounds__(DH == 80 ? 288 : 320, DH == 80 ? 1 : 2) ffa_stream_kernel(const FfaStepParams P)
{
    using G = RowGeom<T, DH>;
    constexpr int EPV = G::EPV, ROWB = G::ROWB, VPR = G::VPR, LPR = G::LPR, VPL = G::VPL, RB = G::RB;
    constexpr bool kPrecise = sizeof(T) == 4;  // natural-log domain, full-precision exp
    constexpr int TENSORS = 2;
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
    // Cluster merge (one-pass, few pairs): the C CTAs that share a (batch, head) are one thread-block
    // cluster; each stores its partial (weighted sum, max, sum) into slot [rank] of CTA 0's shared
    // memory ahead of one cluster barrier, and CTA 0 combines the slots -- no partials in global
    // memory, no fence, no arrival counter, no remote load.  The launcher guarantees grid = B*H*C,
    // so a CTA owns exactly one part of exactly one pair.
    float* clp = reinterpret_cast<float*>(const_cast<int*>(flags) + 4);   // [kMaxClusterCtas][DH + 2]
    const bool cl = P.cluster > 1;
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + S);
    const uint32_t ring = smem_u32(smem);

    if (cl) cluster_arrive();   // "this CTA runs": its peers wait for that before they store into its shared memory
    pdl_release();
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, ncw);
        }
        flags[0] = 0, flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();   // nothing above touches global memory; everything below may read what the previous kernel wrote
    const bool push = P.push_world > 1;
    const uint32_t push_seq = push ? push_step(P) : 0u;

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
                bulk_copy_g2s(ring + stage * stage_bytes + tile_bytes, vc + off, bytes, bar_full + 8 * stage);
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
        __syncwarp();
        if (cl) cluster_wait();   // every thread pairs the arrival above with one wait
    } else {
        // ---------------- consumers ----------------
        const int ctid = threadIdx.x - 32;
        const int lane = ctid & 31;
        const int g = ctid / LPR, li = ctid % LPR;
        constexpr int E2 = EPV / 2;
        constexpr bool kAllLanes = (VPR == LPR * VPL);  // every lane of a group owns VPL vectors
        uint32_t stage = 0, phase = 0;
        long long u = u0;
        bool sent = false;   // cluster merge: this CTA's partial is in CTA 0's shared memory
        float* slot_in_leader = clp + (size_t)(cl ? cluster_rank() : 0u) * (DH + 2);
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
                    vnew[x] = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.v) + src);
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

            auto score_of = [&](float dot) -> float { return kPrecise ? dot * P.scale : dot; };
            auto expo = [&](float x) -> float { return kPrecise ? expf(x) : fast_exp2(x); };

            // RB (four; two for head_dim 80) rows per lane group at a time: all shared-memory loads first, then the
            // packed fp32 FMAs (fma.rn.f32x2), four interleaved butterfly sums, one softmax
            // update.  FULL: every row of the batch exists (no predicates, no clamping).
            auto batch = [&](auto full_tag, const unsigned char* ks, const unsigned char* vs, int base, int nrows) {
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
                {
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
                        for (; base + RB * NG <= nrows; base += RB * NG) batch(std::true_type{}, ks, vs, base, nrows);
                        if (base < nrows) batch(std::false_type{}, ks, vs, base, nrows);
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
                            {
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
                }
            }

            // ---- merge the groups of this CTA ----
            float* mine = red + g * RS;
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
            if (li == 0) mine[DH] = m, mine[DH + 1] = l;
            named_bar_sync(1, nct);
            float M = -CUDART_INF_F;
            for (int gg = 0; gg < NG; ++gg) M = fmaxf(M, red[gg * RS + DH]);
            // one exponential per group, not per group and element: thread gg leaves group gg's weight in the row's pad
            for (int gg = ctid; gg < NG; gg += nct) {
                const float mg = red[gg * RS + DH];
                red[gg * RS + DH + 2] = mg == -CUDART_INF_F ? 0.f : expo(mg - M);
            }
            named_bar_sync(1, nct);
            const bool whole = (j0 == 0 && j1 == upb);
            bool wrote_out = whole;   // this CTA wrote out[bh, :]: a whole pair, or the last arriver's merge
            const int slot = blockIdx.x + bh;
            float* part = P.partials + (size_t)slot * (DH + 2);
            T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
            if (cl && !whole && !sent) cluster_wait();   // CTA 0 runs
            for (int d = ctid; d < DH; d += nct) {
                float A = 0.f, L = 0.f;
                for (int gg = 0; gg < NG; ++gg) {
                    const float w = red[gg * RS + DH + 2];
                    A = fmaf(w, red[gg * RS + d], A);
                    L = fmaf(w, red[gg * RS + DH + 1], L);
                }
                if (whole) {
                    T o;
                    Elem<T>::store(&o, L > 0.f ? A / L : 0.f);
                    outp[d] = o;
                    if (push) push_store<T, DH>(P, push_seq, bh, d, o);
                } else if (cl) {
                    st_peer_smem_f32(slot_in_leader + d, 0, A);
                    if (d == 0) st_peer_smem_f32(slot_in_leader + DH, 0, M), st_peer_smem_f32(slot_in_leader + DH + 1, 0, L);
                } else {
                    part[d] = A;
                    if (d == 0) part[DH] = M, part[DH + 1] = L;
                }
            }
            if (cl && !whole) sent = true;
            if (!whole && !cl) {
                // cross-CTA merge without waiting: whoever arrives last does it.  The barrier orders every thread's
                // partial stores before the first thread's fence, which publishes them with the ticket; its fence after
                // the ticket and the second barrier order the other CTAs' partials before this CTA's reads (the chain a
                // grid-wide barrier is built from).
                named_bar_sync(1, nct);
                const int c_first = cut.first_cta_of(bh), c_last = cut.last_cta_of(bh);
                const int count = c_last - c_first + 1;
                if (ctid == 0) {
                    __threadfence();
                    const int old = atomicAdd(P.tickets + bh, 1);
                    __threadfence();
                    flags[1] = (old == count - 1);
                }
                named_bar_sync(1, nct);
                if (flags[1]) {
                    merge_partials<T, DH, kPrecise>(P, push_seq, bh, P.partials + (size_t)(c_first + bh) * (DH + 2), count, outp, ctid, nct);
                    if (ctid == 0) P.tickets[bh] = 0;  // ready for the next launch on this stream
                    wrote_out = true;
                }
            }
            if (push && wrote_out) __threadfence_system();   // this thread's rows are at the peers before the pair is counted
            named_bar_sync(1, nct);  // `red` and the flag are reused by the next segment
            if (push && wrote_out && ctid == 0) push_pair_done(P, push_seq);
            if (!sr.ok && ctid == 0) atomicOr(P.status, kStatusBadLength);
            u += j1 - j0;
        }
        if (cl && !sent) {   // a CTA without rows (or with a whole pair): its slot says "nothing seen"
            cluster_wait();
            for (int d = ctid; d < DH + 2; d += nct) st_peer_smem_f32(slot_in_leader + d, 0, d == DH ? -CUDART_INF_F : 0.f);
        }
    }
    __syncthreads();
    if (cl) {
        // A pair's C = Q * K CTAs are K clusters of Q.  Inside a cluster: distributed shared memory.
        // Across the K cluster leaders (K > 1: very few pairs): partials in global memory and the
        // arrival counter, as in the non-cluster path, with K instead of C partials to combine.
        const int C = P.parts_per_bh, Q = P.cluster, K = C / Q;
        const int bh = blockIdx.x / C, kc = (blockIdx.x - bh * C) / Q;
        const bool leader = cluster_rank() == 0;
        T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
        float* part = P.partials + ((size_t)bh * K + kc) * (DH + 2);
        cluster_sync_all();   // every CTA's partial has arrived in CTA 0's shared memory
        if (leader) {
            for (int d = threadIdx.x; d < DH; d += blockDim.x) {
                float MM = -CUDART_INF_F;
                for (int c = 0; c < Q; ++c) MM = fmaxf(MM, clp[c * (DH + 2) + DH]);
                float A = 0.f, L = 0.f;
                for (int c = 0; c < Q; ++c) {   // rank order: deterministic
                    const float mc = clp[c * (DH + 2) + DH];
                    const float w = mc == -CUDART_INF_F ? 0.f : (kPrecise ? expf(mc - MM) : fast_exp2(mc - MM));
                    A = fmaf(w, clp[c * (DH + 2) + d], A);
                    L = fmaf(w, clp[c * (DH + 2) + DH + 1], L);
                }
                if (K == 1) {
                    T o;
                    Elem<T>::store(&o, L > 0.f ? A / L : 0.f);
                    outp[d] = o;
                    if (push) push_store<T, DH>(P, push_seq, bh, d, o);
                } else {
                    part[d] = A;
                    if (d == 0) part[DH] = MM, part[DH + 1] = L;
                }
            }
        }
        if (push && leader && K == 1) {
            __threadfence_system();   // rows at the peers before the pair is counted
            __syncthreads();
            if (threadIdx.x == 0) push_pair_done(P, push_seq);
        }
        if (leader && K > 1) {
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) flags[1] = (atomicAdd(P.tickets + bh, 1) == K - 1);
            __syncthreads();
            if (flags[1]) {
                __threadfence();
                merge_partials<T, DH, kPrecise>(P, push_seq, bh, P.partials + (size_t)bh * K * (DH + 2), K, outp, threadIdx.x, blockDim.x);
                if (threadIdx.x == 0) P.tickets[bh] = 0;
                if (push) {
                    __threadfence_system();
                    __syncthreads();
                    if (threadIdx.x == 0) push_pair_done(P, push_seq);
                }
            }
        }
    }
    if (threadIdx.x == 0 && flags[0]) atomicOr(P.status, kStatusWaitTimeout);
}

}  // namespace ffa_dev
