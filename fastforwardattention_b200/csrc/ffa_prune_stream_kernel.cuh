// The streaming pruning kernel: one persistent launch for p > 0 (and the torch-rounding mode) at any size.
#pragma once
#include "ffa_device_common.cuh"

namespace ffa_dev {

// The pruning rule needs the global max and sum of a (batch, head) before any V row may be
// touched (attention.cu:1184-1191): every K row is read, then only the surviving V rows.  The
// reference does both in one CTA per (batch, head) with all scores in shared memory, which caps
// its sequence length; here the K rows of ALL pairs stream through one persistent grid exactly
// like the exact kernel's K and V rows do, and the V rows of a pair are gathered while the K
// rows of the next pairs keep streaming.  A CTA has three roles:
//
//   warp 0              issues the K tiles (1-D bulk copies into a ring of `stages` buffers,
//                       full / empty mbarriers) for this CTA's run of the flat unit list;
//   scorer warps        (4 or 8) consume the tiles, RB rows per lane group at a time: the RB partial
//                       dot products of a group are reduced with a transposed butterfly (5 shuffles
//                       for 4 rows over 16 lanes instead of 16), which leaves every lane with ONE row's
//                       score; that lane stores it to the score scratch in global memory (4 bytes per
//                       row, a 32-byte sector per warp; read back from L2) and folds it into its own
//                       running (max, sum) -- no cross-lane softmax step in the loop.  With K tiles
//                       only, a row-loop iteration carries half the bytes of the exact kernel's, so
//                       the instruction count per row, not HBM, is what this loop has to watch.  The
//                       new token's score and its K append ride along.  A pair cut over several CTAs
//                       is combined by whoever arrives last (partials + ticket, no waiting).  The CTA
//                       that completes a pair's (max, sum) posts a JOB;
//   gather warps        (4) take jobs: a job's rows are dealt round by round to 12 STREAMS; a warp claims a stream
//                       (a counter in shared memory), re-reads its scores, applies the reference rule
//                       (P = cvt_T(e * inv), Theta = cvt_T(p * inv), skip iff leq(P, Theta)), writes the
//                       optional kept mask, lists the survivors in row order, fetches only those V rows
//                       (16-byte cp.async into a staging area), drops the consumed score lines from L2, and
//                       leaves the stream's partial output in shared memory; the warp that completes a job's
//                       last stream adds the 12 partials in stream order, appends the new token's v and
//                       stores the output row.  Who computed which stream never shows in the result.
//
// Scoring never waits for gathering unless two jobs are already queued, so HBM sees one
// continuous K stream with the V reads of earlier pairs mixed in.  When a CTA's scorer warps run out
// of K rows they turn into gather warps for the job they posted last (their staging areas are
// carved from the K ring, which is idle by then): the gather of a CTA's final pair, which nothing
// can overlap, is spread over all its warps instead of four.  Every wait is time-bounded.
//
// Shared memory: [stages][K tile] ring | per gather warp: V-row staging [kPsStageBytes] | scorer groups'
// (max, sum) [2][NG * RB][2] | per gather warp: survivor list [2 * kPsListCap words] | stream partial
// outputs [jobs][streams][DH] | job slots | stream counters: claimed[J], finished[J] | barriers: full[S],
// empty[S], job_full[J], job_empty[J] | flags.
constexpr int kPsGatherWarps = 4;
constexpr int kPsStreams = 12;    // partial sums per job; also the most warps that can work on one job
constexpr int kPsListCap = 256;   // survivor list of a gather warp: 256 (row, probability) entries of 8 bytes, or 512 packed into 4
constexpr int kPsWordsPerRound = kPsListCap / 32;   // 32-row words a gather warp tests per round (twice that for 16-bit tensors)
constexpr int kPsStageBytes = 4096;   // per gather warp: surviving V rows land here (cp.async), up to 16 rows in flight
constexpr int kPsHelperBytes = kPsStageBytes + 2 * kPsListCap * 4;   // staging + list of a scorer warp that helps
constexpr int kPsJobs = 2;        // queued (batch, head) pairs between scorers and gatherers

struct PsJob {
    int bh;       // pair to gather; -1: no more jobs
    float M, L;   // max and sum(exp) over the pair's rows, new token included
    int seq;      // how often this slot has been used before: tells a late warp that the slot has moved on
};

// head_dim 80 keeps five vectors per lane in flight: at most 4 scorer warps there, for the register budget of
// two resident CTAs
constexpr int ps_max_scorer_warps(int dh) { return dh == 80 ? 4 : 8; }

template <typename T, int DH>
__global__ void __launch_bounds__(32 * (1 + ps_max_scorer_warps(DH) + kPsGatherWarps), 2) ffa_prune_stream_kernel(const FfaStepParams P)
{
    using G = RowGeom<T, DH>;
    constexpr int EPV = G::EPV, ROWB = G::ROWB, VPR = G::VPR, LPR = G::LPR, VPL = G::VPL, RB = G::RB;
    constexpr int E2 = EPV / 2;
    constexpr bool kAllLanes = (VPR == LPR * VPL);
    constexpr int NGW = kPsGatherWarps, GPW = 32 / LPR;     // gather warps; lane groups (rows in flight per step) per warp
    constexpr int STEPS = VPL >= 4 ? 1 : 8 / VPL;           // V rows a lane group keeps in flight per batch
    constexpr int SROWS = STEPS * GPW;                      // rows per batch and gather warp
    static_assert(SROWS * ROWB <= kPsStageBytes, "a batch of V rows fits the warp's staging area");

    extern __shared__ __align__(128) unsigned char smem[];
    const int R = P.tile_rows, S = P.stages;
    const int nsw = (blockDim.x >> 5) - 1 - NGW;   // scorer warps
    const int nct = nsw * 32, NG = nct / LPR;      // scorer threads, scorer lane groups
    const uint32_t tile_bytes = (uint32_t)R * ROWB;
    unsigned char* gstage = smem + (size_t)S * tile_bytes;                           // [NGW][kPsStageBytes]
    float* red = reinterpret_cast<float*>(gstage + NGW * kPsStageBytes);             // [2][NG * RB][2], alternating per segment
    uint32_t* lists = reinterpret_cast<uint32_t*>(red + 4 * NG * RB);                // [NGW][2 * kPsListCap] words
    float* gred = reinterpret_cast<float*>(lists + NGW * 2 * kPsListCap);            // [kPsJobs][kPsStreams][DH]
    PsJob* jobs = reinterpret_cast<PsJob*>(gred + kPsJobs * kPsStreams * DH);        // [kPsJobs]
    int* claimed = reinterpret_cast<int*>(jobs + kPsJobs);                           // [kPsJobs] streams handed out, over all uses of the slot
    int* finished = claimed + kPsJobs;                                               // [kPsJobs] streams completed, likewise
    uint64_t* bars = reinterpret_cast<uint64_t*>(finished + kPsJobs);
    volatile int* flags = reinterpret_cast<volatile int*>(bars + 2 * S + 2 * kPsJobs);  // [0] dead, [2] jobs this CTA posted
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + S);
    const uint32_t bar_jfull = smem_u32(bars + 2 * S), bar_jempty = bar_jfull + 8 * kPsJobs;
    const uint32_t ring = smem_u32(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_release();
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, nsw);
        }
        for (int j = 0; j < kPsJobs; ++j) {
            mbar_init(bar_jfull + 8 * j, 1);
            mbar_init(bar_jempty + 8 * j, 1);
            claimed[j] = 0, finished[j] = 0;
        }
        flags[0] = 0, flags[1] = 0, flags[2] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();   // nothing above touches global memory

    const int upb = P.units_per_bh;
    const Partition cut = make_partition(P);
    const long long u0 = cut.first_unit(blockIdx.x), u1 = cut.first_unit(blockIdx.x + 1);
    const bool prune = P.p > 0.f;

    if (warp == 0) {
        // ---------------- producer: K tiles of this CTA's run ----------------
        if (tid == 0) {
            const unsigned char* kc = static_cast<const unsigned char*>(P.k_cache);
            const uint64_t once = l2_policy_evict_first();   // K rows are read once: keep them from displacing the scores in L2
            uint32_t issued = 0, stage = 0, use = 0;
            int cur_b = -1;
            SampleRange sr{0, 0, false};
            int bh = (int)(u0 / upb), j = (int)(u0 - (long long)bh * upb);
            for (long long u = u0; u < u1; ++u, ++j) {
                if (j == upb) j = 0, ++bh;
                const int b = bh / P.H;
                if (b != cur_b) sr = sample_range(P, b), cur_b = b;
                if (!sr.ok) continue;
                const int lo = max(j * R, sr.first), hi = min((j + 1) * R, sr.row);
                if (hi <= lo) continue;
                if (use > 0 && !mbar_wait_bounded(bar_empty + 8 * stage, (use - 1) & 1, flags)) break;
                const uint32_t bytes = (uint32_t)(hi - lo) * ROWB;
                mbar_expect_tx(bar_full + 8 * stage, bytes);
                bulk_copy_g2s_hint(ring + stage * tile_bytes, kc + cache_row_offset(P, bh, lo, ROWB), bytes, bar_full + 8 * stage, once);
                ++issued;
                if (++stage == (uint32_t)S) stage = 0, ++use;
            }
            if (flags[0]) {   // gave up: let the copies already issued land before the CTA releases its shared memory
                const uint32_t pending = issued < (uint32_t)S ? issued : (uint32_t)S;
                for (uint32_t k = 0; k < pending; ++k) {
                    const uint32_t id = issued - 1 - k, st = id % S, us = id / S;
                    for (uint32_t n = 0; n < kDrainPolls && !mbar_try_wait(bar_full + 8 * st, us & 1); ++n) __nanosleep(256);
                }
            }
        }
    }
    // one job to the gather warps (first scorer thread): wait for a free slot, fill it, publish it
    uint32_t pslot = 0, puse = 0;
    auto post_job = [&](int bh, float M, float L) {
        if (puse > 0 && !mbar_wait_bounded(bar_jempty + 8 * pslot, (puse - 1) & 1, flags)) return;
        jobs[pslot].bh = bh, jobs[pslot].M = M, jobs[pslot].L = L, jobs[pslot].seq = (int)puse;
        mbar_arrive(bar_jfull + 8 * pslot);
        if (++pslot == kPsJobs) pslot = 0, ++puse;
    };
    int help_job = -1;   // scorer warps: the job they join once they have no K rows left
    if (warp >= 1 && warp <= nsw) {
        // ---------------- scorers ----------------
        const int ctid = tid - 32;
        const int g = ctid / LPR, li = ctid % LPR;
        const int myrow = transposed_row<LPR, RB>(li);                  // which of a batch's RB rows this lane ends up holding
        const bool store_lane = (li % (LPR / RB)) == 0;                 // one lane per (group, row) writes the score
        uint32_t stage = 0, phase = 0;
        const unsigned char* qbase = static_cast<const unsigned char*>(P.q);
        uint4 qraw[VPL];
#pragma unroll
        for (int x = 0; x < VPL; ++x) {
            qraw[x] = make_uint4(0, 0, 0, 0);
            if (u0 < u1 && li + x * LPR < VPR)
                qraw[x] = *reinterpret_cast<const uint4*>(qbase + (size_t)(u0 / upb) * ROWB + (li + x * LPR) * 16);
        }
        auto score_of = [&](float dot) -> float {
            if (P.round_like_torch) return Elem<T>::round(Elem<T>::round(dot) * P.scale);
            return dot * P.scale;
        };
        long long u = u0;
        int rbuf = 0;   // which half of `red` this segment uses
        while (u < u1) {
            const int bh = (int)(u / upb), j0 = (int)(u - (long long)bh * upb);
            const int j1 = (int)min((long long)upb, j0 + (u1 - u));
            const SampleRange sr = sample_range(P, bh / P.H);
            const int jt = sr.row / R;   // the unit that also owns the new token
            float qf[VPL][EPV];
            float2 q2[VPL][E2];
#pragma unroll
            for (int x = 0; x < VPL; ++x) {
                Elem<T>::unpack(qraw[x], qf[x]);
#pragma unroll
                for (int e = 1; e < EPV; e += 2) q2[x][e >> 1] = make_float2(qf[x][e - 1], qf[x][e]);
            }
            if (u + (j1 - j0) < u1) {   // this CTA goes on with the next (batch, head): fetch its q now
#pragma unroll
                for (int x = 0; x < VPL; ++x)
                    if (li + x * LPR < VPR)
                        qraw[x] = *reinterpret_cast<const uint4*>(qbase + (size_t)(bh + 1) * ROWB + (li + x * LPR) * 16);
            }
            const bool owns_new = sr.ok && j0 <= jt && jt < j1;
            uint4 knew[VPL];
#pragma unroll
            for (int x = 0; x < VPL; ++x) {
                knew[x] = make_uint4(0, 0, 0, 0);
                if (owns_new && li + x * LPR < VPR)
                    knew[x] = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(P.k) + (size_t)bh * ROWB + (li + x * LPR) * 16);
            }
            float m = -CUDART_INF_F, l = 0.f;   // of the rows this lane was handed (see transposed_group_sum)
            float* sc_row = P.scores + (size_t)bh * P.score_stride;

            // RB rows per lane group at a time: shared-memory loads first, packed fp32 FMAs,
            // interleaved butterfly sums; FULL: every row of the batch exists
            auto batch = [&](auto full_tag, const unsigned char* ks, int base, int nrows, int row0) {
                constexpr bool FULL = decltype(full_tag)::value;
                uint4 kraw[RB][VPL];
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    const int r = base + g * RB + uu;   // a lane group owns RB consecutive rows: its scores are one vector store
                    const int rc = FULL ? r : min(r, nrows - 1);
#pragma unroll
                    for (int x = 0; x < VPL; ++x)
                        if (kAllLanes || li + x * LPR < VPR)
                            kraw[uu][x] = *reinterpret_cast<const uint4*>(ks + (size_t)rc * ROWB + (li + x * LPR) * 16);
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
                // every lane ends up with ONE row's total (row `myrow` of the group's RB rows) and keeps the
                // running (max, sum) of the rows it is handed: no cross-lane softmax step in the loop
                const float dot = transposed_group_sum<LPR, RB>(sc, li);
                const bool okr = FULL || base + g * RB + myrow < nrows;
                const float st = okr ? score_of(dot) : -CUDART_INF_F;
                if (okr && store_lane) sc_row[row0 + base + g * RB + myrow] = st;   // RB lanes, RB * 4 contiguous bytes
                const float m_new = fmaxf(m, st);
                if (FULL || m_new != -CUDART_INF_F) {
                    l = l * __expf(m - m_new) + __expf(st - m_new);   // as attention.cu:1113
                    m = m_new;
                }
            };

            if (sr.ok) {
                for (int j = j0; j < j1; ++j) {
                    const int lo = max(j * R, sr.first), hi = min((j + 1) * R, sr.row);
                    if (hi <= lo) continue;
                    const int nrows = hi - lo;
                    const bool ready = mbar_wait_bounded(bar_full + 8 * stage, phase, flags);
                    const unsigned char* ks = smem + (size_t)stage * tile_bytes;
                    if (ready) {
                        int base = 0;
                        for (; base + RB * NG <= nrows; base += RB * NG) batch(std::true_type{}, ks, base, nrows, lo);
                        if (base < nrows) batch(std::false_type{}, ks, base, nrows, lo);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
                    if (++stage == (uint32_t)S) stage = 0, phase ^= 1;
                }
            }
            // the new token: score against k, append k at row sr.row (attention.cu:900-958)
            if (owns_new) {
                float dot = 0.f;
#pragma unroll
                for (int x = 0; x < VPL; ++x) {
                    float kf[EPV];
                    Elem<T>::unpack(knew[x], kf);
#pragma unroll
                    for (int e = 0; e < EPV; ++e) dot = fmaf(qf[x][e], kf[e], dot);
                }
                dot = group_sum<LPR>(dot);
                if (g == 0) {
                    const float st = score_of(dot);
                    if (li == 0) {   // one lane's state takes the new token (lane 0 is a store lane, so it is counted below)
                        const float m_new = fmaxf(m, st);
                        l = l * __expf(m - m_new) + __expf(st - m_new);
                        m = m_new;
                        sc_row[sr.row] = st;
                    }
                    const size_t row_off = cache_row_offset(P, bh, sr.row, ROWB);
#pragma unroll
                    for (int x = 0; x < VPL; ++x)
                        if (li + x * LPR < VPR)
                            *reinterpret_cast<uint4*>(static_cast<unsigned char*>(P.k_cache) + row_off + (li + x * LPR) * 16) = knew[x];
                }
            }
            // ---- (max, sum) of this CTA's piece: the first scorer warp combines the lane groups ----
            // The other scorer warps go straight on to the next segment: `red` alternates between two halves, and a
            // half is written again only after the barrier of the segment in between, which the first warp joins
            // when it is done here.  The scores were stored by all scorer threads; the barrier orders those stores
            // before the first warp's device-wide fence below, which is what makes them visible to whoever is told
            // about them (the same chain a grid-wide barrier is built from).
            float* redb = red + rbuf * 2 * NG * RB;
            if (store_lane) redb[2 * (g * RB + myrow)] = m, redb[2 * (g * RB + myrow) + 1] = l;   // one entry per (group, row class)
            named_bar_sync(1, nct);
            rbuf ^= 1;
            const bool whole = (j0 == 0 && j1 == upb);
            if (warp == 1) {
                __threadfence();
                float Mg = -CUDART_INF_F, Lg = 0.f;
                for (int gg = lane; gg < NG * RB; gg += 32) Mg = fmaxf(Mg, redb[2 * gg]);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) Mg = fmaxf(Mg, __shfl_xor_sync(0xffffffffu, Mg, off));
                for (int gg = lane; gg < NG * RB; gg += 32)
                    if (redb[2 * gg] != -CUDART_INF_F) Lg += redb[2 * gg + 1] * __expf(redb[2 * gg] - Mg);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) Lg += __shfl_xor_sync(0xffffffffu, Lg, off);
                if (!sr.ok) {
                    // the CTA that owns the pair's first unit reports the bad length and clears the output row
                    if (lane == 0 && j0 == 0) atomicOr(P.status, kStatusBadLength);
                    if (j0 == 0)
                        for (int d = lane; d < DH; d += 32) Elem<T>::store(static_cast<T*>(P.out) + (size_t)bh * DH + d, 0.f);
                } else if (whole) {
                    if (lane == 0) post_job(bh, Mg, Lg);
                } else {
                    // a pair cut over several CTAs: partial (max, sum) to global memory; whoever arrives last combines
                    float* part = P.partials + (size_t)(blockIdx.x + bh) * (DH + 2);
                    const int c_first = cut.first_cta_of(bh), c_last = cut.last_cta_of(bh);
                    const int count = c_last - c_first + 1;
                    int last = 0;
                    if (lane == 0) {
                        part[DH] = Mg, part[DH + 1] = Lg;
                        __threadfence();
                        last = atomicAdd(P.tickets + bh, 1) == count - 1;
                    }
                    last = __shfl_sync(0xffffffffu, last, 0);
                    if (last) {
                        __threadfence();
                        const float* pbase = P.partials + (size_t)(c_first + bh) * (DH + 2);
                        float MM = -CUDART_INF_F, LL = 0.f;
                        for (int k = lane; k < count; k += 32) MM = fmaxf(MM, __ldcg(pbase + (size_t)k * (DH + 2) + DH));
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) MM = fmaxf(MM, __shfl_xor_sync(0xffffffffu, MM, off));
                        for (int k = lane; k < count; k += 32) {
                            const float mk = __ldcg(pbase + (size_t)k * (DH + 2) + DH);
                            if (mk != -CUDART_INF_F) LL += __ldcg(pbase + (size_t)k * (DH + 2) + DH + 1) * __expf(mk - MM);
                        }
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) LL += __shfl_xor_sync(0xffffffffu, LL, off);
                        if (lane == 0) {
                            P.tickets[bh] = 0;   // ready for the next launch on this stream
                            post_job(bh, MM, LL);
                        }
                    }
                }
            }
            u += j1 - j0;
        }
        // out of K rows: the ring is idle once every scorer warp is here; join the gather of the job posted last
        if (tid == 32) flags[2] = (int)(puse * kPsJobs + pslot);
        named_bar_sync(1, nct);
        help_job = flags[2] - 1;
    }
    // ---------------- gather: the gather warps take every job, the scorer warps the last one ----------------
    if (warp >= 1) {
        const bool helper = warp <= nsw;
        const int gl = lane / LPR, li = lane % LPR;
        // Survivors of a round, in row order.  16-bit tensors: one word per survivor (row offset within the round,
        // probability as the 16 bits it was rounded to), so a round covers 16 words of 32 rows; fp32: (row, probability).
        constexpr bool kPacked = sizeof(T) == 2;
        constexpr int WPR = kPacked ? 2 * kPsWordsPerRound : kPsWordsPerRound;
        // a scorer warp's staging area and list come out of the K ring (as many warps as fit help)
        const bool has_room = !helper || (size_t)warp * kPsHelperBytes <= (size_t)S * tile_bytes;
        unsigned char* my_stage_p = helper ? smem + (size_t)(warp - 1) * kPsHelperBytes : gstage + (warp - 1 - nsw) * kPsStageBytes;
        uint32_t* my_list = helper ? reinterpret_cast<uint32_t*>(my_stage_p + kPsStageBytes) : lists + (warp - 1 - nsw) * 2 * kPsListCap;
        const uint32_t my_stage = smem_u32(my_stage_p);
        const unsigned char* vc = static_cast<const unsigned char*>(P.v_cache);
        const uint64_t once = l2_policy_evict_first();   // surviving V rows are read once too
        uint32_t gslot = 0, guse = 0;
        if (helper) gslot = (uint32_t)(help_job < 0 ? 0 : help_job % kPsJobs), guse = (uint32_t)(help_job < 0 ? 0 : help_job / kPsJobs);
        const bool idle = helper && (help_job < 0 || !has_room);
        while (!idle) {
            // a gather warp waits for the slot's next job; a helper's job was posted by its own CTA before the barrier above
            if (!helper && !mbar_wait_bounded(bar_jfull + 8 * gslot, guse & 1, flags)) break;
            const int bh = jobs[gslot].bh;
            const float M = jobs[gslot].M, Lsum = jobs[gslot].L;
            const int seq = jobs[gslot].seq;
            if (bh < 0) break;
            if (seq == (int)guse) {   // otherwise the job this warp came for is finished and the slot holds a later one
                const SampleRange sr = sample_range(P, bh / P.H);
                // pruning follows the reference kernel's arithmetic (attention.cu:1113, 1122, 1125, 1185);
                // the torch-rounding mode divides exactly like torch's softmax does
                const float inv = prune ? __fdividef(1.f, Lsum + 1.e-6f) : 1.f / Lsum;
                const float theta = Elem<T>::round(P.p * inv);
                auto prob_of = [&](float sv) -> float {
                    if (prune) return Elem<T>::round(__expf(sv - M) * inv);
                    return Elem<T>::round(expf(sv - M) / Lsum);
                };
                const float* sc_row = P.scores + (size_t)bh * P.score_stride;
                uint32_t* mask_row = P.kept_mask != nullptr ? P.kept_mask + (size_t)bh * P.mask_words : nullptr;
                const int nwords = (sr.row >> 5) + 1;   // 32-row words that hold rows 0..sr.row
                const int ticket_end = ((int)guse + 1) * kPsStreams;
                const int active = min(kPsStreams, (nwords + WPR - 1) / WPR);   // streams that have rows; the rest are empty
                // scores of a round's words, all loads before the first use (written by other threads: read at L2)
                auto load_scores = [&](int w0, float (&sv)[WPR]) {
#pragma unroll
                    for (int k = 0; k < WPR; ++k) {
                        const int i = (w0 + k) * 32 + lane;
                        sv[k] = (w0 + k < nwords && i >= sr.first && i < sr.row) ? __ldcg(sc_row + i) : 0.f;
                    }
                };
                for (;;) {
                    // claim the job's next stream (tickets count over all uses of the slot, so a warp that comes late
                    // can never take one of a later job by mistake)
                    int strm = -1, took = 0;
                    if (lane == 0) {
                        int cur = *reinterpret_cast<volatile int*>(claimed + gslot);
                        while (cur < ticket_end) {
                            const int idx = cur - (int)guse * kPsStreams;
                            const int n_take = idx >= active ? ticket_end - cur : 1;   // the empty streams go in one claim
                            const int old = atomicCAS(claimed + gslot, cur, cur + n_take);
                            if (old == cur) {
                                strm = idx, took = n_take;
                                break;
                            }
                            cur = old;
                        }
                    }
                    strm = __shfl_sync(0xffffffffu, strm, 0);
                    took = __shfl_sync(0xffffffffu, took, 0);
                    if (strm < 0) break;
                    float2 acc2[VPL][E2];
#pragma unroll
                    for (int x = 0; x < VPL; ++x)
#pragma unroll
                        for (int e = 0; e < E2; ++e) acc2[x][e] = make_float2(0.f, 0.f);
                    float sv[WPR];
                    int w0 = strm * WPR;
                    if (w0 < nwords) load_scores(w0, sv);
                    for (; w0 < nwords; w0 += kPsStreams * WPR) {
                        int n = 0;
                        __syncwarp();   // the previous round's list has been consumed by every lane
                        // straight-line code, no branch per word: the 16 (8) words' chains of exponential, rounding and vote
                        // overlap; only the running count n links them
#pragma unroll
                        for (int k = 0; k < WPR; ++k) {
                            const int base = (w0 + k) * 32, i = base + lane;
                            const bool cached = w0 + k < nwords && i >= sr.first && i < sr.row;
                            const float pr = prob_of(sv[k]);
                            const bool keep = cached && (prune ? !Elem<T>::leq(pr, theta) : true);
                            const unsigned bal = __ballot_sync(0xffffffffu, keep);
                            if (mask_row != nullptr && lane == 0 && w0 + k < nwords)
                                mask_row[w0 + k] = bal | ((sr.row >= base && sr.row < base + 32) ? (1u << (sr.row - base)) : 0u);
                            const int pos = n + __popc(bal & ((1u << lane) - 1u));
                            if constexpr (kPacked) {
                                if (keep) my_list[pos] = (uint32_t)(i - w0 * 32) | (Elem<T>::bits(pr) << 16);
                            } else {
                                if (keep) my_list[2 * pos] = (uint32_t)i, my_list[2 * pos + 1] = __float_as_uint(pr);
                            }
                            n += __popc(bal);
                        }
                        // This round's score lines (one per 32-row word; every lane has used its values by now) are not needed
                        // again: spare HBM their write-back.  The word of the new token's row is read once more and left alone.
                        if (lane < WPR && w0 + lane < nwords - 1) l2_discard_line(sc_row + (size_t)(w0 + lane) * 32);
                        // the next round's scores travel while this round's V rows are fetched
                        if (w0 + kPsStreams * WPR < nwords) load_scores(w0 + kPsStreams * WPR, sv);
                        __syncwarp();
                        // survivors in row order; lane group gl takes entries gl, gl + GPW, ...; a batch of SROWS rows is
                        // copied into the warp's staging area (every lane its own 16-byte pieces), then accumulated
                        for (int base = 0; base < n; base += SROWS) {
#pragma unroll
                            for (int st = 0; st < STEPS; ++st) {
                                const int e = base + st * GPW + gl;
                                if (e < n) {
                                    const int row = kPacked ? w0 * 32 + (int)(my_list[e] & 0xffffu) : (int)my_list[2 * e];
                                    const unsigned char* src = vc + cache_row_offset(P, bh, row, ROWB);
#pragma unroll
                                    for (int x = 0; x < VPL; ++x)
                                        if (kAllLanes || li + x * LPR < VPR)
                                            cp_async_16_hint(my_stage + (uint32_t)((st * GPW + gl) * ROWB + (li + x * LPR) * 16), src + (li + x * LPR) * 16, once);
                                }
                            }
                            cp_async_wait_all();
#pragma unroll
                            for (int st = 0; st < STEPS; ++st) {
                                const int e = base + st * GPW + gl;
                                if (e < n) {
                                    const float pe = kPacked ? Elem<T>::from_bits(my_list[e] >> 16) : __uint_as_float(my_list[2 * e + 1]);
                                    const float2 p2 = make_float2(pe, pe);
#pragma unroll
                                    for (int x = 0; x < VPL; ++x)
                                        if (kAllLanes || li + x * LPR < VPR) {
                                            float2 v2[E2];
                                            Elem<T>::unpack2(*reinterpret_cast<const uint4*>(my_stage_p + (st * GPW + gl) * ROWB + (li + x * LPR) * 16), v2);
#pragma unroll
                                            for (int e2 = 0; e2 < E2; ++e2) acc2[x][e2] = __ffma2_rn(p2, v2[e2], acc2[x][e2]);
                                        }
                                }
                            }
                        }
                    }
                    // lane groups of the warp added in index order (butterfly over the group bits), then the
                    // stream's vector to shared memory
#pragma unroll
                    for (int off = LPR; off < 32; off <<= 1)
#pragma unroll
                        for (int x = 0; x < VPL; ++x)
#pragma unroll
                            for (int e = 0; e < E2; ++e) {
                                acc2[x][e].x += __shfl_xor_sync(0xffffffffu, acc2[x][e].x, off);
                                acc2[x][e].y += __shfl_xor_sync(0xffffffffu, acc2[x][e].y, off);
                            }
                    float* mine = gred + ((size_t)gslot * kPsStreams + strm) * DH;
                    if (gl == 0 && strm < active) {
#pragma unroll
                        for (int x = 0; x < VPL; ++x) {
                            const int vec = li + x * LPR;
                            if (vec < VPR) {
#pragma unroll
                                for (int e = 0; e < E2; ++e) {
                                    mine[vec * EPV + 2 * e] = acc2[x][e].x;
                                    mine[vec * EPV + 2 * e + 1] = acc2[x][e].y;
                                }
                            }
                        }
                    }
                    __threadfence_block();
                    __syncwarp();
                    int last = 0;
                    if (lane == 0) last = atomicAdd(finished + gslot, took) + took == ticket_end;
                    last = __shfl_sync(0xffffffffu, last, 0);
                    if (last) {
                        // the job's last stream: add the streams' vectors in order, then the new token, which is
                        // never pruned (attention.cu:1227-1256): append v, add P_t * v
                        __threadfence_block();
                        const float pt = prob_of(__ldcg(sc_row + sr.row));
                        const size_t row_off = cache_row_offset(P, bh, sr.row, ROWB);
                        const T* vnew = static_cast<const T*>(P.v) + (size_t)bh * DH;
                        T* vdst = reinterpret_cast<T*>(static_cast<unsigned char*>(P.v_cache) + row_off);
                        T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
                        for (int d = lane; d < DH; d += 32) {
                            float A = 0.f;
#pragma unroll
                            for (int w = 0; w < kPsStreams; ++w)
                                if (w < active) A += gred[((size_t)gslot * kPsStreams + w) * DH + d];
                            const T vd = vnew[d];
                            vdst[d] = vd;
                            Elem<T>::store(outp + d, fmaf(pt, Elem<T>::to_float(vd), A));
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_jempty + 8 * gslot);   // the slot and its vectors are free again
                    }
                }
            }
            if (helper) break;
            if (++gslot == kPsJobs) gslot = 0, ++guse;
        }
    }
    if (tid == 32) post_job(-1, 0.f, 0.f);   // no more jobs from this CTA
    __syncthreads();
    if (tid == 0 && flags[0]) atomicOr(P.status, kStatusWaitTimeout);
}

}  // namespace ffa_dev
