// Pruning and torch-rounding steps whose slices' scores fit in shared memory: the fused cluster kernel.
#pragma once
#include "ffa_device_common.cuh"

namespace ffa_dev {

// ------------------------------------------------------------------------------------------
// Fused pruning step: one thread-block cluster per (batch, head), scores never leave the SMs
// ------------------------------------------------------------------------------------------
// The pruning rule needs the global max and sum of a (batch, head) before any V row may be
// touched (attention.cu:1184-1191), so the score pass and the value pass cannot be one
// streaming sweep.  Here both live in one kernel: a cluster of C CTAs owns a (batch, head);
// CTA r scores its slice of rows from a K-only bulk-copy ring into its OWN shared memory,
// stores its (max, sum) into every peer's shared memory ahead of a cluster barrier, prunes and
// gathers the V rows of its slice, and stores its partial output into CTA 0's shared memory ahead
// of a second cluster barrier; CTA 0 adds the C partial outputs.  Nothing is loaded remotely.
// No score scratch in HBM, no second launch, no arrival counters.  Where the rule prunes little
// (45 % or more of a slice's first round survive) or nothing (the torch-rounding mode keeps every
// row) the value phase is a second stream instead of a gather: the slice's V tiles follow its K
// tiles through the ring and the rule decides row by row.  Used whenever the slices' scores fit in
// shared memory, except for large pruned steps, which the streaming pruning kernel takes.
//
// Shared memory: [stages][K tile] ring | scores[chunk_rows] | kept list (row indices)
// | ballot words | group reduction area [NG][DH + 4] | partial outputs [C][DH] | (max, sum) [8] | barriers | flags.
constexpr int kFusedThreads = 160;   // 1 copy warp + 4 compute warps
constexpr int kFusedListCap = 1024;  // rows pruned and gathered per round: 32 ballot words, one per lane of the prefix scan

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
    unsigned* words = reinterpret_cast<unsigned*>(list_idx + kFusedListCap);   // one ballot per 32 rows of a round
    float* red = reinterpret_cast<float*>(words + kFusedListCap / 32);
    float* accs = red + NG * RS;                   // [C][DH]: in CTA 0, the partial outputs of all slices
    float* stat = accs + (size_t)C * DH;           // [8][2]: (max, sum) of every slice of the pair
    uint64_t* bars = reinterpret_cast<uint64_t*>(stat + 2 * kMaxClusterCtas);
    volatile int* flags = reinterpret_cast<volatile int*>(bars + 2 * S);  // [0] dead
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + S), ring = smem_u32(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    cluster_arrive();   // "this CTA runs": its peers wait for that before they store into its shared memory
    pdl_release();
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, NCW);
        }
        flags[0] = 0, flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();   // nothing above touches global memory (the per-sample lengths below are)
    const uint32_t rank = cluster_rank();
    const int bh = blockIdx.x / C;
    const SampleRange sr = sample_range(P, bh / P.H);
    const int c0 = (int)rank * chunk;                                   // first absolute row of this slice
    const int lo = sr.ok ? max(c0, sr.first) : 0;
    const int hi = sr.ok ? min(c0 + chunk, sr.row) : 0;                 // cached rows [lo, hi)
    const bool owns_new = sr.ok && sr.row >= c0 && sr.row < c0 + chunk; // the new token's row is in this slice
    const int nrows = max(hi - lo, 0), ntiles = (nrows + R - 1) / R;
    const bool prune = P.p > 0.f;


    const int ctid = tid - 32, g = ctid / LPR, li = ctid % LPR;   // meaningful for compute warps only
    float2 q2[VPL][E2];
    float qf[VPL][EPV];
    float m = -CUDART_INF_F, l = 0.f;

    auto score_of = [&](float dot) -> float {
        if (P.round_like_torch) return Elem<T>::round(Elem<T>::round(dot) * P.scale);
        return dot * P.scale;
    };

    // The copy thread's ring position and the compute warps' (each side walks the same sequence of tiles: the K
    // tiles of the slice, then -- when every row is kept -- its V tiles).
    uint32_t pstage = 0, puse = 0;     // thread 0
    uint32_t cstage = 0, cphase = 0;   // compute warps
    // Issues tile j of the slice from `cache` (thread 0).  Rows of one page are contiguous; a tile that crosses a
    // page boundary arrives as one copy per page, all counted on the same barrier (contiguous caches: one copy).
    auto issue_tile = [&](const unsigned char* cache, int j) -> bool {
        if (puse > 0 && !mbar_wait_bounded(bar_empty + 8 * pstage, (puse - 1) & 1, flags)) return false;
        const int run_rows = P.page_table != nullptr ? P.page_rows : P.Lmax;
        const int n = min(R, nrows - j * R);
        mbar_expect_tx(bar_full + 8 * pstage, (uint32_t)n * ROWB);
        for (int done = 0; done < n;) {
            const int row = lo + j * R + done;
            const int seg = min(n - done, run_rows - row % run_rows);
            bulk_copy_g2s(ring + pstage * tile_bytes + (uint32_t)done * ROWB, cache + cache_row_offset(P, bh, row, ROWB),
                          (uint32_t)seg * ROWB, bar_full + 8 * pstage);
            done += seg;
        }
        if (++pstage == (uint32_t)S) pstage = 0, ++puse;
        return true;
    };
    // Every row kept (the torch-rounding mode): the value phase streams the slice's V tiles through the same ring
    // instead of gathering rows.  The first `dense_ahead` of them are requested as soon as the K tiles release
    // their buffers, so they travel while the statistics are exchanged.
    const bool dense = !prune;
    const int dense_ahead = dense ? min(S, ntiles) : 0;

    // ---------------- phase 1: scores of this slice into shared memory ----------------
    if (warp == 0) {
        if (tid == 0) {
            bool ok = true;
            for (int j = 0; ok && j < ntiles; ++j) ok = issue_tile(static_cast<const unsigned char*>(P.k_cache), j);
            for (int j = 0; ok && j < dense_ahead; ++j) ok = issue_tile(static_cast<const unsigned char*>(P.v_cache), j);
        }
    } else {
        // the new token's k is needed after the score loop and its v after the gather: ask for their lines now
        if (owns_new && g == 0 && li * 128 < ROWB) {
            prefetch_l1(static_cast<const unsigned char*>(P.k) + (size_t)bh * ROWB + li * 128);
            prefetch_l1(static_cast<const unsigned char*>(P.v) + (size_t)bh * ROWB + li * 128);
        }
        load_row_f32<T, DH>(static_cast<const unsigned char*>(P.q) + (size_t)bh * ROWB, li, qf);
#pragma unroll
        for (int x = 0; x < VPL; ++x)
#pragma unroll
            for (int e = 1; e < EPV; e += 2) q2[x][e >> 1] = make_float2(qf[x][e - 1], qf[x][e]);

        for (int j = 0; j < ntiles; ++j) {
            const int n = min(R, nrows - j * R);
            const bool ready = mbar_wait_bounded(bar_full + 8 * cstage, cphase, flags);
            const unsigned char* ks = smem + (size_t)cstage * tile_bytes;
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
            if (lane == 0) mbar_arrive(bar_empty + 8 * cstage);
            if (++cstage == (uint32_t)S) cstage = 0, cphase ^= 1;
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
                const size_t row_off = cache_row_offset(P, bh, sr.row, ROWB);
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
    {
        // (max, sum) of this slice: every warp combines the NG groups with shuffles; warp 0 publishes them
        float Mc = -CUDART_INF_F;
        for (int gg = lane; gg < NG; gg += 32) Mc = fmaxf(Mc, red[gg * RS]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) Mc = fmaxf(Mc, __shfl_xor_sync(0xffffffffu, Mc, off));
        if (warp == 0) {
            float Lc = 0.f;
            for (int gg = lane; gg < NG; gg += 32)
                if (red[gg * RS] != -CUDART_INF_F) Lc += red[gg * RS + 1] * __expf(red[gg * RS] - Mc);
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) Lc += __shfl_xor_sync(0xffffffffu, Lc, off);
            // every CTA of the cluster receives every slice's pair: pushed, so nobody loads remotely after the barrier
            cluster_wait();
            if (lane < C) {
                st_peer_smem_f32(stat + 2 * rank, lane, Mc);
                st_peer_smem_f32(stat + 2 * rank + 1, lane, Lc);
            }
        } else {
            cluster_wait();
        }
        // While the cluster exchanges its statistics, start moving the V rows that can still survive towards L2:
        // a row survives only if its score is within ln(p) of the pair's max (attention.cu:1185), and the pair's max
        // is at least this slice's.  A hint only -- the rule below decides; at most two rows per thread.
        if (prune && Mc != -CUDART_INF_F) {
            const float thr = Mc + __logf(P.p) - 0.25f;
            int sent = 0;
            for (int i = lo + tid; i < hi && sent < 2; i += kFusedThreads)
                if (sc[i - c0] > thr) {
                    const unsigned char* vrow = static_cast<const unsigned char*>(P.v_cache) + cache_row_offset(P, bh, i, ROWB);
#pragma unroll
                    for (int b = 0; b < ROWB; b += 128) prefetch_l2(vrow + b);
                    ++sent;
                }
        }
    }
    cluster_sync_all();   // every slice's (max, sum) is visible cluster-wide; also a CTA barrier

    // ---------------- global statistics of the (batch, head) ----------------
    float M = -CUDART_INF_F, Lsum = 0.f;
    for (int c = 0; c < C; ++c) M = fmaxf(M, stat[2 * c]);
    for (int c = 0; c < C; ++c) {
        const float mc = stat[2 * c];
        if (mc != -CUDART_INF_F) Lsum += stat[2 * c + 1] * __expf(mc - M);
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
    const unsigned char* vc = static_cast<const unsigned char*>(P.v_cache);
    const int hi_mask = sr.ok ? min(c0 + chunk, sr.row + 1) : c0;   // rows whose mask bit this slice writes
    bool stream_v = dense;   // value phase by streaming the slice's V tiles (else: gather the survivors' rows)
    for (int sub = c0; !dense && sub < hi_mask; sub += kFusedListCap) {
        // Survivors are listed in row order (ballots first, then a prefix over the 32-row
        // words), so the order of the floating-point sums below never depends on timing.
        __syncthreads();
        const int sub_hi = min(sub + kFusedListCap, hi_mask);
        constexpr int kWords = kFusedListCap / 32;      // 32: one ballot word per lane of the scan below
#pragma unroll 1
        for (int w = warp; w < kWords; w += kFusedThreads / 32) {
            const int base = sub + w * 32;
            unsigned bal = 0u;
            if (base < sub_hi) {             // warp-uniform
                const int i = base + lane;
                bool keep = false;
                if (i >= lo && i < hi) keep = prune ? !Elem<T>::leq(prob_of(sc[i - c0]), theta) : true;
                bal = __ballot_sync(0xffffffffu, keep);
                if (P.kept_mask != nullptr && lane == 0)
                    P.kept_mask[(size_t)bh * P.mask_words + (base >> 5)] =
                        bal | ((sr.row >= base && sr.row < base + 32) ? (1u << (sr.row - base)) : 0u);
            }
            if (lane == 0) words[w] = bal;
        }
        __syncthreads();
        // every warp scans the 32 word counts itself: exclusive prefix = list position of a word's first survivor
        const int cnt = __popc(words[lane]);
        int incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += up;
        }
        const int n = __shfl_sync(0xffffffffu, incl, 31);
        // Few rows pruned (45 % or more of the first round survive): fetching survivors row by row would cost more
        // than the rows saved, so the slice's V tiles are streamed instead and the rule decides row by row there
        // (bf16 x 128, 1024 pairs, 2 K tokens, 52 % kept: 166 us streamed, 181 us gathered; 8 K tokens, 38 % kept:
        // 625 us streamed, 567 us gathered).
        if (sub == c0 && 20 * n >= 9 * (min(sub_hi, hi) - max(sub, lo)) && n > 0) {
            stream_v = true;
            break;
        }
#pragma unroll 1
        for (int w = warp; w < kWords; w += kFusedThreads / 32) {
            const unsigned bal = words[w];
            const int first = __shfl_sync(0xffffffffu, incl - cnt, w);
            if ((bal >> lane) & 1u) list_idx[first + __popc(bal & ((1u << lane) - 1u))] = sub + w * 32 + lane;
        }
        __syncthreads();
        if (warp > 0) {
            for (int base = 0; base < n; base += RB * NG) {
                uint4 raw[RB][VPL];
                float pr[RB];
                // lane uu of a group looks up row uu of the group's batch and its probability (one exponential per
                // row, not one per lane); shuffles hand both to the whole group
                int row_mine = c0;
                float pr_mine = 0.f;
                if (li < RB && base + li * NG + g < n) {
                    row_mine = list_idx[base + li * NG + g];
                    pr_mine = prob_of(sc[row_mine - c0]);
                }
#pragma unroll
                for (int uu = 0; uu < RB; ++uu) {
                    const int idx = base + uu * NG + g;
                    const bool okr = idx < n;
                    const int row = __shfl_sync(0xffffffffu, row_mine, (lane - li) + uu);
                    pr[uu] = __shfl_sync(0xffffffffu, pr_mine, (lane - li) + uu);
                    const size_t roff = okr ? cache_row_offset(P, bh, row, ROWB) : 0;
#pragma unroll
                    for (int x = 0; x < VPL; ++x) {
                        raw[uu][x] = make_uint4(0, 0, 0, 0);
                        if (okr && (kAllLanes || li + x * LPR < VPR))
                            raw[uu][x] = __ldg(reinterpret_cast<const uint4*>(vc + roff + (li + x * LPR) * 16));
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
    if (stream_v) {
        // The value phase as a stream: thread 0 sends the slice's V tiles through the ring (in the torch-rounding mode
        // the first `dense_ahead` are on their way already), the compute warps weight each row with its rounded
        // probability; a row the rule prunes gets weight 0 and is skipped, never multiplied.
        if (warp == 0) {
            if (tid == 0) {
                bool ok = true;
                for (int j = dense_ahead; ok && j < ntiles; ++j) ok = issue_tile(vc, j);
            }
            if (dense && P.kept_mask != nullptr)   // every cached row of the slice and the new token
                for (int base = c0 + 32 * lane; base < hi_mask; base += 32 * 32) {
                    unsigned bits = 0u;
                    for (int i = max(base, lo); i < min(base + 32, hi); ++i) bits |= 1u << (i - base);
                    if (sr.row >= base && sr.row < base + 32) bits |= 1u << (sr.row - base);
                    P.kept_mask[(size_t)bh * P.mask_words + (base >> 5)] = bits;
                }
        } else {
            if (!dense && P.kept_mask != nullptr)   // the rule's verdict on every row of the slice, 32 rows per vote
                for (int base = c0 + 32 * (warp - 1); base < hi_mask; base += 32 * NCW) {
                    const int i = base + lane;
                    const bool keep = i >= lo && i < hi && !Elem<T>::leq(prob_of(sc[i - c0]), theta);
                    const unsigned bal = __ballot_sync(0xffffffffu, keep);
                    if (lane == 0)
                        P.kept_mask[(size_t)bh * P.mask_words + (base >> 5)] =
                            bal | ((sr.row >= base && sr.row < base + 32) ? (1u << (sr.row - base)) : 0u);
                }
            for (int j = 0; j < ntiles; ++j) {
                const int n = min(R, nrows - j * R);
                const bool ready = mbar_wait_bounded(bar_full + 8 * cstage, cphase, flags);
                const unsigned char* vs = smem + (size_t)cstage * tile_bytes;
                const float* sc_tile = sc + (lo - c0) + j * R;
                if (ready) {
                    for (int base = 0; base < n; base += RB * NG) {
                        // lane uu of a group computes the weight of row uu of the group's batch; shuffles share it
                        const int r_mine = base + li * NG + g;
                        float pr_mine = 0.f;
                        if (li < RB && r_mine < n) {
                            pr_mine = prob_of(sc_tile[r_mine]);
                            if (prune && Elem<T>::leq(pr_mine, theta)) pr_mine = 0.f;
                        }
                        uint4 raw[RB][VPL];
                        float pr[RB];
#pragma unroll
                        for (int uu = 0; uu < RB; ++uu) {
                            const int r = min(base + uu * NG + g, n - 1);   // rows past the tile carry weight 0
                            pr[uu] = __shfl_sync(0xffffffffu, pr_mine, (lane - li) + uu);
#pragma unroll
                            for (int x = 0; x < VPL; ++x)
                                if (kAllLanes || li + x * LPR < VPR)
                                    raw[uu][x] = *reinterpret_cast<const uint4*>(vs + (size_t)r * ROWB + (li + x * LPR) * 16);
                        }
#pragma unroll
                        for (int uu = 0; uu < RB; ++uu) {
                            if (pr[uu] > 0.f) {
                                const float2 p2 = make_float2(pr[uu], pr[uu]);
#pragma unroll
                                for (int x = 0; x < VPL; ++x)
                                    if (kAllLanes || li + x * LPR < VPR) {
                                        float2 v2[E2];
                                        Elem<T>::unpack2(raw[uu][x], v2);
#pragma unroll
                                        for (int e = 0; e < E2; ++e) acc2[x][e] = __ffma2_rn(p2, v2[e], acc2[x][e]);
                                    }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * cstage);
                if (++cstage == (uint32_t)S) cstage = 0, cphase ^= 1;
            }
        }
    }
    // the new token is never pruned (attention.cu:1227-1256): append v, add P_t * v
    if (warp > 0) {
        if (owns_new && g == 0) {
            const float pt = prob_of(sc[sr.row - c0]);
            const size_t row_off = cache_row_offset(P, bh, sr.row, ROWB);
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
        st_peer_smem_f32(accs + (size_t)rank * DH + d, 0, A);   // into CTA 0's shared memory
    }
    cluster_sync_all();   // every slice's partial output has arrived in CTA 0
    if (rank == 0) {
        T* outp = static_cast<T*>(P.out) + (size_t)bh * DH;
        for (int d = tid; d < DH; d += kFusedThreads) {
            float A = 0.f;
            for (int c = 0; c < C; ++c) A += accs[(size_t)c * DH + d];   // slice order: deterministic
            Elem<T>::store(outp + d, sr.ok ? A : 0.f);
        }
    }
    if (tid == 0) {
        if (flags[0]) atomicOr(P.status, kStatusWaitTimeout);
        if (!sr.ok && rank == 0) atomicOr(P.status, kStatusBadLength);
    }
}

}  // namespace ffa_dev
