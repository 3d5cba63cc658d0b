// Host side of the C ABI declared in include/ffa_c_api.h: argument validation, the launch
// planner, workspace carving and the per-step parameter fill.
//
// Replaces the reference's host launch layer: call_attention / call_attention_headdim
// (attention.cu:1454-1554), the template launch switches (attention.cu:1301-1442),
// invokeTranspose4dBatchMajor (attention.cu:1611-1689) and get_launch_params
// (kernel_launch_utils.h:135-180).
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/ffa_c_api.h"
#include "ffa_internal.h"

namespace {

thread_local char g_err[512] = "";
std::atomic<unsigned long long> g_launches{0};

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
int cuda_fail(int e, const char* what)
{
    return fail(FFA_ERR_CUDA, "%s: %s", what, cudaGetErrorString((cudaError_t)e));
}

int elem_size(int dtype) { return dtype == FFA_DTYPE_F32 ? 4 : 2; }
bool dtype_ok(int dtype) { return dtype == FFA_DTYPE_F32 || dtype == FFA_DTYPE_F16 || dtype == FFA_DTYPE_BF16; }
bool head_dim_ok(int d) { return d == 64 || d == 80 || d == 128 || d == 256; }
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
int score_stride(int max_len) { return (max_len + 31) / 32 * 32; }   // a pair's scores are whole 128-byte lines (32 rows each)
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kMaxCtasPerSm = 8;
constexpr int kMaxClusterCtas = 8;   // portable thread-block cluster size
constexpr int kMaxClustersPerPair = 12;
constexpr int kSmemReservePerCta = 1024;  // the driver keeps 1 KB per resident CTA
// below this many tiles per CTA slot the work list is cut on (batch, head) boundaries (measured:
// bf16 x 128, batch 32 x 32 heads: 2 K tokens 154.9 vs 159.3 us, 1 K 81.8 vs 88.3 us, 512 45.6 vs
// 48.9 us in favour of the aligned cut; 8 K tokens 603 vs 594 us against it)
constexpr long long kAlignedBelowUnitsPerSlot = 200;
// pruned steps that stream at least this many bytes of K take the streaming kernel when the score scratch is bound
// (5 % of the V rows kept; streaming vs cluster kernel: fp16 x 64, 320 pairs, 1256 tokens = 51 MB: 27.2 vs 17.5 us;
// 134 MB, three shapes: 42.5-45.2 vs 31.2-37.6 us; 268 MB, five shapes: 52.3-67.3 vs 53.3-63.5 us; bf16 x 128, 1024
// pairs: 2 K tokens = 537 MB 105.3 vs 106.4 us, 4 K 193 vs 212 us, 8 K 342 vs 408 us, 32 K 1393 vs 1713 us).
// The streaming kernel fetches survivors row by row and is slow when the threshold prunes little (nothing pruned: 2 K
// tokens 234 vs 167 us, 8 K 920 vs 667 us -- the cluster kernel streams the V tiles of such slices), so it is the
// default only where it can win by 9 % or more.
constexpr double kStreamPruneAboveBytes = 1e9;

}  // namespace

struct ffa_plan {
    int dtype, B, H, Dh, Lmax, use_default, device, mode;
    int prune_path;  // 0 = choose, 1 = fused cluster kernel only, 2 = streaming kernel only
    int cluster_merge;  // 1 = merge split pairs inside a thread-block cluster when the cut allows it
    // answers of the occupancy query for cluster launches, keyed by (threads, shared memory, cluster size)
    struct { int threads, smem, cluster, clusters; } occ[8];
    int occ_n;
    bool offline;    // planning only: created from given device properties, never launches
    int sms, smem_per_cta, smem_per_sm;
    bool forced;
    ffa_launch_t force;
    // workspace carving
    void* ws;
    size_t ws_bytes;
    int* status;
    int* tickets;
    float* partials;
    float* scores;
    int max_grid;
    // output gather over peer memory
    int peer_world, peer_rank;
    void* peer_buf[FFA_MAX_PEERS];
    void* push_gathered;   // non-null: exact steps push their output rows to the peers (ffa_peer_push_target)
};

namespace {

struct Carve {
    size_t status, tickets, partials, scores, total;
};
Carve carve(const ffa_plan* p, bool with_scores)
{
    const size_t BH = (size_t)p->B * p->H;
    Carve c;
    size_t off = 0;
    c.status = off, off += 256;
    c.tickets = off, off += align_up(BH * sizeof(int), 256);
    c.partials = off, off += align_up(((size_t)p->max_grid + BH) * (p->Dh + 2) * sizeof(float), 256);
    c.scores = off;
    if (with_scores) off += align_up(BH * (size_t)score_stride(p->Lmax) * sizeof(float), 256);
    c.total = off;
    return c;
}

// ---- planner -------------------------------------------------------------------------------
// The streaming kernels take (tile_rows, stages, consumer_warps, ctas_per_sm).  The flat unit
// list is cut evenly over the grid, so the shape questions are: enough bytes in flight per SM
// to cover HBM latency (ring depth x tile size x resident CTAs) but not many more (sweeps on
// B200 lose 4-7 % of bandwidth with a third stage: more concurrent streams, worse DRAM page
// locality), compute warps enough to keep up with the ring, tiles small enough that every CTA
// gets several units when batch*heads*t is small, and the shared-memory budget.
struct Shape {
    int tile_rows, stages, warps, cps;
};

// Fixed analytic rule: 16 KB tiles per tensor (4 rows per lane group and batch at 8 compute
// warps... 8 at 4 warps), a 2-deep ring, 4 compute warps, 2 CTAs per SM.
Shape default_shape(const ffa_plan* p, int row_bytes, long long rows_total, int tensors)
{
    (void)p, (void)rows_total;
    Shape s;
    s.warps = 4;
    s.cps = 2;
    s.stages = 2;
    s.tile_rows = 16384 / row_bytes;
    // head_dim 80 (160- and 320-byte rows): a batch of the row loop is 128 / 64 rows there
    if ((row_bytes / 16) % 5 == 0) s.tile_rows = 20480 / row_bytes;
    if (tensors == 1) {
        // the streaming pruning kernel: K tiles only carry half the bytes per row-loop iteration: twice the compute
        // warps keep up with the ring, and tiles twice as large keep as many bytes in flight with the same two
        // stages -- two row batches per warp and barrier round trip instead of one (bf16 x 128, 1024 pairs, 8 K /
        // 32 K tokens: 362 / 1432 us against 378 / 1479 us for four stages of 16 KB)
        s.warps = 8, s.tile_rows *= 2;
    }
    return s;
}

// Refinements measured on B200 with launch-shape sweeps through ffa_plan_set_launch (CUDA-graph
// timing, replicas rotating so that every launch streams from HBM), keyed by row bytes and by
// the bytes one decode step streams:
//   < 48 MB  (OPT-1.3B fp32 batch 1, 16 MB: 12.9 us vs 17.3 us)  one CTA per SM when there are few
//            (batch, head) pairs: fewer split partials and arrival counters to merge than bytes
//            to stream; more CTAs only to keep it at <= 2 pairs per CTA
//   48-600 MB, 256-byte rows (bf16 x 128, 270 MB: 5.43 vs 5.14 TB/s)  8 KB tiles, 4 CTAs per SM:
//            the ring fills sooner and the tail is shorter
//   48-600 MB, >= 512-byte rows (GPT-J fp16 x 256, 269 MB: 5.53 vs 5.36 TB/s)  8 compute warps
//   otherwise the rule above (bf16 x 128: 7.35 TB/s at 32 K tokens, 7.22 at 8 K, 6.67 at 2 K;
//            fp16 x 64, 103 MB: 4.20 TB/s)
Shape measured_shape(const ffa_plan* p, int row_bytes, long long rows_total, int tensors)
{
    Shape s = default_shape(p, row_bytes, rows_total, tensors);
    if (tensors == 1) return s;   // the refinements below were measured on the exact kernel (K and V tiles)
    const double bytes = (double)rows_total * row_bytes * tensors;
    const long long BH = (long long)p->B * p->H;
    if (bytes < 48e6) {
        // every (batch, head) a CTA walks costs a serial latency chain (merge, store); with many
        // pairs and short sequences let resident CTAs overlap those chains: <= 2 pairs per CTA
        const long long want = (BH + 2LL * p->sms - 1) / (2LL * p->sms);
        s.cps = (int)(want < 1 ? 1 : want > 4 ? 4 : want);
        // a second CTA per SM where that is what lets a pair spread over one whole cluster of 8 (OPT-1.3B fp32 batch 1,
        // 32 pairs on 148 SMs: 8 CTAs per pair 8.85 us, 4 per pair 9.2 us)
        if (s.cps < 2 && 2LL * p->sms / BH >= 8 && 2LL * p->sms / BH < 16 && p->sms / BH < 8) s.cps = 2;
        if (tensors == 2) s.stages = 3;   // OPT-1.3B fp32 batch 1: 10.7 us vs 11.3 us
    } else if (bytes < 600e6) {
        if (row_bytes >= 512 && BH <= p->sms) {
            // GPT-J fp16 x 256, batch 8 (128 pairs, 269 MB): one CTA per pair and per SM with a deep
            // ring of 32 KB tiles, no split to merge: 42.9 us vs 47.5 us for two CTAs per pair
            s.cps = 1, s.warps = 8, s.stages = tensors == 2 ? 3 : 4, s.tile_rows = 32768 / row_bytes;
        } else if (row_bytes >= 512) {
            s.warps = 8;
        } else if (row_bytes == 256) {
            s.tile_rows /= 2, s.cps = 4;
        }
    }
    return s;
}

int fit_launch(const ffa_plan* p, int cap_rows, int tensors, ffa_launch_t* out, bool pow2_tiles = false, int max_parts = 0)
{
    const int rowb = p->Dh * elem_size(p->dtype);
    const long long BH = (long long)p->B * p->H;
    Shape s = p->use_default ? default_shape(p, rowb, BH * cap_rows, tensors)
                             : measured_shape(p, rowb, BH * cap_rows, tensors);
    if (p->forced) {
        if (p->force.tile_rows > 0) s.tile_rows = p->force.tile_rows;
        if (p->force.stages > 0) s.stages = p->force.stages;
        if (p->force.consumer_warps > 0) s.warps = p->force.consumer_warps;
        if (p->force.ctas_per_sm > 0) s.cps = p->force.ctas_per_sm;
    }
    if (s.warps < 1) s.warps = 1;
    if (s.warps > 8) s.warps = 8;   // the kernels are compiled for at most 1 + 8 warps
    if (tensors == 1 && p->Dh == 80 && s.warps > 4) s.warps = 4;   // streaming pruning kernel, five vectors per lane: register budget
    if (tensors == 1 && s.cps > 2) s.cps = 2;   // its 13 warps of 72 registers leave room for two CTAs per SM
    if (s.cps < 1) s.cps = 1;
    if (s.cps > kMaxCtasPerSm) s.cps = kMaxCtasPerSm;
    if (s.stages < 2) s.stages = 2;
    if (s.stages > 16) s.stages = 16;
    if (s.tile_rows < 8) s.tile_rows = 8;
    s.tile_rows = (s.tile_rows + 7) / 8 * 8;  // keeps every tile a multiple of 128 bytes
    const bool tile_forced = p->forced && p->force.tile_rows > 0;
    const bool grid_forced = p->forced && p->force.grid > 0;
    // fewer (batch, head) pairs than CTA slots: each pair will be cut into C aligned parts (below);
    // size the tiles so that a part is about four of them (enough for the 2-stage ring to overlap)
    const long long slots0 = (long long)p->sms * s.cps;
    const bool few_pairs = !grid_forced && BH <= slots0 && BH * (cap_rows / s.tile_rows + 1) < kAlignedBelowUnitsPerSlot * slots0;
    if (!tile_forced) {
        if (few_pairs) {
            const long long c = slots0 / BH;
            long long rows = (cap_rows / c / 4 + 7) / 8 * 8;
            if (rows < 8) rows = 8;
            if (rows < s.tile_rows) s.tile_rows = (int)rows;
        } else {
            // small problems: shrink tiles until every CTA slot has a few units to stream
            while (s.tile_rows > 8 && BH * (cap_rows / s.tile_rows + 1) < 4 * slots0) s.tile_rows = (s.tile_rows / 2 + 7) / 8 * 8;
        }
    }
    if (pow2_tiles) {   // paged caches: tiles must divide the page
        int t2 = 8;
        while (t2 * 2 <= s.tile_rows) t2 *= 2;
        s.tile_rows = t2;
    }
    // shared-memory budget: per CTA and per SM
    for (;;) {
        const int smem = ffa_k_smem_bytes(p->dtype, p->Dh, s.tile_rows, s.stages, s.warps, tensors);
        const bool ok = smem <= p->smem_per_cta && (long long)s.cps * (smem + kSmemReservePerCta) <= p->smem_per_sm;
        if (ok) {
            out->smem_bytes = smem;
            break;
        }
        if (s.stages > 2) --s.stages;
        else if (s.tile_rows > 8) s.tile_rows = (s.tile_rows / 2 + 7) / 8 * 8;
        else if (s.cps > 1) --s.cps;
        else return fail(FFA_ERR_ARG, "no launch shape fits in shared memory");
    }
    // How the work list is cut (see Partition in the kernels).  Large problems: an even cut of the
    // unit list.  Small ones (fewer than 200 units per CTA slot): CTA boundaries on (batch, head)
    // boundaries -- C CTAs per pair when there are fewer pairs than slots, one CTA per pair when
    // a third or fourth resident CTA per SM makes room for all pairs -- because there the serial
    // per-segment latency and the merge of split pairs cost more than imbalance does
    // (OPT-1.3B batch 1: 10.5 us vs 13.1 us; fp16 batch 10: 21.2 us vs 23.1 us).
    const int upb = cap_rows / s.tile_rows + 1;
    const long long units = BH * upb;
    long long grid = (long long)p->sms * s.cps;
    int parts = upb;
    if (!grid_forced && units < kAlignedBelowUnitsPerSlot * grid) {
        if (BH <= grid) {
            long long c = grid / BH;
            // up to 8 CTAs per pair merge inside a thread-block cluster (no partials in global memory);
            // more than 8 run as whole clusters of 8, whose leaders merge through global memory
            if (c > upb) c = upb;
            if (max_parts > 0 && c > max_parts) c = max_parts;
            if (p->cluster_merge && tensors == 2 && c > kMaxClusterCtas) {
                c = c / kMaxClusterCtas * kMaxClusterCtas;
                // the leaders' merge is serial in the number of clusters (bf16 x 128, 4 pairs at 32 K
                // tokens: 13 clusters per pair 20.2 us, 18 clusters 27.9 us)
                if (c > kMaxClustersPerPair * kMaxClusterCtas) c = kMaxClustersPerPair * kMaxClusterCtas;
            }
            parts = (int)c, grid = BH * c;
        } else {
            const int need = (int)((BH + p->sms - 1) / p->sms);
            const int smem = out->smem_bytes;
            if (need <= 4 && (long long)need * (smem + kSmemReservePerCta) <= p->smem_per_sm && !(p->forced && p->force.ctas_per_sm > 0)) {
                s.cps = need, parts = 1, grid = BH;
            } else {
                // more pairs than slots: k whole pairs per persistent CTA, nothing straddles; its copy warp streams across
                // pair boundaries without a bubble.  (One CTA per pair with more CTAs than slots, handed out by the
                // hardware as slots free up, balances better but pays a CTA's start-up per pair: 1024 pairs of 256 KB
                // 48.0 vs 43.5 us, of 1 MB 161.7 vs 161.0 us.)
                const long long k = (BH + grid - 1) / grid;
                parts = 1, grid = (BH + k - 1) / k;
            }
        }
    }
    if (grid > units) grid = units;
    if (grid_forced && p->force.grid < grid) grid = p->force.grid;
    if (grid > p->max_grid) grid = p->max_grid;
    out->parts_per_bh = parts;
    out->tile_rows = s.tile_rows;
    out->stages = s.stages;
    out->consumer_warps = s.warps;
    out->ctas_per_sm = s.cps;
    out->grid = (int)grid;
    return FFA_OK;
}

// Fused pruning kernel: a cluster of C CTAs per (batch, head), C in {1, 2, 4, 8}; each CTA keeps
// the scores of its slice (chunk rows, a multiple of 32 so mask words never straddle slices) in
// shared memory.  The kernel is a score phase and a value phase separated by cluster barriers,
// and the grid is not persistent, so the time is (number of waves) x (one CTA's chain): C is
// the candidate with the smallest  ceil(B*H*C / resident CTAs) x (chunk + fixed cost), the
// fixed cost of a CTA (start, barriers, merge) taken as 512 rows' worth.  Slices stay >= 128
// rows.  False when 8 slices do not fit in shared memory (then the streaming kernel runs).
bool plan_fused(const ffa_plan* p, int cap_rows, FfaStepParams* P, int* smem_out)
{
    const int rowb = p->Dh * elem_size(p->dtype);
    const long long BH = (long long)p->B * p->H;
    int best_c = 0, best_chunk = 0, best_r = 0, best_smem = 0;
    long long best_cost = 0;
    for (int c = 1; c <= 8; c *= 2) {
        const int chunk = (int)(((long long)cap_rows + 1 + c - 1) / c + 31) / 32 * 32;
        if (c > 1 && chunk < 128) break;
        int r = (((rowb / 16) % 5 == 0 ? 20480 : 16384) / rowb) / 8 * 8;   // one 16 KB K tile (20 KB for head_dim 80)
        if (r < 8) r = 8;
        if (r > chunk) r = (chunk + 7) / 8 * 8;
        const int smem = ffa_k_fused_smem_bytes(p->dtype, p->Dh, r, 2, chunk, c);
        if (smem > p->smem_per_cta) continue;
        int resident = p->smem_per_sm / (smem + kSmemReservePerCta);
        if (resident > 7) resident = 7;  // 160 threads x 56 registers
        const long long slots = (long long)p->sms * resident;
        const long long waves = (BH * c + slots - 1) / slots;
        const long long cost = waves * (chunk + 512);
        if (best_c == 0 || cost < best_cost) best_c = c, best_chunk = chunk, best_r = r, best_smem = smem, best_cost = cost;
    }
    if (best_c == 0) return false;
    P->cluster = best_c, P->chunk_rows = best_chunk, P->tile_rows = best_r, P->stages = 2;
    P->grid = (int)(BH * best_c);
    *smem_out = best_smem;
    return true;
}

// Which two-pass kernel a step prefers: the streaming kernel when it is forced, or for pruned steps (p > 0) that stream at
// least kStreamPruneAboveBytes of K while the score scratch is bound; else the cluster kernel (if its slices fit).
bool prefers_stream(const ffa_plan* plan, int cap_rows, float p, bool have_scores)
{
    const double k_bytes = (double)plan->B * plan->H * cap_rows * plan->Dh * elem_size(plan->dtype);
    return plan->prune_path == 2 || (plan->prune_path == 0 && have_scores && p > 0.f && k_bytes >= kStreamPruneAboveBytes);
}

// cudaOccupancyMaxActiveClusters for the one-pass kernel, remembered per launch shape (the query
// costs tens of microseconds); 0 when the device will not say
int max_active_clusters(ffa_plan* p, int threads, int smem, int cluster)
{
    for (int i = 0; i < p->occ_n; ++i)
        if (p->occ[i].threads == threads && p->occ[i].smem == smem && p->occ[i].cluster == cluster) return p->occ[i].clusters;
    int n = 0;
    if (ffa_k_max_active_clusters(p->dtype, p->Dh, threads, smem, cluster, &n) != 0) {
        (void)cudaGetLastError();
        n = 0;
    }
    const int slot = p->occ_n < 8 ? p->occ_n++ : (threads + smem + cluster) % 8;
    p->occ[slot].threads = threads, p->occ[slot].smem = smem, p->occ[slot].cluster = cluster, p->occ[slot].clusters = n;
    return n;
}

// Decides how the parts of the one-pass launch L are grouped into thread-block clusters (0: not at
// all), and takes fewer parts per pair when the device cannot keep all clusters resident at once:
// clusters are placed inside one GPC each, so fewer of them fit than CTA slots / size suggest, and
// a grid that does not fit runs in two waves (bf16 x 128, 192 pairs at 2 K tokens: 3 CTAs per pair
// 48.0 us, 2 per pair 36.7 us).
int fit_clusters(ffa_plan* plan, int cap, bool paged, ffa_launch_t* L, int* cluster)
{
    const long long BH = (long long)plan->B * plan->H;
    for (int tries = 0; tries < 8; ++tries) {
        *cluster = 0;
        if (plan->cluster_merge && L->parts_per_bh >= 2 && (long long)L->grid == BH * L->parts_per_bh) {
            if (L->parts_per_bh <= kMaxClusterCtas) *cluster = L->parts_per_bh;
            else if (L->parts_per_bh % kMaxClusterCtas == 0) *cluster = kMaxClusterCtas;
        }
        if (*cluster == 0 || plan->forced || plan->offline) break;
        const int fit = max_active_clusters(plan, 32 * (L->consumer_warps + 1), L->smem_bytes, *cluster);
        if (fit <= 0 || (long long)L->grid / *cluster <= fit) break;
        const int fewer = L->parts_per_bh <= kMaxClusterCtas ? L->parts_per_bh - 1 : L->parts_per_bh - kMaxClusterCtas;
        const int r = fit_launch(plan, cap, 2, L, paged, fewer);
        if (r != FFA_OK) return r;
        *cluster = 0;   // describes the previous L; recomputed at the top of the next try
    }
    // out of tries right after a refit: the launch runs without clusters (parts merge through global memory)
    if (*cluster > 1 && (L->parts_per_bh % *cluster != 0 || (long long)L->grid != BH * L->parts_per_bh)) *cluster = 0;
    return FFA_OK;
}

}  // namespace

extern "C" {

const char* ffa_last_error(void) { return g_err; }
unsigned long long ffa_launch_count(void) { return g_launches.load(); }

int ffa_cache_bytes(int dtype, int batch, int heads, int max_len, int head_dim, size_t* k_bytes, size_t* v_bytes)
{
    if (!dtype_ok(dtype)) return fail(FFA_ERR_DTYPE, "unsupported dtype code %d", dtype);
    if (!head_dim_ok(head_dim)) return fail(FFA_ERR_HEAD_DIM, "unsupported head_dim %d (64, 80, 128, 256)", head_dim);
    if (batch <= 0 || heads <= 0 || max_len <= 0) return fail(FFA_ERR_RANGE, "batch, heads and max_len must be positive");
    if (k_bytes == nullptr || v_bytes == nullptr) return fail(FFA_ERR_ARG, "null output pointer");
    const size_t n = (size_t)batch * heads * max_len * head_dim * elem_size(dtype);
    *k_bytes = n, *v_bytes = n;
    return FFA_OK;
}

int ffa_cache_copy(int dtype, int batch, int heads, int rows, int src_max_len, int dst_max_len, int head_dim,
                   const void* k_src, const void* v_src, void* k_dst, void* v_dst, void* stream)
{
    if (!dtype_ok(dtype)) return fail(FFA_ERR_DTYPE, "unsupported dtype code %d", dtype);
    if (!head_dim_ok(head_dim)) return fail(FFA_ERR_HEAD_DIM, "unsupported head_dim %d (64, 80, 128, 256)", head_dim);
    if (batch <= 0 || heads <= 0 || dst_max_len <= 0 || rows < 0 || rows > dst_max_len || rows > src_max_len)
        return fail(FFA_ERR_RANGE, "need 0 <= rows (%d) <= source length (%d) and destination length (%d), positive batch, heads",
                    rows, src_max_len, dst_max_len);
    if (rows == 0) return FFA_OK;
    if (!k_src || !v_src || !k_dst || !v_dst) return fail(FFA_ERR_ARG, "null pointer");
    if (!aligned16(k_src) || !aligned16(v_src) || !aligned16(k_dst) || !aligned16(v_dst))
        return fail(FFA_ERR_ARG, "pointers must be 16-byte aligned");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "device query");
    const int r = ffa_k_cache_init(dtype, batch * heads, rows, src_max_len, dst_max_len, head_dim, k_src, v_src, k_dst, v_dst, sms,
                                   static_cast<cudaStream_t>(stream));
    if (r != 0) return cuda_fail(r, "cache copy launch");
    g_launches.fetch_add(1);
    return FFA_OK;
}

int ffa_cache_init(int dtype, int batch, int heads, int prompt_len, int max_len, int head_dim, const void* k_src,
                   const void* v_src, void* k_cache, void* v_cache, void* stream)
{
    if (prompt_len > max_len) return fail(FFA_ERR_RANGE, "need 0 <= prompt_len (%d) <= max_len (%d)", prompt_len, max_len);
    return ffa_cache_copy(dtype, batch, heads, prompt_len, prompt_len, max_len, head_dim, k_src, v_src, k_cache, v_cache, stream);
}

int ffa_plan_create(int dtype, int batch, int heads, int head_dim, int max_len, int use_default_launch, int device,
                    ffa_plan_t** plan)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan pointer");
    *plan = nullptr;
    if (!dtype_ok(dtype)) return fail(FFA_ERR_DTYPE, "unsupported dtype code %d", dtype);
    if (!head_dim_ok(head_dim)) return fail(FFA_ERR_HEAD_DIM, "unsupported head_dim %d (64, 80, 128, 256)", head_dim);
    if (batch <= 0 || heads <= 0 || max_len <= 0) return fail(FFA_ERR_RANGE, "batch, heads and max_len must be positive");
    int prev = 0;
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    int sms = 0, smem_cta = 0, smem_sm = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&smem_cta, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, device);
    int r = 0;
    if (e == cudaSuccess) r = ffa_k_prepare(dtype, head_dim, smem_cta);
    cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_fail(e, "device attribute query");
    if (r != 0) return cuda_fail(r, "kernel preparation (is this an sm_100a device?)");
    ffa_plan* p = new (std::nothrow) ffa_plan();
    if (p == nullptr) return fail(FFA_ERR_ARG, "out of host memory");
    std::memset(p, 0, sizeof(*p));
    p->dtype = dtype, p->B = batch, p->H = heads, p->Dh = head_dim, p->Lmax = max_len;
    p->use_default = use_default_launch != 0, p->device = device, p->mode = FFA_MODE_EXACT;
    p->cluster_merge = 1;
    p->sms = sms, p->smem_per_cta = smem_cta, p->smem_per_sm = smem_sm;
    p->max_grid = sms * kMaxCtasPerSm;
    *plan = p;
    return FFA_OK;
}

int ffa_plan_create_offline(int dtype, int batch, int heads, int head_dim, int max_len, int use_default_launch, int sms,
                            int smem_per_cta, int smem_per_sm, ffa_plan_t** plan)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan pointer");
    *plan = nullptr;
    if (!dtype_ok(dtype)) return fail(FFA_ERR_DTYPE, "unsupported dtype code %d", dtype);
    if (!head_dim_ok(head_dim)) return fail(FFA_ERR_HEAD_DIM, "unsupported head_dim %d (64, 80, 128, 256)", head_dim);
    if (batch <= 0 || heads <= 0 || max_len <= 0) return fail(FFA_ERR_RANGE, "batch, heads and max_len must be positive");
    if (sms <= 0 || smem_per_cta <= 0 || smem_per_sm < smem_per_cta) return fail(FFA_ERR_RANGE, "implausible device properties");
    ffa_plan* p = new (std::nothrow) ffa_plan();
    if (p == nullptr) return fail(FFA_ERR_ARG, "out of host memory");
    std::memset(p, 0, sizeof(*p));
    p->dtype = dtype, p->B = batch, p->H = heads, p->Dh = head_dim, p->Lmax = max_len;
    p->use_default = use_default_launch != 0, p->device = -1, p->mode = FFA_MODE_EXACT;
    p->cluster_merge = 1;
    p->sms = sms, p->smem_per_cta = smem_per_cta, p->smem_per_sm = smem_per_sm;
    p->max_grid = sms * kMaxCtasPerSm;
    p->offline = true;
    *plan = p;
    return FFA_OK;
}

int ffa_plan_get_prune_launch(const ffa_plan_t* plan, int t, int* cluster, int* chunk_rows, int* tile_rows, int* grid,
                              int* smem_bytes)
{
    if (plan == nullptr || !cluster || !chunk_rows || !tile_rows || !grid || !smem_bytes) return fail(FFA_ERR_ARG, "null pointer");
    if (t < 0 || t >= plan->Lmax) return fail(FFA_ERR_RANGE, "t = %d outside [0, %d)", t, plan->Lmax);
    FfaStepParams P;
    std::memset(&P, 0, sizeof(P));
    int smem = 0;
    if (plan->prune_path == 2 || !plan_fused(plan, t, &P, &smem)) {
        *cluster = 0, *chunk_rows = 0, *tile_rows = 0, *grid = 0, *smem_bytes = 0;   // streaming kernel
        return FFA_OK;
    }
    *cluster = P.cluster, *chunk_rows = P.chunk_rows, *tile_rows = P.tile_rows, *grid = P.grid, *smem_bytes = smem;
    return FFA_OK;
}

int ffa_plan_get_prune_path(const ffa_plan_t* plan, int t, float p, int with_scores, int* path)
{
    if (plan == nullptr || path == nullptr) return fail(FFA_ERR_ARG, "null pointer");
    if (t < 0 || t >= plan->Lmax) return fail(FFA_ERR_RANGE, "t = %d outside [0, %d)", t, plan->Lmax);
    FfaStepParams P;
    std::memset(&P, 0, sizeof(P));
    int smem = 0;
    if (prefers_stream(plan, t, p, with_scores != 0)) *path = 2;
    else if (plan->prune_path != 2 && plan_fused(plan, t, &P, &smem)) *path = 1;
    else *path = with_scores ? 2 : 0;
    return FFA_OK;
}

void ffa_plan_destroy(ffa_plan_t* plan) { delete plan; }

int ffa_plan_get_launch(const ffa_plan_t* plan, int t, ffa_launch_t* launch)
{
    if (plan == nullptr || launch == nullptr) return fail(FFA_ERR_ARG, "null pointer");
    if (t < 0 || t >= plan->Lmax) return fail(FFA_ERR_RANGE, "t = %d outside [0, %d)", t, plan->Lmax);
    const int r = fit_launch(plan, t, 2, launch);
    if (r != FFA_OK) return r;
    int cluster = 0;
    return fit_clusters(const_cast<ffa_plan_t*>(plan), t, false, launch, &cluster);   // fills the plan's occupancy cache
}

int ffa_plan_set_launch(ffa_plan_t* plan, const ffa_launch_t* launch)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    plan->forced = launch != nullptr;
    if (launch) plan->force = *launch;
    return FFA_OK;
}

int ffa_plan_set_prune_path(ffa_plan_t* plan, int path)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (path < 0 || path > 2) return fail(FFA_ERR_ARG, "prune path must be 0 (choose), 1 (cluster kernel) or 2 (streaming kernel)");
    plan->prune_path = path;
    return FFA_OK;
}

int ffa_plan_set_cluster_merge(ffa_plan_t* plan, int on)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    plan->cluster_merge = on != 0;
    return FFA_OK;
}

int ffa_plan_set_mode(ffa_plan_t* plan, int mode)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (mode != FFA_MODE_EXACT && mode != FFA_MODE_ROUND_LIKE_TORCH) return fail(FFA_ERR_ARG, "unknown mode %d", mode);
    plan->mode = mode;
    return FFA_OK;
}

size_t ffa_workspace_bytes(const ffa_plan_t* plan, int with_scores)
{
    if (plan == nullptr) return 0;
    return carve(plan, with_scores != 0).total;
}

int ffa_workspace_bind(ffa_plan_t* plan, void* workspace, size_t bytes, void* stream)
{
    if (plan == nullptr || workspace == nullptr) return fail(FFA_ERR_ARG, "null pointer");
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(FFA_ERR_ARG, "workspace must be 256-byte aligned");
    const Carve small = carve(plan, false), big = carve(plan, true);
    if (bytes < small.total) return fail(FFA_ERR_WORKSPACE, "workspace of %zu bytes, need at least %zu", bytes, small.total);
    char* base = static_cast<char*>(workspace);
    // status word + arrival counters start at zero; everything else is written before it is read
    cudaError_t e = cudaMemsetAsync(base, 0, small.partials, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "workspace clear");
    plan->ws = workspace, plan->ws_bytes = bytes;
    plan->status = reinterpret_cast<int*>(base + small.status);
    plan->tickets = reinterpret_cast<int*>(base + small.tickets);
    plan->partials = reinterpret_cast<float*>(base + small.partials);
    plan->scores = bytes >= big.total ? reinterpret_cast<float*>(base + big.scores) : nullptr;
    return FFA_OK;
}

namespace {

// a half of a rank's staging buffer for the output gather: [B][world][H * Dh] elements
size_t peer_half_bytes(const ffa_plan* p, int world)
{
    return align_up((size_t)p->B * world * p->H * p->Dh * elem_size(p->dtype), 256);
}

struct PageArgs {
    const int* table = nullptr;
    int max_pages = 0, page_rows = 0;
};

// One decode step on contiguous caches (pages.table == nullptr) or page pools.
int run_step(ffa_plan_t* plan, const void* q, const void* k, const void* v, void* k_cache, void* v_cache, void* out,
             float softmax_scale, int t, const int* seq_lengths, int right_or_no_padding, float p, uint32_t* kept_mask,
             const PageArgs& pages, void* stream)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (plan->offline) return fail(FFA_ERR_ARG, "this plan was created offline (planning only) and cannot launch");
    if (!q || !k || !v || !k_cache || !v_cache || !out) return fail(FFA_ERR_ARG, "null tensor pointer");
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out))
        return fail(FFA_ERR_ARG, "tensor pointers must be 16-byte aligned");
    if (t < 0 || t >= plan->Lmax) return fail(FFA_ERR_RANGE, "t = %d outside [0, %d)", t, plan->Lmax);
    if (!(p >= 0.f && p <= 1.f)) return fail(FFA_ERR_RANGE, "prob_thresh %g outside [0, 1]", (double)p);
    if (seq_lengths == nullptr && !right_or_no_padding)
        return fail(FFA_ERR_ARG, "left padding (right_or_no_padding = 0) needs seq_lengths");
    if (plan->ws == nullptr) return fail(FFA_ERR_WORKSPACE, "no workspace bound (ffa_workspace_bind)");
    const bool paged = pages.table != nullptr;
    const bool twopass = p > 0.f || plan->mode == FFA_MODE_ROUND_LIKE_TORCH;
    const int cap = t;   // rows the unit list covers: every sample is at row t, or (per-sample lengths) at a row no greater than the bound t
    FfaStepParams P;
    std::memset(&P, 0, sizeof(P));
    P.q = q, P.k = k, P.v = v, P.k_cache = k_cache, P.v_cache = v_cache, P.out = out;
    P.seq_lengths = seq_lengths, P.right_or_no_padding = right_or_no_padding != 0;
    P.B = plan->B, P.H = plan->H, P.Lmax = plan->Lmax, P.t = t;
    P.scale = softmax_scale, P.p = p;
    P.round_like_torch = plan->mode == FFA_MODE_ROUND_LIKE_TORCH && !(p > 0.f);
    P.partials = plan->partials, P.tickets = plan->tickets, P.status = plan->status;
    P.scores = plan->scores, P.score_stride = score_stride(plan->Lmax);
    P.kept_mask = kept_mask, P.mask_words = (plan->Lmax + 31) / 32;
    P.page_table = pages.table, P.max_pages = pages.max_pages, P.page_rows = pages.page_rows;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // p > 0 / torch rounding.  Small steps: the cluster kernel (scores stay in shared memory, nothing but the
    // launch is fixed cost).  Large steps: the streaming kernel (a persistent grid keeps HBM busy; the cluster
    // kernel pays its start, two cluster barriers and the merge once per CTA).  The streaming kernel needs
    // the score scratch; without it the cluster kernel runs whenever it fits.
    // With every row kept (torch rounding, p = 0) the cluster kernel streams the V tiles through its ring like the K
    // tiles and wins at every size it fits (bf16 x 128, 1024 pairs, 512 / 2 K / 8 K / 32 K tokens: 52 / 167 / 651 /
    // 2848 us against 138 / 238 / 921 / 3566 us for the streaming kernel, whose gather warps fetch row by row).
    const bool stream_first = prefers_stream(plan, cap, p, plan->scores != nullptr);
    if (twopass && !stream_first) {
        FfaStepParams F = P;
        int smem_f = 0;
        if (plan_fused(plan, cap, &F, &smem_f)) {
            const int rf = ffa_k_decode_fused_prune(plan->dtype, plan->Dh, F, smem_f, st);
            if (rf != 0) return cuda_fail(rf, "fused pruning launch");
            g_launches.fetch_add(1);
            return FFA_OK;
        }
        if (plan->prune_path == 1) return fail(FFA_ERR_ARG, "the fused pruning kernel does not fit this shape in shared memory");
    }
    if (twopass && plan->scores == nullptr)
        return fail(FFA_ERR_WORKSPACE, "this shape needs the streaming pruning kernel: bind a workspace sized with with_scores = 1");

    ffa_launch_t L;
    // the streaming kernel never lets a tile straddle a page: tiles are powers of two that divide it
    int r = fit_launch(plan, cap, twopass ? 1 : 2, &L, /*pow2_tiles=*/paged);
    if (r != FFA_OK) return r;
    if (paged && pages.page_rows % L.tile_rows != 0) return fail(FFA_ERR_ARG, "tile of %d rows does not divide the page", L.tile_rows);
    P.tile_rows = L.tile_rows, P.stages = L.stages, P.grid = L.grid;
    P.units_per_bh = cap / L.tile_rows + 1;
    P.parts_per_bh = L.parts_per_bh;
    if (!twopass) {
        if (plan->push_gathered != nullptr && plan->peer_world > 1 && !paged) {
            // the kernel's epilogue is the push phase of the output all-gather
            for (int r = 0; r < plan->peer_world; ++r) P.push_peer[r] = plan->peer_buf[r];
            P.push_gathered = plan->push_gathered, P.push_half_bytes = peer_half_bytes(plan, plan->peer_world);
            P.push_world = plan->peer_world, P.push_rank = plan->peer_rank;
        }
        // the C CTAs of a pair merge inside a thread-block cluster when every CTA owns exactly one part
        // (pairs with more than 8 parts: whole clusters of 8, the cluster leaders merge through global memory)
        r = fit_clusters(plan, cap, paged, &L, &P.cluster);
        if (r != FFA_OK) return r;
        P.tile_rows = L.tile_rows, P.stages = L.stages, P.grid = L.grid;
        P.units_per_bh = cap / L.tile_rows + 1;
        P.parts_per_bh = L.parts_per_bh;
        const int threads = 32 * (L.consumer_warps + 1);
        r = ffa_k_decode_onepass(plan->dtype, plan->Dh, P, threads, L.smem_bytes, st);
        if (r != 0) return cuda_fail(r, "attention launch");
        g_launches.fetch_add(1);
        return FFA_OK;
    }
    r = ffa_k_decode_prune_stream(plan->dtype, plan->Dh, P, L.consumer_warps, L.smem_bytes, st);
    if (r != 0) return cuda_fail(r, "streaming pruning launch");
    g_launches.fetch_add(1);
    return FFA_OK;
}

}  // namespace

int ffa_attention(ffa_plan_t* plan, const void* q, const void* k, const void* v, void* k_cache, void* v_cache, void* out,
                  float softmax_scale, int t, const int* seq_lengths, int right_or_no_padding, float p,
                  uint32_t* kept_mask, void* stream)
{
    return run_step(plan, q, k, v, k_cache, v_cache, out, softmax_scale, t, seq_lengths, right_or_no_padding, p, kept_mask,
                    PageArgs{}, stream);
}

int ffa_attention_paged(ffa_plan_t* plan, const void* q, const void* k, const void* v, void* k_pool, void* v_pool,
                        const int* page_table, int max_pages, int page_rows, void* out, float softmax_scale, int t,
                        const int* seq_lengths, int right_or_no_padding, float p, uint32_t* kept_mask, void* stream)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (page_table == nullptr) return fail(FFA_ERR_ARG, "null page table");
    if (page_rows <= 0 || page_rows % 128 != 0) return fail(FFA_ERR_RANGE, "page_rows (%d) must be a positive multiple of 128", page_rows);
    if (max_pages <= 0 || (long long)max_pages * page_rows != plan->Lmax)
        return fail(FFA_ERR_RANGE, "max_pages * page_rows (%d * %d) must equal the plan's max_len (%d)", max_pages, page_rows, plan->Lmax);
    PageArgs pages;
    pages.table = page_table, pages.max_pages = max_pages, pages.page_rows = page_rows;
    return run_step(plan, q, k, v, k_pool, v_pool, out, softmax_scale, t, seq_lengths, right_or_no_padding, p, kept_mask, pages,
                    stream);
}

int ffa_selftest_wait_timeout(ffa_plan_t* plan, unsigned int limit_ms, void* stream)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (plan->ws == nullptr) return fail(FFA_ERR_WORKSPACE, "no workspace bound");
    if (limit_ms == 0 || limit_ms > 2000) return fail(FFA_ERR_RANGE, "limit_ms must be in [1, 2000]");
    const int r = ffa_k_wait_selftest(plan->status, (unsigned long long)limit_ms * 1000000ull, nullptr, static_cast<cudaStream_t>(stream));
    if (r != 0) return cuda_fail(r, "self-test launch");
    g_launches.fetch_add(1);
    return FFA_OK;
}

int ffa_device_status(ffa_plan_t* plan, void* stream, int* status)
{
    if (plan == nullptr || status == nullptr) return fail(FFA_ERR_ARG, "null pointer");
    if (plan->ws == nullptr) return fail(FFA_ERR_WORKSPACE, "no workspace bound");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(status, plan->status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(plan->status, 0, sizeof(int), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(e, "status read");
    if (*status != 0) return fail(FFA_ERR_DEVICE, "device status word = %d", *status);
    return FFA_OK;
}

// ---- output gather over peer memory -------------------------------------------------------------
// Staging buffer of every rank: half 0 | half 1 | flags[FFA_MAX_PEERS], step counter, ticket (256 bytes);
// a half is [B][world][H * Dh] elements.


size_t ffa_peer_gather_bytes(const ffa_plan_t* plan, int world)
{
    if (plan == nullptr || world < 1 || world > FFA_MAX_PEERS) return 0;
    return 2 * peer_half_bytes(plan, world) + 256;
}

int ffa_peer_mem_alloc(size_t bytes, void** ptr, unsigned char* handle)
{
    if (ptr == nullptr || handle == nullptr || bytes == 0) return fail(FFA_ERR_ARG, "null pointer or zero size");
    static_assert(sizeof(cudaIpcMemHandle_t) == FFA_PEER_HANDLE_BYTES, "handle size");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "peer buffer allocation");
    e = cudaMemset(p, 0, bytes);   // arrival flags start at zero
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(e, "peer buffer export");
    }
    std::memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return FFA_OK;
}

int ffa_peer_mem_open(const unsigned char* handle, void** ptr)
{
    if (ptr == nullptr || handle == nullptr) return fail(FFA_ERR_ARG, "null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    const cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e, "peer buffer import");
    return FFA_OK;
}

int ffa_peer_mem_close(void* ptr)
{
    if (ptr == nullptr) return FFA_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? FFA_OK : cuda_fail(e, "peer buffer close");
}

int ffa_peer_mem_free(void* ptr)
{
    if (ptr == nullptr) return FFA_OK;
    const cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? FFA_OK : cuda_fail(e, "peer buffer free");
}

int ffa_peer_gather_attach(ffa_plan_t* plan, int world, int rank, void* const* buffers, size_t bytes_each)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (world == 0) {   // detach
        plan->peer_world = 0, plan->push_gathered = nullptr;
        return FFA_OK;
    }
    if (buffers == nullptr) return fail(FFA_ERR_ARG, "null buffer list");
    if (world < 1 || world > FFA_MAX_PEERS) return fail(FFA_ERR_RANGE, "world %d outside [1, %d]", world, FFA_MAX_PEERS);
    if (rank < 0 || rank >= world) return fail(FFA_ERR_RANGE, "rank %d outside [0, %d)", rank, world);
    if (bytes_each < ffa_peer_gather_bytes(plan, world))
        return fail(FFA_ERR_WORKSPACE, "peer buffers of %zu bytes, need %zu", bytes_each, ffa_peer_gather_bytes(plan, world));
    for (int r = 0; r < world; ++r) {
        if (buffers[r] == nullptr) return fail(FFA_ERR_ARG, "buffer of rank %d is null", r);
        if ((reinterpret_cast<uintptr_t>(buffers[r]) & 255u) != 0) return fail(FFA_ERR_ARG, "buffer of rank %d is not 256-byte aligned", r);
    }
    for (int r = 0; r < world; ++r) plan->peer_buf[r] = buffers[r];
    plan->peer_world = world, plan->peer_rank = rank;
    return FFA_OK;
}

int ffa_peer_push_target(ffa_plan_t* plan, void* gathered)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (gathered != nullptr && plan->peer_world < 1) return fail(FFA_ERR_ARG, "no peer buffers attached (ffa_peer_gather_attach)");
    if (gathered != nullptr && !aligned16(gathered)) return fail(FFA_ERR_ARG, "gathered must be a 16-byte aligned pointer");
    plan->push_gathered = gathered;
    return FFA_OK;
}

int ffa_peer_gather(ffa_plan_t* plan, const void* out_local, void* gathered, int phases, unsigned int wait_limit_ms, void* stream)
{
    if (plan == nullptr) return fail(FFA_ERR_ARG, "null plan");
    if (plan->peer_world < 1) return fail(FFA_ERR_ARG, "no peer buffers attached (ffa_peer_gather_attach)");
    if (plan->ws == nullptr) return fail(FFA_ERR_WORKSPACE, "no workspace bound (ffa_workspace_bind)");
    if (phases < 1 || phases > 3) return fail(FFA_ERR_ARG, "phases must be 1 (push), 2 (wait) or 3 (both)");
    if ((phases & 1) && (out_local == nullptr || !aligned16(out_local))) return fail(FFA_ERR_ARG, "out_local must be a 16-byte aligned pointer");
    if (gathered == nullptr || !aligned16(gathered)) return fail(FFA_ERR_ARG, "gathered must be a 16-byte aligned pointer");
    if (wait_limit_ms == 0 || wait_limit_ms > 2000) return fail(FFA_ERR_RANGE, "wait_limit_ms must be in [1, 2000]");
    const int world = plan->peer_world;
    FfaPeerGatherParams G;
    std::memset(&G, 0, sizeof(G));
    G.out_local = out_local, G.gathered = gathered;
    for (int r = 0; r < world; ++r) G.peer_base[r] = plan->peer_buf[r];
    G.half_bytes = peer_half_bytes(plan, world);
    G.status = plan->status;
    G.wait_limit_ns = (unsigned long long)wait_limit_ms * 1000000ull;
    G.world = world, G.rank = plan->peer_rank, G.B = plan->B;
    G.row_bytes = plan->H * plan->Dh * elem_size(plan->dtype);
    G.phases = phases;
    const int r = ffa_k_peer_gather(G, static_cast<cudaStream_t>(stream));
    if (r != 0) return cuda_fail(r, "peer gather launch");
    g_launches.fetch_add(1);
    return FFA_OK;
}

}  // extern "C"
