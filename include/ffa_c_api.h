/*
 * C ABI of the B200 decode-attention engine (libffa_b200.so).
 *
 * One decode step of masked multi-head attention for a single new token per (batch, head):
 * append k/v at row t of the KV cache, attend over rows 0..t, optional probability pruning.
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless stated otherwise.
 * All calls are asynchronous on the given stream (a cudaStream_t passed as void*; NULL is the
 * legacy default stream) and return an int status: 0 on success, a negative FFA_ERR_* code
 * otherwise, with a human-readable reason available from ffa_last_error().
 *
 * Each entry point cites the reference interface it replaces (paths inside the
 * FastForwardAttention checkout).
 */
#ifndef FFA_C_API_H
#define FFA_C_API_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element type of q/k/v, the caches and the output.  The reference dispatches on
 * sizeof(T) with T in {float, uint16_t-as-half} (attention.cu:1512-1554); bf16 is new. */
enum { FFA_DTYPE_F32 = 0, FFA_DTYPE_F16 = 1, FFA_DTYPE_BF16 = 2 };

enum {
    FFA_OK = 0,
    FFA_ERR_DTYPE = -1,     /* unknown dtype code */
    FFA_ERR_HEAD_DIM = -2,  /* head_dim not in {64, 80, 128, 256} (attention.cu:1515-1531) */
    FFA_ERR_RANGE = -3,     /* t outside [0, max_len), sizes <= 0, p outside [0, 1] */
    FFA_ERR_ARG = -4,       /* null or misaligned pointer, bad flag combination */
    FFA_ERR_CUDA = -5,      /* a CUDA runtime call failed; ffa_last_error() has its text */
    FFA_ERR_WORKSPACE = -6, /* no workspace bound, or bound workspace too small */
    FFA_ERR_DEVICE = -7     /* the kernel recorded an error in the device status word */
};

/* Arithmetic modes (ffa_plan_set_mode). */
enum {
    /* fp32 arithmetic throughout, one rounding to the storage type at the end.  Default. */
    FFA_MODE_EXACT = 0,
    /* Re-applies the four roundings of torch's same-dtype softmax(QK^T*scale)V on fp16/bf16
     * operands (scores, scaled scores, probabilities, output), so results track the
     * reference's torch path (example.py:6-7) rather than the exact value.  Two kernels. */
    FFA_MODE_ROUND_LIKE_TORCH = 1
};

/* Bits of the device status word (ffa_device_status). */
enum {
    FFA_STATUS_WAIT_TIMEOUT = 1, /* a bounded wait on a copy barrier ran out */
    FFA_STATUS_BAD_LENGTH = 2    /* a per-sample length was outside [0, max_len) or above the stated bound */
};

typedef struct ffa_plan ffa_plan_t;

/* Launch shape of the streaming kernels, chosen by the planner per (dtype, sizes, t). */
typedef struct ffa_launch {
    int tile_rows;      /* cache rows per pipeline stage (K rows and V rows each) */
    int stages;         /* depth of the shared-memory ring */
    int consumer_warps; /* compute warps per CTA, 1..8 (one more warp issues the bulk copies) */
    int ctas_per_sm;    /* resident CTAs per SM the grid is sized for */
    int grid;           /* number of CTAs; the work list is cut into this many contiguous runs */
    int smem_bytes;     /* dynamic shared memory per CTA */
    int parts_per_bh;   /* parts a (batch, head) is cut into; CTA runs are whole parts (output only) */
} ffa_launch_t;

/* Bytes of the two cache slabs, each laid out [batch, heads, max_len, head_dim] (row t of
 * one (batch, head) is head_dim contiguous elements; rows are 16-byte aligned).
 * Replaces the torch::empty shapes in init_attention_cache (torch_ffa_api.cpp:65-66, 85-86). */
int ffa_cache_bytes(int dtype, int batch, int heads, int max_len, int head_dim, size_t* k_bytes,
                    size_t* v_bytes);

/* Copies prompt K and V, each [batch, heads, prompt_len, head_dim] contiguous, into rows
 * [0, prompt_len) of the caches; rows >= prompt_len are left untouched.
 * Replaces invokeTranspose4dBatchMajor<T> (attention.cu:1611-1689). */
int ffa_cache_init(int dtype, int batch, int heads, int prompt_len, int max_len, int head_dim,
                   const void* k_src, const void* v_src, void* k_cache, void* v_cache, void* stream);

/* Copies rows [0, rows) of every (batch, head) between two cache slabs of different lengths
 * ([batch, heads, src_max_len, head_dim] -> [batch, heads, dst_max_len, head_dim]): how a cache
 * grows.  No counterpart in the reference, whose cache length is fixed at construction
 * (torch_ffa_api.cpp:65-66). */
int ffa_cache_copy(int dtype, int batch, int heads, int rows, int src_max_len, int dst_max_len, int head_dim,
                   const void* k_src, const void* v_src, void* k_dst, void* v_dst, void* stream);

/* Creates the per-engine plan: validates the shape, queries the device once, prepares the
 * kernels.  use_default_launch != 0 selects the fixed analytic launch rule, 0 the table
 * measured on B200.  Host memory only; no device allocation.
 * Replaces get_launch_params (kernel_launch_utils.h:135-180) and the launch members kept by
 * the FastForwardAttn constructor (torch_ffa_api.cpp:162-177, 196-201). */
int ffa_plan_create(int dtype, int batch, int heads, int head_dim, int max_len, int use_default_launch,
                    int device, ffa_plan_t** plan);
/* The same planner without a device: the caller states the multiprocessor count and the
 * shared-memory limits (per CTA opt-in, per SM).  For capacity planning and for testing the
 * launch rules on hosts without a GPU; such a plan cannot be passed to ffa_attention. */
int ffa_plan_create_offline(int dtype, int batch, int heads, int head_dim, int max_len, int use_default_launch, int sms,
                            int smem_per_cta, int smem_per_sm, ffa_plan_t** plan);
void ffa_plan_destroy(ffa_plan_t* plan);

/* The launch shape the planner picks for step t (after any override). */
int ffa_plan_get_launch(const ffa_plan_t* plan, int t, ffa_launch_t* launch);
/* Forces a launch shape (fields <= 0 keep the planner's choice); NULL removes the override.
 * Used by the tuning sweep; the reference exposes tpb/tpv/tpk the same way
 * (c_ffa_api.h:17-20). */
int ffa_plan_set_launch(ffa_plan_t* plan, const ffa_launch_t* launch);
int ffa_plan_set_mode(ffa_plan_t* plan, int mode);
/* p > 0 and the torch-rounding mode need the global softmax statistics before any V row is
 * read.  Two implementations, one launch each: 1 = a thread-block cluster per (batch, head)
 * with the scores in shared memory (needs no score scratch; small steps); 2 = the streaming
 * kernel: a persistent grid streams the K rows of all pairs, leaves fp32 scores in the
 * workspace's score scratch, and its gather warps fetch the surviving V rows of finished
 * pairs while the K stream goes on (any size).  0 (default) picks 2 for pruned steps (p > 0) that
 * stream at least 1 GB of K when the score scratch is bound, else 1 whenever a slice fits in shared
 * memory (with every row kept, i.e. torch rounding with p = 0, implementation 1 streams V tiles
 * instead of gathering rows and is the faster one at every size).  The reference does both phases in one CTA per (batch, head) (attention.cu:1077-1257),
 * which is what caps its sequence length. */
int ffa_plan_set_prune_path(ffa_plan_t* plan, int path);
/* Exact steps whose (batch, head) pairs are split over 2..8 CTAs merge the splits inside a
 * thread-block cluster through distributed shared memory (on = 1, the default) or through
 * partial results in global memory and an arrival counter (on = 0; kept for comparison). */
int ffa_plan_set_cluster_merge(ffa_plan_t* plan, int on);
/* The fused pruning launch the planner picks for step t: CTAs per (batch, head) cluster, cache
 * rows per CTA, tile rows, grid and dynamic shared memory; all zero when the streaming kernel
 * would run instead (path 2, or no cluster shape fits). */
int ffa_plan_get_prune_launch(const ffa_plan_t* plan, int t, int* cluster, int* chunk_rows, int* tile_rows, int* grid,
                              int* smem_bytes);
/* Which implementation a step at row t with threshold p takes (p = 0: a torch-rounding step): 1 or 2 as in
 * ffa_plan_set_prune_path, 0 when neither can run (the cluster kernel's slices do not fit in shared memory and no
 * score scratch is bound).  with_scores: whether the workspace was sized with the score scratch. */
int ffa_plan_get_prune_path(const ffa_plan_t* plan, int t, float p, int with_scores, int* path);

/* Scratch the engine needs in device memory: split partials, arrival counters, the status
 * word and, when with_scores != 0 (needed for p > 0 and FFA_MODE_ROUND_LIKE_TORCH), one fp32
 * score per cache row (the streaming pruning kernel's scratch; ffa_attention returns
 * FFA_ERR_WORKSPACE if a call needs it and it is missing).  The caller allocates it (256-byte aligned) and binds it once;
 * binding clears the counters on the stream.  One workspace serves one stream at a time. */
size_t ffa_workspace_bytes(const ffa_plan_t* plan, int with_scores);
int ffa_workspace_bind(ffa_plan_t* plan, void* workspace, size_t bytes, void* stream);

/* One decode step.  q, k, v: batch*heads*head_dim contiguous elements in (batch, head, dim)
 * order.  Writes k and v into row `row` of the caches and out[batch, heads, head_dim], where
 *   seq_lengths == NULL                      : row = t for every sample, all keys visible;
 *   seq_lengths != NULL, right_or_no_padding : row = seq_lengths[b] (per-sample lengths); t is then
 *                                              the host's upper bound on every seq_lengths[b]: the
 *                                              work is laid out for rows 0..t, so a tight bound keeps
 *                                              all CTAs busy when the cache is mostly empty; pass
 *                                              max_len - 1 when nothing is known.  A sample whose
 *                                              length exceeds t is skipped and reported as
 *                                              FFA_STATUS_BAD_LENGTH, never cut short;
 *   seq_lengths != NULL, !right_or_no_padding: row = t, keys < seq_lengths[b] are masked
 *                                              (left padding).
 * q, k, v and out may also point into pinned (page-locked, device-addressable) host memory: the
 * kernels read and write them in place, which saves a host-driven loop its staging copies.
 * p is the pruning threshold as a fraction of the largest probability; p == 0 is exact
 * attention.  kept_mask, if not NULL and p > 0, receives one bit per cache row,
 * [batch*heads, ceil(max_len/32)] words, bit set = row contributed to the output.
 * Replaces call_attention<T> (attention.cu:1512-1554) / do_attention<T> (c_ffa_api.h:17-20);
 * the tpv/tpk/tpb arguments of those live in the plan. */
int ffa_attention(ffa_plan_t* plan, const void* q, const void* k, const void* v, void* k_cache, void* v_cache,
                  void* out, float softmax_scale, int t, const int* seq_lengths, int right_or_no_padding,
                  float p, uint32_t* kept_mask, void* stream);

/* ffa_attention on PAGED caches; p, kept_mask and the plan's mode mean what they mean there.
 * k_pool and v_pool are page pools laid out [pages, heads, page_rows, head_dim]; page_table
 * [batch, max_pages] (int32, device) names the pool page that holds rows
 * [i*page_rows, (i+1)*page_rows) of sequence b.  Only pages that hold rows 0..row of a sequence
 * are dereferenced, so sequences of different lengths share one pool and a sequence takes
 * memory as it grows.  page_rows is a multiple of 128 and max_pages * page_rows equals the
 * plan's max_len.  No counterpart in the reference, which allocates max_len rows per sequence
 * up front (torch_ffa_api.cpp:65-66). */
int ffa_attention_paged(ffa_plan_t* plan, const void* q, const void* k, const void* v, void* k_pool, void* v_pool,
                        const int* page_table, int max_pages, int page_rows, void* out, float softmax_scale, int t,
                        const int* seq_lengths, int right_or_no_padding, float p, uint32_t* kept_mask, void* stream);

/* The exact (p == 0, no per-sample lengths) decode step with NO caller-provided workspace and
 * no allocation of any kind inside the call.  It has no counterpart in the reference; it
 * exists for hosts that cannot allocate device memory when they call the engine: a server
 * whose own pool allocator took the whole GPU at start-up (a cudaMalloc from a plug-in then
 * fails or is against policy), a latency-critical decode thread that must not pay the
 * device-wide synchronisation of cudaMalloc / cudaFree, or a bare C host that owns only the
 * six tensors of the call.  The scratch (split partials, arrival counters, status word)
 * lives in a 4 MiB static device array that every GPU loading this library holds until
 * process exit.  Limits and rules:
 *   - sizes whose scratch need exceeds 4 MiB are rejected with FFA_ERR_RANGE (need =
 *     256 + 4*batch*heads + 4*(grid + batch*heads)*(head_dim + 2) bytes, grid <= 2 CTAs per SM;
 *     e.g. batch*heads = 1024 at head_dim 128 needs 0.7 MiB); use ffa_attention beyond that;
 *   - the array is shared by every call on that GPU and keeps the previous call's contents;
 *     each call clears the arrival counters on `stream` before launching, and calls whose
 *     kernels overlap on one GPU (other streams, other host threads) race -- keep them
 *     stream-ordered;
 *   - the first call on each device performs a one-time set-up (device address of the array,
 *     device queries, kernel attributes); make that first call outside any stream capture.
 * Arguments as for ffa_attention.  device_status: optional DEVICE int the kernel ORs its
 * FFA_STATUS_* bits into (caller-owned, caller-cleared); with NULL the bits accumulate in a
 * status word inside the static array, which no call clears and ffa_static_scratch_status
 * reads.  error_text: optional HOST buffer that receives the reason for a non-zero return. */
int ffa_attention_static_scratch(int dtype, int batch, int heads, int head_dim, int max_len, const void* q,
                                 const void* k, const void* v, void* k_cache, void* v_cache, void* out,
                                 float softmax_scale, int t, int* device_status, void* stream, char* error_text,
                                 size_t error_text_len);

/* Companion of ffa_attention_static_scratch (no counterpart in the reference either): copies the
 * static array's status word of the current device to the HOST int *status, clears the word,
 * synchronises `stream`.  Allocates nothing.  FFA_OK when *status == 0, FFA_ERR_DEVICE when a
 * FFA_STATUS_* bit was set by any static-scratch call since the last read. */
int ffa_static_scratch_status(void* stream, int* status);
/* Diagnostic for that status word, like ffa_selftest_wait_timeout below: one warp waits at most
 * limit_ms (1..2000) on a copy barrier nothing completes, gives up and records
 * FFA_STATUS_WAIT_TIMEOUT in the static status word.  Nothing faults or hangs. */
int ffa_static_scratch_selftest_wait_timeout(unsigned int limit_ms, void* stream);

/* Synchronises the stream and returns the device status word (0 = clean) in *status, then
 * clears it.  The reference only printf()s cudaGetLastError (attention.cu:1444-1451). */
int ffa_device_status(ffa_plan_t* plan, void* stream, int* status);

/* ---- All-gather of the step outputs over peer memory (heads sharded over the GPUs of a node).
 * No counterpart in the reference, which runs on one GPU.  Every rank allocates one staging
 * buffer of ffa_peer_gather_bytes(plan, world) bytes with ffa_peer_mem_alloc (device memory,
 * zero-filled, plus a 64-byte handle another process of the node can open with
 * ffa_peer_mem_open), collects the `world` buffer pointers in rank order (its own included)
 * and attaches them to its plan (world = 0 detaches).
 * ffa_peer_gather then stores this rank's out_local [batch, heads, head_dim] (heads = the
 * plan's local head count) into every peer's staging buffer, raises one arrival flag per peer,
 * waits -- for at most wait_limit_ms (1..2000), after which FFA_STATUS_WAIT_TIMEOUT is set in
 * the status word and the kernel returns -- until every peer's slice of the same step has
 * arrived, and writes gathered [batch, world*heads, head_dim] (this rank's own memory; rank r's
 * heads at [r*heads, (r+1)*heads)).  out_local may be NULL when phases == 2.  Every rank must make the same sequence of calls.  The
 * step number lives in device memory and is advanced by the kernel, so all launch arguments
 * are the same for every step and the call may be recorded in a CUDA graph.
 * phases: 3 = both; 1 = store and signal only, 2 = wait and collect only (refers to the latest
 * push; same `gathered`) -- the split exists so that several ranks can be driven from ONE
 * stream of one GPU, all pushes before all waits; a kernel that waits must never be queued
 * ahead of the kernel that signals it on the same GPU.
 * Teardown: no rank may unmap or free a buffer while a peer can still store into it, and an
 * exported buffer must outlive every mapping of it: synchronise the device, pass a host
 * barrier, ffa_peer_mem_close the peers' buffers, pass a second barrier, ffa_peer_mem_free the
 * own. */
#define FFA_MAX_PEERS 8
#define FFA_PEER_HANDLE_BYTES 64
size_t ffa_peer_gather_bytes(const ffa_plan_t* plan, int world);
int ffa_peer_mem_alloc(size_t bytes, void** ptr, unsigned char* handle /* [FFA_PEER_HANDLE_BYTES] */);
int ffa_peer_mem_open(const unsigned char* handle, void** ptr);
int ffa_peer_mem_close(void* ptr);
int ffa_peer_mem_free(void* ptr);
int ffa_peer_gather_attach(ffa_plan_t* plan, int world, int rank, void* const* buffers, size_t bytes_each);
int ffa_peer_gather(ffa_plan_t* plan, const void* out_local, void* gathered, int phases, unsigned int wait_limit_ms,
                    void* stream);
/* Folds the push phase into the attention kernel itself: while `gathered` (this rank's [batch, world*heads, head_dim]
 * result, device memory or pinned host memory) is set, every EXACT step of ffa_attention (p == 0, exact mode, contiguous
 * caches) stores each output row, from the CTA that computes it, into this rank's slot of every peer's staging buffer and
 * of `gathered`, and the CTA that finishes the step's last (batch, head) pair raises the arrival flags -- one kernel does the
 * attention and the sending half of the collective, and rows leave as they are produced.  Complete the step with
 * ffa_peer_gather(plan, NULL, gathered, 2, ...) (wait and collect only).  Pruned and torch-rounding steps do not push: follow
 * those with phases = 3 as before.  A push must always be followed by its wait before the next step (the two staging
 * halves alternate on that assumption).  NULL switches the push off.  Plain 2..16-byte peer stores; no multicast. */
int ffa_peer_push_target(ffa_plan_t* plan, void* gathered);

/* Diagnostic, no counterpart in the reference: launches one warp that waits, for at most
 * limit_ms (1..2000), on a copy barrier nothing completes.  The wait must give up, the kernel
 * must return normally, and the next ffa_device_status() must report FFA_STATUS_WAIT_TIMEOUT
 * -- the path the streaming kernels take if a bulk copy never lands.  Nothing faults or hangs. */
int ffa_selftest_wait_timeout(ffa_plan_t* plan, unsigned int limit_ms, void* stream);

/* Kernels launched by this library since it was loaded (for launch accounting in benchmarks). */
unsigned long long ffa_launch_count(void);

/* Reason for the most recent non-zero return on this thread. */
const char* ffa_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* FFA_C_API_H */
