// Internal interface between the C ABI (ffa_c_api.cu) and the kernels (ffa_decode_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Everything one decode step needs on the device.  Plain data, passed by value to kernels.
struct FfaStepParams {
    const void* q;        // [B*H, Dh]
    const void* k;        // [B*H, Dh]
    const void* v;        // [B*H, Dh]
    void* k_cache;        // [B*H, Lmax, Dh]
    void* v_cache;        // [B*H, Lmax, Dh]
    void* out;            // [B*H, Dh]
    const int* seq_lengths;  // [B] or null
    int right_or_no_padding;
    int B, H, Lmax, t;
    // work decomposition: every (batch, head) owns units_per_bh tiles of tile_rows cache rows, grouped
    // into parts_per_bh parts; the flat list of B*H*parts_per_bh parts is cut into `grid` equal runs
    int tile_rows, stages, units_per_bh, parts_per_bh, grid;
    float scale;
    float p;
    int round_like_torch;
    // scratch
    float* partials;   // [(grid + B*H)] x (Dh + 2): weighted sum, running max, running sum
    int* tickets;      // [B*H] arrival counters, zero between launches
    int* status;       // device status word
    float* scores;     // [B*H, score_stride] fp32 scores (streaming pruning kernel); a pair's scores are whole 128-byte lines
    int score_stride;  // Lmax rounded up to a multiple of 32
    uint32_t* kept_mask;  // [B*H, mask_words] or null
    int mask_words;
    // thread-block cluster size: CTAs per (batch, head) (fused pruning kernel; streaming kernel when
    // it merges split pairs inside a cluster, 0 otherwise); fused pruning: cache rows per CTA (multiple of 32)
    int cluster, chunk_rows;
    // paged caches: k_cache / v_cache are page pools [pages, H, page_rows, Dh] and
    // page_table [B, max_pages] names the page of every page_rows rows of a sequence; null = contiguous
    const int* page_table;
    int max_pages, page_rows;
    // Output push over peer memory (heads sharded over the GPUs of a node; exact kernel only): the CTA that writes
    // out[b, h, :] also stores the row into this rank's slot of every peer's staging half and of the own gathered
    // result, and the CTA that finishes the step's last pair raises the arrival flags.  push_world <= 1: off.
    void* push_peer[8];     // every rank's staging buffer (layout: see FfaPeerGatherParams)
    void* push_gathered;    // [B][push_world * H][Dh]: this rank's own result tensor
    size_t push_half_bytes;
    int push_world, push_rank;
};

// 32-bit words of the 256-byte tail of a staging buffer: arrival flags (one per peer), the step counter, the ticket that
// advances it, one ticket per peer that elects the CTA raising that peer's flag, and the count of (batch, head)
// pairs whose output the attention kernel has pushed in the current step
enum { kPeerTailFlags = 0, kPeerTailCounter = 16, kPeerTailTicket = 17, kPeerTailPushTickets = 24, kPeerTailPairsDone = 32 };

// One all-gather of the step outputs over peer memory.  Every rank owns a staging buffer: two
// halves [B][world * row_bytes] (used alternately), then flags[8], the step counter, a ticket.
struct FfaPeerGatherParams {
    const void* out_local;     // [B][row_bytes]: this rank's outputs
    void* gathered;            // [B][world * row_bytes]: the result, this rank's own memory
    void* peer_base[8];        // every rank's staging buffer (own included)
    size_t half_bytes;
    int* status;               // device status word
    unsigned long long wait_limit_ns;
    int world, rank, B, row_bytes;
    int phases;                // bit 0: push the slice and raise the flags; bit 1: wait for the peers' flags, collect
    int slices;                // CTAs per peer (set by the launcher)
};

// dtype codes as in ffa_c_api.h.  Return a cudaError_t as int.
int ffa_k_prepare(int dtype, int head_dim, int max_smem_bytes);
int ffa_k_cache_init(int dtype, int BH, int prompt_len, int src_len, int max_len, int head_dim, const void* k_src,
                     const void* v_src, void* k_cache, void* v_cache, int sms, cudaStream_t stream);
// p == 0, exact mode: one launch.
int ffa_k_decode_onepass(int dtype, int head_dim, const FfaStepParams& P, int threads, int smem, cudaStream_t stream);
// how many clusters of `cluster` CTAs of the one-pass kernel the device keeps resident at once
int ffa_k_max_active_clusters(int dtype, int head_dim, int threads, int smem, int cluster, int* clusters);
// p > 0 or round-like-torch at any size: the streaming pruning kernel (scores through the scratch), one launch.
int ffa_k_decode_prune_stream(int dtype, int head_dim, const FfaStepParams& P, int scorer_warps, int smem, cudaStream_t stream);
int ffa_k_prune_stream_threads(int scorer_warps);
// shared-memory bytes a launch shape needs (tensors_per_stage 2: the exact kernel, K and V tiles; 1: the
// streaming pruning kernel, K tiles only)
int ffa_k_smem_bytes(int dtype, int head_dim, int tile_rows, int stages, int consumer_warps, int tensors_per_stage);
// p > 0 or round-like-torch, small steps whose slices' scores fit in shared memory: one cluster launch.
int ffa_k_decode_fused_prune(int dtype, int head_dim, const FfaStepParams& P, int smem, cudaStream_t stream);
int ffa_k_fused_smem_bytes(int dtype, int head_dim, int tile_rows, int stages, int chunk_rows, int cluster);
// diagnostic: a bounded wait that must time out (see ffa_selftest_wait_timeout)
int ffa_k_wait_selftest(int* status, unsigned long long limit_ns, unsigned long long* waited_ns, cudaStream_t stream);
// all-gather of the step outputs: a few CTAs per rank
int ffa_k_peer_gather(FfaPeerGatherParams G, cudaStream_t stream);
