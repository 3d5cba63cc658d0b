// Torch extension `ff_attention`: the FastForwardAttn class over the C ABI of libffa_b200.so.
//
// Mirrors the reference's pybind class (torch_ffa_api.cpp:161-214): same constructor
// (K, V, max_timesteps, use_default_kernel_launch), the same three attention overloads in
// the same argument order, get_cache().  Differences, all on purpose:
//   * bf16 is accepted next to fp32 and fp16 (torch_ffa_api.cpp:100-101 rejects it);
//   * arguments are validated and errors raise instead of printf + garbage (:101, :129);
//   * kernels run on torch's current stream under a device guard (the reference launches on
//     the legacy stream 0, attention.cu:1504);
//   * both caches are token-major [B, H, max_len, Dh] (the reference's K cache is
//     [B, H, Dh/x, max_len, x], torch_ffa_api.cpp:65);
//   * prob_thresh defaults to 0 in Python too.
// torch is used for memory, streams and the binding only; all arithmetic is in the library.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "ffa_c_api.h"

namespace {

int dtype_code(const torch::Tensor& x)
{
    switch (x.scalar_type()) {
        case torch::kFloat: return FFA_DTYPE_F32;
        case torch::kHalf: return FFA_DTYPE_F16;
        case torch::kBFloat16: return FFA_DTYPE_BF16;
        default: TORCH_CHECK(false, "FastForwardAttn: unsupported tensor type ", x.scalar_type(), " (float32, float16, bfloat16)");
    }
}

void check(int rc, const char* what) { TORCH_CHECK(rc == FFA_OK, "FastForwardAttn: ", what, ": ", ffa_last_error()); }

struct FastForwardAttn {
    FastForwardAttn(torch::Tensor K, torch::Tensor V, int64_t max_timesteps, bool use_default_kernel_launch)
    {
        TORCH_CHECK(K.is_cuda() && V.is_cuda(), "FastForwardAttn: K and V must be CUDA tensors");
        TORCH_CHECK(K.dim() == 4 && V.sizes() == K.sizes(), "FastForwardAttn: K and V must both be [batch, heads, prompt_len, head_dim]");
        TORCH_CHECK(K.scalar_type() == V.scalar_type() && K.device() == V.device(), "FastForwardAttn: K and V differ in dtype or device");
        K = K.contiguous(), V = V.contiguous();
        B = K.size(0), H = K.size(1), Dh = K.size(3);
        const int64_t Lp = K.size(2);
        Lmax = max_timesteps;
        TORCH_CHECK(Lmax >= Lp && Lmax > 0, "FastForwardAttn: max_timesteps (", Lmax, ") is smaller than the prompt (", Lp, ")");
        TORCH_CHECK(Lmax < (int64_t(1) << 31) && B * H < (int64_t(1) << 31), "FastForwardAttn: sizes exceed int range");
        dtype = dtype_code(K);
        c10::cuda::CUDAGuard guard(K.device());
        device = K.device();
        use_default = use_default_kernel_launch;
        check(ffa_plan_create(dtype, (int)B, (int)H, (int)Dh, (int)Lmax, use_default_kernel_launch, K.device().index(), &plan),
              "plan");
        k_cache = torch::empty({B, H, Lmax, Dh}, K.options());
        v_cache = torch::empty({B, H, Lmax, Dh}, K.options());
        auto stream = at::cuda::getCurrentCUDAStream();
        check(ffa_cache_init(dtype, (int)B, (int)H, (int)Lp, (int)Lmax, (int)Dh, K.data_ptr(), V.data_ptr(), k_cache.data_ptr(),
                             v_cache.data_ptr(), stream.stream()),
              "cache init");
        bind_workspace(false);
        // one-time: the caches and the cleared workspace are complete before the constructor
        // returns, so the first step may run on any stream
        stream.synchronize();
    }
    // Adopts caches the caller already filled (a prefill that writes K and V straight into
    // [batch, heads, max_len, head_dim] slabs needs no copy at all): rows [0, t) are whatever the
    // caller put there.  Replaces the copy in init_attention_cache (torch_ffa_api.cpp:68-77, 88-97).
    struct AdoptTag {};
    FastForwardAttn(AdoptTag, torch::Tensor kc, torch::Tensor vc, bool use_default_kernel_launch)
    {
        TORCH_CHECK(kc.is_cuda() && vc.is_cuda() && kc.dim() == 4 && vc.sizes() == kc.sizes() && kc.scalar_type() == vc.scalar_type() &&
                        kc.device() == vc.device() && kc.is_contiguous() && vc.is_contiguous(),
                    "FastForwardAttn.adopt: caches must be two contiguous CUDA tensors [batch, heads, max_len, head_dim] of one dtype");
        B = kc.size(0), H = kc.size(1), Lmax = kc.size(2), Dh = kc.size(3);
        TORCH_CHECK(Lmax > 0 && Lmax < (int64_t(1) << 31) && B * H < (int64_t(1) << 31), "FastForwardAttn.adopt: sizes out of range");
        dtype = dtype_code(kc);
        c10::cuda::CUDAGuard guard(kc.device());
        device = kc.device();
        use_default = use_default_kernel_launch;
        check(ffa_plan_create(dtype, (int)B, (int)H, (int)Dh, (int)Lmax, use_default, device.index(), &plan), "plan");
        k_cache = kc, v_cache = vc;
        bind_workspace(false);
        at::cuda::getCurrentCUDAStream().synchronize();
    }

    // Grows both caches to new_max_len rows (contents kept), re-plans and re-binds the workspace; mode,
    // pruning path, cluster merge and any launch override carry over.  Tensors handed out by
    // get_cache() before the call keep pointing at the old slabs, and a CUDA graph recorded before
    // it holds the old slabs' and workspace's addresses: record it again after growing.
    void grow(int64_t new_max_len)
    {
        TORCH_CHECK(new_max_len > Lmax && new_max_len < (int64_t(1) << 31), "FastForwardAttn.grow: new length ", new_max_len,
                    " must exceed the current ", Lmax);
        c10::cuda::CUDAGuard guard(device);
        auto stream = at::cuda::getCurrentCUDAStream();
        torch::Tensor nk = torch::empty({B, H, new_max_len, Dh}, k_cache.options());
        torch::Tensor nv = torch::empty({B, H, new_max_len, Dh}, k_cache.options());
        check(ffa_cache_copy(dtype, (int)B, (int)H, (int)Lmax, (int)Lmax, (int)new_max_len, (int)Dh, k_cache.data_ptr(),
                             v_cache.data_ptr(), nk.data_ptr(), nv.data_ptr(), stream.stream()),
              "cache copy");
        ffa_plan_t* np = nullptr;
        check(ffa_plan_create(dtype, (int)B, (int)H, (int)Dh, (int)new_max_len, use_default, device.index(), &np), "plan");
        check(ffa_plan_set_mode(np, mode), "mode");
        check(ffa_plan_set_prune_path(np, prune_path), "prune path");
        check(ffa_plan_set_cluster_merge(np, cluster_merge ? 1 : 0), "cluster merge");
        if (launch_forced) check(ffa_plan_set_launch(np, &forced_launch), "launch override");
        if (peer_world > 0) {
            std::vector<void*> bufs(peer_ptrs.begin(), peer_ptrs.end());
            check(ffa_peer_gather_attach(np, peer_world, peer_rank, bufs.data(), peer_bytes), "peer gather");
        }
        stream.synchronize();   // the old slabs may be freed once the copy is done
        ffa_plan_destroy(plan);
        plan = np, k_cache = nk, v_cache = nv, Lmax = new_max_len;
        kept_mask = torch::Tensor();   // one bit per row of the old length; re-created on the next recorded call
        push_tensor = torch::Tensor();
        bind_workspace(has_scores);
        stream.synchronize();
    }
    int64_t max_len() const { return Lmax; }

    ~FastForwardAttn()
    {
        peer_gather_free();   // the owner keeps the engine alive while any peer may still gather
        ffa_plan_destroy(plan);
    }
    FastForwardAttn(const FastForwardAttn&) = delete;
    FastForwardAttn& operator=(const FastForwardAttn&) = delete;

    void bind_workspace(bool with_scores)
    {
        const size_t n = ffa_workspace_bytes(plan, with_scores);
        workspace = torch::empty({(int64_t)n}, torch::TensorOptions().dtype(torch::kUInt8).device(device));
        check(ffa_workspace_bind(plan, workspace.data_ptr(), n, at::cuda::getCurrentCUDAStream().stream()), "workspace");
        has_scores = with_scores;
    }

    // memory the engine's kernels can address: its own device, or pinned (page-locked) host memory
    bool reachable(const torch::Tensor& x) const { return (x.is_cuda() && x.device() == device) || (x.is_cpu() && x.is_pinned()); }

    // gather_into: when given (heads sharded, peer_gather_attach done), the step also completes the all-gather of the
    // outputs and returns gather_into = [B, world*H, Dh].  Exact steps push their rows from the attention kernel's
    // epilogue (ffa_peer_push_target) and only the wait-and-collect kernel follows; pruned and torch-rounding steps are
    // followed by the whole gather kernel.
    torch::Tensor run(const torch::Tensor& q_, const torch::Tensor& k_, const torch::Tensor& v_, torch::Tensor& kc,
                      torch::Tensor& vc, double softmax_scale, int64_t t, const torch::Tensor* seq_lengths,
                      bool right_or_no_padding, double p, c10::optional<torch::Tensor> out_opt,
                      c10::optional<torch::Tensor> gather_into = c10::nullopt)
    {
        const int64_t n = B * H * Dh;
        // q, k, v (and out) may also live in pinned host memory: the kernel then reads (writes) them
        // in place over PCIe, which saves the staging copies of a host-driven decode loop
        auto prep = [&](const torch::Tensor& x, const char* name) {
            TORCH_CHECK(reachable(x), "FastForwardAttn: ", name, " is not on the engine's device (nor in pinned host memory)");
            TORCH_CHECK(dtype_code(x) == dtype, "FastForwardAttn: ", name, " has a different dtype than the cache");
            TORCH_CHECK(x.numel() == n, "FastForwardAttn: ", name, " must hold batch*heads*head_dim = ", n, " elements, got ", x.numel());
            TORCH_CHECK(x.is_cuda() || x.is_contiguous(), "FastForwardAttn: ", name, " in pinned host memory must be contiguous");
            return x.contiguous();
        };
        torch::Tensor q = prep(q_, "q"), k = prep(k_, "k"), v = prep(v_, "v");
        for (const torch::Tensor* c : {&kc, &vc}) {
            TORCH_CHECK(c->is_cuda() && c->device() == device && dtype_code(*c) == dtype && c->is_contiguous() &&
                            c->dim() == 4 && c->size(0) == B && c->size(1) == H && c->size(2) == Lmax && c->size(3) == Dh,
                        "FastForwardAttn: cache tensors must be the [batch, heads, max_len, head_dim] tensors returned by get_cache()");
        }
        TORCH_CHECK(t >= 0 && t < Lmax, "FastForwardAttn: curr_timestep ", t, " outside [0, ", Lmax, ")");
        TORCH_CHECK(p >= 0.0 && p <= 1.0, "FastForwardAttn: prob_thresh ", p, " outside [0, 1]");
        torch::Tensor sl;
        if (seq_lengths != nullptr) {
            TORCH_CHECK(seq_lengths->is_cuda() && seq_lengths->device() == device && seq_lengths->scalar_type() == torch::kInt &&
                            seq_lengths->numel() == B,
                        "FastForwardAttn: seq_lengths must be an int32 CUDA tensor with one entry per batch element");
            sl = seq_lengths->contiguous();
        }
        c10::cuda::CUDAGuard guard(device);
        torch::Tensor out;
        if (out_opt.has_value()) {
            out = *out_opt;
            TORCH_CHECK(reachable(out) && dtype_code(out) == dtype && out.is_contiguous() && out.numel() == n,
                        "FastForwardAttn: out must be a contiguous tensor of batch*heads*head_dim elements on the engine's device "
                        "(or in pinned host memory)");
        } else {
            out = torch::empty({B, H, Dh}, kc.options());
        }
        uint32_t* mask_ptr = nullptr;
        if (want_mask && p > 0.0) {
            if (!kept_mask.defined()) kept_mask = torch::zeros({B, H, (Lmax + 31) / 32}, torch::TensorOptions().dtype(torch::kInt).device(device));
            mask_ptr = reinterpret_cast<uint32_t*>(kept_mask.data_ptr());
        }
        // large pruned steps go through an fp32 score scratch (4 bytes per cache row, under 1 % of the caches): bound
        // the first time a pruned step is asked for.  (Torch-rounding steps keep their scores in shared memory; the
        // retry below binds the scratch for the rare shape that does not fit there.)
        if (p > 0.0 && !has_scores) bind_workspace(true);
        auto call = [&]() {
            return ffa_attention(plan, q.data_ptr(), k.data_ptr(), v.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                 (float)softmax_scale, (int)t, seq_lengths ? sl.data_ptr<int>() : nullptr, right_or_no_padding,
                                 (float)p, mask_ptr, at::cuda::getCurrentCUDAStream().stream());
        };
        bool pushed = false;
        if (gather_into.has_value()) {
            TORCH_CHECK(peer_world > 0, "FastForwardAttn: gather_into needs peer_gather_attach first");
            TORCH_CHECK(reachable(*gather_into) && dtype_code(*gather_into) == dtype && gather_into->is_contiguous() &&
                            gather_into->numel() == (int64_t)peer_world * n,
                        "FastForwardAttn: gather_into must be a contiguous [batch, world*heads, head_dim] tensor of the cache's dtype on the "
                        "engine's device (or in pinned host memory)");
            if (peer_world > 1 && !(p > 0.0) && mode == FFA_MODE_EXACT && !push_tensor.defined()) {
                check(ffa_peer_push_target(plan, gather_into->data_ptr()), "push target");
                pushed = true;
            }
        }
        int rc = call();
        if (rc == FFA_ERR_WORKSPACE && !has_scores) {
            // a shape the fused pruning kernel cannot hold: grow the workspace by the score scratch, once
            bind_workspace(true);
            rc = call();
        }
        if (pushed) ffa_peer_push_target(plan, nullptr);
        check(rc, "attention");
        if (gather_into.has_value()) {
            check(ffa_peer_gather(plan, out.data_ptr(), gather_into->data_ptr(), pushed ? 2 : 3, 2000,
                                  at::cuda::getCurrentCUDAStream().stream()),
                  "peer gather");
            return *gather_into;
        }
        return out;
    }

    // Low-level switch of the fused push (the gather_into keyword does this per call): while set, every exact step pushes
    // its rows into `gathered` and the peers' staging buffers; the caller then issues peer_gather(..., phases=2).
    void set_push_target(c10::optional<torch::Tensor> gathered)
    {
        if (!gathered.has_value()) {
            check(ffa_peer_push_target(plan, nullptr), "push target");
            push_tensor = torch::Tensor();
            return;
        }
        TORCH_CHECK(peer_world > 0, "FastForwardAttn: peer_gather_attach first");
        TORCH_CHECK(reachable(*gathered) && dtype_code(*gathered) == dtype && gathered->is_contiguous() &&
                        gathered->numel() == (int64_t)peer_world * B * H * Dh,
                    "FastForwardAttn: the push target must be a contiguous [batch, world*heads, head_dim] tensor of the cache's dtype");
        check(ffa_peer_push_target(plan, gathered->data_ptr()), "push target");
        push_tensor = *gathered;
    }

    // torch_ffa_api.cpp:189-192
    torch::Tensor attention(torch::Tensor q, torch::Tensor k, torch::Tensor v, double softmax_scale, int64_t curr_timestep,
                            double prob_thresh, c10::optional<torch::Tensor> out, c10::optional<torch::Tensor> gather_into)
    {
        return run(q, k, v, k_cache, v_cache, softmax_scale, curr_timestep, nullptr, true, prob_thresh, out, gather_into);
    }
    // torch_ffa_api.cpp:179-182
    torch::Tensor attention_cache(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kc, torch::Tensor vc,
                                  double softmax_scale, int64_t curr_timestep, double prob_thresh, c10::optional<torch::Tensor> out)
    {
        return run(q, k, v, kc, vc, softmax_scale, curr_timestep, nullptr, true, prob_thresh, out);
    }
    // torch_ffa_api.cpp:184-187: left padding, keys below seq_lengths[b] are masked
    torch::Tensor attention_varlen(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor kc, torch::Tensor vc,
                                   double softmax_scale, int64_t curr_timestep, torch::Tensor seq_lengths, double prob_thresh,
                                   c10::optional<torch::Tensor> out)
    {
        return run(q, k, v, kc, vc, softmax_scale, curr_timestep, &seq_lengths, false, prob_thresh, out);
    }
    // c_ffa_api.h:17-20 semantics (per-sample lengths, right padding); not exported by the
    // reference's Python class, exported here so the mode is reachable from Python
    // max_row: what the host knows about the lengths (every seq_lengths[b] <= max_row); the work is
    // laid out for rows 0..max_row.  -1 = nothing known = max_len - 1.
    torch::Tensor attention_per_sample(torch::Tensor q, torch::Tensor k, torch::Tensor v, double softmax_scale,
                                       torch::Tensor seq_lengths, double prob_thresh, c10::optional<torch::Tensor> out,
                                       int64_t max_row, c10::optional<torch::Tensor> gather_into)
    {
        TORCH_CHECK(max_row >= -1 && max_row < Lmax, "FastForwardAttn: max_row ", max_row, " outside [-1, ", Lmax, ")");
        return run(q, k, v, k_cache, v_cache, softmax_scale, max_row < 0 ? Lmax - 1 : max_row, &seq_lengths, true, prob_thresh, out,
                   gather_into);
    }

    std::pair<torch::Tensor, torch::Tensor> get_cache() { return std::make_pair(k_cache, v_cache); }

    void set_mode(const std::string& m)
    {
        TORCH_CHECK(m == "exact" || m == "round_like_torch", "FastForwardAttn: mode must be 'exact' or 'round_like_torch'");
        mode = m == "exact" ? FFA_MODE_EXACT : FFA_MODE_ROUND_LIKE_TORCH;
        check(ffa_plan_set_mode(plan, mode), "mode");
    }
    void set_prune_path(int path)
    {
        check(ffa_plan_set_prune_path(plan, path), "prune path");
        prune_path = path;
    }
    void set_cluster_merge(bool on)
    {
        check(ffa_plan_set_cluster_merge(plan, on ? 1 : 0), "cluster merge");
        cluster_merge = on;
    }
    void set_launch(int tile_rows, int stages, int consumer_warps, int ctas_per_sm, int grid)
    {
        ffa_launch_t l{tile_rows, stages, consumer_warps, ctas_per_sm, grid, 0, 0};
        const bool any = tile_rows > 0 || stages > 0 || consumer_warps > 0 || ctas_per_sm > 0 || grid > 0;
        check(ffa_plan_set_launch(plan, any ? &l : nullptr), "launch override");
        launch_forced = any, forced_launch = l;
    }
    py::dict launch_shape(int64_t t)
    {
        c10::cuda::CUDAGuard guard(device);   // the planner may ask this device about cluster occupancy
        ffa_launch_t l;
        check(ffa_plan_get_launch(plan, (int)t, &l), "launch shape");
        py::dict d;
        d["tile_rows"] = l.tile_rows, d["stages"] = l.stages, d["consumer_warps"] = l.consumer_warps;
        d["ctas_per_sm"] = l.ctas_per_sm, d["grid"] = l.grid, d["smem_bytes"] = l.smem_bytes, d["parts_per_bh"] = l.parts_per_bh;
        return d;
    }
    void record_kept_mask(bool on) { want_mask = on; }
    torch::Tensor get_kept_mask()
    {
        TORCH_CHECK(kept_mask.defined(), "FastForwardAttn: no kept mask recorded (record_kept_mask(True), then a call with prob_thresh > 0)");
        return kept_mask;
    }
    int device_status()
    {
        c10::cuda::CUDAGuard guard(device);
        int s = 0;
        const int rc = ffa_device_status(plan, at::cuda::getCurrentCUDAStream().stream(), &s);
        TORCH_CHECK(rc == FFA_OK || rc == FFA_ERR_DEVICE, "FastForwardAttn: status: ", ffa_last_error());
        return s;
    }

    // ---- all-gather of the outputs over peer memory (ffa_peer_gather_* of the C ABI) ----
    // Allocates this rank's buffer; the returned 64-byte handle is what the other ranks open.
    py::bytes peer_gather_alloc(int64_t world)
    {
        TORCH_CHECK(peer_own == nullptr, "FastForwardAttn: the peer buffer is already allocated");
        c10::cuda::CUDAGuard guard(device);
        const size_t n = ffa_peer_gather_bytes(plan, (int)world);
        TORCH_CHECK(n > 0, "FastForwardAttn: world ", world, " outside [1, ", FFA_MAX_PEERS, "]");
        unsigned char handle[FFA_PEER_HANDLE_BYTES];
        check(ffa_peer_mem_alloc(n, &peer_own, handle), "peer buffer");
        peer_bytes = n;
        return py::bytes(reinterpret_cast<const char*>(handle), sizeof(handle));
    }
    int64_t peer_gather_ptr() const { return (int64_t)reinterpret_cast<uintptr_t>(peer_own); }
    int64_t peer_mem_open(const std::string& handle)
    {
        TORCH_CHECK(handle.size() == FFA_PEER_HANDLE_BYTES, "FastForwardAttn: a peer handle has ", FFA_PEER_HANDLE_BYTES, " bytes");
        c10::cuda::CUDAGuard guard(device);
        void* p = nullptr;
        check(ffa_peer_mem_open(reinterpret_cast<const unsigned char*>(handle.data()), &p), "peer buffer");
        return (int64_t)reinterpret_cast<uintptr_t>(p);
    }
    void peer_mem_close(int64_t ptr)
    {
        c10::cuda::CUDAGuard guard(device);
        check(ffa_peer_mem_close(reinterpret_cast<void*>((uintptr_t)ptr)), "peer buffer");
    }
    // ptrs: every rank's buffer in rank order (ptrs[rank] is this rank's own); close_on_free: the
    // other ranks' pointers came from peer_mem_open and are closed by peer_gather_free
    void peer_gather_attach(int64_t world, int64_t rank, std::vector<int64_t> ptrs, bool close_on_free)
    {
        TORCH_CHECK(peer_own != nullptr, "FastForwardAttn: peer_gather_alloc first");
        TORCH_CHECK((int64_t)ptrs.size() == world && rank >= 0 && rank < world, "FastForwardAttn: need one buffer pointer per rank");
        TORCH_CHECK(ptrs[rank] == peer_gather_ptr(), "FastForwardAttn: ptrs[rank] must be this rank's own buffer");
        std::vector<void*> bufs;
        for (int64_t x : ptrs) bufs.push_back(reinterpret_cast<void*>((uintptr_t)x));
        check(ffa_peer_gather_attach(plan, (int)world, (int)rank, bufs.data(), peer_bytes), "peer gather");
        peer_ptrs = bufs, peer_world = (int)world, peer_rank = (int)rank, peer_close = close_on_free;
    }
    // out_local [B, H, Dh] -> [B, world*H, Dh] holding every rank's outputs (a fresh tensor, or
    // `out`).  Every launch argument is the same for every step, so the call can be recorded in a
    // CUDA graph when `out` is given.
    torch::Tensor peer_gather(const torch::Tensor& out_local, int64_t phases, int64_t wait_limit_ms, c10::optional<torch::Tensor> out_opt)
    {
        TORCH_CHECK(peer_world > 0, "FastForwardAttn: peer_gather_attach first");
        TORCH_CHECK(out_local.is_cuda() && out_local.device() == device && dtype_code(out_local) == dtype && out_local.is_contiguous() &&
                        out_local.numel() == B * H * Dh,
                    "FastForwardAttn: out_local must be a contiguous [batch, heads, head_dim] tensor of the cache's dtype and device");
        c10::cuda::CUDAGuard guard(device);
        torch::Tensor out = out_opt.has_value() ? *out_opt : torch::empty({B, (int64_t)peer_world * H, Dh}, out_local.options());
        TORCH_CHECK(reachable(out) && dtype_code(out) == dtype && out.is_contiguous() && out.numel() == (int64_t)peer_world * B * H * Dh,
                    "FastForwardAttn: out must be a contiguous [batch, world*heads, head_dim] tensor of the cache's dtype on the engine's "
                    "device (or in pinned host memory)");
        check(ffa_peer_gather(plan, out_local.data_ptr(), out.data_ptr(), (int)phases, (unsigned)wait_limit_ms,
                              at::cuda::getCurrentCUDAStream().stream()),
              "peer gather");
        return out;
    }
    // Teardown is collective and has two steps with a host barrier before each: (1) every rank has
    // synchronised its device, so no store is in flight -> peer_gather_detach unmaps the peers'
    // buffers; (2) every rank has unmapped -> peer_gather_free releases this rank's own buffer (an
    // exported allocation must outlive every mapping of it).
    void peer_gather_detach()
    {
        if (peer_world == 0) return;
        c10::cuda::CUDAGuard guard(device);
        ffa_peer_gather_attach(plan, 0, 0, nullptr, 0);
        if (peer_close)
            for (int r = 0; r < peer_world; ++r)
                if (r != peer_rank) ffa_peer_mem_close(peer_ptrs[r]);
        peer_world = 0, peer_ptrs.clear();
    }
    void peer_gather_free()
    {
        peer_gather_detach();
        if (peer_own == nullptr) return;
        c10::cuda::CUDAGuard guard(device);
        ffa_peer_mem_free(peer_own);
        peer_own = nullptr;
    }

    ffa_plan_t* plan = nullptr;
    torch::Tensor k_cache, v_cache, workspace, kept_mask, push_tensor;
    c10::Device device{c10::kCUDA, 0};
    int64_t B = 0, H = 0, Dh = 0, Lmax = 0;
    int dtype = 0, mode = FFA_MODE_EXACT, prune_path = 0;
    bool has_scores = false, want_mask = false, use_default = false, cluster_merge = true, launch_forced = false;
    ffa_launch_t forced_launch{};
    void* peer_own = nullptr;
    std::vector<void*> peer_ptrs;
    size_t peer_bytes = 0;
    int peer_world = 0, peer_rank = 0;
    bool peer_close = false;
};

// Decode steps over PAGED caches (exact or pruned): the K and V pools are
// [pages, heads, page_rows, head_dim]; a page table [batch, max_pages] maps every page_rows rows of a
// sequence to a pool page.  The pools and the table belong to the caller (see paged.py for an
// allocator); this class holds the plan and the workspace.  The reference has nothing like it:
// its caches are max_len rows per sequence, allocated up front (torch_ffa_api.cpp:65-66).
struct PagedEngine {
    PagedEngine(torch::Tensor k_pool, torch::Tensor v_pool, int64_t batch, int64_t max_pages, bool use_default_kernel_launch)
    {
        TORCH_CHECK(k_pool.is_cuda() && v_pool.is_cuda() && k_pool.dim() == 4 && v_pool.sizes() == k_pool.sizes() &&
                        k_pool.scalar_type() == v_pool.scalar_type() && k_pool.device() == v_pool.device() &&
                        k_pool.is_contiguous() && v_pool.is_contiguous(),
                    "PagedEngine: pools must be two contiguous CUDA tensors [pages, heads, page_rows, head_dim] of one dtype");
        kp = k_pool, vp = v_pool;
        B = batch, H = k_pool.size(1), page_rows = k_pool.size(2), Dh = k_pool.size(3), this->max_pages = max_pages;
        TORCH_CHECK(B > 0 && max_pages > 0 && max_pages * page_rows < (int64_t(1) << 31), "PagedEngine: sizes out of range");
        dtype = dtype_code(k_pool);
        device = k_pool.device();
        c10::cuda::CUDAGuard guard(device);
        check(ffa_plan_create(dtype, (int)B, (int)H, (int)Dh, (int)(max_pages * page_rows), use_default_kernel_launch, device.index(), &plan),
              "plan");
        bind_workspace(false);
        at::cuda::getCurrentCUDAStream().synchronize();
    }
    ~PagedEngine() { ffa_plan_destroy(plan); }
    void bind_workspace(bool with_scores)
    {
        const size_t n = ffa_workspace_bytes(plan, with_scores);
        workspace = torch::empty({(int64_t)n}, torch::TensorOptions().dtype(torch::kUInt8).device(device));
        check(ffa_workspace_bind(plan, workspace.data_ptr(), n, at::cuda::getCurrentCUDAStream().stream()), "workspace");
        has_scores = with_scores;
    }
    PagedEngine(const PagedEngine&) = delete;
    PagedEngine& operator=(const PagedEngine&) = delete;

    torch::Tensor run(const torch::Tensor& q_, const torch::Tensor& k_, const torch::Tensor& v_, const torch::Tensor& table,
                      double softmax_scale, int64_t t, const torch::Tensor* rows, double p, c10::optional<torch::Tensor> out_opt)
    {
        const int64_t n = B * H * Dh;
        TORCH_CHECK(p >= 0.0 && p <= 1.0, "PagedEngine: prob_thresh ", p, " outside [0, 1]");
        auto prep = [&](const torch::Tensor& x, const char* name) {
            TORCH_CHECK(x.is_cuda() && x.device() == device && dtype_code(x) == dtype && x.numel() == n, "PagedEngine: ", name,
                        " must hold batch*heads*head_dim = ", n, " elements of the pool's dtype on the pool's device");
            return x.contiguous();
        };
        torch::Tensor q = prep(q_, "q"), k = prep(k_, "k"), v = prep(v_, "v");
        TORCH_CHECK(table.is_cuda() && table.device() == device && table.scalar_type() == torch::kInt && table.is_contiguous() &&
                        table.dim() == 2 && table.size(0) == B && table.size(1) == max_pages,
                    "PagedEngine: page_table must be a contiguous int32 CUDA tensor [batch, max_pages]");
        torch::Tensor sl;
        if (rows != nullptr) {
            TORCH_CHECK(rows->is_cuda() && rows->device() == device && rows->scalar_type() == torch::kInt && rows->numel() == B,
                        "PagedEngine: rows must be an int32 CUDA tensor with one entry per sequence");
            sl = rows->contiguous();
        }
        TORCH_CHECK(t >= 0 && t < max_pages * page_rows, "PagedEngine: curr_timestep ", t, " outside [0, ", max_pages * page_rows, ")");
        c10::cuda::CUDAGuard guard(device);
        torch::Tensor out = out_opt.has_value() ? *out_opt : torch::empty({B, H, Dh}, q.options());
        TORCH_CHECK(out.is_cuda() && out.device() == device && dtype_code(out) == dtype && out.is_contiguous() && out.numel() == n,
                    "PagedEngine: out must be a contiguous tensor of batch*heads*head_dim elements on the pool's device");
        uint32_t* mask_ptr = nullptr;
        if (want_mask && p > 0.0) {
            if (!kept_mask.defined())
                kept_mask = torch::zeros({B, H, (max_pages * page_rows + 31) / 32}, torch::TensorOptions().dtype(torch::kInt).device(device));
            mask_ptr = reinterpret_cast<uint32_t*>(kept_mask.data_ptr());
        }
        if (p > 0.0 && !has_scores) bind_workspace(true);   // torch-rounding steps keep their scores in shared memory
        auto call = [&]() {
            return ffa_attention_paged(plan, q.data_ptr(), k.data_ptr(), v.data_ptr(), kp.data_ptr(), vp.data_ptr(),
                                       table.data_ptr<int>(), (int)max_pages, (int)page_rows, out.data_ptr(), (float)softmax_scale,
                                       (int)t, rows ? sl.data_ptr<int>() : nullptr, 1, (float)p, mask_ptr,
                                       at::cuda::getCurrentCUDAStream().stream());
        };
        int rc = call();
        if (rc == FFA_ERR_WORKSPACE && !has_scores) {
            // a shape the fused pruning kernel cannot hold: grow the workspace by the score scratch, once
            bind_workspace(true);
            rc = call();
        }
        check(rc, "paged attention");
        return out;
    }
    torch::Tensor attention(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor table, double scale, int64_t t,
                            double prob_thresh, c10::optional<torch::Tensor> out)
    {
        return run(q, k, v, table, scale, t, nullptr, prob_thresh, out);
    }
    // max_row: the host's upper bound on rows[b] (-1: nothing known = the last row of the last page)
    torch::Tensor attention_per_sample(torch::Tensor q, torch::Tensor k, torch::Tensor v, torch::Tensor table, double scale,
                                       torch::Tensor rows, double prob_thresh, c10::optional<torch::Tensor> out, int64_t max_row)
    {
        TORCH_CHECK(max_row >= -1 && max_row < max_pages * page_rows, "PagedEngine: max_row ", max_row, " outside [-1, ",
                    max_pages * page_rows, ")");
        return run(q, k, v, table, scale, max_row < 0 ? max_pages * page_rows - 1 : max_row, &rows, prob_thresh, out);
    }
    void set_mode(const std::string& m)
    {
        TORCH_CHECK(m == "exact" || m == "round_like_torch", "PagedEngine: mode must be 'exact' or 'round_like_torch'");
        mode = m == "exact" ? FFA_MODE_EXACT : FFA_MODE_ROUND_LIKE_TORCH;
        check(ffa_plan_set_mode(plan, mode), "mode");
    }
    void set_prune_path(int path) { check(ffa_plan_set_prune_path(plan, path), "prune path"); }
    void record_kept_mask(bool on) { want_mask = on; }
    torch::Tensor get_kept_mask()
    {
        TORCH_CHECK(kept_mask.defined(), "PagedEngine: no kept mask recorded (record_kept_mask(True), then a call with prob_thresh > 0)");
        return kept_mask;
    }
    int device_status()
    {
        c10::cuda::CUDAGuard guard(device);
        int st = 0;
        const int rc = ffa_device_status(plan, at::cuda::getCurrentCUDAStream().stream(), &st);
        TORCH_CHECK(rc == FFA_OK || rc == FFA_ERR_DEVICE, "PagedEngine: status: ", ffa_last_error());
        return st;
    }

    ffa_plan_t* plan = nullptr;
    torch::Tensor kp, vp, workspace, kept_mask;
    c10::Device device{c10::kCUDA, 0};
    int64_t B = 0, H = 0, Dh = 0, page_rows = 0, max_pages = 0;
    int dtype = 0, mode = FFA_MODE_EXACT;
    bool has_scores = false, want_mask = false;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.doc() = "B200 decode masked multi-head attention behind the FastForwardAttention interface";
    m.def("launch_count", []() { return ffa_launch_count(); }, "kernels launched by the engine since load");
    py::class_<FastForwardAttn>(m, "FastForwardAttn")
        .def(py::init<torch::Tensor, torch::Tensor, int64_t, bool>(), py::arg("K"), py::arg("V"), py::arg("max_timesteps"),
             py::arg("use_default_kernel_launch") = false)
        .def_static("adopt", [](torch::Tensor kc, torch::Tensor vc, bool use_default_kernel_launch) {
                        return std::make_unique<FastForwardAttn>(FastForwardAttn::AdoptTag{}, kc, vc, use_default_kernel_launch);
                    }, py::arg("k_cache"), py::arg("v_cache"), py::arg("use_default_kernel_launch") = false,
                    "engine over caches [batch, heads, max_len, head_dim] the caller has already filled (no copy)")
        .def("grow", &FastForwardAttn::grow, py::arg("new_max_len"), "reallocate both caches to a longer max_len, contents kept")
        .def_property_readonly("max_len", &FastForwardAttn::max_len)
        .def("get_cache", &FastForwardAttn::get_cache, "the live (k_cache, v_cache) tensors, [batch, heads, max_len, head_dim]")
        .def("attention", &FastForwardAttn::attention, "decode step on the engine's own caches", py::arg("q"), py::arg("k"),
             py::arg("v"), py::arg("softmax_scale"), py::arg("curr_timestep"), py::arg("prob_thresh") = 0.0,
             py::arg("out") = py::none(), py::arg("gather_into") = py::none())
        .def("attention", &FastForwardAttn::attention_cache, "decode step on caches passed back by the caller", py::arg("q"),
             py::arg("k"), py::arg("v"), py::arg("k_cache"), py::arg("v_cache"), py::arg("softmax_scale"),
             py::arg("curr_timestep"), py::arg("prob_thresh") = 0.0, py::arg("out") = py::none())
        .def("attention", &FastForwardAttn::attention_varlen, "decode step with left padding: keys below seq_lengths[b] are masked",
             py::arg("q"), py::arg("k"), py::arg("v"), py::arg("k_cache"), py::arg("v_cache"), py::arg("softmax_scale"),
             py::arg("curr_timestep"), py::arg("seq_lengths"), py::arg("prob_thresh") = 0.0, py::arg("out") = py::none())
        .def("attention_per_sample", &FastForwardAttn::attention_per_sample,
             "decode step with per-sample cache lengths (right padding): sample b appends at row seq_lengths[b]", py::arg("q"),
             py::arg("k"), py::arg("v"), py::arg("softmax_scale"), py::arg("seq_lengths"), py::arg("prob_thresh") = 0.0,
             py::arg("out") = py::none(), py::arg("max_row") = -1, py::arg("gather_into") = py::none())
        .def("set_push_target", &FastForwardAttn::set_push_target, py::arg("gathered") = py::none(),
             "while set, exact steps push their output rows to the peers from the attention kernel (follow with peer_gather(phases=2))")
        .def("set_mode", &FastForwardAttn::set_mode, "'exact' (default) or 'round_like_torch'")
        .def("set_prune_path", &FastForwardAttn::set_prune_path, "0 choose, 1 cluster kernel, 2 streaming kernel")
        .def("set_cluster_merge", &FastForwardAttn::set_cluster_merge, "merge split pairs inside a thread-block cluster (default on)")
        .def("set_launch", &FastForwardAttn::set_launch, py::arg("tile_rows") = 0, py::arg("stages") = 0,
             py::arg("consumer_warps") = 0, py::arg("ctas_per_sm") = 0, py::arg("grid") = 0)
        .def("launch_shape", &FastForwardAttn::launch_shape, py::arg("t"))
        .def("record_kept_mask", &FastForwardAttn::record_kept_mask)
        .def("get_kept_mask", &FastForwardAttn::get_kept_mask)
        .def("device_status", &FastForwardAttn::device_status, "synchronises; 0 when the kernels recorded no error")
        .def("peer_gather_alloc", &FastForwardAttn::peer_gather_alloc, py::arg("world"))
        .def("peer_gather_ptr", &FastForwardAttn::peer_gather_ptr)
        .def("peer_mem_open", &FastForwardAttn::peer_mem_open, py::arg("handle"))
        .def("peer_mem_close", &FastForwardAttn::peer_mem_close, py::arg("ptr"))
        .def("peer_gather_attach", &FastForwardAttn::peer_gather_attach, py::arg("world"), py::arg("rank"), py::arg("ptrs"),
             py::arg("close_on_free") = true)
        .def("peer_gather", &FastForwardAttn::peer_gather, py::arg("out_local"), py::arg("phases") = 3, py::arg("wait_limit_ms") = 2000,
             py::arg("out") = py::none(), "all-gather of the outputs over peer memory: [B, H, Dh] -> [B, world*H, Dh]")
        .def("peer_gather_detach", &FastForwardAttn::peer_gather_detach, "unmap the peers' buffers (teardown step 1)")
        .def("peer_gather_free", &FastForwardAttn::peer_gather_free, "release this rank's buffer (teardown step 2)");
    py::class_<PagedEngine>(m, "PagedEngine")
        .def(py::init<torch::Tensor, torch::Tensor, int64_t, int64_t, bool>(), py::arg("k_pool"), py::arg("v_pool"), py::arg("batch"),
             py::arg("max_pages"), py::arg("use_default_kernel_launch") = false)
        .def("attention", &PagedEngine::attention, "decode step, every sequence at row curr_timestep", py::arg("q"), py::arg("k"),
             py::arg("v"), py::arg("page_table"), py::arg("softmax_scale"), py::arg("curr_timestep"), py::arg("prob_thresh") = 0.0,
             py::arg("out") = py::none())
        .def("attention_per_sample", &PagedEngine::attention_per_sample, "decode step, sequence b at row rows[b]", py::arg("q"),
             py::arg("k"), py::arg("v"), py::arg("page_table"), py::arg("softmax_scale"), py::arg("rows"),
             py::arg("prob_thresh") = 0.0, py::arg("out") = py::none(), py::arg("max_row") = -1)
        .def("set_mode", &PagedEngine::set_mode, "'exact' (default) or 'round_like_torch'")
        .def("set_prune_path", &PagedEngine::set_prune_path, "0 choose, 1 cluster kernel, 2 streaming kernel")
        .def("record_kept_mask", &PagedEngine::record_kept_mask)
        .def("get_kept_mask", &PagedEngine::get_kept_mask)
        .def("device_status", &PagedEngine::device_status);
}
