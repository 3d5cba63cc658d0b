// ffa_attention_static_scratch: the exact (p = 0) decode step for callers that cannot hand
// the engine any scratch memory.
//
// The regular entry point needs a caller-allocated workspace (split partials, arrival
// counters, status word).  Some hosts have nowhere to get one from: an inference server that
// gave the whole GPU to its own pool allocator at start-up, so a cudaMalloc issued by a plug-in
// fails or is forbidden by policy; a latency-critical decode thread that must not take the
// device-wide synchronisation cudaMalloc/cudaFree imply; a bare C host of the kind
// c_ffa_api.h serves, which owns exactly the six tensors of the call and no allocator.  For
// them the scratch lives in the file-scope device array below, which every GPU that loads
// this library holds (4 MiB) until the process exits.
//
// Consequences of sharing one array:
//   * it keeps the previous call's contents, so every call first clears the part that must
//     start at zero (the arrival counters) on the caller's stream; the status word is NOT
//     cleared by a call -- error bits stay until ffa_static_scratch_status reads and clears them;
//   * two calls whose kernels overlap on the same GPU (different streams, or different host
//     threads) race on it -- keep calls on one GPU stream-ordered;
//   * sizes that do not fit are rejected, nothing is grown.
// The first call on each device does a one-time set-up (resolves the array's device address,
// queries the device, raises the kernels' shared-memory limit); make that first call outside
// any stream capture.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/ffa_c_api.h"
#include "ffa_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;  // the stated maximum: 4 MiB per GPU
// In host code this name is only a handle for the runtime, never a device address; the
// address the kernel gets comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_ffa_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_ffa_static_scratch on this device
    int sms = 0, smem_cta = 0, smem_sm = 0;
    unsigned prepared = 0;  // bit (dtype * 4 + head-dim index): kernel attributes raised
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

// writes the reason for a non-zero return into the caller's (host) buffer, if one was given
int report(char* buf, size_t len, int code, const char* fmt, ...)
{
    if (buf != nullptr && len > 0) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, len, fmt, ap);
        va_end(ap);
    }
    return code;
}

int head_dim_index(int d) { return d == 64 ? 0 : d == 80 ? 1 : d == 128 ? 2 : d == 256 ? 3 : -1; }
size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// One-time set-up for the current device: the array's device address and the device's limits.
// Returns 0 and fills *out, or a cudaError_t; *what names the call that failed.
int device_state(int* dev_out, DeviceState* out, const char** what)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    *what = "cudaGetDevice";
    if (e != cudaSuccess) return (int)e;
    *what = "device ordinal beyond the supported 64";
    if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState& d = g_dev[dev];
    if (!d.ready) {
        unsigned char* ptr = nullptr;
        *what = "cudaGetSymbolAddress(static scratch)";
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_ffa_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (ptr == nullptr) return (int)cudaErrorInvalidSymbol;
        *what = "device attribute query";
        e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.smem_cta, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
        if (e != cudaSuccess) return (int)e;
        d.scratch = ptr;
        d.ready = true;
    }
    *dev_out = dev, *out = d;
    return 0;
}

}  // namespace

// Reads the status word the static-scratch calls on the current device OR their FFA_STATUS_*
// bits into (calls made with device_status == NULL), then clears it: one 4-byte copy to the
// caller's host int and one 4-byte clear, both on `stream`, then a stream synchronisation.
// Allocates nothing.  Returns FFA_OK with *status == 0 when clean, FFA_ERR_DEVICE when a bit was set.
extern "C" int ffa_static_scratch_status(void* stream, int* status)
{
    if (status == nullptr) return FFA_ERR_ARG;
    int dev = 0;
    DeviceState st;
    const char* what = "";
    if (device_state(&dev, &st, &what) != 0) return FFA_ERR_CUDA;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(status, st.scratch, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(st.scratch, 0, sizeof(int), s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return FFA_ERR_CUDA;
    return *status != 0 ? FFA_ERR_DEVICE : FFA_OK;
}

// Diagnostic twin of ffa_selftest_wait_timeout for the static array: one warp waits, for at most
// limit_ms, on a copy barrier nothing completes, gives up, and ORs FFA_STATUS_WAIT_TIMEOUT into the
// static status word -- what a static-scratch decode step does when a bulk copy never lands.
// Nothing faults or hangs; the next ffa_static_scratch_status must report the bit.
extern "C" int ffa_static_scratch_selftest_wait_timeout(unsigned int limit_ms, void* stream)
{
    if (limit_ms == 0 || limit_ms > 2000) return FFA_ERR_RANGE;
    int dev = 0;
    DeviceState st;
    const char* what = "";
    if (device_state(&dev, &st, &what) != 0) return FFA_ERR_CUDA;
    const int r = ffa_k_wait_selftest(reinterpret_cast<int*>(st.scratch), (unsigned long long)limit_ms * 1000000ull, nullptr,
                                      static_cast<cudaStream_t>(stream));
    return r == 0 ? FFA_OK : FFA_ERR_CUDA;
}

extern "C" int ffa_attention_static_scratch(int dtype, int batch, int heads, int head_dim, int max_len, const void* q,
                                            const void* k, const void* v, void* k_cache, void* v_cache, void* out,
                                            float softmax_scale, int t, int* device_status, void* stream,
                                            char* error_text, size_t error_text_len)
{
    auto fail = [&](int code, const char* fmt, auto... a) { return report(error_text, error_text_len, code, fmt, a...); };
    if (error_text != nullptr && error_text_len > 0) error_text[0] = 0;
    if (dtype != FFA_DTYPE_F32 && dtype != FFA_DTYPE_F16 && dtype != FFA_DTYPE_BF16) return fail(FFA_ERR_DTYPE, "unsupported dtype code %d", dtype);
    const int dhi = head_dim_index(head_dim);
    if (dhi < 0) return fail(FFA_ERR_HEAD_DIM, "unsupported head_dim %d (64, 80, 128, 256)", head_dim);
    if (batch <= 0 || heads <= 0 || max_len <= 0 || t < 0 || t >= max_len)
        return fail(FFA_ERR_RANGE, "need positive batch, heads, max_len and 0 <= t (%d) < max_len (%d)", t, max_len);
    if (!q || !k || !v || !k_cache || !v_cache || !out) return fail(FFA_ERR_ARG, "null tensor pointer");
    for (const void* p : {q, k, v, (const void*)k_cache, (const void*)v_cache, (const void*)out})
        if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return fail(FFA_ERR_ARG, "tensor pointers must be 16-byte aligned");

    // ---- one-time set-up for the current device ----
    int dev = 0;
    DeviceState st;
    const char* what = "";
    int ce = device_state(&dev, &st, &what);
    if (ce != 0) return fail(FFA_ERR_CUDA, "%s: %s", what, cudaGetErrorString((cudaError_t)ce));
    {
        std::lock_guard<std::mutex> lock(g_mu);
        const unsigned bit = 1u << (dtype * 4 + dhi);
        if (!(g_dev[dev].prepared & bit)) {
            const int r = ffa_k_prepare(dtype, head_dim, st.smem_cta);
            if (r != 0) return fail(FFA_ERR_CUDA, "kernel preparation: %s", cudaGetErrorString((cudaError_t)r));
            g_dev[dev].prepared |= bit;
        }
    }
    cudaError_t e = cudaSuccess;

    // ---- launch shape: the engine's fixed rule (16 KB tiles, 4 compute warps, 2 CTAs/SM, 2 stages) ----
    const int es = dtype == FFA_DTYPE_F32 ? 4 : 2, rowb = head_dim * es;
    const long long BH = (long long)batch * heads;
    int tile_rows = ((rowb / 16) % 5 == 0 ? 20480 : 16384) / rowb, stages = 2, cps = 2;
    const int warps = 4;
    tile_rows = (tile_rows + 7) / 8 * 8;
    while (tile_rows > 8 && BH * (t / tile_rows + 1) < 4LL * st.sms * cps) tile_rows = (tile_rows / 2 + 7) / 8 * 8;
    int smem = 0;
    for (;;) {
        smem = ffa_k_smem_bytes(dtype, head_dim, tile_rows, stages, warps, 2);
        if (smem <= st.smem_cta && (long long)cps * (smem + 1024) <= st.smem_sm) break;
        if (stages > 2) --stages;
        else if (tile_rows > 8) tile_rows = (tile_rows / 2 + 7) / 8 * 8;
        else if (cps > 1) --cps;
        else return fail(FFA_ERR_ARG, "no launch shape fits in shared memory");
    }
    const int upb = t / tile_rows + 1;
    long long grid = (long long)st.sms * cps;
    if (grid > BH * upb) grid = BH * upb;

    // ---- carve the static array; reject what does not fit ----
    const size_t tickets_off = 256, partials_off = tickets_off + align_up((size_t)BH * sizeof(int), 256);
    const size_t need = partials_off + (size_t)(grid + BH) * (head_dim + 2) * sizeof(float);
    if (need > kStaticScratchBytes)
        return fail(FFA_ERR_RANGE,
                    "batch*heads = %lld with head_dim %d needs %zu bytes of scratch; the static scratch holds %zu "
                    "(use ffa_attention with a caller-allocated workspace)", BH, head_dim, need, kStaticScratchBytes);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array still holds the previous call's state: the arrival counters must start at zero (the
    // status word is left alone so that error bits survive until ffa_static_scratch_status reads them)
    e = cudaMemsetAsync(st.scratch + tickets_off, 0, partials_off - tickets_off, s);
    if (e != cudaSuccess) return fail(FFA_ERR_CUDA, "scratch clear: %s", cudaGetErrorString(e));

    FfaStepParams P;
    std::memset(&P, 0, sizeof(P));
    P.q = q, P.k = k, P.v = v, P.k_cache = k_cache, P.v_cache = v_cache, P.out = out;
    P.seq_lengths = nullptr, P.right_or_no_padding = 1;
    P.B = batch, P.H = heads, P.Lmax = max_len, P.t = t;
    P.tile_rows = tile_rows, P.stages = stages, P.units_per_bh = upb, P.parts_per_bh = upb, P.grid = (int)grid;
    P.scale = softmax_scale, P.p = 0.f;
    P.status = device_status != nullptr ? device_status : reinterpret_cast<int*>(st.scratch);
    P.tickets = reinterpret_cast<int*>(st.scratch + tickets_off);
    P.partials = reinterpret_cast<float*>(st.scratch + partials_off);
    const int r = ffa_k_decode_onepass(dtype, head_dim, P, 32 * (warps + 1), smem, s);
    if (r != 0) return fail(FFA_ERR_CUDA, "attention launch: %s", cudaGetErrorString((cudaError_t)r));
    return FFA_OK;
}
