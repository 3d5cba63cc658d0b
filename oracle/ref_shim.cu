// TEST / BASELINE INFRASTRUCTURE ONLY -- not part of the shipped library.
//
// Gives C names to the reference's C++ entry points so the reference's own CUDA kernel,
// compiled unmodified from its checkout, can be driven through ctypes on a GPU box:
//   call_attention<float|uint16_t>              attention.cu:1512-1554
//   invokeTranspose4dBatchMajor<float|uint16_t> attention.cu:1649-1689
//   get_launch_params                           kernel_launch_utils.h:135-180
// The declarations below repeat the prototypes the reference's torch binding declares
// (torch_ffa_api.cpp:4-47); no reference code is contained in this file.
#include <cfloat>
#include <cstdint>
#include <cstdlib>
#include <sstream>  // kernel_launch_utils.h uses std::stringstream without including it
#include <cuda_runtime.h>
#include "kernel_launch_utils.h"

template<typename T>
void call_attention(int batch_size, int head_num, int size_per_head, int seq_length, float softmax_scale,
                    int curr_timestep, T* q, T* k, T* v, T* k_cache, T* v_cache, T* out, int* seq_lengths,
                    float prob_thresh, int tpv, int tpk, int tpb, bool right_or_no_padding);
template<> void call_attention<float>(int, int, int, int, float, int, float*, float*, float*, float*, float*, float*,
                                      int*, float, int, int, int, bool);
template<> void call_attention<uint16_t>(int, int, int, int, float, int, uint16_t*, uint16_t*, uint16_t*, uint16_t*,
                                         uint16_t*, uint16_t*, int*, float, int, int, int, bool);

template<typename T>
void invokeTranspose4dBatchMajor(T* k_dst, T* v_dst, const T* k_src, const T* v_src, const int local_batch_size,
                                 const int seq_len, const int max_seq_len, const int size_per_head,
                                 const int local_head_num);
template<> void invokeTranspose4dBatchMajor<float>(float*, float*, const float*, const float*, const int, const int,
                                                   const int, const int, const int);
template<> void invokeTranspose4dBatchMajor<uint16_t>(uint16_t*, uint16_t*, const uint16_t*, const uint16_t*,
                                                      const int, const int, const int, const int, const int);

extern "C" {

// elem_size: 4 = float, 2 = half-as-uint16_t.  Returns cudaGetLastError().
int ffa_ref_cache_init(int elem_size, void* k_dst, void* v_dst, const void* k_src, const void* v_src, int batch,
                       int seq_len, int max_seq_len, int head_dim, int heads)
{
    if (elem_size == 4)
        invokeTranspose4dBatchMajor<float>((float*)k_dst, (float*)v_dst, (const float*)k_src, (const float*)v_src,
                                           batch, seq_len, max_seq_len, head_dim, heads);
    else
        invokeTranspose4dBatchMajor<uint16_t>((uint16_t*)k_dst, (uint16_t*)v_dst, (const uint16_t*)k_src,
                                              (const uint16_t*)v_src, batch, seq_len, max_seq_len, head_dim, heads);
    return (int)cudaGetLastError();
}

void ffa_ref_launch_params(int precision, int batch, int heads, int head_dim, int prompt_len, int use_default_ft,
                           int* tpb, int* tpv, int* tpk)
{
    int b = 0, v = 0, k = 0;
    get_launch_params(precision, batch, heads, head_dim, prompt_len, b, v, k, use_default_ft != 0);
    *tpb = b; *tpv = v; *tpk = k;
}

int ffa_ref_attention(int elem_size, int batch, int heads, int head_dim, int max_seq_len, float softmax_scale,
                      int t, void* q, void* k, void* v, void* k_cache, void* v_cache, void* out, int* seq_lengths,
                      float prob_thresh, int tpv, int tpk, int tpb, int right_or_no_padding)
{
    if (elem_size == 4)
        call_attention<float>(batch, heads, head_dim, max_seq_len, softmax_scale, t, (float*)q, (float*)k, (float*)v,
                              (float*)k_cache, (float*)v_cache, (float*)out, seq_lengths, prob_thresh, tpv, tpk, tpb,
                              right_or_no_padding != 0);
    else
        call_attention<uint16_t>(batch, heads, head_dim, max_seq_len, softmax_scale, t, (uint16_t*)q, (uint16_t*)k,
                                 (uint16_t*)v, (uint16_t*)k_cache, (uint16_t*)v_cache, (uint16_t*)out, seq_lengths,
                                 prob_thresh, tpv, tpk, tpb, right_or_no_padding != 0);
    return (int)cudaGetLastError();
}

}  // extern "C"
