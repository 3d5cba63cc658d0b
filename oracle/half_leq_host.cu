// TEST INFRASTRUCTURE ONLY -- not part of the shipped library.
//
// Pins the fp16 comparison inside the reference's pruning rule.  The reference writes
//     inline __device__ bool leq(uint16_t a, uint16_t b) { return __hle(a, b); }
// (attention.cu:466-469): two raw fp16 bit patterns are passed to a function that takes
// __half, so each goes through the toolkit's numeric `__half(unsigned short)` constructor
// before the comparison.  This file evaluates that same expression with the CUDA toolkit's
// own HOST implementation of cuda_fp16.h, so the numpy restatement in ffa_oracle.py can be
// checked against it without a GPU.  Built with the reference's half-operator flags
// (setup.py:10).
#include <cuda_fp16.h>
#include <cstddef>
#include <cstdint>

extern "C" void ffa_ref_half_leq(const uint16_t* a, const uint16_t* b, uint8_t* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        uint16_t x = a[i], y = b[i];
        out[i] = __hle(x, y) ? 1 : 0;
    }
}

// The number the comparison sees for one bit pattern, returned as the bits of the __half.
extern "C" void ffa_ref_half_from_bits_numeric(const uint16_t* a, uint16_t* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        __half h = a[i];
        out[i] = __half_as_ushort(h);
    }
}
