// Shared helpers for the OMMX B200 kernels: error reporting, bf16 bit tricks, and the two
// table-driven decisions of the quantizer (power-of-two exponent, FP4 E2M1 encode).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>

#include "../../include/ommx_b200.h"
#include "ommx_tables.inc"

namespace ommx {

// ---- host-side error text (thread local) and launch counter --------------------------------
char *last_error_buf();
int fail(int code, const char *fmt, ...);
extern std::atomic<long long> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define OMMX_CUDA_TRY(expr)                                                              \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess)                                                           \
            return ::ommx::fail(OMMX_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// ---- quantizer decision tables --------------------------------------------------------------
// Host copies (used by the host twins in the C ABI) and device copies in constant memory.
static const uint32_t kPow2CutHost[256] = {OMMX_POW2_CUT_VALUES};
static const uint32_t kFp4ThreshHost[7] = {OMMX_FP4_THRESH_VALUES};

// round_half_even(log2(x)) for positive normal x: exponent + (mantissa >= cut[exponent]).
__host__ __device__ inline int pow2_exponent_tbl(float x, const uint32_t *cut) {
#ifdef __CUDA_ARCH__
    uint32_t b = __float_as_uint(x);
#else
    uint32_t b;
    memcpy(&b, &x, 4);
#endif
    uint32_t E = (b >> 23) & 0xFFu;
    return (int)E - 127 + ((b & 0x7FFFFFu) >= cut[E] ? 1 : 0);
}

// FP4 E2M1 code (sign<<3 | exp<<1 | mant): nearest level in log magnitude, ties to the lower.
__host__ __device__ inline int fp4_encode_tbl(float m, const uint32_t *th) {
#ifdef __CUDA_ARCH__
    uint32_t a = __float_as_uint(m) & 0x7FFFFFFFu;
#else
    uint32_t a;
    memcpy(&a, &m, 4);
    a &= 0x7FFFFFFFu;
#endif
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 7; ++i) idx += (a >= th[i]) ? 1 : 0;
    int sign = (m < 0.0f) ? 1 : 0;
    return (sign << 3) | idx;          // idx = exp * 2 + mant: the level's rank among the eight magnitudes is its code
}

// ---- device-side bf16 helpers -----------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }
// fp32 -> bf16 (round to nearest even) -> fp32, finite inputs
__device__ __forceinline__ float bf16_round_f32(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}
__device__ __forceinline__ void or_status(int32_t *status, int bits) {
    if (status != nullptr) atomicOr(status, bits);
}
#endif

}  // namespace ommx
