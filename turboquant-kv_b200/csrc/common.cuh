// common.cuh -- shared helpers of libtqb200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <algorithm>

#include "../../include/tqb200.h"

namespace tqb {

// ---- error reporting ---------------------------------------------------------------------
char* last_error_buffer();              // thread-local, 512 bytes
extern std::atomic<int64_t> g_launches; // kernels launched by this library

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(last_error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// Checks the launch itself (configuration errors); execution errors surface at the caller's
// next synchronisation, as with any stream-ordered API.
inline int check_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TQB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return TQB_OK;
}

#define TQB_REQUIRE(cond, ...)                                  \
    do {                                                        \
        if (!(cond)) return ::tqb::fail(TQB_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define TQB_CUDA(call)                                                                          \
    do {                                                                                        \
        cudaError_t e__ = (call);                                                               \
        if (e__ != cudaSuccess)                                                                 \
            return ::tqb::fail(TQB_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__));         \
    } while (0)

inline int bytes_per_plane(int dim) { return (dim + 7) / 8; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// SM count of the current device (cached per device id).
int sm_count();

// ---- device helpers ------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// A 32-lane ballot holds dimension l at bit l.  The packed layout wants dimension 8m+t at bit
// 7-t of byte m (little-endian word): reverse all 32 bits, then swap the four bytes back.
__device__ __forceinline__ uint32_t ballot_to_plane_word(uint32_t ballot) {
    return __byte_perm(__brev(ballot), 0u, 0x0123);
}

// Row mapping of tqb_rowmap evaluated on the device.  Returns -1 for a skipped row.
struct RowMap {
    int64_t inner, stride_a, stride_b, offset, pos_div;
    const int32_t* pos;
    const int64_t* slots;
    int32_t block_size;
    __device__ __forceinline__ int64_t operator()(int64_t r) const {
        const int64_t a = r / inner, b = r - a * inner;
        if (slots) {
            const int64_t s = slots[a];
            if (s < 0) return -1;
            return ((s / block_size) * inner + b) * block_size + s % block_size;
        }
        int64_t o = a * stride_a + b * stride_b + offset;
        if (pos) o += pos[a / pos_div];
        return o;
    }
};

inline RowMap make_rowmap(const tqb_rowmap* m) {
    RowMap r;
    if (m) {
        r.inner = m->inner > 0 ? m->inner : 1;
        r.stride_a = m->stride_a; r.stride_b = m->stride_b; r.offset = m->offset;
        r.pos = m->pos; r.pos_div = m->pos_div > 0 ? m->pos_div : 1;
        r.slots = m->slots; r.block_size = m->block_size > 0 ? m->block_size : 1;
    } else {
        r.inner = 1; r.stride_a = 1; r.stride_b = 0; r.offset = 0;
        r.pos = nullptr; r.pos_div = 1; r.slots = nullptr; r.block_size = 1;
    }
    return r;
}

}  // namespace tqb
