// rowgemm.cuh -- the small dense contraction shared by quantize and dequantize:
//   acc[i][q] += sum_k ub[k][i] * T[k][lane + 32 q]
// for the RW rows a warp owns.  T is a (k, DP+1)-pitched tile of a (dim x dim) matrix in shared
// memory, ub a per-warp [k][RW] buffer of the rows' k-th input coordinate.
#pragma once
#include "common.cuh"

namespace tqb {

constexpr int RW = 8;           // rows per warp
constexpr int KC = 128;         // k-chunk of the transposed matrix kept in shared memory
// T[kk][j] = M[j][c0 + kk] for kk < kc, j < DP (zero beyond dim).  Row pitch DP + 1 keeps both the
// transposing stores and the row reads free of bank conflicts.  Eight loads are issued before the
// first store so that their latencies overlap (this runs once per CTA and, for the few rows of a
// decode-step append, is most of the kernel).
template <int DP>
__device__ __forceinline__ void load_transposed_chunk(float* T, const float* __restrict__ M, int dim,
                                                      int c0, int kc) {
    const int total = DP * kc;
    const int step = blockDim.x;
    for (int base = threadIdx.x; base < total; base += step * 8) {
        float v[8];
        int dst[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = base + u * step;
            const int j = idx / kc, kk = idx - j * kc;
            dst[u] = idx < total ? kk * (DP + 1) + j : -1;
            v[u] = (idx < total && j < dim) ? M[(int64_t)j * dim + c0 + kk] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (dst[u] >= 0) T[dst[u]] = v[u];
    }
}

template <int NQ>
__device__ __forceinline__ void accumulate_chunk(float (&acc)[RW][NQ], const float* T, const float* ub,
                                                 int c0, int kc, int lane) {
    constexpr int DP = NQ * 32;
#pragma unroll 4
    for (int kk = 0; kk < kc; kk++) {
        float r[NQ];
#pragma unroll
        for (int q = 0; q < NQ; q++) r[q] = T[kk * (DP + 1) + lane + 32 * q];
        const float4 u0 = *reinterpret_cast<const float4*>(ub + (c0 + kk) * RW);
        const float4 u1 = *reinterpret_cast<const float4*>(ub + (c0 + kk) * RW + 4);
        const float u[RW] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int i = 0; i < RW; i++)
#pragma unroll
            for (int q = 0; q < NQ; q++) acc[i][q] = fmaf(u[i], r[q], acc[i][q]);
    }
}


// T[kk][j] = M[c0 + kk][j]: the matrix as stored (used by the inverse rotation x = y @ R).
template <int DP>
__device__ __forceinline__ void load_direct_chunk(float* T, const float* __restrict__ M, int dim,
                                                  int c0, int kc) {
    const int total = DP * kc;
    const int step = blockDim.x;
    for (int base = threadIdx.x; base < total; base += step * 8) {
        float v[8];
        int dst[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int idx = base + u * step;
            const int kk = idx / DP, j = idx - kk * DP;
            dst[u] = idx < total ? kk * (DP + 1) + j : -1;
            v[u] = (idx < total && j < dim) ? M[(int64_t)(c0 + kk) * dim + j] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (dst[u] >= 0) T[dst[u]] = v[u];
    }
}

}  // namespace tqb
