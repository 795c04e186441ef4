// dequantize.cu -- inverse of Algorithm 1 / Algorithm 2:
//   unpack codes -> centroid lookup -> inverse rotation x = y @ R -> (Prod) + sqrt(pi/2)/d * ||r|| *
//   (signs @ S) -> * norm.   Upstream: turboquant_kv/reference.py:320-367 and :472-533.
//
// Same decomposition as quantize.cu: a warp owns 8 rows, lane l owns output coordinates l + 32 q,
// the (dim x dim) matrix sits in shared memory as stored (row j = rotated coordinate j).
#include "rowgemm.cuh"

namespace tqb {

struct DequantArgs {
    const uint8_t* packed; const uint8_t* signs;
    const float* norms; const float* res_norms;
    int64_t n;
    const float* rot; const float* cent; const float* qjl;
    int mse_bits;
    void* out;
};

template <int NQ>
__device__ __forceinline__ void gemm_pass(float (&acc)[RW][NQ], float* Tm, const float* M, const float* ub,
                                          int dim, int nchunks, bool resident, int lane) {
    constexpr int DP = NQ * 32;
#pragma unroll
    for (int i = 0; i < RW; i++)
#pragma unroll
        for (int q = 0; q < NQ; q++) acc[i][q] = 0.0f;
    if (resident) {
        accumulate_chunk<NQ>(acc, Tm, ub, 0, dim, lane);
    } else {
        for (int c = 0; c < nchunks; c++) {
            const int kc = min(KC, dim - c * KC);
            __syncthreads();
            load_direct_chunk<DP>(Tm, M, dim, c * KC, kc);
            __syncthreads();
            accumulate_chunk<NQ>(acc, Tm, ub, c * KC, kc, lane);
        }
    }
}

template <int NQ, typename OutT, bool PROD>
__global__ void __launch_bounds__(256) dequantize_kernel(DequantArgs a, int dim) {
    constexpr int DP = NQ * 32;
    extern __shared__ __align__(16) float smem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kc_max = dim < KC ? dim : KC;
    const int nchunks = (dim + KC - 1) / KC;
    const bool resident = nchunks == 1;
    float* Tm = smem;
    float* Tm2 = Tm + kc_max * (DP + 1);
    float* ub_all = (PROD && resident) ? Tm2 + kc_max * (DP + 1) : Tm2;
    float* ub = ub_all + warp * (DP * RW);
    float* sc = ub_all + warps * (DP * RW);  // centroids (16)
    const int bpp = (dim + 7) >> 3;
    const int pd = a.mse_bits * bpp;
    const float qjl_scale = 1.2533141373155003f / (float)dim;  // sqrt(pi/2) / d, reference.py:528

    if (threadIdx.x < 16) sc[threadIdx.x] = threadIdx.x < (1 << a.mse_bits) ? a.cent[threadIdx.x] : 0.0f;
    if (resident) {
        load_direct_chunk<DP>(Tm, a.rot, dim, 0, dim);
        if (PROD) load_direct_chunk<DP>(Tm2, a.qjl, dim, 0, dim);
    }
    __syncthreads();

    const int64_t rows_per_cta = (int64_t)warps * RW;
    const int64_t nblocks = (a.n + rows_per_cta - 1) / rows_per_cta;
    OutT* out = reinterpret_cast<OutT*>(a.out);

    for (int64_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        const int64_t row0 = blk * rows_per_cta + (int64_t)warp * RW;
#pragma unroll
        for (int i = 0; i < RW; i++) {
            const int64_t r = row0 + i;
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const int j = lane + 32 * q;
                float y = 0.0f;
                if (r < a.n && j < dim) {
                    const uint8_t* p = a.packed + r * pd + (j >> 3);
                    uint32_t c = 0;
                    for (int b = 0; b < a.mse_bits; b++) c |= ((p[b * bpp] >> (7 - (j & 7))) & 1u) << b;
                    y = sc[c];
                }
                ub[j * RW + i] = y;
            }
        }
        __syncwarp();
        float acc[RW][NQ];
        gemm_pass<NQ>(acc, Tm, a.rot, ub, dim, nchunks, resident, lane);
        __syncwarp();
        if (PROD) {
#pragma unroll
            for (int i = 0; i < RW; i++) {
                const int64_t r = row0 + i;
#pragma unroll
                for (int q = 0; q < NQ; q++) {
                    const int j = lane + 32 * q;
                    float s = 0.0f;
                    if (r < a.n && j < dim)
                        s = ((a.signs[r * bpp + (j >> 3)] >> (7 - (j & 7))) & 1u) ? 1.0f : -1.0f;
                    ub[j * RW + i] = s;
                }
            }
            __syncwarp();
            float acc2[RW][NQ];
            gemm_pass<NQ>(acc2, resident ? Tm2 : Tm, a.qjl, ub, dim, nchunks, resident, lane);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < RW; i++) {
                const int64_t r = row0 + i;
                const float coef = (r < a.n) ? qjl_scale * a.res_norms[r] : 0.0f;
#pragma unroll
                for (int q = 0; q < NQ; q++) acc[i][q] = acc[i][q] + coef * acc2[i][q];
            }
        }
#pragma unroll
        for (int i = 0; i < RW; i++) {
            const int64_t r = row0 + i;
            if (r >= a.n) continue;
            const float nr = a.norms[r];
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const int k = lane + 32 * q;
                if (k < dim) out[r * dim + k] = from_f32<OutT>(acc[i][q] * nr);
            }
        }
    }
}

template <int NQ, typename OutT, bool PROD>
static int launch_dequantize(const DequantArgs& a, int dim, cudaStream_t st) {
    constexpr int DP = NQ * 32;
    const int warps = 8;
    const int kc_max = dim < KC ? dim : KC;
    const int nchunks = (dim + KC - 1) / KC;
    const int mats = (PROD && nchunks == 1) ? 2 : 1;
    const size_t smem = sizeof(float) * ((size_t)mats * kc_max * (DP + 1) + (size_t)warps * DP * RW + 16);
    auto kern = dequantize_kernel<NQ, OutT, PROD>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t nblocks = ceil_div(a.n, (int64_t)warps * RW);
    const int per_sm = std::max<int>(1, (int)(200 * 1024 / smem));
    const int gx = (int)std::min<int64_t>(nblocks, (int64_t)sm_count() * per_sm);
    kern<<<gx, warps * 32, smem, st>>>(a, dim);
    return check_launch("dequantize");
}

template <typename OutT, bool PROD>
static int dq_dispatch_nq(const DequantArgs& a, int dim, cudaStream_t st) {
    if (dim <= 32) return launch_dequantize<1, OutT, PROD>(a, dim, st);
    if (dim <= 64) return launch_dequantize<2, OutT, PROD>(a, dim, st);
    if (dim <= 128) return launch_dequantize<4, OutT, PROD>(a, dim, st);
    return launch_dequantize<8, OutT, PROD>(a, dim, st);
}

template <bool PROD>
static int dq_dispatch(int dtype, const DequantArgs& a, int dim, cudaStream_t st) {
    switch (dtype) {
        case TQB_F32: return dq_dispatch_nq<float, PROD>(a, dim, st);
        case TQB_F16: return dq_dispatch_nq<__half, PROD>(a, dim, st);
        case TQB_BF16: return dq_dispatch_nq<__nv_bfloat16, PROD>(a, dim, st);
    }
    return fail(TQB_ERR_INVALID, "dequantize: unknown dtype %d", dtype);
}

}  // namespace tqb

extern "C" int tqb_dequantize_mse(const uint8_t* packed, const float* norms, int64_t n, int dim,
                                  const float* rotation, const float* centroids, int bits, void* out,
                                  int out_dtype, void* stream) {
    TQB_REQUIRE(n >= 0, "dequantize_mse: negative row count");
    TQB_REQUIRE(bits >= 1 && bits <= 4, "dequantize_mse: bit_width must be 1-4, got %d", bits);
    if (dim < 8 || dim > 256 || (dim & 7))
        return tqb::fail(TQB_ERR_UNSUPPORTED, "dequantize_mse: dim must be a multiple of 8 in 8..256, got %d", dim);
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(packed && norms && rotation && centroids && out, "dequantize_mse: null pointer");
    tqb::DequantArgs a{};
    a.packed = packed; a.norms = norms; a.n = n; a.rot = rotation; a.cent = centroids; a.mse_bits = bits; a.out = out;
    return tqb::dq_dispatch<false>(out_dtype, a, dim, (cudaStream_t)stream);
}

extern "C" int tqb_dequantize_prod(const uint8_t* mse_packed, const uint8_t* signs, const float* res_norms,
                                   const float* norms, int64_t n, int dim, const float* rotation,
                                   const float* centroids, const float* qjl, int bits, void* out,
                                   int out_dtype, void* stream) {
    TQB_REQUIRE(n >= 0, "dequantize_prod: negative row count");
    TQB_REQUIRE(bits >= 2 && bits <= 5, "dequantize_prod: bit_width must be 2-5, got %d", bits);
    if (dim < 8 || dim > 256 || (dim & 7))
        return tqb::fail(TQB_ERR_UNSUPPORTED, "dequantize_prod: dim must be a multiple of 8 in 8..256, got %d", dim);
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(mse_packed && signs && res_norms && norms && rotation && centroids && qjl && out,
                "dequantize_prod: null pointer");
    tqb::DequantArgs a{};
    a.packed = mse_packed; a.signs = signs; a.norms = norms; a.res_norms = res_norms; a.n = n; a.rot = rotation;
    a.cent = centroids; a.qjl = qjl; a.mse_bits = bits - 1; a.out = out;
    return tqb::dq_dispatch<true>(out_dtype, a, dim, (cudaStream_t)stream);
}
