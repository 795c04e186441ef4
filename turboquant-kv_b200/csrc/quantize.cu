// quantize.cu -- Algorithm 1 / Algorithm 2 quantisation, fused:
//   norm -> unit vector -> rotation (d x d contraction) -> Lloyd-Max code selection
//   -> (Prod) residual in rotated space -> QJL projection -> sign bits -> bit-plane pack.
//
// Arithmetic follows upstream turboquant_kv/reference.py:293-317 (MSE) and :429-469 (Prod) in
// float32.  Work decomposition: a warp owns RW = 8 consecutive rows; lane l owns the rotated
// coordinates j = l + 32 q.  The NORM of a row is summed in one fixed order that every quantising kernel
// of this library shares (this one, the tensor-core kernel, the decode step's append), so that they all
// store the same norm and select the same codes: when dim is a multiple of 32, lane l squares and adds
// the dim/32 CONSECUTIVE elements starting at l * dim/32 (fused multiply-add chain), else the elements
// l + 32 q; then a butterfly over the lanes.  The transposed rotation T[k][j] = R[j][k] sits in shared memory, so a
// k step costs NQ conflict-free LDS.32 (T row) + 2 broadcast LDS.128 (the 8 rows' k-th unit
// coordinate) for 8*NQ FMAs per lane.  Codes are packed with one __ballot_sync per (plane, q):
// the ballot of 32 lanes is exactly one 32-bit word of a bit-plane after a bit reversal.
//
// The Prod path keeps the residual in ROTATED space: residual = unit - R^T c, so
// S residual = (S R^T)(R unit - c); the caller passes qjl_rot = S R^T.  ||residual|| is the same in
// both spaces because R is orthogonal.
#include "rowgemm.cuh"
#include "tiled_layout.cuh"

namespace tqb {

constexpr int MAX_BND = 16;     // boundaries / centroids staged in shared memory

// quantize_tc.cu: the tensor-core kernel for large MSE calls (dim 64 / 128, 2-4 bits).  TQB_ERR_UNSUPPORTED
// means "not a shape for that path" and sends the call to the kernel below.
int quantize_tc_try(const void* x, int dtype, int64_t n, int dim, int64_t x_stride, const float* rot, const float* bnd,
                    int bits, uint8_t* packed, float* norms, const RowMap& map, int tiled, int kb, int vb, cudaStream_t st);

struct QuantArgs {
    const void* x;              // (n, dim) rows, x_stride elements apart
    int64_t n, x_stride;
    const float* rot;           // (dim, dim)
    const float* bnd;           // (2^mb - 1)
    const float* cent;          // (2^mb)      Prod only
    const float* qjl_rot;       // (dim, dim)  Prod only
    int mse_bits;               // bits of the Lloyd-Max part
    uint8_t* packed; float* norms;
    uint8_t* signs; float* res_norms;  // Prod only (dense)
    RowMap map;
    int tiled;                  // 0: upstream rows; 1 / 2: key / value section of the tiled KV store
    int kb, vb;                 // tiled store geometry (bits of keys and values)
};

// Store one bit-plane group: lane (p * NQ + q) holds the 4 bytes at row offset p * bpp + 4 q.
template <int NQ>
__device__ __forceinline__ void store_planes(uint8_t* row, uint32_t word, int planes, int bpp, int lane) {
    if (lane < planes * NQ) {
        const int p = lane / NQ, q = lane - p * NQ;
        const int nb = min(4, bpp - 4 * q);
        if (nb == 4 && (bpp & 3) == 0) {
            *reinterpret_cast<uint32_t*>(row + p * bpp + 4 * q) = word;
        } else {
            for (int t = 0; t < nb; t++) row[p * bpp + 4 * q + t] = (uint8_t)(word >> (8 * t));
        }
    }
}

template <int NQ, typename T, bool PROD>
__global__ void __launch_bounds__(256) quantize_kernel(QuantArgs a0, QuantArgs a1, int dim) {
    constexpr int DP = NQ * 32;
    extern __shared__ __align__(16) float smem[];
    const QuantArgs& a = (blockIdx.y == 0) ? a0 : a1;
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kc_max = dim < KC ? dim : KC;
    const int nchunks = (dim + KC - 1) / KC;
    float* Tm = smem;                                   // kc_max x (DP+1)
    float* Tm2 = Tm + kc_max * (DP + 1);                 // Prod: second matrix (only when nchunks == 1)
    float* ub_all = (PROD && nchunks == 1) ? Tm2 + kc_max * (DP + 1) : Tm2;
    float* ub = ub_all + warp * (DP * RW);             // [k][RW] per warp
    float* sb = ub_all + warps * (DP * RW);            // boundaries (16) + centroids (16)
    const int nbnd = (1 << a.mse_bits) - 1;
    const int bpp = (dim + 7) >> 3;
    const int pd = a.mse_bits * bpp;

    if (threadIdx.x < MAX_BND) {
        sb[threadIdx.x] = threadIdx.x < nbnd ? a.bnd[threadIdx.x] : __int_as_float(0x7f800000);
        if (PROD) sb[MAX_BND + threadIdx.x] = threadIdx.x <= nbnd ? a.cent[threadIdx.x] : 0.0f;
    }
    if (nchunks == 1) {
        load_transposed_chunk<DP>(Tm, a.rot, dim, 0, dim);
        if (PROD) load_transposed_chunk<DP>(Tm2, a.qjl_rot, dim, 0, dim);
    }
    __syncthreads();

    const int64_t rows_per_cta = (int64_t)warps * RW;
    const int64_t nblocks = (a.n + rows_per_cta - 1) / rows_per_cta;
    const T* x = reinterpret_cast<const T*>(a.x);

    for (int64_t blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        const int64_t row0 = blk * rows_per_cta + (int64_t)warp * RW;
        float nrm[RW], n2[RW];
        // ---- norms and unit vectors into the per-warp transposed buffer ----
#pragma unroll
        for (int i = 0; i < RW; i++) {
            const int64_t r = row0 + i;
            float v[NQ], ss = 0.0f;
            const bool blocked = (dim & 31) == 0;             // lane owns dim/32 consecutive elements
            const int per_lane = dim >> 5;
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const int j = blocked ? lane * per_lane + q : lane + 32 * q;
                v[q] = (r < a.n && j < dim && (!blocked || q < per_lane)) ? to_f32<T>(x[r * a.x_stride + j]) : 0.0f;
                ss = fmaf(v[q], v[q], ss);
            }
            nrm[i] = sqrtf(warp_sum(ss));
            const float den = fmaxf(nrm[i], 1e-10f);
            float s2 = 0.0f;
#pragma unroll
            for (int q = 0; q < NQ; q++) { v[q] = v[q] / den; s2 = fmaf(v[q], v[q], s2); }
            n2[i] = 1.0f;
            if (PROD) {  // quantize_mse normalises the unit vector once more (reference.py:441 -> :294)
                n2[i] = sqrtf(warp_sum(s2));
                const float den2 = fmaxf(n2[i], 1e-10f);
#pragma unroll
                for (int q = 0; q < NQ; q++) v[q] = v[q] / den2;
            }
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const int j = blocked ? lane * per_lane + q : lane + 32 * q;
                if (j < DP && (!blocked || q < per_lane)) ub[j * RW + i] = v[q];
            }
        }
        __syncwarp();

        // ---- rotation: y[i][q] = sum_k unit[i][k] R[lane+32q][k] ----
        float acc[RW][NQ];
#pragma unroll
        for (int i = 0; i < RW; i++)
#pragma unroll
            for (int q = 0; q < NQ; q++) acc[i][q] = 0.0f;
        if (nchunks == 1) {
            accumulate_chunk<NQ>(acc, Tm, ub, 0, dim, lane);
        } else {
            for (int c = 0; c < nchunks; c++) {
                const int kc = min(KC, dim - c * KC);
                __syncthreads();
                load_transposed_chunk<DP>(Tm, a.rot, dim, c * KC, kc);
                __syncthreads();
                accumulate_chunk<NQ>(acc, Tm, ub, c * KC, kc, lane);
            }
        }
        __syncwarp();

        // ---- code selection, packing, (Prod) residual ----
        float rn[RW];
#pragma unroll
        for (int i = 0; i < RW; i++) {
            const int64_t r = row0 + i;
            uint32_t code[NQ];
            float ee = 0.0f;
#pragma unroll
            for (int q = 0; q < NQ; q++) {
                const float y = acc[i][q];
                uint32_t c = 0;
                for (int step = 1 << (a.mse_bits - 1); step > 0; step >>= 1)
                    if (sb[c + step - 1] < y) c += step;
                if (lane + 32 * q >= dim) c = 0;
                code[q] = c;
                if (PROD) {
                    const float e = (lane + 32 * q < dim) ? fmaf(n2[i], y, -sb[MAX_BND + c]) : 0.0f;
                    ee = fmaf(e, e, ee);
                    ub[(lane + 32 * q) * RW + i] = e;
                }
            }
            if (PROD) rn[i] = sqrtf(warp_sum(ee));
            if (!PROD && a.tiled) {
                if (r < a.n) {
                    const int64_t slot = a.map(r);
                    if (slot >= 0) tiled_store_row<NQ>(a.packed, a.tiled, a.kb, a.vb, slot, code, nrm[i], lane, dim);
                }
                continue;
            }
            uint32_t mine = 0;
            for (int p = 0; p < a.mse_bits; p++)
#pragma unroll
                for (int q = 0; q < NQ; q++) {
                    const uint32_t w = ballot_to_plane_word(__ballot_sync(0xffffffffu, (code[q] >> p) & 1u));
                    if (lane == p * NQ + q) mine = w;
                }
            if (r < a.n) {
                const int64_t orow = a.map(r);
                if (orow >= 0) {
                    store_planes<NQ>(a.packed + orow * pd, mine, a.mse_bits, bpp, lane);
                    if (lane == 0) a.norms[orow] = nrm[i];
                }
            }
        }

        if (PROD) {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < RW; i++)
#pragma unroll
                for (int q = 0; q < NQ; q++) acc[i][q] = 0.0f;
            if (nchunks == 1) {
                accumulate_chunk<NQ>(acc, Tm2, ub, 0, dim, lane);
            } else {
                for (int c = 0; c < nchunks; c++) {
                    const int kc = min(KC, dim - c * KC);
                    __syncthreads();
                    load_transposed_chunk<DP>(Tm, a.qjl_rot, dim, c * KC, kc);
                    __syncthreads();
                    accumulate_chunk<NQ>(acc, Tm, ub, c * KC, kc, lane);
                }
            }
#pragma unroll
            for (int i = 0; i < RW; i++) {
                const int64_t r = row0 + i;
                uint32_t mine = 0;
#pragma unroll
                for (int q = 0; q < NQ; q++) {
                    const bool s = (lane + 32 * q < dim) && (acc[i][q] >= 0.0f);
                    const uint32_t w = ballot_to_plane_word(__ballot_sync(0xffffffffu, s));
                    if (lane == q) mine = w;
                }
                if (r < a.n) {
                    store_planes<NQ>(a.signs + r * bpp, mine, 1, bpp, lane);
                    if (lane == 0) a.res_norms[r] = rn[i];
                }
            }
            __syncwarp();
        }
    }
}

template <int NQ, typename T, bool PROD>
static int launch_quantize(const QuantArgs& a0, const QuantArgs& a1, int ntensors, int dim, cudaStream_t st) {
    constexpr int DP = NQ * 32;
    const int64_t n = a0.n;
    const int warps = 8;
    const int kc_max = dim < KC ? dim : KC;
    const int nchunks = (dim + KC - 1) / KC;
    const int mats = (PROD && nchunks == 1) ? 2 : 1;
    const size_t smem = sizeof(float) * ((size_t)mats * kc_max * (DP + 1) + (size_t)warps * DP * RW + 2 * MAX_BND);
    auto kern = quantize_kernel<NQ, T, PROD>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t nblocks = ceil_div(n, (int64_t)warps * RW);
    const int per_sm = std::max<int>(1, (int)(200 * 1024 / smem));
    const int gx = (int)std::min<int64_t>(nblocks, (int64_t)sm_count() * per_sm);
    dim3 grid(gx, ntensors);
    kern<<<grid, warps * 32, smem, st>>>(a0, a1, dim);
    return check_launch("quantize");
}

template <typename T, bool PROD>
static int dispatch_nq(const QuantArgs& a0, const QuantArgs& a1, int nt, int dim, cudaStream_t st) {
    if (dim <= 32) return launch_quantize<1, T, PROD>(a0, a1, nt, dim, st);
    if (dim <= 64) return launch_quantize<2, T, PROD>(a0, a1, nt, dim, st);
    if (dim <= 128) return launch_quantize<4, T, PROD>(a0, a1, nt, dim, st);
    return launch_quantize<8, T, PROD>(a0, a1, nt, dim, st);
}

template <bool PROD>
static int dispatch_dtype(int dtype, const QuantArgs& a0, const QuantArgs& a1, int nt, int dim, cudaStream_t st) {
    switch (dtype) {
        case TQB_F32: return dispatch_nq<float, PROD>(a0, a1, nt, dim, st);
        case TQB_F16: return dispatch_nq<__half, PROD>(a0, a1, nt, dim, st);
        case TQB_BF16: return dispatch_nq<__nv_bfloat16, PROD>(a0, a1, nt, dim, st);
    }
    return fail(TQB_ERR_INVALID, "quantize: unknown dtype %d", dtype);
}

static int check_common(const char* who, int64_t n, int dim, int bits, int lo, int hi) {
    TQB_REQUIRE(n >= 0, "%s: negative row count", who);
    TQB_REQUIRE(bits >= lo && bits <= hi, "%s: bit_width must be %d-%d, got %d", who, lo, hi, bits);
    if (dim < 8 || dim > 256 || (dim & 7))
        return fail(TQB_ERR_UNSUPPORTED, "%s: dim must be a multiple of 8 in 8..256, got %d", who, dim);
    return TQB_OK;
}

}  // namespace tqb

extern "C" int tqb_quantize_mse(const void* x, int dtype, int64_t n, int dim, int64_t x_stride,
                                const float* rotation, const float* boundaries, int bits,
                                uint8_t* packed, float* norms, const tqb_rowmap* map, void* stream) {
    if (int e = tqb::check_common("quantize_mse", n, dim, bits, 1, 4)) return e;
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(x && rotation && boundaries && packed && norms, "quantize_mse: null pointer");
    TQB_REQUIRE(x_stride >= dim, "quantize_mse: row stride %lld < dim %d", (long long)x_stride, dim);
    tqb::QuantArgs a{};
    a.x = x; a.n = n; a.x_stride = x_stride; a.rot = rotation; a.bnd = boundaries; a.mse_bits = bits;
    a.packed = packed; a.norms = norms; a.map = tqb::make_rowmap(map);
    const int rc = tqb::quantize_tc_try(x, dtype, n, dim, x_stride, rotation, boundaries, bits, packed, norms, a.map, 0, 0, 0,
                                        (cudaStream_t)stream);
    if (rc != TQB_ERR_UNSUPPORTED) return rc;
    return tqb::dispatch_dtype<false>(dtype, a, a, 1, dim, (cudaStream_t)stream);
}

extern "C" int tqb_kv_append(const void* key, const void* value, int dtype, int64_t n, int dim,
                             int64_t x_stride, const float* rot_k, const float* bnd_k, int kbits,
                             const float* rot_v, const float* bnd_v, int vbits, uint8_t* store,
                             const tqb_rowmap* map, void* stream) {
    TQB_REQUIRE(n >= 0, "kv_append: negative row count");
    if (dim != 64 && dim != 128) return tqb::fail(TQB_ERR_UNSUPPORTED, "kv_append: head_dim must be 64 or 128, got %d", dim);
    if (kbits < 2 || kbits > 4 || (vbits != 0 && (vbits < 2 || vbits > 4)))
        return tqb::fail(TQB_ERR_UNSUPPORTED, "kv_append: key bits must be 2..4 and value bits 2..4 (or 0: key-only records), got %d/%d",
                         kbits, vbits);
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(key && rot_k && bnd_k && store, "kv_append: null pointer");
    TQB_REQUIRE(vbits == 0 || (value && rot_v && bnd_v), "kv_append: null pointer");
    TQB_REQUIRE(x_stride >= dim, "kv_append: row stride %lld < dim %d", (long long)x_stride, dim);
    TQB_REQUIRE((uintptr_t)store % 16 == 0, "kv_append: the record store must be 16-byte aligned");
    tqb::QuantArgs a{}, b{};
    a.x = key; a.n = n; a.x_stride = x_stride; a.rot = rot_k; a.bnd = bnd_k; a.mse_bits = kbits;
    a.packed = store; a.norms = nullptr; a.map = tqb::make_rowmap(map); a.tiled = 1; a.kb = kbits; a.vb = vbits;
    b = a;
    b.x = value; b.rot = rot_v; b.bnd = bnd_v; b.mse_bits = vbits; b.tiled = 2;
    // large calls: keys, then values, through the tensor-core kernel
    int rc = tqb::quantize_tc_try(key, dtype, n, dim, x_stride, rot_k, bnd_k, kbits, store, nullptr, a.map, 1, kbits, vbits,
                                  (cudaStream_t)stream);
    if (rc == TQB_OK && vbits)
        rc = tqb::quantize_tc_try(value, dtype, n, dim, x_stride, rot_v, bnd_v, vbits, store, nullptr, a.map, 2, kbits, vbits,
                                  (cudaStream_t)stream);
    if (rc != TQB_ERR_UNSUPPORTED) return rc;
    return tqb::dispatch_dtype<false>(dtype, a, b, vbits ? 2 : 1, dim, (cudaStream_t)stream);
}

extern "C" int tqb_quantize_prod(const void* x, int dtype, int64_t n, int dim, int64_t x_stride,
                                 const float* rotation, const float* boundaries, const float* centroids,
                                 const float* qjl_rot, int bits, uint8_t* mse_packed, uint8_t* signs,
                                 float* res_norms, float* norms, void* stream) {
    if (bits < 2) return tqb::fail(TQB_ERR_INVALID, "Prod mode requires bits >= 2, got %d", bits);
    if (int e = tqb::check_common("quantize_prod", n, dim, bits, 2, 5)) return e;
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(x && rotation && boundaries && centroids && qjl_rot && mse_packed && signs && res_norms && norms,
                "quantize_prod: null pointer");
    TQB_REQUIRE(x_stride >= dim, "quantize_prod: row stride %lld < dim %d", (long long)x_stride, dim);
    tqb::QuantArgs a{};
    a.x = x; a.n = n; a.x_stride = x_stride; a.rot = rotation; a.bnd = boundaries; a.cent = centroids;
    a.qjl_rot = qjl_rot; a.mse_bits = bits - 1; a.packed = mse_packed; a.norms = norms; a.signs = signs;
    a.res_norms = res_norms; a.map = tqb::make_rowmap(nullptr);
    return tqb::dispatch_dtype<true>(dtype, a, a, 1, dim, (cudaStream_t)stream);
}
