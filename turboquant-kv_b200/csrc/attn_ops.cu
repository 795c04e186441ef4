// attn_ops.cu -- operator-level attention over ONE packed stream shared by all (batch, head)
// queries: the two ops of upstream turboquant_kv/ops.py:131-246 (csrc/cuda/attn_scores.cu,
// csrc/cuda/attn_values.cu).  Any dim that is a multiple of 8 up to 512, bits 1..4.
//
// scores: a CTA owns one query and a slice of the sequence.  It rotates the query, builds the table
// T[j][c] = (R q)_j * centroid_c in shared memory, then every thread walks rows of the slice byte
// column by byte column, exactly the loop structure of turboquant::search_packed
// (csrc/core/turboquant_core.cpp:455-495).  values: a CTA owns one query; threads are laid out as
// (sequence slice) x (dimension), partial sums are combined in shared memory and multiplied by
// rotation_T.
#include "common.cuh"

namespace tqb {

constexpr int OPS_MAX_DIM = 512;

__global__ void __launch_bounds__(256) scores_packed_kernel(const float* __restrict__ query, int dim,
                                                            const uint8_t* __restrict__ packed,
                                                            const float* __restrict__ norms, int64_t seq,
                                                            const float* __restrict__ cent,
                                                            const float* __restrict__ R, int bits,
                                                            float* __restrict__ scores, int64_t rows_per_cta) {
    extern __shared__ float sm[];
    float* q = sm;               // dim
    float* qr = sm + dim;        // dim
    float* T = sm + 2 * dim;     // dim * levels
    const int levels = 1 << bits, bpp = (dim + 7) >> 3, pd = bits * bpp;
    const int64_t i = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int k = threadIdx.x; k < dim; k += blockDim.x) q[k] = query[i * dim + k];
    __syncthreads();
    for (int j = warp; j < dim; j += nwarps) {
        float s = 0.0f;
        for (int k = lane; k < dim; k += 32) s = fmaf(R[(int64_t)j * dim + k], q[k], s);
        s = warp_sum(s);
        if (lane == 0) qr[j] = s;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < dim * levels; e += blockDim.x) T[e] = qr[e / levels] * cent[e % levels];
    __syncthreads();
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_cta;
    const int64_t r1 = min(seq, r0 + rows_per_cta);
    for (int64_t r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
        const uint8_t* row = packed + r * pd;
        float dot = 0.0f;
        for (int m = 0; m < bpp; m++) {
            uint32_t pl[4] = {0, 0, 0, 0};
            for (int b = 0; b < bits; b++) pl[b] = row[b * bpp + m];
            const int lim = min(8, dim - 8 * m);
            for (int t = 0; t < lim; t++) {
                const int sh = 7 - t;
                const uint32_t c = ((pl[0] >> sh) & 1u) | (((pl[1] >> sh) & 1u) << 1) |
                                   (((pl[2] >> sh) & 1u) << 2) | (((pl[3] >> sh) & 1u) << 3);
                dot += T[(8 * m + t) * levels + c];
            }
        }
        scores[i * seq + r] = dot * norms[r];
    }
}

// blockDim = (dim padded to 32) x slices, at most 1024 threads.
__global__ void values_packed_kernel(const float* __restrict__ weights, int64_t seq, int dim,
                                     const uint8_t* __restrict__ packed, const float* __restrict__ norms,
                                     const float* __restrict__ cent, const float* __restrict__ RT, int bits,
                                     float* __restrict__ out) {
    extern __shared__ float sm[];
    const int dp = blockDim.x, slices = blockDim.y;
    float* part = sm;                 // slices * dp
    float* c = sm + slices * dp;      // 16
    const int j = threadIdx.x, sl = threadIdx.y;
    const int bpp = (dim + 7) >> 3, pd = bits * bpp;
    const int64_t i = blockIdx.x;
    if (sl == 0 && j < 16) c[j] = j < (1 << bits) ? cent[j] : 0.0f;
    __syncthreads();
    float acc = 0.0f;
    if (j < dim) {
        const int m = j >> 3, sh = 7 - (j & 7);
        for (int64_t s = sl; s < seq; s += slices) {
            const uint8_t* row = packed + s * pd + m;
            uint32_t code = 0;
            for (int b = 0; b < bits; b++) code |= ((row[b * bpp] >> sh) & 1u) << b;
            acc = fmaf(weights[i * seq + s] * norms[s], c[code], acc);
        }
    }
    part[sl * dp + j] = acc;
    __syncthreads();
    if (sl == 0) {
        float a = 0.0f;
        for (int s = 0; s < slices; s++) a += part[s * dp + j];
        part[j] = a;
    }
    __syncthreads();
    if (sl == 0 && j < dim) {
        float o = 0.0f;
        for (int jj = 0; jj < dim; jj++) o = fmaf(part[jj], RT[(int64_t)jj * dim + j], o);
        out[i * dim + j] = o;
    }
}

}  // namespace tqb

extern "C" int tqb_attention_scores_packed(const float* query, int64_t bh, int dim, const uint8_t* packed_keys,
                                           const float* key_norms, int64_t seq, const float* centroids,
                                           const float* rotation, int bits, float* scores, void* stream) {
    TQB_REQUIRE(bits >= 1 && bits <= 4, "attention_scores_packed: bit_width must be 1-4, got %d", bits);
    TQB_REQUIRE(bh >= 0 && seq >= 0, "attention_scores_packed: negative size");
    if (dim < 8 || dim > tqb::OPS_MAX_DIM || (dim & 7))
        return tqb::fail(TQB_ERR_UNSUPPORTED, "attention_scores_packed: dim must be a multiple of 8 in 8..512, got %d", dim);
    if (bh == 0 || seq == 0) return TQB_OK;
    TQB_REQUIRE(query && packed_keys && key_norms && centroids && rotation && scores, "attention_scores_packed: null pointer");
    TQB_REQUIRE(bh <= 0x7fffffff, "attention_scores_packed: too many queries");
    const size_t smem = sizeof(float) * ((size_t)2 * dim + (size_t)dim * (1 << bits));
    int64_t slices = std::max<int64_t>(1, (int64_t)tqb::sm_count() * 4 / bh);
    slices = std::min<int64_t>(slices, tqb::ceil_div(seq, 1024));
    slices = std::min<int64_t>(std::max<int64_t>(slices, 1), 65535);
    const int64_t rows_per_cta = tqb::ceil_div(seq, slices);
    dim3 grid((unsigned)bh, (unsigned)tqb::ceil_div(seq, rows_per_cta));
    tqb::scores_packed_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(query, dim, packed_keys, key_norms, seq,
                                                                         centroids, rotation, bits, scores, rows_per_cta);
    return tqb::check_launch("attention_scores_packed");
}

extern "C" int tqb_attention_values_packed(const float* weights, int64_t bh, int64_t seq, int dim,
                                           const uint8_t* packed_values, const float* value_norms,
                                           const float* centroids, const float* rotation_T, int bits,
                                           float* out, void* stream) {
    TQB_REQUIRE(bits >= 1 && bits <= 4, "attention_values_packed: bit_width must be 1-4, got %d", bits);
    TQB_REQUIRE(bh >= 0 && seq >= 0, "attention_values_packed: negative size");
    if (dim < 8 || dim > tqb::OPS_MAX_DIM || (dim & 7))
        return tqb::fail(TQB_ERR_UNSUPPORTED, "attention_values_packed: dim must be a multiple of 8 in 8..512, got %d", dim);
    if (bh == 0) return TQB_OK;
    TQB_REQUIRE(weights && packed_values && value_norms && centroids && rotation_T && out, "attention_values_packed: null pointer");
    TQB_REQUIRE(bh <= 0x7fffffff, "attention_values_packed: too many queries");
    const int dp = (dim + 31) / 32 * 32;
    const int slices = std::max(1, 1024 / dp);
    const size_t smem = sizeof(float) * ((size_t)slices * dp + 16);
    dim3 block(dp, slices);
    tqb::values_packed_kernel<<<(unsigned)bh, block, smem, (cudaStream_t)stream>>>(weights, seq, dim, packed_values, value_norms,
                                                                                  centroids, rotation_T, bits, out);
    return tqb::check_launch("attention_values_packed");
}
