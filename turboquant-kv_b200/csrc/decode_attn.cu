// decode_attn.cu -- fused decode attention over a packed KV cache (one new token per sequence).
//
// Replaces "dequantise every cached key and value, then attend" (upstream
// turboquant_kv/cache.py:216-339) by three launches that never materialise dense K/V:
//
//   1. rotate_query_kernel   q_rot = R_k q per head, normalised to |.| <= 1, written directly as
//                            mma.sync B fragments (fp16) + one fp32 scale per head.
//   2. decode_partial_kernel persistent warps stream 16-token tiles of packed K / V codes and norms
//                            through a per-warp ring of shared-memory stages filled by TMA bulk copies
//                            (cp.async.bulk + mbarrier).  Per tile: scores = K-codes x q on tensor
//                            cores (codes -> fp16 centroids through a 256-entry shared-memory table
//                            indexed by one byte = 2 codes), online softmax in the log2 domain with a
//                            lazy running maximum, P^T via movmatrix, O^T += V^T-codes x P^T on tensor
//                            cores, all in ROTATED space.  One (m, l, acc) partial per (unit, chunk).
//   3. decode_merge_kernel   combines the chunks of a (sequence, query head), divides by l and applies
//                            the inverse value rotation acc @ R_v (reference.py:362).
//
// A unit is one (sequence, KV head); its `group` query heads ride along as the N dimension of the
// MMA (grouped-query attention: decode cost is paid once per KV head).  HBM traffic per token and
// KV head is the packed K row + packed V row + two float norms; everything else lives in L2/SMEM.
//
// Every wait is bounded: a warp that gives up records it in the status word at the start of the
// workspace, drains nothing further and returns, so a lost copy cannot hang the device.
#include "common.cuh"
#include "decode_bits.cuh"

namespace tqb {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_INF = -__builtin_huge_valf();
constexpr float RESCALE_SLACK = 4.0f;   // lazy max: rescale only when a score exceeds m + 4 (log2)
constexpr int TILE = 16;                // tokens per MMA tile
constexpr uint32_t WAIT_LIMIT = 1u << 20;

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// TMA bulk copy global -> this CTA's shared memory, completion counted on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
// half2 {lo, hi} with saturation to the largest finite fp16 instead of infinity.
__device__ __forceinline__ uint32_t pack_half2_sat(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ---- launch parameters --------------------------------------------------------------------------
struct DecodeParams {
    const uint8_t* k_packed; const float* k_norms;
    const uint8_t* v_packed; const float* v_norms;
    const int32_t* seq_lens; const int32_t* block_tables;
    int64_t max_seq;                 // row pitch of a unit (contiguous cache)
    int batch, q_heads, kv_heads, group, max_blocks, block_size;
    int chunk, nchunks;              // tokens per (unit, chunk) work item
    const float* cent_k; const float* cent_v;
    // workspace views
    int* status; const uint32_t* qfrag; const float* qscale;
    float* part_m; float* part_l; float* part_acc;
};

// Workspace layout shared by the size query and the launcher.
struct DecodeWorkspace {
    size_t off_status, off_qfrag, off_qscale, off_m, off_l, off_acc, total;
    int chunk, nchunks;
};


// =================================================================================================
// 1. query rotation -> B fragments
// =================================================================================================
// One CTA (4 warps) per unit.  Fragment element (ks, lane = 4g+t, half) of head g holds the rotated,
// normalised query coordinates pair_dims(D, t, 2ks+half); heads >= group are zero columns.
template <typename T>
__global__ void __launch_bounds__(128) rotate_query_kernel(const T* __restrict__ q, int q_heads, int kv_heads,
                                                           int group, int dim, const float* __restrict__ R,
                                                           float scale, uint32_t* __restrict__ qfrag,
                                                           float* __restrict__ qscale, int* status) {
    __shared__ float qin[8][128];
    __shared__ float qr[8][128];
    __shared__ float qmax[8];
    const int u = blockIdx.x, b = u / kv_heads, h = u - b * kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (u == 0 && threadIdx.x == 0) *status = 0;
    for (int idx = threadIdx.x; idx < group * dim; idx += blockDim.x) {
        const int n = idx / dim, k = idx - n * dim;
        qin[n][k] = to_f32<T>(q[((int64_t)b * q_heads + h * group + n) * dim + k]);
    }
    __syncthreads();
    const int nq = dim >> 5;
    for (int j = warp; j < dim; j += 4) {
        float r[4];
        for (int i = 0; i < nq; i++) r[i] = R[(int64_t)j * dim + lane + 32 * i];
        for (int n = 0; n < group; n++) {
            float s = 0.0f;
            for (int i = 0; i < nq; i++) s = fmaf(r[i], qin[n][lane + 32 * i], s);
            s = warp_sum(s);
            if (lane == 0) qr[n][j] = s;
        }
    }
    __syncthreads();
    for (int n = warp; n < 8; n += 4) {
        float mx = 0.0f;
        if (n < group)
            for (int k = lane; k < dim; k += 32) mx = fmaxf(mx, fabsf(qr[n][k]));
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) {
            qmax[n] = mx;
            qscale[(int64_t)u * 8 + n] = (n < group) ? mx * scale * LOG2E : 0.0f;
        }
    }
    __syncthreads();
    const int ksteps = dim >> 4;
    for (int idx = threadIdx.x; idx < ksteps * 64; idx += blockDim.x) {
        const int ks = idx >> 6, rem = idx & 63, fl = rem >> 1, half = rem & 1;
        const int g = fl >> 2, t = fl & 3;
        float lo = 0.0f, hi = 0.0f;
        if (g < group && qmax[g] > 0.0f) {
            int dlo, dhi;
            pair_dims(dim, t, 2 * ks + half, dlo, dhi);
            const float inv = 1.0f / qmax[g];
            lo = qr[g][dlo] * inv;
            hi = qr[g][dhi] * inv;
        }
        qfrag[((int64_t)u * ksteps + ks) * 64 + rem] = pack_half2(lo, hi);
    }
}


// =================================================================================================
// 2. streaming partial attention
// =================================================================================================
template <int D, int KB, int VB>
struct DecodeCfg {
    static constexpr int PK = KB * D / 8;                 // packed key row bytes
    static constexpr int PV = VB * D / 8;
    static constexpr int KT = TILE * PK;                  // tile bytes
    static constexpr int VT = TILE * PV;
    static constexpr int STAGE = KT + VT + 2 * TILE * 4;  // + key norms + value norms
    static constexpr int LUTK_ENTRIES = 1 << (2 * KB);
    static constexpr int LUTV_ENTRIES = 1 << (VB == 2 ? 8 : 2 * VB);
    static constexpr int LUTV_WORDS = VB == 2 ? 2 : 1;    // 8-byte entries for 2-bit values
    static constexpr int LUTK_BYTES = LUTK_ENTRIES * 32 * 4;
    static constexpr int LUTV_BYTES = LUTV_ENTRIES * 32 * 4 * LUTV_WORDS;
    static constexpr int MT = D / 16;                     // m-tiles of O^T / k-steps of the scores
    static constexpr int BV = D / 64;                     // value byte columns per thread
};

// Position of a warp in its stream of tiles: items (unit, chunk) are dealt round-robin to warps,
// tiles inside an item are consecutive.
struct TileCursor {
    int64_t item, total_items, stride;
    int tile, ntiles;         // inside the current item
    int unit, b, h, chunk_idx, tok0, tok_end;
    __device__ __forceinline__ bool valid() const { return item < total_items; }
    __device__ __forceinline__ void open(const DecodeParams& p) {
        // find the next item that has tokens
        while (item < total_items) {
            unit = (int)(item / p.nchunks);
            chunk_idx = (int)(item - (int64_t)unit * p.nchunks);
            b = unit / p.kv_heads;
            h = unit - b * p.kv_heads;
            const int S = p.seq_lens[b];
            tok0 = chunk_idx * p.chunk;
            tok_end = min(S, tok0 + p.chunk);
            if (tok0 < tok_end) {
                ntiles = (tok_end - tok0 + TILE - 1) / TILE;
                tile = 0;
                return;
            }
            item += stride;
        }
    }
    __device__ __forceinline__ void next(const DecodeParams& p) {
        if (++tile == ntiles) { item += stride; open(p); }
    }
};

template <int D, int KB, int VB, bool PAGED, int WARPS, int NS>
__global__ void __launch_bounds__(WARPS * 32, 1) decode_partial_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, KB, VB>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint32_t* lutK = reinterpret_cast<uint32_t*>(smem_raw);
    uint32_t* lutV = reinterpret_cast<uint32_t*>(smem_raw + C::LUTK_BYTES);
    uint8_t* ring_all = smem_raw + C::LUTK_BYTES + C::LUTV_BYTES;
    uint64_t* bars_all = reinterpret_cast<uint64_t*>(ring_all + (size_t)WARPS * NS * C::STAGE);
    __shared__ float s_ck[16], s_cv[16];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t* ring = ring_all + (size_t)warp * NS * C::STAGE;
    const uint32_t bar0 = smem_u32(bars_all + warp * NS);

    if (threadIdx.x < 16) {
        s_ck[threadIdx.x] = threadIdx.x < (1 << KB) ? p.cent_k[threadIdx.x] : 0.0f;
        s_cv[threadIdx.x] = threadIdx.x < (1 << VB) ? p.cent_v[threadIdx.x] : 0.0f;
    }
    if (lane == 0)
        for (int s = 0; s < NS; s++) mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // ---- lookup tables: entry x replicated for the 32 lanes at word x*32 + lane (no bank conflicts)
    for (int x = warp; x < C::LUTK_ENTRIES; x += WARPS) {
        int clo, chi;
        pair_index_codes<KB>((uint32_t)x, clo, chi);
        lutK[x * 32 + lane] = pack_half2(s_ck[clo], s_ck[chi]);
    }
    for (int x = warp; x < C::LUTV_ENTRIES; x += WARPS) {
        if (VB == 2) {
            int ag, bg, ag8, bg8;
            quad_index_codes_v2((uint32_t)x, ag, bg, ag8, bg8);
            reinterpret_cast<uint2*>(lutV)[x * 32 + lane] =
                make_uint2(pack_half2(s_cv[ag], s_cv[bg]), pack_half2(s_cv[ag8], s_cv[bg8]));
        } else {
            int ca, cb;
            token_pair_codes<VB>((uint32_t)x, ca, cb);
            lutV[x * 32 + lane] = pack_half2(s_cv[ca], s_cv[cb]);
        }
    }
    __syncthreads();

    const int64_t total_warps = (int64_t)gridDim.x * WARPS;
    TileCursor pc, cc;  // producer / consumer cursors over the same stream
    pc.item = (int64_t)blockIdx.x * WARPS + warp;
    pc.total_items = (int64_t)p.batch * p.kv_heads * p.nchunks;
    pc.stride = total_warps;
    pc.tile = pc.ntiles = 0;
    pc.open(p);
    cc = pc;

    // issue the copies of the producer cursor's tile into stage s (lane 0 only)
    auto issue = [&](const TileCursor& cur, int s) {
        if (lane == 0) {
            const int tok = cur.tok0 + cur.tile * TILE;
            int64_t row;
            if (PAGED) {
                const int blk = p.block_tables[(int64_t)cur.b * p.max_blocks + tok / p.block_size];
                row = ((int64_t)blk * p.kv_heads + cur.h) * p.block_size + tok % p.block_size;
            } else {
                row = (int64_t)cur.unit * p.max_seq + tok;
            }
            const uint32_t dst = smem_u32(ring + (size_t)s * C::STAGE);
            const uint32_t bar = bar0 + 8 * s;
            // order this warp's earlier generic-proxy reads of the stage before the async-proxy overwrite
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, C::STAGE);
            bulk_g2s(dst, p.k_packed + row * C::PK, C::KT, bar);
            bulk_g2s(dst + C::KT, p.v_packed + row * C::PV, C::VT, bar);
            bulk_g2s(dst + C::KT + C::VT, p.k_norms + row, TILE * 4, bar);
            bulk_g2s(dst + C::KT + C::VT + TILE * 4, p.v_norms + row, TILE * 4, bar);
        }
    };

    uint32_t issued = 0, consumed = 0;
    while (issued < NS && pc.valid()) { issue(pc, issued % NS); pc.next(p); issued++; }

    // per-item state
    float m0 = NEG_INF, m1 = NEG_INF, l0 = 0.0f, l1 = 0.0f, qs0 = 0.0f, qs1 = 0.0f;
    float O[C::MT][4];
    uint32_t qf[C::MT][2];
    bool failed = false;

    while (cc.valid()) {
        if (cc.tile == 0) {
            m0 = m1 = NEG_INF; l0 = l1 = 0.0f;
#pragma unroll
            for (int mt = 0; mt < C::MT; mt++) { O[mt][0] = O[mt][1] = O[mt][2] = O[mt][3] = 0.0f; }
            const uint2* qsrc = reinterpret_cast<const uint2*>(p.qfrag) + ((int64_t)cc.unit * C::MT) * 32 + lane;
#pragma unroll
            for (int ks = 0; ks < C::MT; ks++) { const uint2 v = qsrc[ks * 32]; qf[ks][0] = v.x; qf[ks][1] = v.y; }
            qs0 = p.qscale[(int64_t)cc.unit * 8 + 2 * t];
            qs1 = p.qscale[(int64_t)cc.unit * 8 + 2 * t + 1];
        }
        const int s = consumed % NS;
        if (!mbar_wait(bar0 + 8 * s, (consumed / NS) & 1)) failed = true;
        if (__any_sync(0xffffffffu, failed)) { failed = true; break; }

        const uint8_t* kt = ring + (size_t)s * C::STAGE;
        const uint8_t* vt = kt + C::KT;
        const float* nk = reinterpret_cast<const float*>(vt + C::VT);
        const float* nv = nk + TILE;
        const int tokb = cc.tok0 + cc.tile * TILE;
        const bool val_g = tokb + g < cc.tok_end, val_g8 = tokb + g + 8 < cc.tok_end;

        // ---- scores: 16 tokens x 8 heads ----
        float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        {
            uint32_t P[KeyWords<D>::NW][4];
            gather_key_words<D, KB>(kt, C::PK, g, t, P);
            uint32_t iw[KeyWords<D>::NW][4];
#pragma unroll
            for (int w = 0; w < KeyWords<D>::NW; w++)
#pragma unroll
                for (int u = 0; u < 4; u++) iw[w][u] = pair_index_word<KB>(P[w], u);
#pragma unroll
            for (int ks = 0; ks < C::MT; ks++) {
                uint32_t a[4];
#pragma unroll
                for (int half = 0; half < 2; half++)
#pragma unroll
                    for (int second = 0; second < 2; second++) {
                        int u, w, bl;
                        key_element_slot<D>(2 * ks + half, second != 0, u, w, bl);
                        const uint32_t x = (iw[w][u] >> (8 * bl)) & 0xFFu;
                        a[2 * half + second] = lutK[x * 32 + lane];
                    }
                mma_f16(sc, a, qf[ks][0], qf[ks][1]);
            }
        }
        const float nkg = val_g ? nk[g] : 0.0f, nkg8 = val_g8 ? nk[g + 8] : 0.0f;
        float s0 = val_g ? sc[0] * (nkg * qs0) : NEG_INF, s1 = val_g ? sc[1] * (nkg * qs1) : NEG_INF;
        float s2 = val_g8 ? sc[2] * (nkg8 * qs0) : NEG_INF, s3 = val_g8 ? sc[3] * (nkg8 * qs1) : NEG_INF;

        // ---- online softmax, lazy maximum ----
        float tm0 = fmaxf(s0, s2), tm1 = fmaxf(s1, s3);
        if (__any_sync(0xffffffffu, (tm0 > m0 + RESCALE_SLACK) || (tm1 > m1 + RESCALE_SLACK))) {
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, o));
                tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, o));
            }
            const float mn0 = fmaxf(m0, tm0), mn1 = fmaxf(m1, tm1);
            const float f0 = (mn0 == NEG_INF) ? 1.0f : exp2f(m0 - mn0);
            const float f1 = (mn1 == NEG_INF) ? 1.0f : exp2f(m1 - mn1);
            l0 *= f0; l1 *= f1;
#pragma unroll
            for (int mt = 0; mt < C::MT; mt++) { O[mt][0] *= f0; O[mt][2] *= f0; O[mt][1] *= f1; O[mt][3] *= f1; }
            m0 = mn0; m1 = mn1;
        }
        const float mu0 = (m0 == NEG_INF) ? 0.0f : m0, mu1 = (m1 == NEG_INF) ? 0.0f : m1;
        const float p0 = exp2f(s0 - mu0), p1 = exp2f(s1 - mu1), p2 = exp2f(s2 - mu0), p3 = exp2f(s3 - mu1);
        l0 += p0 + p2; l1 += p1 + p3;
        const float nvg = val_g ? nv[g] : 0.0f, nvg8 = val_g8 ? nv[g + 8] : 0.0f;
        // P^T as B operand: (k = tokens, col = head) through two 8x8 transposes
        const uint32_t pb0 = movmatrix_trans(pack_half2_sat(p0 * nvg, p1 * nvg));
        const uint32_t pb1 = movmatrix_trans(pack_half2_sat(p2 * nvg8, p3 * nvg8));

        // ---- O^T += V^T P^T : (dims x tokens) x (tokens x heads) ----
#pragma unroll
        for (int i = 0; i < C::BV; i++) {
            const int c = C::BV * g + i;
            const uint32_t WA0 = gather_value_word<D, VB>(vt, C::PV, 2 * t, c);
            const uint32_t WB0 = gather_value_word<D, VB>(vt, C::PV, 2 * t + 1, c);
            const uint32_t WA1 = gather_value_word<D, VB>(vt, C::PV, 2 * t + 8, c);
            const uint32_t WB1 = gather_value_word<D, VB>(vt, C::PV, 2 * t + 9, c);
            if (VB == 2) {
                const uint32_t W0 = WA0 | (WB0 << 16), W1 = WA1 | (WB1 << 16);
                const uint2* lut2 = reinterpret_cast<const uint2*>(lutV);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const uint2 e0 = lut2[quad_index_v2(W0, u) * 32 + lane];
                    const uint2 e1 = lut2[quad_index_v2(W1, u) * 32 + lane];
                    const uint32_t a[4] = {e0.x, e0.y, e1.x, e1.y};
                    mma_f16(O[4 * i + u], a, pb0, pb1);
                }
            } else {
                uint32_t Ze0, Zo0, Ze1, Zo1;
                token_pair_words(WA0, WB0, Ze0, Zo0);
                token_pair_words(WA1, WB1, Ze1, Zo1);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    uint32_t a[4];
                    a[0] = lutV[token_pair_index(Ze0, Zo0, 2 * u + 1) * 32 + lane];
                    a[1] = lutV[token_pair_index(Ze0, Zo0, 2 * u) * 32 + lane];
                    a[2] = lutV[token_pair_index(Ze1, Zo1, 2 * u + 1) * 32 + lane];
                    a[3] = lutV[token_pair_index(Ze1, Zo1, 2 * u) * 32 + lane];
                    mma_f16(O[4 * i + u], a, pb0, pb1);
                }
            }
        }

        // ---- stage is free: refill it with the tile NS ahead ----
        __syncwarp();
        if (pc.valid()) { issue(pc, s); pc.next(p); issued++; }
        consumed++;

        // ---- end of item: write the partial (rotated space, unnormalised) ----
        if (cc.tile + 1 == cc.ntiles) {
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, o);
                l1 += __shfl_xor_sync(0xffffffffu, l1, o);
            }
            const int64_t pbase = ((int64_t)cc.unit * p.nchunks + cc.chunk_idx) * p.group;
            const int h0 = 2 * t, h1 = 2 * t + 1;
            if (g == 0) {
                if (h0 < p.group) { p.part_m[pbase + h0] = m0; p.part_l[pbase + h0] = l0; }
                if (h1 < p.group) { p.part_m[pbase + h1] = m1; p.part_l[pbase + h1] = l1; }
            }
#pragma unroll
            for (int mt = 0; mt < C::MT; mt++) {
                int dg, dg8;
                value_dims(D, g, mt, dg, dg8);
                if (h0 < p.group) {
                    p.part_acc[(pbase + h0) * D + dg] = O[mt][0];
                    p.part_acc[(pbase + h0) * D + dg8] = O[mt][2];
                }
                if (h1 < p.group) {
                    p.part_acc[(pbase + h1) * D + dg] = O[mt][1];
                    p.part_acc[(pbase + h1) * D + dg8] = O[mt][3];
                }
            }
        }
        cc.next(p);
    }

    if (failed) {
        // A copy never arrived.  Record it; give the copies still in flight a bounded chance to land
        // before this CTA's shared memory is released.
        if (lane == 0) atomicExch(p.status, 1);
        for (uint32_t i = consumed; i < issued; i++) (void)mbar_wait(bar0 + 8 * (i % NS), (i / NS) & 1);
    }
}


// =================================================================================================
// 3. merge of the chunks + inverse value rotation
// =================================================================================================
// One CTA of D threads per (unit, query head of the group).
template <typename OutT>
__global__ void decode_merge_kernel(const DecodeParams p, int dim, const float* __restrict__ Rv,
                                    OutT* __restrict__ out) {
    __shared__ float y[128];
    __shared__ float red[2];
    const int u = blockIdx.x / p.group, n = blockIdx.x - u * p.group;
    const int b = u / p.kv_heads, h = u - b * p.kv_heads;
    const int S = p.seq_lens[b];
    const int nch = (S + p.chunk - 1) / p.chunk;
    const int j = threadIdx.x;
    const int64_t pbase = (int64_t)u * p.nchunks * p.group + n;
    float M = NEG_INF;
    for (int c = 0; c < nch; c++) M = fmaxf(M, p.part_m[pbase + (int64_t)c * p.group]);
    float acc = 0.0f, L = 0.0f;
    for (int c = 0; c < nch; c++) {
        const int64_t pi = pbase + (int64_t)c * p.group;
        const float mc = p.part_m[pi];
        const float w = (mc == NEG_INF) ? 0.0f : exp2f(mc - M);
        L = fmaf(w, p.part_l[pi], L);
        acc = fmaf(w, p.part_acc[pi * dim + j], acc);
    }
    y[j] = (L > 0.0f) ? acc / L : 0.0f;
    (void)red;
    __syncthreads();
    float o = 0.0f;
    for (int jj = 0; jj < dim; jj++) o = fmaf(y[jj], Rv[(int64_t)jj * dim + j], o);
    out[((int64_t)b * p.q_heads + h * p.group + n) * dim + j] = from_f32<OutT>(o);
}

// ---- host side -------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 8;

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tokens per work item: small enough that every warp of the grid gets several items, large enough
// that the per-item partial (group x (D+2) floats) stays a few percent of the streamed bytes.
static int choose_chunk(int64_t units, int64_t max_len, int64_t total_warps) {
    int best = 64;
    double best_cost = 1e300;
    for (int L = 64; L <= 4096; L *= 2) {
        const int64_t nch = (max_len + L - 1) / L;
        const int64_t rounds = (units * nch + total_warps - 1) / total_warps;
        const double cost = (double)rounds * ((double)std::min<int64_t>(L, max_len) + 24.0);
        if (cost <= best_cost) { best_cost = cost; best = L; }
        if (L >= max_len) break;
    }
    return best;
}

static DecodeWorkspace plan_workspace(int batch, int q_heads, int kv_heads, int dim, int64_t max_len) {
    DecodeWorkspace w{};
    const int64_t units = (int64_t)batch * kv_heads;
    const int group = q_heads / kv_heads;
    w.chunk = choose_chunk(units, std::max<int64_t>(max_len, 1), (int64_t)sm_count() * DEC_WARPS);
    w.nchunks = (int)std::max<int64_t>(1, (max_len + w.chunk - 1) / w.chunk);
    size_t off = 0;
    w.off_status = off; off = align_up(off + 256, 256);
    w.off_qfrag = off;  off = align_up(off + (size_t)units * dim * 16, 256);   // (dim/16) x 64 words
    w.off_qscale = off; off = align_up(off + (size_t)units * 8 * 4, 256);
    const size_t parts = (size_t)units * w.nchunks * group;
    w.off_m = off;   off = align_up(off + parts * 4, 256);
    w.off_l = off;   off = align_up(off + parts * 4, 256);
    w.off_acc = off; off = align_up(off + parts * dim * 4, 256);
    w.total = off;
    return w;
}

template <int D, int KB, int VB, bool PAGED>
static int launch_partial(const DecodeParams& p, cudaStream_t st) {
    using C = DecodeCfg<D, KB, VB>;
    constexpr int NS = (C::STAGE * DEC_WARPS * 8 + C::LUTK_BYTES + C::LUTV_BYTES <= 200 * 1024) ? 8 : 4;
    const size_t smem = (size_t)C::LUTK_BYTES + C::LUTV_BYTES + (size_t)DEC_WARPS * NS * C::STAGE + DEC_WARPS * NS * 8;
    auto kern = decode_partial_kernel<D, KB, VB, PAGED, DEC_WARPS, NS>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t items = (int64_t)p.batch * p.kv_heads * p.nchunks;
    const int grid = (int)std::min<int64_t>(sm_count(), ceil_div(items, DEC_WARPS));
    kern<<<grid, DEC_WARPS * 32, smem, st>>>(p);
    return check_launch("decode_partial");
}

template <int D, bool PAGED>
static int dispatch_bits(int kbits, int vbits, const DecodeParams& p, cudaStream_t st) {
#define TQB_CASE(kb, vb) if (kbits == kb && vbits == vb) return launch_partial<D, kb, vb, PAGED>(p, st);
    TQB_CASE(4, 2) TQB_CASE(4, 3) TQB_CASE(4, 4)
    TQB_CASE(3, 2) TQB_CASE(3, 3) TQB_CASE(3, 4)
    TQB_CASE(2, 2) TQB_CASE(2, 3) TQB_CASE(2, 4)
#undef TQB_CASE
    return fail(TQB_ERR_UNSUPPORTED, "decode_attention: key/value bits must be 2..4, got %d/%d", kbits, vbits);
}

}  // namespace tqb

extern "C" size_t tqb_decode_attention_workspace_bytes(int batch, int q_heads, int kv_heads, int dim,
                                                       int64_t max_len) {
    if (batch <= 0 || kv_heads <= 0 || q_heads <= 0 || dim <= 0 || q_heads % kv_heads) return 0;
    return tqb::plan_workspace(batch, q_heads, kv_heads, dim, max_len).total;
}

extern "C" int tqb_decode_attention(const void* query, int q_dtype, int batch, int q_heads, int kv_heads,
                                    int dim, const uint8_t* k_packed, const float* k_norms,
                                    const uint8_t* v_packed, const float* v_norms, int64_t max_seq,
                                    const int32_t* seq_lens, int64_t max_len, const int32_t* block_tables,
                                    int max_blocks, int block_size, const float* rot_k, const float* cent_k,
                                    int kbits, const float* rot_v, const float* cent_v, int vbits, float scale,
                                    void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                                    void* stream) {
    using namespace tqb;
    TQB_REQUIRE(batch >= 0 && q_heads > 0 && kv_heads > 0, "decode_attention: bad head counts");
    TQB_REQUIRE(q_heads % kv_heads == 0, "decode_attention: q_heads (%d) must be a multiple of kv_heads (%d)",
                q_heads, kv_heads);
    const int group = q_heads / kv_heads;
    if (dim != 64 && dim != 128)
        return fail(TQB_ERR_UNSUPPORTED, "decode_attention: head_dim must be 64 or 128, got %d", dim);
    if (group > 8) return fail(TQB_ERR_UNSUPPORTED, "decode_attention: at most 8 query heads per KV head, got %d", group);
    if (batch == 0) return TQB_OK;
    TQB_REQUIRE(query && k_packed && k_norms && v_packed && v_norms && seq_lens && rot_k && cent_k && rot_v &&
                cent_v && workspace && out, "decode_attention: null pointer");
    TQB_REQUIRE(max_len >= 0, "decode_attention: negative max_len");
    const bool paged = block_tables != nullptr;
    if (paged) {
        TQB_REQUIRE(block_size > 0 && block_size % 16 == 0, "decode_attention: block_size must be a multiple of 16, got %d", block_size);
        TQB_REQUIRE(max_blocks > 0 && (int64_t)max_blocks * block_size >= max_len, "decode_attention: block table shorter than max_len");
    } else {
        TQB_REQUIRE(max_seq % 16 == 0 && max_seq >= max_len, "decode_attention: max_seq (%lld) must be a multiple of 16 and >= max_len (%lld)",
                    (long long)max_seq, (long long)max_len);
    }
    TQB_REQUIRE(((uintptr_t)k_packed | (uintptr_t)v_packed | (uintptr_t)k_norms | (uintptr_t)v_norms) % 16 == 0,
                "decode_attention: cache arrays must be 16-byte aligned");
    TQB_REQUIRE((uintptr_t)workspace % 256 == 0, "decode_attention: workspace must be 256-byte aligned");
    const DecodeWorkspace w = plan_workspace(batch, q_heads, kv_heads, dim, max_len);
    if (workspace_bytes < w.total)
        return fail(TQB_ERR_WORKSPACE, "decode_attention: workspace %zu bytes < required %zu", workspace_bytes, w.total);

    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    DecodeParams p{};
    p.k_packed = k_packed; p.k_norms = k_norms; p.v_packed = v_packed; p.v_norms = v_norms;
    p.seq_lens = seq_lens; p.block_tables = block_tables; p.max_seq = max_seq;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = group;
    p.max_blocks = max_blocks; p.block_size = block_size; p.chunk = w.chunk; p.nchunks = w.nchunks;
    p.cent_k = cent_k; p.cent_v = cent_v;
    p.status = reinterpret_cast<int*>(ws + w.off_status);
    uint32_t* qfrag = reinterpret_cast<uint32_t*>(ws + w.off_qfrag);
    float* qscale = reinterpret_cast<float*>(ws + w.off_qscale);
    p.qfrag = qfrag; p.qscale = qscale;
    p.part_m = reinterpret_cast<float*>(ws + w.off_m);
    p.part_l = reinterpret_cast<float*>(ws + w.off_l);
    p.part_acc = reinterpret_cast<float*>(ws + w.off_acc);
    cudaStream_t st = (cudaStream_t)stream;
    const int units = batch * kv_heads;

    switch (q_dtype) {
        case TQB_F32: rotate_query_kernel<float><<<units, 128, 0, st>>>((const float*)query, q_heads, kv_heads, group, dim, rot_k, scale, qfrag, qscale, p.status); break;
        case TQB_F16: rotate_query_kernel<__half><<<units, 128, 0, st>>>((const __half*)query, q_heads, kv_heads, group, dim, rot_k, scale, qfrag, qscale, p.status); break;
        case TQB_BF16: rotate_query_kernel<__nv_bfloat16><<<units, 128, 0, st>>>((const __nv_bfloat16*)query, q_heads, kv_heads, group, dim, rot_k, scale, qfrag, qscale, p.status); break;
        default: return fail(TQB_ERR_INVALID, "decode_attention: unknown query dtype %d", q_dtype);
    }
    if (int e = check_launch("rotate_query")) return e;

    if (max_len > 0) {
        int e;
        if (dim == 64) e = paged ? dispatch_bits<64, true>(kbits, vbits, p, st) : dispatch_bits<64, false>(kbits, vbits, p, st);
        else e = paged ? dispatch_bits<128, true>(kbits, vbits, p, st) : dispatch_bits<128, false>(kbits, vbits, p, st);
        if (e) return e;
    }

    switch (out_dtype) {
        case TQB_F32: decode_merge_kernel<float><<<units * group, dim, 0, st>>>(p, dim, rot_v, (float*)out); break;
        case TQB_F16: decode_merge_kernel<__half><<<units * group, dim, 0, st>>>(p, dim, rot_v, (__half*)out); break;
        case TQB_BF16: decode_merge_kernel<__nv_bfloat16><<<units * group, dim, 0, st>>>(p, dim, rot_v, (__nv_bfloat16*)out); break;
        default: return fail(TQB_ERR_INVALID, "decode_attention: unknown output dtype %d", out_dtype);
    }
    return check_launch("decode_merge");
}
