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
#include "tiled_layout.cuh"

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
    const uint8_t* store;            // tiled records (tiled_layout.cuh)
    const int32_t* seq_lens; const int32_t* block_tables;
    int64_t max_seq;                 // token pitch of a unit (contiguous cache), multiple of 16
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
// normalised query coordinates (16ks + 8half + 2t, +1); heads >= group are zero columns.
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
            const int dlo = 16 * ks + 8 * half + 2 * t, dhi = dlo + 1;   // k index = dimension
            const float inv = 1.0f / qmax[g];
            lo = qr[g][dlo] * inv;
            hi = qr[g][dhi] * inv;
        }
        qfrag[((int64_t)u * ksteps + ks) * 64 + rem] = pack_half2(lo, hi);
    }
}


// =================================================================================================
// 2. streaming partial attention over tiled records
// =================================================================================================
template <int D, int KB, int VB>
struct DecodeCfg {
    static constexpr int KL = D * KB / 16, VL = D * VB / 16;       // bytes per lane
    static constexpr int KSEC = 32 * KL, VSEC = 32 * VL;
    static constexpr int REC = KSEC + VSEC + 128;                   // one 16-token record
    static constexpr int LUTK_ENTRIES = 1 << (2 * KB);
    static constexpr int LUTV_ENTRIES = VB == 2 ? 256 : (1 << (2 * VB));
    static constexpr int LUTV_WORDS = VB == 2 ? 2 : 1;             // 8-byte entries for 2-bit values
    static constexpr int LUTK_BYTES = LUTK_ENTRIES * 32 * 4;
    static constexpr int LUTV_BYTES = LUTV_ENTRIES * 32 * 4 * LUTV_WORDS;
    static constexpr int MT = D / 16;                               // m-tiles of O^T / k-steps of the scores
    static constexpr int WARPS = D == 64 ? 16 : 8;
    static constexpr int RPS = D == 64 ? 4 : 2;                     // records per pipeline stage
    static constexpr int NS = D == 64 ? 2 : 4;                      // stages per warp
    static constexpr int STAGE = RPS * REC;
    static constexpr size_t SMEM = (size_t)LUTK_BYTES + LUTV_BYTES + (size_t)WARPS * NS * STAGE + WARPS * NS * 8 + 128;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// A lane's chunk of NB bytes -> 32-bit registers, with the widest loads the chunk's alignment allows.
template <int NB>
__device__ __forceinline__ void load_chunk(const uint8_t* p, uint32_t (&w)[NB / 4]) {
    if (NB % 16 == 0) {
#pragma unroll
        for (int i = 0; i < NB / 16; i++) {
            const uint4 v = reinterpret_cast<const uint4*>(p)[i];
            w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
        }
    } else if (NB % 8 == 0) {
#pragma unroll
        for (int i = 0; i < NB / 8; i++) {
            const uint2 v = reinterpret_cast<const uint2*>(p)[i];
            w[2 * i] = v.x; w[2 * i + 1] = v.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < NB / 4; i++) w[i] = reinterpret_cast<const uint32_t*>(p)[i];
    }
}

// Byte offset of a table entry: (field value) << SHIFT, taken straight out of the chunk registers.
// `bit` and `bits` are compile-time constants after unrolling, so this is one shift and one mask
// (a funnel shift when the field straddles two registers).
template <int NW, int SHIFT>
__device__ __forceinline__ uint32_t lut_offset(const uint32_t (&w)[NW], int bit, int bits) {
    const int i = bit >> 5, s = bit & 31;
    uint32_t v;
    if (s + bits <= 32) v = (s >= SHIFT) ? (w[i] >> (s - SHIFT)) : (w[i] << (SHIFT - s));
    else v = __funnelshift_r(w[i], w[(i + 1) < NW ? (i + 1) : i], s) << SHIFT;
    return v & (((1u << bits) - 1u) << SHIFT);
}

// Position of a warp in its stream of pipeline stages: items (unit, chunk) are dealt round-robin to
// warps; an item is cut into blocks of RPS records.
template <int RPS>
struct StageCursor {
    int64_t item, total_items, stride;
    int blk, nblk, ntiles;
    int unit, b, h, chunk_idx, tok0, tok_end;
    __device__ __forceinline__ bool valid() const { return item < total_items; }
    __device__ __forceinline__ int tiles_here() const { return min(RPS, ntiles - blk * RPS); }
    __device__ __forceinline__ void open(const DecodeParams& p) {
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
                nblk = (ntiles + RPS - 1) / RPS;
                blk = 0;
                return;
            }
            item += stride;
        }
    }
    __device__ __forceinline__ void next(const DecodeParams& p) {
        if (++blk == nblk) { item += stride; open(p); }
    }
};

template <int D, int KB, int VB, bool PAGED>
__global__ void __launch_bounds__(DecodeCfg<D, KB, VB>::WARPS * 32, 1) decode_partial_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, KB, VB>;
    constexpr int WARPS = C::WARPS, NS = C::NS, RPS = C::RPS;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* lutK_b = smem_raw;
    uint8_t* lutV_b = smem_raw + C::LUTK_BYTES;
    uint8_t* ring_all = lutV_b + C::LUTV_BYTES;
    uint64_t* bars_all = reinterpret_cast<uint64_t*>(ring_all + (size_t)WARPS * NS * C::STAGE);
    float* s_c = reinterpret_cast<float*>(bars_all + WARPS * NS);   // 16 key + 16 value centroids

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t* ring = ring_all + (size_t)warp * NS * C::STAGE;
    const uint32_t bar0 = smem_u32(bars_all + warp * NS);

    if (threadIdx.x < 16) {
        s_c[threadIdx.x] = threadIdx.x < (1 << KB) ? p.cent_k[threadIdx.x] : 0.0f;
        s_c[16 + threadIdx.x] = threadIdx.x < (1 << VB) ? p.cent_v[threadIdx.x] : 0.0f;
    }
    if (lane == 0)
        for (int s = 0; s < NS; s++) mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // ---- lookup tables: entry x replicated for the 32 lanes at word x*32 + lane (no bank conflicts)
    {
        uint32_t* lutK = reinterpret_cast<uint32_t*>(lutK_b);
        for (int x = warp; x < C::LUTK_ENTRIES; x += WARPS) {
            int clo, chi;
            tl_key_field_codes((uint32_t)x, KB, clo, chi);
            lutK[x * 32 + lane] = pack_half2(s_c[clo], s_c[chi]);
        }
        for (int x = warp; x < C::LUTV_ENTRIES; x += WARPS) {
            if (VB == 2) {
                int ag, bg, ag8, bg8;
                tl_val_quad_codes((uint32_t)x, ag, bg, ag8, bg8);
                reinterpret_cast<uint2*>(lutV_b)[x * 32 + lane] =
                    make_uint2(pack_half2(s_c[16 + ag], s_c[16 + bg]), pack_half2(s_c[16 + ag8], s_c[16 + bg8]));
            } else {
                int ca, cb;
                tl_val_pair_codes((uint32_t)x, VB, ca, cb);
                reinterpret_cast<uint32_t*>(lutV_b)[x * 32 + lane] = pack_half2(s_c[16 + ca], s_c[16 + cb]);
            }
        }
    }
    __syncthreads();
    const uint8_t* lutK_lane = lutK_b + lane * 4;
    const uint8_t* lutV_lane = lutV_b + lane * 4 * C::LUTV_WORDS;

    StageCursor<RPS> pc, cc;   // producer / consumer cursors over the same stream
    pc.item = (int64_t)blockIdx.x * WARPS + warp;
    pc.total_items = (int64_t)p.batch * p.kv_heads * p.nchunks;
    pc.stride = (int64_t)gridDim.x * WARPS;
    pc.blk = pc.nblk = pc.ntiles = 0;
    pc.open(p);
    cc = pc;

    // lane 0 issues the bulk copies of one stage: a run of records of one unit (contiguous cache) or
    // record by record through the block table (paged cache)
    auto issue = [&](const StageCursor<RPS>& cur, int s) {
        if (lane == 0) {
            const int nt = cur.tiles_here();
            const int tile0 = cur.tok0 / TILE + cur.blk * RPS;
            const uint32_t dst = smem_u32(ring + (size_t)s * C::STAGE);
            const uint32_t bar = bar0 + 8 * s;
            // order this warp's earlier generic-proxy reads of the stage before the async-proxy overwrite
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar, (uint32_t)(nt * C::REC));
            if (PAGED) {
                const int rpb = p.block_size / TILE;   // records per page
                for (int i = 0; i < nt; i++) {
                    const int tile = tile0 + i;
                    const int blk = p.block_tables[(int64_t)cur.b * p.max_blocks + tile / rpb];
                    const int64_t rec = ((int64_t)blk * p.kv_heads + cur.h) * rpb + tile % rpb;
                    bulk_g2s(dst + i * C::REC, p.store + rec * C::REC, C::REC, bar);
                }
            } else {
                const int64_t rec = (int64_t)cur.unit * (p.max_seq / TILE) + tile0;
                bulk_g2s(dst, p.store + rec * C::REC, (uint32_t)(nt * C::REC), bar);
            }
        }
    };

    uint32_t issued = 0, consumed = 0;
    while (issued < NS && pc.valid()) { issue(pc, issued % NS); pc.next(p); issued++; }

    float m0 = NEG_INF, m1 = NEG_INF, l0 = 0.0f, l1 = 0.0f, qs0 = 0.0f, qs1 = 0.0f;
    float O[C::MT][4];
    uint32_t qf[C::MT][2];
    bool failed = false;

    while (cc.valid()) {
        if (cc.blk == 0) {
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
        const int nt = cc.tiles_here();
        const int tok_blk = cc.tok0 + cc.blk * RPS * TILE;

#pragma unroll 1
        for (int i = 0; i < nt; i++) {
            const uint8_t* rec = ring + (size_t)s * C::STAGE + i * C::REC;
            const float* nk = reinterpret_cast<const float*>(rec + C::KSEC + C::VSEC);
            const float* nv = nk + TILE;
            const int tokb = tok_blk + i * TILE;
            const bool val_g = tokb + g < cc.tok_end, val_g8 = tokb + g + 8 < cc.tok_end;

            // ---- scores: 16 tokens x 8 heads ----
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                uint32_t kw[C::KL / 4];
                load_chunk<C::KL>(rec + lane * C::KL, kw);
#pragma unroll
                for (int ks = 0; ks < C::MT; ks++) {
                    uint32_t a[4];
#pragma unroll
                    for (int half = 0; half < 2; half++)
#pragma unroll
                        for (int second = 0; second < 2; second++) {
                            const uint32_t off = lut_offset<C::KL / 4, 7>(kw, tl_key_field_bit(D, KB, ks, half, second), 2 * KB);
                            a[2 * half + second] = *reinterpret_cast<const uint32_t*>(lutK_lane + off);
                        }
                    mma_f16(sc, a, qf[ks][0], qf[ks][1]);
                }
            }
            const float nkg = val_g ? nk[g] : 0.0f, nkg8 = val_g8 ? nk[g + 8] : 0.0f;
            const float s0 = val_g ? sc[0] * (nkg * qs0) : NEG_INF, s1 = val_g ? sc[1] * (nkg * qs1) : NEG_INF;
            const float s2 = val_g8 ? sc[2] * (nkg8 * qs0) : NEG_INF, s3 = val_g8 ? sc[3] * (nkg8 * qs1) : NEG_INF;

            // ---- online softmax, lazy maximum ----
            float tm0 = fmaxf(s0, s2), tm1 = fmaxf(s1, s3);
            if (__any_sync(0xffffffffu, (tm0 > m0 + RESCALE_SLACK) || (tm1 > m1 + RESCALE_SLACK))) {
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, o));
                    tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, o));
                }
                const float mn0 = fmaxf(m0, tm0), mn1 = fmaxf(m1, tm1);
                const float f0 = (mn0 == NEG_INF) ? 1.0f : ex2_approx(m0 - mn0);
                const float f1 = (mn1 == NEG_INF) ? 1.0f : ex2_approx(m1 - mn1);
                l0 *= f0; l1 *= f1;
#pragma unroll
                for (int mt = 0; mt < C::MT; mt++) { O[mt][0] *= f0; O[mt][2] *= f0; O[mt][1] *= f1; O[mt][3] *= f1; }
                m0 = mn0; m1 = mn1;
            }
            const float mu0 = (m0 == NEG_INF) ? 0.0f : m0, mu1 = (m1 == NEG_INF) ? 0.0f : m1;
            const float p0 = ex2_approx(s0 - mu0), p1 = ex2_approx(s1 - mu1);
            const float p2 = ex2_approx(s2 - mu0), p3 = ex2_approx(s3 - mu1);
            l0 += p0 + p2; l1 += p1 + p3;
            const float nvg = val_g ? nv[g] : 0.0f, nvg8 = val_g8 ? nv[g + 8] : 0.0f;
            // P^T as B operand: (k = tokens, col = head) through two 8x8 transposes
            const uint32_t pb0 = movmatrix_trans(pack_half2_sat(p0 * nvg, p1 * nvg));
            const uint32_t pb1 = movmatrix_trans(pack_half2_sat(p2 * nvg8, p3 * nvg8));

            // ---- O^T += V^T P^T : (dims x tokens) x (tokens x heads) ----
            {
                uint32_t vw[C::VL / 4];
                load_chunk<C::VL>(rec + C::KSEC + lane * C::VL, vw);
#pragma unroll
                for (int mt = 0; mt < C::MT; mt++) {
                    uint32_t a[4];
                    if (VB == 2) {
                        const uint2 e0 = *reinterpret_cast<const uint2*>(
                            lutV_lane + lut_offset<C::VL / 4, 8>(vw, tl_val_field_bit(VB, mt, 0, 0), 8));
                        const uint2 e1 = *reinterpret_cast<const uint2*>(
                            lutV_lane + lut_offset<C::VL / 4, 8>(vw, tl_val_field_bit(VB, mt, 1, 0), 8));
                        a[0] = e0.x; a[1] = e0.y; a[2] = e1.x; a[3] = e1.y;
                    } else {
#pragma unroll
                        for (int half = 0; half < 2; half++)
#pragma unroll
                            for (int rs = 0; rs < 2; rs++)
                                a[2 * half + rs] = *reinterpret_cast<const uint32_t*>(
                                    lutV_lane + lut_offset<C::VL / 4, 7>(vw, tl_val_field_bit(VB, mt, half, rs), 2 * VB));
                    }
                    mma_f16(O[mt], a, pb0, pb1);
                }
            }
        }

        // ---- stage is free: refill it with the stage NS ahead ----
        __syncwarp();
        if (pc.valid()) { issue(pc, s); pc.next(p); issued++; }
        consumed++;

        // ---- end of item: write the partial (rotated space, unnormalised) ----
        if (cc.blk + 1 == cc.nblk) {
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
                const int dg = 16 * mt + g, dg8 = dg + 8;
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
    w.chunk = choose_chunk(units, std::max<int64_t>(max_len, 1), (int64_t)sm_count() * (dim == 64 ? 16 : 8));
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
    auto kern = decode_partial_kernel<D, KB, VB, PAGED>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
    const int64_t items = (int64_t)p.batch * p.kv_heads * p.nchunks;
    const int grid = (int)std::min<int64_t>(sm_count(), ceil_div(items, C::WARPS));
    kern<<<grid, C::WARPS * 32, C::SMEM, st>>>(p);
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
                                    int dim, const uint8_t* store, int64_t max_seq,
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
    TQB_REQUIRE(query && store && seq_lens && rot_k && cent_k && rot_v &&
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
    TQB_REQUIRE((uintptr_t)store % 16 == 0, "decode_attention: the record store must be 16-byte aligned");
    TQB_REQUIRE((uintptr_t)workspace % 256 == 0, "decode_attention: workspace must be 256-byte aligned");
    const DecodeWorkspace w = plan_workspace(batch, q_heads, kv_heads, dim, max_len);
    if (workspace_bytes < w.total)
        return fail(TQB_ERR_WORKSPACE, "decode_attention: workspace %zu bytes < required %zu", workspace_bytes, w.total);

    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    DecodeParams p{};
    p.store = store;
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
