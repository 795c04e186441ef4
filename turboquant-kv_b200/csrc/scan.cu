// scan.cu -- packed-code inner-product scan with top-k (TurboQuantIndex.search).
//
// Replaces turboquant::search_packed (upstream csrc/core/turboquant_core.cpp:407-514): for every
// query, score_i = norm_i * sum_j (R q)_j * centroid[code_ij] over all database rows, keep the k best.
//
// Three launches:
//   1. scan_prepare_kernel  rotates the queries (sequential float32 sums, the upstream order), and
//                           writes them as mma.sync B fragments split into fp16 hi + lo parts.
//   2. scan_kernel          persistent warps stream 16-row tiles of packed codes + norms through a
//                           per-warp TMA ring (cp.async.bulk + mbarrier).  Codes become fp16 centroid
//                           pairs through a 256-entry shared-memory table indexed by one byte (= two
//                           codes); one MMA per 16 dims (c_fp16 x [q_hi | q_lo]) scores 4 queries at
//                           once.  Each warp keeps a sorted candidate list of kk = k + 8 entries per
//                           query; insertions are warp-cooperative and rare once the threshold has risen.
//   3. scan_merge_kernel    per query: selects the best k + 24 of all lists' candidates, RE-SCORES them in
//                           float32 in exactly the upstream summation order (table[j][code] added for
//                           j = 0..d-1, then * norm), sorts by (score desc, id asc) and emits k.
// The reported scores are therefore bit-identical to the upstream C++ arithmetic; the tensor-core
// pass only has to RANK: its scores carry the fp16 rounding of the 16 centroids (relative 2^-12 per
// term, the queries keep 22 bits).  A true top-k row is lost only if more rows than the margin overtake
// it through that rounding: 8 within the few thousand rows one warp sees, 24 within the whole database.
//
// Dims 64 and 128 with 2..4 bits take the tensor-core path; every other supported shape takes
// scan_generic_kernel (one row per lane, float32 table lookups) with the same list and merge code; so do
// Prod-mode rows (tqb_scan_topk_prod), with a second term for the QJL sign plane.
//
// scan_records_kernel is the same scan over the key-only records of tiled_layout.cuh (what TurboQuantIndex
// stores): one table lookup per two codes, one MMA per 16 dims on the centroids' fp16 values, and eight
// queries per pass as single fp16 columns for batched calls (four as hi + lo pairs for short calls).
// A call with many query groups gives each group few, large CTAs in full waves (rec_ctas_per_group), and the
// warps of a CTA share a threshold per query (the r-th best of every warp bounds what the CTA can emit).
#include "common.cuh"
#include "decode_bits.cuh"
#include "pipe.cuh"
#include "tiled_layout.cuh"

#include <cmath>
#include <mutex>

namespace tqb {

constexpr int SCAN_TILE = 16;
constexpr int SCAN_MARGIN = 8;          // extra candidates a list keeps beyond k
constexpr int SCAN_SELECT_MARGIN = 24;  // extra candidates the merge re-scores exactly beyond k
constexpr int SCAN_WARPS = 8;
constexpr int QG = 4;                   // queries per tensor-core pass over upstream rows (fp16 hi + lo query columns)
constexpr int RQ = 8;                   // queries per pass over records (one fp16 column each: the pass only ranks)
// A CTA of the record scan that merges its warps' lists emits its best REC_OUT_LISTS * kk candidates, as that many
// sorted lists: with few CTAs per query the margin beyond k has to come from within the CTA.
constexpr int REC_OUT_LISTS = 2;
constexpr float CENT_SCALE = 1024.0f;   // keeps the fp16 lo parts out of the subnormal range
constexpr float QUERY_SCALE = 16.0f;
constexpr int ID_NONE = 0x7fffffff;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void s_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void s_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool s_mbar_wait(uint32_t bar, uint32_t parity) { return mbar_wait(bar, parity); }
__device__ __forceinline__ void s_bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void s_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                      uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t s_pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Candidates kept per list for a top-k request.
__host__ __device__ inline int scan_kk(int k) { return k + SCAN_MARGIN; }

// (score, id) ordering used everywhere: higher score first, lower id first among equal scores.
__device__ __forceinline__ bool better(float s, int id, float ts, int tid) {
    return s > ts || (s == ts && id < tid);
}

struct ScanParams {
    const uint8_t* packed; const float* norms; int64_t n;
    const uint8_t* records;             // non-null: the database as key-only 16-row records (tiled_layout.cuh)
    int combine;                        // record scan: sorted candidate lists a CTA emits after merging its warps'
                                        // (1 or REC_OUT_LISTS); 0 = every warp writes its own list
    int dim, bits, nq, k, kk;           // kk = scan_kk(k) candidates kept per list
    const float* rot; const float* cent; const float* queries;
    // Prod-mode rows (Algorithm 2): `packed` holds the MSE codes at `bits` (= bit_width - 1), plus one QJL sign
    // per dimension, the residual norm, and the query projected by the QJL matrix (qsign = S q).  Null: MSE rows.
    const uint8_t* signs; const float* res_norms; const float* qsign; float sign_coef;
    int64_t id_offset;
    int lists_per_query;                // candidate lists written per query (= warps in the grid)
    // workspace views
    int* status; float* qrot; uint32_t* qfrag; float* qscale;
    float* cand_s; int* cand_id;        // (nq, lists_per_query, kk)
    float* out_scores; int64_t* out_ids;
};

// ---- warp-cooperative sorted list in shared memory ----------------------------------------------
// ls / li: kk entries sorted best-first.  Inserts (s, id) if it beats the last entry.  All 32 lanes
// call with the same arguments.
__device__ __forceinline__ void list_insert(float* ls, int* li, int kk, float s, int id, int lane) {
    if (!better(s, id, ls[kk - 1], li[kk - 1])) return;
    // position = number of entries better than the candidate
    int cnt = 0;
    for (int e = lane; e < kk; e += 32) cnt += better(ls[e], li[e], s, id) ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    const int pos = cnt;
    // shift [pos, kk-1) down by one: read everything first, then write
    float ts[(TQB_SCAN_MAX_K + SCAN_MARGIN + 31) / 32];
    int ti[(TQB_SCAN_MAX_K + SCAN_MARGIN + 31) / 32];
    int c = 0;
    for (int e = lane; e < kk; e += 32, c++) {
        if (e > pos) { ts[c] = ls[e - 1]; ti[c] = li[e - 1]; }
    }
    __syncwarp();
    c = 0;
    for (int e = lane; e < kk; e += 32, c++) {
        if (e > pos) { ls[e] = ts[c]; li[e] = ti[c]; }
        else if (e == pos) { ls[e] = s; li[e] = id; }
    }
    __syncwarp();
}


// =================================================================================================
// 1. query rotation (+ B fragments for the tensor-core path)
// =================================================================================================
// One CTA per group of QN queries (QN for scans over upstream rows, RQ for scans over records).  q_rot[j] = sum_k q[k] * R[j][k], accumulated in k order with
// separate multiply and add, the arithmetic of csrc/core/turboquant_core.cpp:425-433.
// Fragment word layout: qfrag[group][ks][lane] = uint2 {half 0, half 1} of the B operand;
// QN = QN: MMA column n = lane/4 holds query n/2 of the group: even n its fp16 hi part, odd n its lo part,
// so that the two columns of a query add up to a 22-bit query against the fp16 centroids.
// QN = RQ: column n holds query n, fp16 (the pass over records only ranks; survivors are re-scored exactly).
template <int QN>
__global__ void __launch_bounds__(128) scan_prepare_kernel(const ScanParams p, int use_mma) {
    extern __shared__ float sm[];
    float* qr = sm + p.dim;             // QN * dim (rotated queries); the raw queries follow
    __shared__ float qmax[QN];
    const int grp = blockIdx.x;
    pdl_wait();
    pdl_trigger();
    if (grp == 0 && threadIdx.x == 0) *p.status = 0;
    // all QN queries of the group go through one pass over R: row j is read once (128-bit loads), each
    // query keeps its own sum, accumulated in k order with separate multiply and add
    float* qin_all = qr + QN * p.dim;        // QN * dim (the caller sizes the shared memory for it)
    for (int e = threadIdx.x; e < QN * p.dim; e += blockDim.x) {
        const int jq = e / p.dim, k = e - jq * p.dim, q = grp * QN + jq;
        qin_all[e] = q < p.nq ? p.queries[(int64_t)q * p.dim + k] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < p.dim; j += blockDim.x) {
        const float4* row = reinterpret_cast<const float4*>(p.rot + (int64_t)j * p.dim);
        float s[QN];
#pragma unroll
        for (int jq = 0; jq < QN; jq++) s[jq] = 0.0f;
        const int nvalid = min(QN, p.nq - grp * QN);     // queries of this group that exist
#pragma unroll 8
        for (int k4 = 0; k4 < p.dim / 4; k4++) {
            const float4 r = __ldg(row + k4);
#pragma unroll
            for (int jq = 0; jq < QN; jq++) {
                if (jq >= nvalid) break;
                const float* qv = qin_all + jq * p.dim + 4 * k4;
                s[jq] = __fadd_rn(s[jq], __fmul_rn(qv[0], r.x));
                s[jq] = __fadd_rn(s[jq], __fmul_rn(qv[1], r.y));
                s[jq] = __fadd_rn(s[jq], __fmul_rn(qv[2], r.z));
                s[jq] = __fadd_rn(s[jq], __fmul_rn(qv[3], r.w));
            }
        }
#pragma unroll
        for (int jq = 0; jq < QN; jq++) {
            const int q = grp * QN + jq;
            if (q < p.nq) p.qrot[(int64_t)q * p.dim + j] = s[jq];
            qr[jq * p.dim + j] = q < p.nq ? s[jq] : 0.0f;
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int jq = warp; jq < QN; jq += (int)(blockDim.x >> 5)) {
        float mx = 0.0f;
        for (int k = lane; k < p.dim; k += 32) mx = fmaxf(mx, fabsf(qr[jq * p.dim + k]));
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) {
            qmax[jq] = mx;
            const int q = grp * QN + jq;
            if (q < p.nq) p.qscale[q] = mx / (CENT_SCALE * QUERY_SCALE);
        }
    }
    __syncthreads();
    if (!use_mma) return;
    const int ksteps = p.dim >> 4;
    for (int idx = threadIdx.x; idx < ksteps * 32; idx += blockDim.x) {
        const int ks = idx >> 5, fl = idx & 31, g = fl >> 2, t = fl & 3;
        const int jq = QN == RQ ? g : g >> 1, part = QN == RQ ? 0 : g & 1;
        const float inv = qmax[jq] > 0.0f ? QUERY_SCALE / qmax[jq] : 0.0f;
        uint32_t w[2];
        for (int half = 0; half < 2; half++) {
            int dlo, dhi;
            if (use_mma == 2) { dlo = 16 * ks + 8 * half + 2 * t; dhi = dlo + 1; }   // record layout: dims in order
            else pair_dims(p.dim, t, 2 * ks + half, dlo, dhi);
            const float a = qr[jq * p.dim + dlo] * inv, b = qr[jq * p.dim + dhi] * inv;
            const float ah = __half2float(__float2half_rn(a)), bh = __half2float(__float2half_rn(b));
            w[half] = part ? s_pack_half2(a - ah, b - bh) : s_pack_half2(ah, bh);
        }
        reinterpret_cast<uint2*>(p.qfrag)[((int64_t)grp * ksteps + ks) * 32 + fl] = make_uint2(w[0], w[1]);
    }
}

// =================================================================================================
// 2a. tensor-core scan
// =================================================================================================
template <int D, int BITS>
struct ScanCfg {
    static constexpr int PD = BITS * D / 8;
    static constexpr int RT = SCAN_TILE * PD;              // rows of a tile
    static constexpr int STAGE = RT + SCAN_TILE * 4;       // + norms
    static constexpr int LUT_ENTRIES = 1 << (2 * BITS);
    static constexpr int LUT_BYTES = LUT_ENTRIES * 32 * 4; // one fp16 pair per lane and entry
    static constexpr int KS = D / 16;
};

template <int D, int BITS, int NS>
__global__ void __launch_bounds__(SCAN_WARPS * 32, 1) scan_kernel(const ScanParams p) {
    using C = ScanCfg<D, BITS>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem_raw);
    uint8_t* ring_all = smem_raw + C::LUT_BYTES;
    uint64_t* bars_all = reinterpret_cast<uint64_t*>(ring_all + (size_t)SCAN_WARPS * NS * C::STAGE);
    float* lists_s = reinterpret_cast<float*>(bars_all + SCAN_WARPS * NS);
    int* lists_i = reinterpret_cast<int*>(lists_s + SCAN_WARPS * QG * p.kk);
    __shared__ float s_c[16];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int grp = blockIdx.y;
    uint8_t* ring = ring_all + (size_t)warp * NS * C::STAGE;
    const uint32_t bar0 = s_u32(bars_all + warp * NS);
    float* ls = lists_s + (size_t)warp * QG * p.kk;
    int* li = lists_i + (size_t)warp * QG * p.kk;

    if (threadIdx.x < 16) s_c[threadIdx.x] = threadIdx.x < (1 << BITS) ? p.cent[threadIdx.x] * CENT_SCALE : 0.0f;
    if (lane == 0)
        for (int s = 0; s < NS; s++) s_mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int e = lane; e < QG * p.kk; e += 32) { ls[e] = -__builtin_huge_valf(); li[e] = ID_NONE; }
    __syncthreads();
    for (int x = warp; x < C::LUT_ENTRIES; x += SCAN_WARPS) {
        int clo, chi;
        pair_index_codes<BITS>((uint32_t)x, clo, chi);
        lut[x * 32 + lane] = s_pack_half2(s_c[clo], s_c[chi]);
    }
    __syncthreads();

    // B fragments of this query group stay in registers for the whole scan
    uint2 qf[C::KS];
    {
        const uint2* src = reinterpret_cast<const uint2*>(p.qfrag) + ((int64_t)grp * C::KS) * 32 + lane;
#pragma unroll
        for (int ks = 0; ks < C::KS; ks++) qf[ks] = src[ks * 32];
    }
    const int myq = grp * QG + t;                       // the query whose scores this lane receives
    const float qsc = myq < p.nq ? p.qscale[myq] : 0.0f;
    float thr_s = -__builtin_huge_valf();
    int thr_i = ID_NONE;

    // full tiles only: the last n % 16 rows are scored by the merge kernel
    const int64_t ntiles = p.n / SCAN_TILE;
    const int64_t wstride = (int64_t)gridDim.x * SCAN_WARPS;
    const int64_t first = (int64_t)blockIdx.x * SCAN_WARPS + warp;

    auto issue = [&](int64_t tile, int s) {
        if (lane == 0) {
            const int64_t row = tile * SCAN_TILE;
            const uint32_t dst = s_u32(ring + (size_t)s * C::STAGE);
            const uint32_t bar = bar0 + 8 * s;
            // order this warp's earlier generic-proxy reads of the stage before the async-proxy overwrite
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            s_mbar_expect_tx(bar, C::STAGE);
            s_bulk_g2s(dst, p.packed + row * C::PD, C::RT, bar);
            s_bulk_g2s(dst + C::RT, p.norms + row, SCAN_TILE * 4, bar);
        }
    };

    int64_t ptile = first, ctile = first;
    uint32_t issued = 0, consumed = 0;
    while (issued < NS && ptile < ntiles) { issue(ptile, issued % NS); ptile += wstride; issued++; }
    bool failed = false;

    for (; ctile < ntiles; ctile += wstride) {
        const int s = consumed % NS;
        if (!s_mbar_wait(bar0 + 8 * s, (consumed / NS) & 1)) failed = true;
        if (__any_sync(0xffffffffu, failed)) { failed = true; break; }
        const uint8_t* rt = ring + (size_t)s * C::STAGE;
        const float* nr = reinterpret_cast<const float*>(rt + C::RT);
        const int64_t row0 = ctile * SCAN_TILE;

        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t P[KeyWords<D>::NW][4];
        gather_key_words<D, BITS>(rt, C::PD, g, t, P);
        uint32_t iw[KeyWords<D>::NW][4];
#pragma unroll
        for (int w = 0; w < KeyWords<D>::NW; w++)
#pragma unroll
            for (int u = 0; u < 4; u++) iw[w][u] = pair_index_word<BITS>(P[w], u);
#pragma unroll
        for (int ks = 0; ks < C::KS; ks++) {
            uint32_t e[4];
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int second = 0; second < 2; second++) {
                    int u, w, bl;
                    key_element_slot<D>(2 * ks + half, second != 0, u, w, bl);
                    e[2 * half + second] = lut[((iw[w][u] >> (8 * bl)) & 0xFFu) * 32 + lane];
                }
            s_mma(acc, e[0], e[1], e[2], e[3], qf[ks].x, qf[ks].y);
        }
        const bool v0 = row0 + g < p.n, v1 = row0 + g + 8 < p.n;
        const float sc0 = v0 ? (acc[0] + acc[1]) * (nr[g] * qsc) : 0.0f;
        const float sc1 = v1 ? (acc[2] + acc[3]) * (nr[g + 8] * qsc) : 0.0f;
        const int id0 = (int)(row0 + g), id1 = id0 + 8;

        // ---- candidates: lanes whose score beats their query's threshold ----
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float sc = r ? sc1 : sc0;
            const int id = r ? id1 : id0;
            const bool ok = (r ? v1 : v0) && myq < p.nq && better(sc, id, thr_s, thr_i);
            uint32_t mask = __ballot_sync(0xffffffffu, ok);
            while (mask) {
                const int leader = __ffs(mask) - 1;
                mask &= mask - 1;
                const float bs = __shfl_sync(0xffffffffu, sc, leader);
                const int bid = __shfl_sync(0xffffffffu, id, leader);
                const int bq = leader & 3;
                list_insert(ls + bq * p.kk, li + bq * p.kk, p.kk, bs, bid, lane);
                if (t == bq) { thr_s = ls[bq * p.kk + p.kk - 1]; thr_i = li[bq * p.kk + p.kk - 1]; }
            }
        }

        __syncwarp();
        if (ptile < ntiles) { issue(ptile, s); ptile += wstride; issued++; }
        consumed++;
    }

    if (failed) {
        if (lane == 0) atomicExch(p.status, 1);
        for (uint32_t i = consumed; i < issued; i++) (void)s_mbar_wait(bar0 + 8 * (i % NS), (i / NS) & 1);
    }
    // ---- this warp's candidates -> global ----
    __syncwarp();
    const int64_t wid = (int64_t)blockIdx.x * SCAN_WARPS + warp;
    for (int jq = 0; jq < QG; jq++) {
        const int q = grp * QG + jq;
        if (q >= p.nq) break;
        const int64_t base = ((int64_t)q * p.lists_per_query + wid) * p.kk;
        for (int e = lane; e < p.kk; e += 32) { p.cand_s[base + e] = ls[jq * p.kk + e]; p.cand_id[base + e] = li[jq * p.kk + e]; }
    }
}


// =================================================================================================
// 2c. record scan: the database stored as key-only 16-row records (tiled_layout.cuh)
// =================================================================================================
// Same arithmetic as scan_kernel (one MMA per 16 dims, fp16 centroids x 22-bit queries), but the rows
// arrive in the order the MMA lanes consume them: one shared-memory load brings a lane's code fields of a
// record, and each field (two codes) is the index of a table entry holding the two centroids as an fp16
// pair.  For 4-bit codes a field is one byte and a single byte permute forms the entry's shared address
// (entries 256 bytes apart in a 64 KB window on a 64 KB boundary; the lanes' copies fill the first 128
// bytes of an entry).  One persistent CTA per SM and query group: a
// producer warp streams stages of SR records with one TMA bulk copy each; GROUPS groups of consumer
// warps take the stages in turn, RPW records per warp.  Every wait is bounded.
template <int D, int BITS>
struct RecScanCfg {
    static constexpr int KL = D * BITS / 16;                 // code bytes per lane and record
    static constexpr int KSEC = 32 * KL;
    static constexpr int REC = KSEC + 64;                    // + 16 norms
    static constexpr bool KBYTE = (2 * BITS == 8);
    static constexpr int LUT_ENTRIES = 1 << (2 * BITS);
    static constexpr int LUT_BYTES = LUT_ENTRIES * 256;      // 32 lanes x 4 bytes per entry, entries 256 bytes apart
    static constexpr int KS = D / 16;
    static constexpr int NT = D == 64 ? 4 : 2;               // records a warp has in flight at once
    // Two consumer groups share the ring: with 8 stages each group has 4 stages in flight, which covers
    // the memory latency (a group finishes a stage well within one round trip to HBM).
    static constexpr int WARPS = 16, GROUPS = 2, WPG = WARPS / GROUPS, RPW = NT, SR = WPG * RPW;
    static constexpr int STAGE = SR * REC;
    static constexpr int THREADS = (WARPS + 1) * 32;         // + the producer warp
    static constexpr int DYN = 227 * 1024;
    static constexpr int MAX_NS = 8;
    static constexpr int SHARE_OFF = 8 * (8 + 8 + 8) + 64;   // barriers, stage headers, centroids come first
    static constexpr int FIXED = SHARE_OFF + 8 * (WARPS + 1) * RQ;   // + shared thresholds (one key per warp and query, one per query)
};

// NT records at once: acc[i] = this lane's part of the 16 x 8 score tile of record i.
// qf[ks] = B fragment {half 0, half 1}: column n = query n of the group, fp16.
template <int D, int BITS, int NT>
__device__ __forceinline__ void rec_scan_tiles(uint32_t rec0, uint32_t tab, const uint2 (&qf)[D / 16],
                                               int lane, float (&acc)[NT][4]) {
    using C = RecScanCfg<D, BITS>;
    uint32_t kw[NT][C::KL / 4];
#pragma unroll
    for (int i = 0; i < NT; i++) {
        load_key_chunk<C::KL>(rec0 + i * C::REC, lane, kw[i]);
        acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    }
#pragma unroll
    for (int ks = 0; ks < C::KS; ks++) {
        uint32_t ah[NT][4];
#pragma unroll
        for (int i = 0; i < NT; i++)
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int second = 0; second < 2; second++) {
                    const int bit = tl_key_field_bit(D, BITS, ks, half, second);
                    const uint32_t addr = C::KBYTE ? entry_addr<true>(kw[i], bit, 8, tab)
                                                   : lut_offset<C::KL / 4, 8>(kw[i], bit, 2 * BITS) + tab;
                    ah[i][2 * half + second] = lds32(addr);
                }
#pragma unroll
        for (int i = 0; i < NT; i++) mma_f16(acc[i], ah[i], qf[ks].x, qf[ks].y);
    }
}

// Candidate lists of up to 32 entries live in registers: lane e holds entry e (best first) of each of the
// RQ queries.  Insertion of (s, id) into the list of query bq (warp-uniform): the entries better than the
// candidate form a prefix, everything behind it moves down one lane.
struct RegLists {
    float s[RQ];
    int i[RQ];
};
template <int JQ>
__device__ __forceinline__ void reg_list_insert(RegLists& L, int kk, float s, int id, int lane) {
    const uint32_t ahead = __ballot_sync(0xffffffffu, lane < kk && better(L.s[JQ], L.i[JQ], s, id));
    const int pos = __popc(ahead);
    const float us = __shfl_up_sync(0xffffffffu, L.s[JQ], 1);
    const int ui = __shfl_up_sync(0xffffffffu, L.i[JQ], 1);
    if (lane < kk) {
        if (lane > pos) { L.s[JQ] = us; L.i[JQ] = ui; }
        else if (lane == pos) { L.s[JQ] = s; L.i[JQ] = id; }
    }
}

// The rare path of the record scan, kept out of line so that the streaming loop stays small enough for
// the instruction cache: lanes flagged `ok` offer (sc, id) to the list of the query their lane serves
// (query = lane % 4).  Returns the caller's updated threshold (the tail of its query's list).
struct ScanThreshold { float s; int i; };
// (score, id) as one 64-bit key whose unsigned order is the order of better(): larger key = better candidate
__device__ __forceinline__ unsigned long long thr_key(float s, int id) {
    uint32_t b = __float_as_uint(s + 0.0f);          // (-0 becomes +0: better() holds them equal)
    b ^= (b >> 31) ? 0xffffffffu : 0x80000000u;
    return ((unsigned long long)b << 32) | (uint32_t)(ID_NONE - id);
}
__device__ __forceinline__ ScanThreshold key_thr(unsigned long long k) {
    uint32_t b = (uint32_t)(k >> 32);
    b ^= (b >> 31) ? 0x80000000u : 0xffffffffu;
    return {__uint_as_float(b), ID_NONE - (int)(uint32_t)k};
}
__device__ __forceinline__ ScanThreshold thr_max(ScanThreshold a, ScanThreshold b) {
    return better(b.s, b.i, a.s, a.i) ? b : a;
}
__device__ __noinline__ ScanThreshold rec_scan_offer(float* ls, int* li, int kk, float sc, int id, bool ok,
                                                     ScanThreshold thr, int lane) {
    const int t = lane & 3;
    uint32_t mask = __ballot_sync(0xffffffffu, ok);
    while (mask) {
        const int leader = __ffs(mask) - 1;
        mask &= mask - 1;
        const float bs = __shfl_sync(0xffffffffu, sc, leader);
        const int bid = __shfl_sync(0xffffffffu, id, leader);
        const int bq = leader & 3;
        list_insert(ls + bq * kk, li + bq * kk, kk, bs, bid, lane);
        if (t == bq) { thr.s = ls[bq * kk + kk - 1]; thr.i = li[bq * kk + kk - 1]; }
    }
    return thr;
}

// NQ = RQ: eight queries per pass, one fp16 column each (calls with more than four queries and register lists);
// NQ = QG: four queries per pass in hi + lo column pairs.  REGL: candidate lists of up to 32 entries in
// registers (k <= 24), else in shared memory.
template <int D, int BITS, int NQ, bool REGL>
__global__ void __launch_bounds__(RecScanCfg<D, BITS>::THREADS, 1) scan_records_kernel(const ScanParams p) {
    constexpr bool PAIR = NQ == RQ;                  // a lane serves two queries (columns 2t, 2t+1)
    static_assert(!PAIR || REGL, "eight queries per pass need the register lists");
    using C = RecScanCfg<D, BITS>;
    constexpr int WARPS = C::WARPS, GROUPS = C::GROUPS, WPG = C::WPG, RPW = C::RPW, SR = C::SR, NT = C::NT;
    constexpr uint32_t F_END = 1u << 31;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int grp = blockIdx.y;

    // ---- carve the shared window: [ring A | table (64 KB aligned for byte fields) | misc, lists | ring B] ----
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t end = base + C::DYN;
    uint32_t tab_base, misc, ringA = base;
    int slotsA = 0;
    if (C::KBYTE) {
        tab_base = (base + 65535u) & ~65535u;
        slotsA = (int)((tab_base - base) / C::STAGE);
    } else {
        tab_base = base;
    }
    misc = tab_base + C::LUT_BYTES;
    const uint32_t full_addr = misc, empty_addr = misc + 64, meta_addr = misc + 128, cent_addr = misc + 192;
    // Thresholds shared by the CTA's warps.  A CTA emits its best `nout` candidates per query, so a candidate
    // below the r-th best of EVERY warp (r = ceil(nout / WARPS): WARPS * r candidates of distinct rows are
    // better) cannot be among them.  Each warp publishes its r-th best per query (warp_key), the minimum over the
    // warps is the CTA's threshold (cta_key), far tighter than the tail of a warp's own list while the lists
    // fill.  Keys only ever grow; a stale or overwritten smaller value is a looser, still valid bound.
    unsigned long long* const warp_key = reinterpret_cast<unsigned long long*>(smem_raw - base + misc + C::SHARE_OFF);
    unsigned long long* const cta_key = warp_key + WARPS * RQ;
    const bool share = REGL && p.combine > 0;
    const int share_lane = share ? (p.combine * p.kk + WARPS - 1) / WARPS - 1 : 0;
    // Candidate lists of up to 32 entries live in registers while the rows stream; they are written to
    // shared memory only once the stream has ended, over the then idle second part of the ring.
    constexpr bool reg_lists = REGL;                 // (the host picks REGL = (kk <= 32))
    const uint32_t lists_bytes = (uint32_t)WARPS * NQ * p.kk * 8;
    const uint32_t ringB = (misc + C::FIXED + (reg_lists ? 0u : lists_bytes) + 127u) & ~127u;
    const uint32_t lists_addr = reg_lists ? ringB : misc + C::FIXED;
    const int slotsB = ringB < end ? (int)((end - ringB) / C::STAGE) : 0;
    const int NS = min(C::MAX_NS, slotsA + slotsB);
    uint8_t* const smem_gen = smem_raw - base;       // generic pointer of shared address 0
    float* lists_s = reinterpret_cast<float*>(smem_gen + lists_addr);
    int* lists_i = reinterpret_cast<int*>(lists_s + WARPS * NQ * p.kk);
    if (NS < 2 || lists_addr + lists_bytes > end) {  // the host sizes kk so that this cannot happen
        if (threadIdx.x == 0) atomicExch(p.status, 2);
        return;
    }
    auto slot_addr = [&](int slot) -> uint32_t {
        return slot < slotsA ? ringA + slot * C::STAGE : ringB + (slot - slotsA) * C::STAGE;
    };

    pdl_trigger();
    if (threadIdx.x < 16)
        reinterpret_cast<float*>(smem_gen + cent_addr)[threadIdx.x] =
            threadIdx.x < (1 << BITS) ? p.cent[threadIdx.x] * CENT_SCALE : 0.0f;
    if (threadIdx.x < (WARPS + 1) * RQ) warp_key[threadIdx.x] = thr_key(-__builtin_huge_valf(), ID_NONE);
    if (threadIdx.x < C::MAX_NS) {
        mbar_init(full_addr + threadIdx.x * 8, 1);
        mbar_init(empty_addr + threadIdx.x * 8, WPG);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!reg_lists)
        for (int e = threadIdx.x; e < WARPS * NQ * p.kk; e += blockDim.x) { lists_s[e] = -__builtin_huge_valf(); lists_i[e] = ID_NONE; }
    __syncthreads();
    {
        const float* cf = reinterpret_cast<const float*>(smem_gen + cent_addr);
        for (int x = warp; x < C::LUT_ENTRIES; x += WARPS + 1) {
            int clo, chi;
            tl_key_field_codes((uint32_t)x, BITS, clo, chi);
            *reinterpret_cast<uint32_t*>(smem_gen + tab_base + x * 256 + lane * 4) = pack_half2(cf[clo], cf[chi]);
        }
    }
    pdl_wait();                                      // the query fragments come from the preparation kernel
    __syncthreads();

    const int64_t nrec = p.n / SCAN_TILE;            // full records; the last n % 16 rows belong to the merge kernel
    const int64_t nstages = (nrec + SR - 1) / SR;
    RegLists RL;
#pragma unroll
    for (int jq = 0; jq < RQ; jq++) { RL.s[jq] = -__builtin_huge_valf(); RL.i[jq] = ID_NONE; }

    if (warp == WARPS) {
        // ---- producer: stage index blockIdx.x, + gridDim.x, ...; one bulk copy per stage ----
        if (lane == 0) {
            bool ok = true;
            int end_marks = 0;
            uint32_t n = 0;
            int64_t st = blockIdx.x;
            int s = 0;                                // slot of stage n and the parity of its previous use
            uint32_t par = 1;                         // (no division by the run-time ring size in the loop)
            for (;; n++, s++) {
                if (s == NS) { s = 0; par ^= 1; }
                if (n >= (uint32_t)NS) ok = mbar_wait(empty_addr + 8 * s, par);
                if (!ok) break;
                uint2* meta = reinterpret_cast<uint2*>(smem_gen + meta_addr + s * 8);
                if (st >= nstages) {                  // end of stream: one marker per consumer group
                    *meta = make_uint2(0u, F_END);
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_addr + 8 * s) : "memory");
                    if (++end_marks == GROUPS) break;
                    continue;
                }
                const int64_t r0 = st * SR;
                const int nt = (nrec - r0) < SR ? (int)(nrec - r0) : SR;
                *meta = make_uint2((uint32_t)r0, (uint32_t)nt);
                mbar_expect_tx(full_addr + 8 * s, (uint32_t)(nt * C::REC));
                bulk_g2s(slot_addr(s), p.records + r0 * C::REC, (uint32_t)(nt * C::REC), full_addr + 8 * s);
                st += gridDim.x;
            }
            if (!ok) {
                atomicExch(p.status, 1);
                for (uint32_t i = (n > (uint32_t)NS ? n - NS : 0); i < n; i++)
                    (void)mbar_wait(full_addr + 8 * (i % NS), (i / NS) & 1);
            }
        }
    } else {
        // ---- consumers ----
        const uint32_t tab = C::KBYTE ? (tab_base | (uint32_t)(lane * 4)) : tab_base + lane * 4;
        uint2 qf[C::KS];
        {
            const uint2* src = reinterpret_cast<const uint2*>(p.qfrag) + ((int64_t)grp * C::KS) * 32 + lane;
#pragma unroll
            for (int ks = 0; ks < C::KS; ks++) qf[ks] = src[ks * 32];
        }
        float* ls = lists_s + (size_t)warp * NQ * p.kk;
        int* li = lists_i + (size_t)warp * NQ * p.kk;
        // PAIR: this lane receives the scores of queries 2t and 2t+1 of the group (MMA columns 2t, 2t+1);
        // else of query t (columns 2t, 2t+1 = its fp16 hi and lo parts, added up)
        const int qa = PAIR ? grp * NQ + 2 * t : grp * NQ + t, qb = qa + 1;
        const bool live_a = qa < p.nq, live_b = PAIR && qb < p.nq;
        const float qsc_a = live_a ? p.qscale[qa] : 0.0f, qsc_b = live_b ? p.qscale[qb] : 0.0f;
        ScanThreshold thr_a{-__builtin_huge_valf(), ID_NONE}, thr_b{-__builtin_huge_valf(), ID_NONE};
        const int r0w = RPW * (warp % WPG);
        int s = warp / WPG - GROUPS;                  // slot of this group's current stage and its parity
        uint32_t par = 0;
        const int ja = PAIR ? 2 * t : t;              // this lane's queries within the group
        bool fresh = false;                           // this warp's lists changed since it last looked at the others'
        for (;;) {
            s += GROUPS;
            if (s >= NS) { s -= NS; par ^= 1; }
            if (share && fresh) {
                // CTA threshold of each query = the minimum over the warps' published keys
                fresh = false;
                const int w = lane & 15, half = lane >> 4;
                unsigned long long m[4];
#pragma unroll
                for (int j = 0; j < 4; j++) m[j] = warp_key[w * RQ + (half * 4 + j) % NQ];
#pragma unroll
                for (int off = 8; off; off >>= 1)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const unsigned long long o = __shfl_xor_sync(0xffffffffu, m[j], off);
                        m[j] = o < m[j] ? o : m[j];
                    }
                if (w == 0 && half * 4 < NQ) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        if (m[j] > cta_key[half * 4 + j]) cta_key[half * 4 + j] = m[j];
                }
                __syncwarp();
                thr_a = thr_max(thr_a, key_thr(cta_key[ja]));
                if (PAIR) thr_b = thr_max(thr_b, key_thr(cta_key[ja + 1]));
            }
            const bool ok = mbar_wait(full_addr + 8 * s, par);
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) atomicExch(p.status, 1);
                break;
            }
            uint2 meta;
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(meta.x), "=r"(meta.y) : "r"(meta_addr + s * 8));
            if (meta.y & F_END) {                     // release the marker's slot too: the producer may need it
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_addr + 8 * s) : "memory");
                break;
            }
            const int nt = (int)meta.y;
            const int mine = min(RPW, nt - r0w);
            for (int i0 = 0; i0 < mine; i0 += NT) {
                const uint32_t rec = slot_addr(s) + (r0w + i0) * C::REC;
                float acc[NT][4];
                // (records past the stage's end hold stale bytes: computed but never inserted)
                rec_scan_tiles<D, BITS, NT>(rec, tab, qf, lane, acc);
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    if (i0 + i >= mine) break;
                    uint2 nr;                          // norms of rows g and g + 8
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(nr.x), "=r"(nr.y) : "r"(rec + i * C::REC + C::KSEC + 8 * g));
                    const float n0 = __uint_as_float(nr.x), n1 = __uint_as_float(nr.y);
                    // candidate c: row (c >> 1 ? g + 8 : g), query (c & 1 ? qb : qa)
                    const float sc[4] = {PAIR ? acc[i][0] * (n0 * qsc_a) : (acc[i][0] + acc[i][1]) * (n0 * qsc_a),
                                         PAIR ? acc[i][1] * (n0 * qsc_b) : 0.0f,
                                         PAIR ? acc[i][2] * (n1 * qsc_a) : (acc[i][2] + acc[i][3]) * (n1 * qsc_a),
                                         PAIR ? acc[i][3] * (n1 * qsc_b) : 0.0f};
                    const int id0 = (int)(meta.x + r0w + i0 + i) * SCAN_TILE + g, id1 = id0 + 8;
                    const bool any = (live_a && (better(sc[0], id0, thr_a.s, thr_a.i) || better(sc[2], id1, thr_a.s, thr_a.i))) ||
                                     (live_b && (better(sc[1], id0, thr_b.s, thr_b.i) || better(sc[3], id1, thr_b.s, thr_b.i)));
                    if (__any_sync(0xffffffffu, any)) {
#pragma unroll 1
                        for (int c = 0; c < 4; c += PAIR ? 1 : 2) {
                            const int col = c & 1, id = c >> 1 ? id1 : id0;
                            const float v = c == 0 ? sc[0] : c == 1 ? sc[1] : c == 2 ? sc[2] : sc[3];
                            const bool lv = col ? live_b : live_a;
                            const ScanThreshold th = col ? thr_b : thr_a;
                            const bool offer = lv && better(v, id, th.s, th.i);
                            if (reg_lists) {
                                uint32_t mask = __ballot_sync(0xffffffffu, offer);
                                while (mask) {
                                    const int leader = __ffs(mask) - 1;
                                    mask &= mask - 1;
                                    const float bs = __shfl_sync(0xffffffffu, v, leader);
                                    const int bid = __shfl_sync(0xffffffffu, id, leader);
                                    // (a candidate that no longer beats its list's tail finds no place: harmless)
                                    switch (PAIR ? 2 * (leader & 3) + col : leader & 3) {
                                        case 0: reg_list_insert<0>(RL, p.kk, bs, bid, lane); break;
                                        case 1: reg_list_insert<1>(RL, p.kk, bs, bid, lane); break;
                                        case 2: reg_list_insert<2>(RL, p.kk, bs, bid, lane); break;
                                        case 3: reg_list_insert<3>(RL, p.kk, bs, bid, lane); break;
                                        case 4: reg_list_insert<4>(RL, p.kk, bs, bid, lane); break;
                                        case 5: reg_list_insert<5>(RL, p.kk, bs, bid, lane); break;
                                        case 6: reg_list_insert<6>(RL, p.kk, bs, bid, lane); break;
                                        default: reg_list_insert<7>(RL, p.kk, bs, bid, lane); break;
                                    }
                                }
                            } else {
                                thr_a = rec_scan_offer(ls, li, p.kk, v, id, offer, thr_a, lane);
                            }
                        }
                        if (reg_lists) {
                            // every lane's thresholds = the tails of the lists of the two queries it serves
                            float ts[RQ];
                            int tj[RQ];
#pragma unroll
                            for (int jq = 0; jq < NQ; jq++) {
                                ts[jq] = __shfl_sync(0xffffffffu, RL.s[jq], p.kk - 1);
                                tj[jq] = __shfl_sync(0xffffffffu, RL.i[jq], p.kk - 1);
                            }
                            if (PAIR) {
                                thr_a.s = t == 0 ? ts[0] : t == 1 ? ts[2] : t == 2 ? ts[4] : ts[6];
                                thr_a.i = t == 0 ? tj[0] : t == 1 ? tj[2] : t == 2 ? tj[4] : tj[6];
                                thr_b.s = t == 0 ? ts[1] : t == 1 ? ts[3] : t == 2 ? ts[5] : ts[7];
                                thr_b.i = t == 0 ? tj[1] : t == 1 ? tj[3] : t == 2 ? tj[5] : tj[7];
                            } else {
                                thr_a.s = t == 0 ? ts[0] : t == 1 ? ts[1] : t == 2 ? ts[2] : ts[3];
                                thr_a.i = t == 0 ? tj[0] : t == 1 ? tj[1] : t == 2 ? tj[2] : tj[3];
                            }
                            if (share) {
                                fresh = true;
                                if (lane == share_lane) {
#pragma unroll
                                    for (int jq = 0; jq < NQ; jq++) warp_key[warp * RQ + jq] = thr_key(RL.s[jq], RL.i[jq]);
                                }
                                thr_a = thr_max(thr_a, key_thr(cta_key[ja]));
                                if (PAIR) thr_b = thr_max(thr_b, key_thr(cta_key[ja + 1]));
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_addr + 8 * s) : "memory");
        }
    }

    // ---- candidates -> global (every thread of the CTA gets here) ----
    __syncthreads();                                  // nobody reads a stage any more: the ring may be reused
    if (reg_lists && warp < WARPS && lane < p.kk) {
#pragma unroll
        for (int jq = 0; jq < NQ; jq++) {
            lists_s[(warp * NQ + jq) * p.kk + lane] = RL.s[jq];
            lists_i[(warp * NQ + jq) * p.kk + lane] = RL.i[jq];
        }
    }
    __syncthreads();
    if (p.combine) {
        // p.combine sorted lists per CTA and query (ranks 0..kk-1, kk..2kk-1, ...): every candidate is ranked
        // among the CTA's WARPS * kk by counting
        const int per_q = WARPS * p.kk, nout = p.combine * p.kk;
        for (int idx = threadIdx.x; idx < NQ * nout; idx += blockDim.x) {
            const int jq = idx / nout, e = idx - jq * nout, q = grp * NQ + jq;
            if (q >= p.nq) continue;
            const int64_t o = ((int64_t)q * p.lists_per_query + (int64_t)blockIdx.x * p.combine) * p.kk + e;
            p.cand_s[o] = -__builtin_huge_valf();
            p.cand_id[o] = ID_NONE;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < NQ * per_q; idx += blockDim.x) {
            const int jq = idx / per_q, c = idx - jq * per_q, q = grp * NQ + jq;
            if (q >= p.nq) continue;
            const int w = c / p.kk, e = c - w * p.kk;
            const float s = lists_s[(w * NQ + jq) * p.kk + e];
            const int id = lists_i[(w * NQ + jq) * p.kk + e];
            if (id == ID_NONE) continue;
            int rank = 0;
            for (int w2 = 0; w2 < WARPS; w2++) {
                const float* s2 = lists_s + (w2 * NQ + jq) * p.kk;
                const int* i2 = lists_i + (w2 * NQ + jq) * p.kk;
                for (int e2 = 0; e2 < p.kk; e2++) rank += better(s2[e2], i2[e2], s, id) ? 1 : 0;
            }
            if (rank < nout) {
                const int64_t o = ((int64_t)q * p.lists_per_query + (int64_t)blockIdx.x * p.combine) * p.kk + rank;
                p.cand_s[o] = s;
                p.cand_id[o] = id;
            }
        }
    } else if (warp < WARPS) {
        const int64_t wid = (int64_t)blockIdx.x * WARPS + warp;
        for (int jq = 0; jq < NQ; jq++) {
            const int q = grp * NQ + jq;
            if (q >= p.nq) break;
            const int64_t o = ((int64_t)q * p.lists_per_query + wid) * p.kk;
            for (int e = lane; e < p.kk; e += 32) {
                p.cand_s[o + e] = lists_s[(warp * NQ + jq) * p.kk + e];
                p.cand_id[o + e] = lists_i[(warp * NQ + jq) * p.kk + e];
            }
        }
    }
}


// =================================================================================================
// 2b. generic scan: any dim (multiple of 8, <= 512), bits 1..4.  One query per blockIdx.y, one row per
// lane; the float32 table and the summation order are the upstream ones, so these scores are exact.
// =================================================================================================
__global__ void __launch_bounds__(SCAN_WARPS * 32) scan_generic_kernel(const ScanParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int levels = 1 << p.bits, bpp = (p.dim + 7) >> 3, pd = p.bits * bpp;
    float* T = reinterpret_cast<float*>(smem_raw);                    // dim * levels
    const bool prod = p.signs != nullptr;
    float* Ts = T + p.dim * levels;                                   // Prod: the query projected by S, dim floats
    float* lists_s = Ts + (prod ? p.dim : 0);
    int* lists_i = reinterpret_cast<int*>(lists_s + SCAN_WARPS * p.kk);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q = blockIdx.y;
    if (prod)
        for (int e = threadIdx.x; e < p.dim; e += blockDim.x) Ts[e] = p.qsign[(int64_t)q * p.dim + e];
    float* ls = lists_s + warp * p.kk;
    int* li = lists_i + warp * p.kk;
    for (int e = threadIdx.x; e < p.dim * levels; e += blockDim.x)
        T[e] = __fmul_rn(p.qrot[(int64_t)q * p.dim + e / levels], p.cent[e % levels]);
    for (int e = lane; e < p.kk; e += 32) { ls[e] = -__builtin_huge_valf(); li[e] = ID_NONE; }
    __syncthreads();
    float thr_s = -__builtin_huge_valf();
    int thr_i = ID_NONE;
    const int64_t n_main = p.n - p.n % SCAN_TILE;   // the tail belongs to the merge kernel
    const int64_t stride = (int64_t)gridDim.x * SCAN_WARPS * 32;
    for (int64_t base = ((int64_t)blockIdx.x * SCAN_WARPS + warp) * 32; base < n_main; base += stride) {
        const int64_t r = base + lane;
        const bool valid = r < n_main;
        float sc = 0.0f;
        if (valid) {
            const uint8_t* row = p.packed + r * pd;
            float dot = 0.0f;
            for (int m = 0; m < bpp; m++) {
                uint32_t pl[4] = {0, 0, 0, 0};
                for (int b = 0; b < p.bits; b++) pl[b] = row[b * bpp + m];
                const int lim = min(8, p.dim - 8 * m);
                for (int t = 0; t < lim; t++) {
                    const int sh = 7 - t;
                    const uint32_t c = ((pl[0] >> sh) & 1u) | (((pl[1] >> sh) & 1u) << 1) |
                                       (((pl[2] >> sh) & 1u) << 2) | (((pl[3] >> sh) & 1u) << 3);
                    dot = __fadd_rn(dot, T[(8 * m + t) * levels + c]);
                }
            }
            if (prod) {
                // <q, x~> = norm * ( <R q, c[codes]> + sqrt(pi/2)/d * ||r|| * <S q, signs> ),  sign = 2 bit - 1
                const uint8_t* srow = p.signs + r * bpp;
                float ds = 0.0f;
                for (int m = 0; m < bpp; m++) {
                    const uint32_t byte = srow[m];
                    const int lim = min(8, p.dim - 8 * m);
                    for (int t = 0; t < lim; t++) {
                        const float v = Ts[8 * m + t];
                        ds += (byte >> (7 - t)) & 1u ? v : -v;
                    }
                }
                sc = p.norms[r] * fmaf(p.sign_coef * p.res_norms[r], ds, dot);
            } else {
                sc = __fmul_rn(dot, p.norms[r]);
            }
        }
        uint32_t mask = __ballot_sync(0xffffffffu, valid && better(sc, (int)r, thr_s, thr_i));
        while (mask) {
            const int leader = __ffs(mask) - 1;
            mask &= mask - 1;
            const float bs = __shfl_sync(0xffffffffu, sc, leader);
            const int bid = __shfl_sync(0xffffffffu, (int)r, leader);
            list_insert(ls, li, p.kk, bs, bid, lane);
            thr_s = ls[p.kk - 1]; thr_i = li[p.kk - 1];
        }
    }
    __syncwarp();
    const int64_t wid = (int64_t)blockIdx.x * SCAN_WARPS + warp;
    const int64_t out = ((int64_t)q * p.lists_per_query + wid) * p.kk;
    for (int e = lane; e < p.kk; e += 32) { p.cand_s[out + e] = ls[e]; p.cand_id[out + e] = li[e]; }
}

// =================================================================================================
// 3. merge: best kk candidates per query -> exact float32 re-score -> sort -> top k
// =================================================================================================
constexpr int MERGE_THREADS = 256;
constexpr int MERGE_MAX = TQB_SCAN_MAX_K + SCAN_SELECT_MARGIN + SCAN_TILE;   // selected + tail rows
constexpr int SURV_MAX = 1024;          // candidates the fast selection path ranks among themselves

__global__ void __launch_bounds__(MERGE_THREADS) scan_merge_kernel(const ScanParams p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int levels = 1 << p.bits, bpp = (p.dim + 7) >> 3, pd = p.bits * bpp;
    float* T = reinterpret_cast<float*>(smem_raw);     // dim * levels
    __shared__ float sel_s[MERGE_MAX];
    __shared__ int sel_i[MERGE_MAX];
    __shared__ float red_s[MERGE_THREADS / 32];
    __shared__ int red_i[MERGE_THREADS / 32];
    __shared__ float cur_s;
    __shared__ int cur_i;
    const int q = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    pdl_wait();
    for (int e = tid; e < p.dim * levels; e += blockDim.x)
        T[e] = __fmul_rn(p.qrot[(int64_t)q * p.dim + e / levels], p.cent[e % levels]);
    const int64_t ncand = (int64_t)p.lists_per_query * p.kk;
    const float* cs = p.cand_s + (int64_t)q * ncand;
    const int* ci = p.cand_id + (int64_t)q * ncand;
    // ---- selection by the scan's scores: the best ksel candidates go on to the exact re-score ----
    // Fast path: every list is sorted best-first, so the ksel-th best of the list HEADS is a lower bound of
    // the ksel-th best candidate overall; the few candidates not below it are ranked among themselves.
    const int ksel = p.k + SCAN_SELECT_MARGIN;
    __shared__ float sv_s[SURV_MAX];
    __shared__ int sv_i[SURV_MAX];
    __shared__ int surv_n;
    __shared__ float tau_s;
    __shared__ int tau_i;
    if (tid == 0) { surv_n = 0; tau_s = -__builtin_huge_valf(); tau_i = ID_NONE; }
    __syncthreads();
    const int L = p.lists_per_query;
    if (L <= SURV_MAX) {                    // (more lists than that: no pruning, the general path takes over)
        // the heads go through shared memory (the survivor buffers are free until the next phase)
        for (int l = tid; l < L; l += blockDim.x) { sv_s[l] = cs[(int64_t)l * p.kk]; sv_i[l] = ci[(int64_t)l * p.kk]; }
        __syncthreads();
        for (int l = tid; l < L; l += blockDim.x) {
            const float hs = sv_s[l];
            const int hi = sv_i[l];
            if (hi == ID_NONE) continue;
            int rank = 0;
            for (int l2 = 0; l2 < L; l2++) rank += better(sv_s[l2], sv_i[l2], hs, hi) ? 1 : 0;
            if (rank == ksel - 1) { tau_s = hs; tau_i = hi; }      // (ranks are distinct: at most one writer)
        }
    }
    __syncthreads();
    for (int64_t e0 = tid; e0 < ncand; e0 += (int64_t)blockDim.x * 8) {   // eight candidates per thread in flight
        float sc[8];
        int id[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int64_t e = e0 + (int64_t)u * blockDim.x;
            sc[u] = e < ncand ? cs[e] : 0.0f;
            id[u] = e < ncand ? ci[e] : ID_NONE;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            if (id[u] == ID_NONE || better(tau_s, tau_i, sc[u], id[u])) continue;
            const int pos = atomicAdd(&surv_n, 1);
            if (pos < SURV_MAX) { sv_s[pos] = sc[u]; sv_i[pos] = id[u]; }
        }
    }
    __syncthreads();
    int nsel = 0;
    const bool fast = surv_n <= SURV_MAX;
    if (fast) {
        nsel = min(ksel, surv_n);
        for (int e = tid; e < surv_n; e += blockDim.x) {
            int rank = 0;
            for (int o = 0; o < surv_n; o++) rank += better(sv_s[o], sv_i[o], sv_s[e], sv_i[e]) ? 1 : 0;
            if (rank < ksel) sel_i[rank] = sv_i[e];
        }
        __syncthreads();
    }
    // General path (more survivors than the buffer holds): round r takes the best candidate worse than round r-1's.
    float prev_s = __builtin_huge_valf();
    int prev_i = -1;
    for (int r = 0; !fast && r < ksel; r++) {
        float bs = -__builtin_huge_valf();
        int bi = ID_NONE;
        for (int64_t e = tid; e < ncand; e += blockDim.x) {
            const float s = cs[e];
            const int id = ci[e];
            if (id != ID_NONE && better(prev_s, prev_i, s, id) && better(s, id, bs, bi)) { bs = s; bi = id; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(os, oi, bs, bi)) { bs = os; bi = oi; }
        }
        if (lane == 0) { red_s[warp] = bs; red_i[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < MERGE_THREADS / 32; w++)
                if (better(red_s[w], red_i[w], bs, bi)) { bs = red_s[w]; bi = red_i[w]; }
            cur_s = bs; cur_i = bi;
            if (bi != ID_NONE) { sel_i[r] = bi; }
        }
        __syncthreads();
        prev_s = cur_s; prev_i = cur_i;
        if (prev_i == ID_NONE) break;
        nsel = r + 1;
    }
    // ---- tail rows (n % 16) always take part ----
    const int tail = (int)(p.n % SCAN_TILE);
    if (tid < tail) sel_i[nsel + tid] = (int)(p.n - tail + tid);
    const int total = nsel + tail;
    __syncthreads();
    // ---- exact re-score, upstream order: dims ascending, add table entries, then * norm ----
    // A warp per candidate: the lanes look the table entries up in parallel, lane 0 adds them in order.
    __shared__ float vals[MERGE_THREADS / 32][512];
    for (int e = warp; e < total; e += MERGE_THREADS / 32) {
        const int id = sel_i[e];
        float nrm;
        if (p.records) {
            const int ksec = tl_key_section(p.dim, p.bits);
            const uint8_t* rec = p.records + (int64_t)(id >> 4) * tl_record_bytes(p.dim, p.bits, 0);
            for (int d = lane; d < p.dim; d += 32) {
                int base, bit;
                tl_key_slot(p.dim, p.bits, id & 15, d, base, bit);
                vals[warp][d] = T[d * levels + tl_read_bits(rec + base, bit, p.bits)];
            }
            nrm = *reinterpret_cast<const float*>(rec + ksec + tl_norm_offset(0, 0, id & 15));
        } else {
            const uint8_t* row = p.packed + (int64_t)id * pd;
            for (int d = lane; d < p.dim; d += 32) {
                const int m = d >> 3, sh = 7 - (d & 7);
                uint32_t c = 0;
                for (int b = 0; b < p.bits; b++) c |= ((row[b * bpp + m] >> sh) & 1u) << b;
                vals[warp][d] = T[d * levels + c];
            }
            nrm = p.norms[id];
        }
        float ds = 0.0f;
        if (p.signs) {                                  // Prod rows: the sign term, summed across the warp
            const uint8_t* srow = p.signs + (int64_t)id * bpp;
            for (int d = lane; d < p.dim; d += 32) {
                const float v = p.qsign[(int64_t)q * p.dim + d];
                ds += (srow[d >> 3] >> (7 - (d & 7))) & 1u ? v : -v;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ds += __shfl_xor_sync(0xffffffffu, ds, o);
        }
        __syncwarp();
        if (lane == 0) {
            float dot = 0.0f;
            for (int d = 0; d < p.dim; d++) dot = __fadd_rn(dot, vals[warp][d]);
            sel_s[e] = p.signs ? nrm * fmaf(p.sign_coef * p.res_norms[id], ds, dot) : __fmul_rn(dot, nrm);
        }
        __syncwarp();
    }
    __syncthreads();
    // ---- rank by counting, emit the first k ----
    for (int e = tid; e < total; e += blockDim.x) {
        int rank = 0;
        for (int o = 0; o < total; o++) rank += better(sel_s[o], sel_i[o], sel_s[e], sel_i[e]) ? 1 : 0;
        if (rank < p.k) {
            p.out_scores[(int64_t)q * p.k + rank] = sel_s[e];
            p.out_ids[(int64_t)q * p.k + rank] = (int64_t)sel_i[e] + p.id_offset;
        }
    }
    for (int e = total + tid; e < p.k; e += blockDim.x) {   // fewer rows than k: pad like upstream
        p.out_scores[(int64_t)q * p.k + e] = -__builtin_huge_valf();
        p.out_ids[(int64_t)q * p.k + e] = -1;
    }
}

}  // namespace tqb

// =================================================================================================
// 4. merge of per-shard top-k lists (row-sharded search: one list per shard, gathered by the caller)
// =================================================================================================
namespace tqb {

__device__ __forceinline__ bool better64(float s, int64_t id, float ts, int64_t tid) {
    // padding entries (-1) lose against everything real
    if (id < 0) return false;
    if (tid < 0) return true;
    return s > ts || (s == ts && id < tid);
}

__global__ void topk_merge_kernel(const float* __restrict__ scores, const int64_t* __restrict__ ids, int parts,
                                  int k, float* __restrict__ out_scores, int64_t* __restrict__ out_ids) {
    const int q = blockIdx.x;
    const int total = parts * k;
    const float* s = scores + (int64_t)q * total;
    const int64_t* id = ids + (int64_t)q * total;
    for (int e = threadIdx.x; e < k; e += blockDim.x) {   // defaults: padding
        out_scores[(int64_t)q * k + e] = -__builtin_huge_valf();
        out_ids[(int64_t)q * k + e] = -1;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
        if (id[e] < 0) continue;
        int rank = 0;
        for (int o = 0; o < total; o++) rank += (o != e && better64(s[o], id[o], s[e], id[e])) ? 1 : 0;
        if (rank < k) { out_scores[(int64_t)q * k + rank] = s[e]; out_ids[(int64_t)q * k + rank] = id[e]; }
    }
}

struct ScanPlan {
    size_t off_status, off_qrot, off_qfrag, off_qscale, off_cs, off_ci, total;
    int kk, lists, ngroups;
    bool mma;
};

static inline size_t s_align(size_t v) { return (v + 255) / 256 * 256; }

static ScanPlan plan_scan(int nq, int64_t n, int dim, int bits, int k) {
    ScanPlan pl{};
    pl.mma = (dim == 64 || dim == 128) && bits >= 2 && bits <= 4;
    pl.kk = scan_kk(k);
    pl.lists = sm_count() * SCAN_WARPS;
    pl.ngroups = (nq + QG - 1) / QG;
    size_t off = 0;
    pl.off_status = off; off = s_align(off + 256);
    pl.off_qrot = off;   off = s_align(off + (size_t)nq * dim * 4);
    pl.off_qfrag = off;  off = s_align(off + (size_t)pl.ngroups * (dim / 16 + 1) * 32 * 16);
    pl.off_qscale = off; off = s_align(off + (size_t)nq * 4);
    const size_t cand = (size_t)nq * pl.lists * pl.kk;
    pl.off_cs = off; off = s_align(off + cand * 4);
    pl.off_ci = off; off = s_align(off + cand * 4);
    pl.total = off;
    (void)n;
    return pl;
}

template <int D, int BITS>
static int launch_scan(const ScanParams& p, int ngroups, cudaStream_t st) {
    using C = ScanCfg<D, BITS>;
    const size_t lists = (size_t)SCAN_WARPS * QG * p.kk * 8;
    const size_t fixed = (size_t)C::LUT_BYTES + lists;
    const int NS8 = (fixed + (size_t)SCAN_WARPS * 8 * (C::STAGE + 8) <= 200 * 1024);
    const int ns = NS8 ? 8 : 4;
    const size_t smem = fixed + (size_t)SCAN_WARPS * ns * (C::STAGE + 8);
    if (smem > 220 * 1024) return fail(TQB_ERR_UNSUPPORTED, "scan_topk: k = %d needs %zu bytes of shared memory", p.k, smem);
    dim3 grid(p.lists_per_query / SCAN_WARPS, ngroups);
    if (ns == 8) {
        auto kern = scan_kernel<D, BITS, 8>;
        TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, SCAN_WARPS * 32, smem, st>>>(p);
    } else {
        auto kern = scan_kernel<D, BITS, 4>;
        TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, SCAN_WARPS * 32, smem, st>>>(p);
    }
    return check_launch("scan");
}

}  // namespace tqb

namespace tqb {

// Record scan: candidate lists are merged per CTA inside the scan kernel while that is cheap
// (rank by counting among 16 * kk entries); beyond that every consumer warp writes its own list.
static bool rec_combine(int kk) { return 16 * kk <= 1024; }

// Eight queries per pass (one fp16 column each) for calls with more than four queries whose candidate lists fit
// the registers; else four (hi + lo columns): a single query then pays for no columns it does not use.
static int rec_queries_per_pass(int kk, int nq) { return kk <= 32 && nq > QG ? RQ : QG; }

static ScanPlan plan_scan_records(int nq, int dim, int bits, int k) {
    ScanPlan pl{};
    pl.mma = true;
    pl.kk = scan_kk(k);
    pl.lists = sm_count() * (rec_combine(pl.kk) ? REC_OUT_LISTS : 16);
    const int per = rec_queries_per_pass(pl.kk, nq);
    pl.ngroups = (nq + per - 1) / per;
    size_t off = 0;
    pl.off_status = off; off = s_align(off + 256);
    pl.off_qrot = off;   off = s_align(off + (size_t)nq * dim * 4);
    pl.off_qfrag = off;  off = s_align(off + (size_t)pl.ngroups * (dim / 16 + 1) * 32 * 16);
    pl.off_qscale = off; off = s_align(off + (size_t)nq * 4);
    const size_t cand = (size_t)nq * pl.lists * pl.kk;
    pl.off_cs = off; off = s_align(off + cand * 4);
    pl.off_ci = off; off = s_align(off + cand * 4);
    pl.total = off;
    (void)bits;
    return pl;
}

// CTAs per query group.  A CTA has an SM to itself and all CTAs of a launch take equally long, so a launch
// costs (waves of CTAs) x (time of one CTA), and a CTA's time is its share of the records plus a fixed part:
// the lookup table, the pipeline fill and above all the candidate lists of its warps, which take insertions
// until their thresholds have tightened (about k ln(rows) of them whatever the share).  Measured with groups
// of eight queries, that part is worth REC_CTA_FIXED records of streaming (0.45 ms against 33 ns per record).
// One group therefore takes every SM, and many groups take few, large CTAs each in as few full waves as
// possible: 5 groups over 4 M rows 1.51 ms with 118 CTAs each, 0.85 ms with 29; 64 groups 5.9 ms with 9 CTAs
// each, 4.8 ms with 2.  At least two CTAs per group keep the candidate margin the exact re-scoring relies on.
constexpr int64_t REC_CTA_FIXED = 14000;
static int rec_ctas_per_group(int ngroups, int64_t nrec, int sms) {
    int best = 2;
    int64_t best_cost = INT64_MAX;
    for (int x = 2; x <= sms; ++x) {
        const int64_t waves = ceil_div((int64_t)ngroups * x, (int64_t)sms);
        const int64_t cost = waves * (REC_CTA_FIXED + ceil_div(nrec, (int64_t)x));
        if (cost < best_cost) { best_cost = cost; best = x; }
    }
    return best;
}

template <int D, int BITS>
static int launch_scan_records(const ScanParams& p, int ngroups, int grid_x, cudaStream_t st) {
    using C = RecScanCfg<D, BITS>;
    const bool regl = p.kk <= 32, pair = rec_queries_per_pass(p.kk, p.nq) == RQ;
    // at least two stages must fit beside the table and the candidate lists
    const size_t lists = regl ? 0 : (size_t)C::WARPS * QG * p.kk * 8;
    const size_t worst = (C::KBYTE ? 2 * 65536 : C::LUT_BYTES + 4096) + C::FIXED + lists + 256;
    const size_t tail = worst < (size_t)C::DYN ? (size_t)C::DYN - worst : 0;
    const size_t stages = tail / C::STAGE + (C::KBYTE ? (65536 - 4096) / C::STAGE : 0);
    if (stages < 2 || worst >= (size_t)C::DYN)
        return fail(TQB_ERR_UNSUPPORTED, "scan_records_topk: k = %d leaves no room for the pipeline in shared memory", p.k);
    auto kern = pair ? scan_records_kernel<D, BITS, RQ, true>
                     : regl ? scan_records_kernel<D, BITS, QG, true> : scan_records_kernel<D, BITS, QG, false>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::DYN));
    dim3 grid(grid_x, ngroups);
    // (programmatic dependent launch: the table build overlaps the end of the preparation kernel)
    TQB_CUDA(launch_pdl(1, kern, grid, dim3(C::THREADS), (size_t)C::DYN, st, p));
    return check_launch("scan_records");
}

}  // namespace tqb

extern "C" size_t tqb_scan_records_workspace_bytes(int nq, int dim, int bits, int k) {
    if (nq <= 0 || (dim != 64 && dim != 128) || bits < 2 || bits > 4 || k <= 0 || k > TQB_SCAN_MAX_K) return 0;
    return tqb::plan_scan_records(nq, dim, bits, k).total;
}

extern "C" int tqb_scan_records_ctas_per_group(int groups, int64_t n, int sms) {
    if (groups <= 0 || n < 0) return 0;
    return tqb::rec_ctas_per_group(groups, tqb::ceil_div(n, (int64_t)16), sms > 0 ? sms : tqb::sm_count());
}

extern "C" int tqb_scan_records_topk(const float* queries, int nq, const uint8_t* records, int64_t n, int dim,
                                     int bits, const float* rotation, const float* centroids, int k,
                                     int64_t id_offset, void* workspace, size_t workspace_bytes,
                                     float* out_scores, int64_t* out_ids, void* stream) {
    using namespace tqb;
    TQB_REQUIRE(nq >= 0 && n >= 0, "scan_records_topk: negative size");
    if (dim != 64 && dim != 128) return fail(TQB_ERR_UNSUPPORTED, "scan_records_topk: dim must be 64 or 128, got %d", dim);
    if (bits < 2 || bits > 4) return fail(TQB_ERR_UNSUPPORTED, "scan_records_topk: bit_width must be 2-4, got %d", bits);
    TQB_REQUIRE(k >= 1, "scan_records_topk: k must be positive, got %d", k);
    if (k > TQB_SCAN_MAX_K) return fail(TQB_ERR_UNSUPPORTED, "scan_records_topk: k = %d exceeds the limit %d", k, TQB_SCAN_MAX_K);
    if (n >= 0x7fffffff - 16) return fail(TQB_ERR_UNSUPPORTED, "scan_records_topk: at most 2^31-18 rows per call (shard the index)");
    if (nq == 0) return TQB_OK;
    TQB_REQUIRE(queries && rotation && centroids && workspace && out_scores && out_ids, "scan_records_topk: null pointer");
    TQB_REQUIRE(n == 0 || records, "scan_records_topk: null database");
    TQB_REQUIRE((uintptr_t)records % 16 == 0, "scan_records_topk: the record store must be 16-byte aligned");
    TQB_REQUIRE((uintptr_t)workspace % 256 == 0, "scan_records_topk: workspace must be 256-byte aligned");
    const ScanPlan pl = plan_scan_records(nq, dim, bits, k);
    if (workspace_bytes < pl.total)
        return fail(TQB_ERR_WORKSPACE, "scan_records_topk: workspace %zu bytes < required %zu", workspace_bytes, pl.total);

    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    ScanParams p{};
    p.records = records; p.n = n; p.dim = dim; p.bits = bits; p.nq = nq; p.k = k; p.kk = pl.kk;
    p.rot = rotation; p.cent = centroids; p.queries = queries; p.id_offset = id_offset;
    p.status = reinterpret_cast<int*>(ws + pl.off_status);
    p.qrot = reinterpret_cast<float*>(ws + pl.off_qrot);
    p.qfrag = reinterpret_cast<uint32_t*>(ws + pl.off_qfrag);
    p.qscale = reinterpret_cast<float*>(ws + pl.off_qscale);
    p.cand_s = reinterpret_cast<float*>(ws + pl.off_cs);
    p.cand_id = reinterpret_cast<int*>(ws + pl.off_ci);
    p.out_scores = out_scores; p.out_ids = out_ids;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid_x = rec_ctas_per_group(pl.ngroups, ceil_div(n, (int64_t)16), sm_count());
    // with few CTAs per query the margin beyond k has to come from within the CTA: it then emits more lists
    p.combine = rec_combine(pl.kk) ? (grid_x < 16 ? REC_OUT_LISTS : 1) : 0;
    p.lists_per_query = grid_x * (p.combine ? p.combine : 16);

    if (rec_queries_per_pass(pl.kk, nq) == RQ)
        scan_prepare_kernel<RQ><<<pl.ngroups, 128, sizeof(float) * (size_t)(1 + 2 * RQ) * dim, st>>>(p, 2);
    else
        scan_prepare_kernel<QG><<<pl.ngroups, 128, sizeof(float) * (size_t)(1 + 2 * QG) * dim, st>>>(p, 2);
    if (int e = check_launch("scan_prepare")) return e;
    int e = TQB_ERR_UNSUPPORTED;
#define TQB_CASE(d, b) if (dim == d && bits == b) e = launch_scan_records<d, b>(p, pl.ngroups, grid_x, st);
    TQB_CASE(64, 2) TQB_CASE(64, 3) TQB_CASE(64, 4) TQB_CASE(128, 2) TQB_CASE(128, 3) TQB_CASE(128, 4)
#undef TQB_CASE
    if (e) return e;
    const size_t msmem = sizeof(float) * (size_t)dim * (1 << bits);
    TQB_CUDA(cudaFuncSetAttribute(scan_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max<size_t>(msmem, 48 * 1024)));
    TQB_CUDA(launch_pdl(1, scan_merge_kernel, dim3(nq), dim3(MERGE_THREADS), msmem, st, p));
    return check_launch("scan_merge");
}

extern "C" size_t tqb_scan_topk_workspace_bytes(int nq, int64_t n, int dim, int bits, int k) {
    if (nq <= 0 || dim <= 0 || k <= 0 || k > TQB_SCAN_MAX_K) return 0;
    return tqb::plan_scan(nq, n, dim, bits, k).total;
}

extern "C" int tqb_scan_topk(const float* queries, int nq, const uint8_t* packed, const float* norms,
                             int64_t n, int dim, int bits, const float* rotation, const float* centroids,
                             int k, int64_t id_offset, void* workspace, size_t workspace_bytes,
                             float* out_scores, int64_t* out_ids, void* stream) {
    using namespace tqb;
    TQB_REQUIRE(nq >= 0 && n >= 0, "scan_topk: negative size");
    TQB_REQUIRE(bits >= 1 && bits <= 4, "scan_topk: bit_width must be 1-4, got %d", bits);
    TQB_REQUIRE(k >= 1, "scan_topk: k must be positive, got %d", k);
    if (k > TQB_SCAN_MAX_K) return fail(TQB_ERR_UNSUPPORTED, "scan_topk: k = %d exceeds the limit %d", k, TQB_SCAN_MAX_K);
    if (dim < 8 || dim > 512 || (dim & 7))
        return fail(TQB_ERR_UNSUPPORTED, "scan_topk: dim must be a multiple of 8 in 8..512, got %d", dim);
    if (n >= 0x7fffffff) return fail(TQB_ERR_UNSUPPORTED, "scan_topk: at most 2^31-2 rows per call (shard the index)");
    if (nq == 0) return TQB_OK;
    TQB_REQUIRE(queries && rotation && centroids && workspace && out_scores && out_ids, "scan_topk: null pointer");
    TQB_REQUIRE(n == 0 || (packed && norms), "scan_topk: null database");
    TQB_REQUIRE((uintptr_t)workspace % 256 == 0, "scan_topk: workspace must be 256-byte aligned");
    const ScanPlan pl = plan_scan(nq, n, dim, bits, k);
    if (workspace_bytes < pl.total)
        return fail(TQB_ERR_WORKSPACE, "scan_topk: workspace %zu bytes < required %zu", workspace_bytes, pl.total);
    if (pl.mma) TQB_REQUIRE(((uintptr_t)packed | (uintptr_t)norms) % 16 == 0, "scan_topk: database arrays must be 16-byte aligned");

    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    ScanParams p{};
    p.packed = packed; p.norms = norms; p.n = n; p.dim = dim; p.bits = bits; p.nq = nq; p.k = k; p.kk = pl.kk;
    p.rot = rotation; p.cent = centroids; p.queries = queries; p.id_offset = id_offset;
    p.status = reinterpret_cast<int*>(ws + pl.off_status);
    p.qrot = reinterpret_cast<float*>(ws + pl.off_qrot);
    p.qfrag = reinterpret_cast<uint32_t*>(ws + pl.off_qfrag);
    p.qscale = reinterpret_cast<float*>(ws + pl.off_qscale);
    p.cand_s = reinterpret_cast<float*>(ws + pl.off_cs);
    p.cand_id = reinterpret_cast<int*>(ws + pl.off_ci);
    p.out_scores = out_scores; p.out_ids = out_ids;
    cudaStream_t st = (cudaStream_t)stream;

    const int64_t ntiles = n / SCAN_TILE;
    const int gx = (int)std::max<int64_t>(1, std::min<int64_t>(sm_count(), ceil_div(ntiles, SCAN_WARPS)));
    p.lists_per_query = gx * SCAN_WARPS;

    scan_prepare_kernel<QG><<<pl.ngroups, 128, sizeof(float) * (size_t)(1 + 2 * QG) * dim, st>>>(p, pl.mma ? 1 : 0);
    if (int e = check_launch("scan_prepare")) return e;

    if (pl.mma) {
        int e = TQB_ERR_UNSUPPORTED;
#define TQB_CASE(d, b) if (dim == d && bits == b) e = launch_scan<d, b>(p, pl.ngroups, st);
        TQB_CASE(64, 2) TQB_CASE(64, 3) TQB_CASE(64, 4) TQB_CASE(128, 2) TQB_CASE(128, 3) TQB_CASE(128, 4)
#undef TQB_CASE
        if (e) return e;
    } else {
        const size_t smem = sizeof(float) * (size_t)dim * (1 << bits) + (size_t)SCAN_WARPS * p.kk * 8;
        TQB_CUDA(cudaFuncSetAttribute(scan_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dim3 grid(gx, nq);
        scan_generic_kernel<<<grid, SCAN_WARPS * 32, smem, st>>>(p);
        if (int e = check_launch("scan_generic")) return e;
    }
    const size_t msmem = sizeof(float) * (size_t)dim * (1 << bits);
    TQB_CUDA(cudaFuncSetAttribute(scan_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max<size_t>(msmem, 48 * 1024)));
    scan_merge_kernel<<<nq, MERGE_THREADS, msmem, st>>>(p);
    return check_launch("scan_merge");
}

extern "C" size_t tqb_scan_topk_prod_workspace_bytes(int nq, int64_t n, int dim, int bits, int k) {
    if (nq <= 0 || dim <= 0 || bits < 2 || bits > 5 || k <= 0 || k > TQB_SCAN_MAX_K) return 0;
    // the MSE scan's workspace plus the queries projected by the QJL matrix
    return tqb::plan_scan(nq, n, dim, bits - 1, k).total + tqb::s_align((size_t)nq * dim * 4);
}

extern "C" int tqb_scan_topk_prod(const float* queries, int nq, const uint8_t* mse_packed, const uint8_t* signs,
                                  const float* res_norms, const float* norms, int64_t n, int dim, int bits,
                                  const float* rotation, const float* centroids, const float* S, int k,
                                  int64_t id_offset, void* workspace, size_t workspace_bytes, float* out_scores,
                                  int64_t* out_ids, void* stream) {
    using namespace tqb;
    TQB_REQUIRE(nq >= 0 && n >= 0, "scan_topk_prod: negative size");
    TQB_REQUIRE(bits >= 2 && bits <= 5, "scan_topk_prod: bit_width must be 2-5 (1-4 MSE bits + the sign bit), got %d", bits);
    TQB_REQUIRE(k >= 1, "scan_topk_prod: k must be positive, got %d", k);
    if (k > TQB_SCAN_MAX_K) return fail(TQB_ERR_UNSUPPORTED, "scan_topk_prod: k = %d exceeds the limit %d", k, TQB_SCAN_MAX_K);
    if (dim < 8 || dim > 512 || (dim & 7))
        return fail(TQB_ERR_UNSUPPORTED, "scan_topk_prod: dim must be a multiple of 8 in 8..512, got %d", dim);
    if (n >= 0x7fffffff) return fail(TQB_ERR_UNSUPPORTED, "scan_topk_prod: at most 2^31-2 rows per call (shard the index)");
    if (nq == 0) return TQB_OK;
    TQB_REQUIRE(queries && rotation && centroids && S && workspace && out_scores && out_ids, "scan_topk_prod: null pointer");
    TQB_REQUIRE(n == 0 || (mse_packed && signs && res_norms && norms), "scan_topk_prod: null database");
    TQB_REQUIRE((uintptr_t)workspace % 256 == 0, "scan_topk_prod: workspace must be 256-byte aligned");
    const int mb = bits - 1;
    const ScanPlan pl = plan_scan(nq, n, dim, mb, k);
    const size_t need = pl.total + s_align((size_t)nq * dim * 4);
    if (workspace_bytes < need)
        return fail(TQB_ERR_WORKSPACE, "scan_topk_prod: workspace %zu bytes < required %zu", workspace_bytes, need);

    uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
    ScanParams p{};
    p.packed = mse_packed; p.norms = norms; p.n = n; p.dim = dim; p.bits = mb; p.nq = nq; p.k = k; p.kk = pl.kk;
    p.rot = rotation; p.cent = centroids; p.queries = queries; p.id_offset = id_offset;
    p.signs = signs; p.res_norms = res_norms;
    p.sign_coef = (float)(std::sqrt(M_PI / 2.0) / (double)dim);
    p.status = reinterpret_cast<int*>(ws + pl.off_status);
    p.qrot = reinterpret_cast<float*>(ws + pl.off_qrot);
    p.qfrag = reinterpret_cast<uint32_t*>(ws + pl.off_qfrag);
    p.qscale = reinterpret_cast<float*>(ws + pl.off_qscale);
    p.cand_s = reinterpret_cast<float*>(ws + pl.off_cs);
    p.cand_id = reinterpret_cast<int*>(ws + pl.off_ci);
    float* qsign = reinterpret_cast<float*>(ws + pl.total);
    p.qsign = qsign;
    p.out_scores = out_scores; p.out_ids = out_ids;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t ntiles = n / SCAN_TILE;
    const int gx = (int)std::max<int64_t>(1, std::min<int64_t>(sm_count(), ceil_div(ntiles, SCAN_WARPS)));
    p.lists_per_query = gx * SCAN_WARPS;

    // R q and S q: the same kernel twice (row j of the matrix times the query, float32, k ascending)
    const size_t psmem = sizeof(float) * (size_t)(1 + 2 * QG) * dim;
    scan_prepare_kernel<QG><<<pl.ngroups, 128, psmem, st>>>(p, 0);
    if (int e = check_launch("scan_prepare")) return e;
    ScanParams ps = p;
    ps.rot = S; ps.qrot = qsign;
    scan_prepare_kernel<QG><<<pl.ngroups, 128, psmem, st>>>(ps, 0);
    if (int e = check_launch("scan_prepare")) return e;

    const size_t smem = sizeof(float) * ((size_t)dim * (1 << mb) + dim) + (size_t)SCAN_WARPS * p.kk * 8;
    TQB_CUDA(cudaFuncSetAttribute(scan_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(gx, nq);
    scan_generic_kernel<<<grid, SCAN_WARPS * 32, smem, st>>>(p);
    if (int e = check_launch("scan_generic")) return e;
    const size_t msmem = sizeof(float) * (size_t)dim * (1 << mb);
    TQB_CUDA(cudaFuncSetAttribute(scan_merge_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max<size_t>(msmem, 48 * 1024)));
    scan_merge_kernel<<<nq, MERGE_THREADS, msmem, st>>>(p);
    return check_launch("scan_merge");
}

extern "C" int tqb_topk_merge(const float* scores, const int64_t* ids, int nq, int parts, int k,
                              float* out_scores, int64_t* out_ids, void* stream) {
    TQB_REQUIRE(nq >= 0 && parts >= 1 && k >= 1, "topk_merge: bad sizes");
    if (nq == 0) return TQB_OK;
    TQB_REQUIRE(scores && ids && out_scores && out_ids, "topk_merge: null pointer");
    tqb::topk_merge_kernel<<<nq, 128, 0, (cudaStream_t)stream>>>(scores, ids, parts, k, out_scores, out_ids);
    return tqb::check_launch("topk_merge");
}

// ---- scan with built-in scratch ------------------------------------------------------------------
// Same computation as tqb_scan_topk, for callers that cannot hand over a workspace because they cannot
// allocate one: a host that has already given every free byte of device memory to its own pools (an
// allocation there fails or forces the pool to shrink), or a latency-critical loop in which a device
// allocation would stall all streams of the process while the driver maps memory.  The scratch is a
// fixed array in the module's device image, so this entry point never calls an allocating routine.
//
// Set-up: the first call on each device looks up the array's address with cudaGetSymbolAddress while
// that device is current (this may load the module on that device).  Make that first call early, on
// every device that will be used, before any stream capture is begun.
//
// Sharing: all calls on one device use the same array.  The status word at its start is cleared on the
// caller's stream at the beginning of each call; candidate lists and query fragments are rewritten by
// every call before they are read.  Calls that may overlap on the device (different streams, different
// host threads) race on the array and must be serialised by the caller; calls on one stream are safe.
namespace tqb {
constexpr size_t SCAN_STATIC_BYTES = (size_t)4 << 20;          // 4 MiB: whatever tqb_scan_topk_workspace_bytes says fits
constexpr int SCAN_STATIC_MAX_DEVICES = 64;
static __device__ __align__(256) unsigned char g_scan_scratch[SCAN_STATIC_BYTES];
static void* g_scan_scratch_ptr[SCAN_STATIC_MAX_DEVICES] = {};
static std::mutex g_scan_scratch_mutex;

static int scan_static_scratch(void** out) {
    int dev = -1;
    TQB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= SCAN_STATIC_MAX_DEVICES)
        return fail(TQB_ERR_UNSUPPORTED, "scan_topk_static: device ordinal %d not supported (limit %d)", dev,
                    SCAN_STATIC_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_scan_scratch_mutex);
    if (!g_scan_scratch_ptr[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_scan_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(TQB_ERR_CUDA, "scan_topk_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                        cudaGetErrorString(e));
        g_scan_scratch_ptr[dev] = ptr;
    }
    *out = g_scan_scratch_ptr[dev];
    return TQB_OK;
}
}  // namespace tqb

extern "C" size_t tqb_scan_topk_static_capacity(void) { return tqb::SCAN_STATIC_BYTES; }

extern "C" int tqb_scan_topk_static(const float* queries, int nq, const uint8_t* packed, const float* norms,
                                    int64_t n, int dim, int bits, const float* rotation, const float* centroids,
                                    int k, int64_t id_offset, float* out_scores, int64_t* out_ids, void* stream) {
    using namespace tqb;
    TQB_REQUIRE(nq >= 0 && n >= 0, "scan_topk_static: negative size");
    if (nq == 0) return TQB_OK;
    TQB_REQUIRE(dim > 0 && k >= 1, "scan_topk_static: dim and k must be positive, got dim %d, k %d", dim, k);
    if (k > TQB_SCAN_MAX_K)      // (the code tqb_scan_topk returns for the same request)
        return fail(TQB_ERR_UNSUPPORTED, "scan_topk_static: k = %d exceeds the limit %d", k, TQB_SCAN_MAX_K);
    const size_t need = tqb_scan_topk_workspace_bytes(nq, n, dim, bits, k);
    if (need == 0 || need > SCAN_STATIC_BYTES)
        return fail(TQB_ERR_WORKSPACE,
                    "scan_topk_static: this call needs %zu bytes of scratch but the built-in scratch holds %zu; "
                    "use fewer queries per call or tqb_scan_topk with a workspace of your own", need,
                    SCAN_STATIC_BYTES);
    void* scratch = nullptr;
    if (int e = scan_static_scratch(&scratch)) return e;
    TQB_CUDA(cudaMemsetAsync(scratch, 0, 256, (cudaStream_t)stream));   // the status word starts at zero
    return tqb_scan_topk(queries, nq, packed, norms, n, dim, bits, rotation, centroids, k, id_offset, scratch,
                         SCAN_STATIC_BYTES, out_scores, out_ids, stream);
}
