// decode_attn.cu -- fused decode attention over a packed KV cache (one new token per sequence).
//
// Replaces "dequantise every cached key and value, then attend" (upstream
// turboquant_kv/cache.py:216-339) by three launches that never materialise dense K/V:
//
//   1. decode_prepare_kernel q_rot = R_k q per head, times scale * log2(e), written directly as
//                            mma.sync B fragments (fp16); for a fused step it also quantises and
//                            stores the new token's key and value.
//   2. decode_partial_kernel one persistent CTA per SM.  A producer warp streams the 16-token records
//                            of the CTA's work items into a ring of shared-memory stages, one TMA bulk
//                            copy (cp.async.bulk + mbarrier) of up to 28 KB per stage; two groups of
//                            consumer warps take alternate stages, four records per warp.  Per record:
//                            scores = K-codes x q on tensor cores (codes -> fp16 centroids through a
//                            256-entry shared-memory table indexed by one byte = 2 codes), online
//                            softmax in the log2 domain with a lazy running maximum, P^T via movmatrix,
//                            O^T += V^T-codes x P^T on tensor cores, all in ROTATED space.  One
//                            (m, l, acc) partial per (unit, chunk, consumer warp).
//   3. decode_merge_kernel   combines the partials of a (sequence, query head), divides by l and
//                            applies the inverse value rotation acc @ R_v (reference.py:362).
//
// A unit is one (sequence, KV head); its `group` query heads ride along as the N dimension of the
// MMA (grouped-query attention: decode cost is paid once per KV head).  HBM traffic per token and
// KV head is the packed K row + packed V row + two float norms; everything else lives in L2/SMEM.
//
// Every wait is bounded: a warp that gives up records it in the status word at the start of the
// workspace and returns, so a lost copy cannot hang the device.
#include "common.cuh"
#include "pipe.cuh"
#include "tiled_layout.cuh"

namespace tqb {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_INF = -__builtin_huge_valf();
constexpr float RESCALE_SLACK = 4.0f;   // lazy max: rescale only when a score exceeds m + 4 (log2)
constexpr int TILE = 16;                // tokens per MMA tile

// Which launches carry the attribute (bit 0 preparation, 1 streaming kernel, 2 merge).  Measured on the
// benchmark step (1 GPU, ms per step): none 1.366, streaming + merge 1.317, all three 1.414 -- early-resident
// preparation CTAs of the next call get in the way of the merge, so the preparation is launched plainly.
static constexpr int PDL_MASK = 6;
static constexpr int pdl_mask() { return PDL_MASK; }

// ---- launch parameters --------------------------------------------------------------------------
struct DecodeParams {
    const uint8_t* store;            // tiled records (tiled_layout.cuh)
    const int32_t* seq_lens; const int32_t* block_tables;
    int64_t max_seq;                 // token pitch of a unit (contiguous cache), multiple of 16
    int batch, q_heads, kv_heads, group, max_blocks, block_size;
    int chunk, nchunks;              // tokens per (unit, chunk) work item
    int sets;                        // partials per work item (consumer warps of the streaming kernel)
    const float* cent_k; const float* cent_v;
    // workspace views
    int* status; const uint32_t* qfrag;
    float* part_m; float* part_l; float* part_acc;
};

// Workspace layout shared by the size query and the launcher.
struct DecodeWorkspace {
    size_t off_status, off_lens, off_qfrag, off_m, off_l, off_acc, total;
    int chunk, nchunks;
};


// =================================================================================================
// 1. query rotation -> B fragments
// =================================================================================================
// Fragments carry q_rot * scale * log2(e): fp16 keeps 11 significant bits whatever the magnitude and
// the products stay far inside its range, so no separate per-head factor is needed.
__device__ __forceinline__ void write_query_fragments(const float (*qr)[128], int u, int group, int dim,
                                                      float scale, uint32_t* __restrict__ qfrag) {
    const float fold = scale * LOG2E;
    const int ksteps = dim >> 4;
    for (int idx = threadIdx.x; idx < ksteps * 64; idx += blockDim.x) {
        const int ks = idx >> 6, rem = idx & 63, fl = rem >> 1, half = rem & 1;
        const int g = fl >> 2, t = fl & 3;
        float lo = 0.0f, hi = 0.0f;
        if (g < group) {
            const int dlo = 16 * ks + 8 * half + 2 * t, dhi = dlo + 1;   // k index = dimension
            lo = qr[g][dlo] * fold;
            hi = qr[g][dhi] * fold;
        }
        qfrag[((int64_t)u * ksteps + ks) * 64 + rem] = pack_half2_sat(lo, hi);
    }
}

// -------------------------------------------------------------------------------------------------
// One CTA (8 warps) per unit rotates the unit's queries into B fragments: element (ks, lane = 4g+t, half)
// of head g holds the rotated query coordinates (16ks + 8half + 2t, +1); heads >= group are zero columns.
// With key != nullptr it is one decode step's whole preparation: it also quantises and stores the new
// token's key and value of the unit.
//
// The code selection repeats quantize.cu's arithmetic exactly (norm by per-lane partial sums and a
// butterfly, unit = x / max(norm, 1e-10), y_j as one fused-multiply-add chain over k ascending,
// code = number of boundaries below y_j), so the stored codes are those tqb_kv_append would store.
// The token goes to position lens_in[b] of its unit; lens_now[b] = lens_in[b] + 1 is what the
// attention kernels of this step read.  A full unit (position >= max_seq) stores nothing, raises
// status 3 and attends to the tokens it has.
template <typename T, int NQ>
__global__ void __launch_bounds__(256) decode_prepare_kernel(
    const T* __restrict__ q, const T* __restrict__ key, const T* __restrict__ value, int64_t kv_stride,
    int q_heads, int kv_heads, int group, int dim, const float* __restrict__ Rk, const float* __restrict__ Rv,
    const float* __restrict__ bnd_k, const float* __restrict__ bnd_v, int kbits, int vbits, float scale,
    uint8_t* __restrict__ store, int64_t max_seq, const int32_t* __restrict__ lens_in,
    int32_t* __restrict__ lens_now, uint32_t* __restrict__ qfrag, int* status) {
    __shared__ float vec[10][128];            // rows 0..group-1: queries; 8: unit key; 9: unit value
    __shared__ float qr[8][128];
    __shared__ float bnd[2][16];
    __shared__ float nrm[2];
    __shared__ uint32_t codes[2][128];
    const int u = blockIdx.x, b = u / kv_heads, h = u - b * kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();          // inputs may come from the previous kernel; the workspace is still read by it
    pdl_trigger();
    if (u == 0 && threadIdx.x == 0) *status = 0;
    const bool step = key != nullptr;
    const int pos = step ? lens_in[b] : 0;
    const bool room = step && pos < max_seq;
    if (step && h == 0 && threadIdx.x == 0) lens_now[b] = room ? pos + 1 : pos;
    if (step && !room && threadIdx.x == 0) atomicExch(status, 3);
    if (step && threadIdx.x < 32) {            // (the boundary tables are null without a new token)
        const int which = threadIdx.x >> 4, i = threadIdx.x & 15;
        const int nb = (1 << (which ? vbits : kbits)) - 1;
        bnd[which][i] = i < nb ? (which ? bnd_v : bnd_k)[i] : __int_as_float(0x7f800000);
    }
    for (int idx = threadIdx.x; idx < group * dim; idx += blockDim.x) {
        const int n = idx / dim, k = idx - n * dim;
        vec[n][k] = to_f32<T>(q[((int64_t)b * q_heads + h * group + n) * dim + k]);
    }
    if (step && (warp == 6 || warp == 7)) {    // warps 6, 7: norm and unit vector of the key, the value
        const int which = warp - 6;
        const T* x = (which ? value : key) + (int64_t)u * kv_stride;
        float v[NQ], ss = 0.0f;
#pragma unroll
        for (int qq = 0; qq < NQ; qq++) {
            const int j = lane + 32 * qq;
            v[qq] = j < dim ? to_f32<T>(x[j]) : 0.0f;
            ss = fmaf(v[qq], v[qq], ss);
        }
        const float n = sqrtf(warp_sum(ss));
        const float den = fmaxf(n, 1e-10f);
#pragma unroll
        for (int qq = 0; qq < NQ; qq++)
            if (lane + 32 * qq < dim) vec[8 + which][lane + 32 * qq] = v[qq] / den;
        if (lane == 0) nrm[which] = n;
    }
    __syncthreads();
    // one thread per output coordinate of (group + 2) vectors
    const int total = (group + (step ? 2 : 0)) * dim;
    for (int o = threadIdx.x; o < total; o += blockDim.x) {
        const int vi = o / dim, j = o - vi * dim;
        const float* src = vec[vi < group ? vi : 8 + (vi - group)];
        const float4* row = reinterpret_cast<const float4*>((vi <= group ? Rk : Rv) + (int64_t)j * dim);
        float acc = 0.0f;
#pragma unroll 8
        for (int k4 = 0; k4 < dim / 4; k4++) {
            const float4 r = __ldg(row + k4);
            acc = fmaf(src[4 * k4], r.x, acc);
            acc = fmaf(src[4 * k4 + 1], r.y, acc);
            acc = fmaf(src[4 * k4 + 2], r.z, acc);
            acc = fmaf(src[4 * k4 + 3], r.w, acc);
        }
        if (vi < group) {
            qr[vi][j] = acc;
        } else {
            const int which = vi - group;
            uint32_t c = 0;
            for (int step = 1 << ((which ? vbits : kbits) - 1); step > 0; step >>= 1)
                if (bnd[which][c + step - 1] < acc) c += step;
            codes[which][j] = c;
        }
    }
    __syncthreads();
    if (warp < 2 && room) {                    // warp 0 stores the key, warp 1 the value
        uint32_t code[NQ];
#pragma unroll
        for (int qq = 0; qq < NQ; qq++) code[qq] = lane + 32 * qq < dim ? codes[warp][lane + 32 * qq] : 0u;
        tiled_store_row<NQ>(store, warp + 1, kbits, vbits, (int64_t)u * max_seq + pos, code, nrm[warp], lane, dim);
    }
    write_query_fragments(qr, u, group, dim, scale, qfrag);
}


// =================================================================================================
// 2. streaming partial attention over tiled records
// =================================================================================================
template <int D, int KB, int VB>
struct DecodeCfg {
    static constexpr int KL = D * KB / 16, VL = D * VB / 16;       // bytes per lane
    static constexpr int KSEC = 32 * KL, VSEC = 32 * VL;
    static constexpr int REC = KSEC + VSEC + 128;                   // one 16-token record
    // Lookup tables.  An entry is replicated for the 32 lanes (bank = lane: no conflicts).
    // BYTE tables (8-bit fields): entries 256 bytes apart in a 64 KB table that starts on a 64 KB boundary
    // of the shared window, so that ONE byte-permute assembles the complete shared address of an entry:
    // byte 0 = lane offset, byte 1 = the field, bytes 2-3 = table base.  Other tables: 128 bytes apart,
    // address = base + (field << 7) + lane offset.
    static constexpr bool KBYTE = (2 * KB == 8);
    static constexpr bool VQUAD = (VB == 2);                        // 2 dims x 2 tokens per 8-bit field
    static constexpr bool VBYTE = VQUAD || (2 * VB == 8);
    static constexpr int LUTK_ENTRIES = 1 << (2 * KB);
    static constexpr int LUTV_ENTRIES = VQUAD ? 256 : (1 << (2 * VB));
    static constexpr int LUTV_WORDS = VQUAD ? 2 : 1;               // 8-byte entries for 2-bit values
    // When both tables are BYTE tables they share ONE 64 KB region: the 256 bytes of entry x hold the key
    // entry in [0,128) (32 lanes x 4 B) and the value entry in [128,256) (32 lanes x 4 B, or 16 lane slots
    // x 8 B: a 64-bit shared load is served half a warp at a time, so lanes l and l+16 can share a slot).
    static constexpr int NALIGNED = (KBYTE || VBYTE) ? 1 : 0;
    static constexpr int SMALL_K = KBYTE ? 0 : LUTK_ENTRIES * 128;  // tables that need no alignment
    static constexpr int SMALL_V = VBYTE ? 0 : LUTV_ENTRIES * 128;
    static constexpr int MT = D / 16;                               // m-tiles of O^T / k-steps of the scores
    // head_dim 64: 16 consumer warps (96 registers each).  head_dim 128 keeps twice the accumulators: 8
    // consumer warps with four records in flight each measured faster than 12 warps with two (0.76 vs
    // 0.85 ms per layer at batch 64 x 32,768 tokens, K4/V3).
    static constexpr int WARPS = D == 64 ? 16 : 8;                  // consumer warps
    static constexpr int NTMAX = 4;                                 // records a warp processes at once
    static constexpr int GROUPS = 2;                                // consumer warp groups; stage n goes to group n % GROUPS
    static constexpr int WPG = WARPS / GROUPS;
    static constexpr int RPW = 4;                                   // records per warp per stage
    static constexpr int SR = WPG * RPW;                            // records per stage (one bulk copy)
    static constexpr int STAGE = SR * REC;
    static constexpr int STAGE_TOKENS = SR * 16;
    static constexpr int THREADS = (WARPS + 1) * 32;                // consumer warps + one producer warp
    // Shared-memory plan (dynamic, the whole opt-in maximum):  [ring A | aligned tables | misc | ring B]
    static constexpr int DYN = 227 * 1024;
    static constexpr int LENS_MAX = 512;
    static constexpr int MISC = SMALL_K + SMALL_V + 256 /*centroids*/ + 8 * (8 + 8 + 16) /*barriers, stage headers*/
                                + LENS_MAX * 4;
    static constexpr int BASE_MAX = 4096;                           // assumed upper bound of the window offset
    static constexpr int SLOTS_A = NALIGNED ? (65536 - BASE_MAX) / STAGE : 0;
    static constexpr int TAIL = NALIGNED ? DYN - 2 * 65536 : DYN - BASE_MAX;
    static constexpr int SLOTS_B = (TAIL - MISC) / STAGE;
    static constexpr int NS_FIT = SLOTS_A + SLOTS_B;
    static constexpr int NS = NS_FIT > 8 ? 8 : NS_FIT;              // stages in the ring
    static_assert(NS >= 2, "shared memory: the ring needs at least two stages");
    static_assert(SR <= 32, "a paged stage is issued as one copy per producer lane");
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Position of a CTA in its stream of pipeline stages: items (unit, chunk) are dealt round-robin to CTAs;
// an item is streamed in stages of up to SR records, which the consumer warps share (RPW records each).
template <int SR, int GROUPS>
struct StageCursor {
    int item, total_items, stride;     // (the host checks that the item count fits 31 bits)
    int tiles_left, tile0;              // tiles of the item not yet taken; index of the next one in its unit
    int unit, b, h, chunk_idx, tok_end;
    int stage_idx, stages;              // position in the item; an item takes at least GROUPS stages (empty ones
                                        // if need be) so that every consumer group sees its start and its end
    __device__ __forceinline__ bool valid() const { return item < total_items; }
    __device__ __forceinline__ int tiles_here() const { return min(SR, tiles_left); }
    // `lens`: the sequence lengths (a shared-memory copy when the batch fits, else the global array)
    __device__ __forceinline__ void open(const DecodeParams& p, const int32_t* lens) {
        while (item < total_items) {
            unit = item / p.nchunks;
            chunk_idx = item - unit * p.nchunks;
            b = unit / p.kv_heads;
            h = unit - b * p.kv_heads;
            const int S = lens[b];
            const int tok0 = chunk_idx * p.chunk;
            tok_end = min(S, tok0 + p.chunk);
            if (tok0 < tok_end) {
                tiles_left = (tok_end - tok0 + TILE - 1) / TILE;
                tile0 = tok0 / TILE;
                stage_idx = 0;
                stages = max(GROUPS, (tiles_left + SR - 1) / SR);
                return;
            }
            item += stride;
        }
    }
    __device__ __forceinline__ void next(const DecodeParams& p, const int32_t* lens) {
        const int n = tiles_here();
        tiles_left -= n; tile0 += n; stage_idx++;
        if (stage_idx == stages) { item += stride; open(p, lens); }
    }
};

// Per-warp softmax state of the item being processed.
template <int MT>
struct WarpState {
    float m0, m1, l0, l1;      // running maximum (log2 domain; 0 before the first token) and row sums
    float thr;                 // rescale when a shifted score exceeds this: -inf before the first token, then the slack
    float O[MT][4];
    uint32_t qf[MT][2];
};

// NT (1, 2 or 4) 16-token records at once: scores, online softmax, accumulation.  Both records go through
// every phase together so that their independent instruction chains interleave.  MASKED handles the
// partial last tile of an item (tokens >= valid contribute nothing).
template <int D, int KB, int VB, int NT, bool MASKED>
__device__ __forceinline__ void process_tiles(WarpState<D / 16>& st, uint32_t rec0, uint32_t tabK, uint32_t tabV,
                                               int lane, int g, int valid) {
    using C = DecodeCfg<D, KB, VB>;
    float sc[NT][4];
    // ---- scores: 16 tokens x 8 heads per record ----
    {
        uint32_t kw[NT][C::KL / 4];
#pragma unroll
        for (int i = 0; i < NT; i++) {
            load_key_chunk<C::KL>(rec0 + i * C::REC, lane, kw[i]);
            sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
        }
#pragma unroll
        for (int ks = 0; ks < C::MT; ks++) {
            uint32_t a[NT][4];
#pragma unroll
            for (int i = 0; i < NT; i++)
#pragma unroll
                for (int half = 0; half < 2; half++)
#pragma unroll
                    for (int second = 0; second < 2; second++)
                        a[i][2 * half + second] = lds32(entry_addr<C::KBYTE>(kw[i], tl_key_field_bit(D, KB, ks, half, second), 2 * KB, tabK));
#pragma unroll
            for (int i = 0; i < NT; i++) mma_f16(sc[i], a[i], st.qf[ks][0], st.qf[ks][1]);
        }
    }
    // shifted scores s' = score * key_norm - m  (one FFMA each); the running maximum m is lazy: it only
    // moves when some s' exceeds the slack, so most tiles skip the cross-lane reduction and the rescale
    float s[NT][4], nvg[NT], nvg8[NT];
    float tm0 = NEG_INF, tm1 = NEG_INF;
#pragma unroll
    for (int i = 0; i < NT; i++) {
        const uint32_t nk = rec0 + i * C::REC + C::KSEC + C::VSEC + 4 * g;   // key norms, then 16 value norms
        const bool val_g = !MASKED || 16 * i + g < valid, val_g8 = !MASKED || 16 * i + g + 8 < valid;
        float nkg = ldsf(nk), nkg8 = ldsf(nk + 32);
        nvg[i] = ldsf(nk + 64);
        nvg8[i] = ldsf(nk + 96);
        if (MASKED) {
            if (!val_g) { nkg = 0.0f; nvg[i] = 0.0f; }
            if (!val_g8) { nkg8 = 0.0f; nvg8[i] = 0.0f; }
        }
        s[i][0] = fmaf(sc[i][0], nkg, -st.m0); s[i][1] = fmaf(sc[i][1], nkg, -st.m1);
        s[i][2] = fmaf(sc[i][2], nkg8, -st.m0); s[i][3] = fmaf(sc[i][3], nkg8, -st.m1);
        if (MASKED) {
            if (!val_g) { s[i][0] = NEG_INF; s[i][1] = NEG_INF; }
            if (!val_g8) { s[i][2] = NEG_INF; s[i][3] = NEG_INF; }
        }
        tm0 = fmaxf(tm0, fmaxf(s[i][0], s[i][2]));
        tm1 = fmaxf(tm1, fmaxf(s[i][1], s[i][3]));
    }
    if (__any_sync(0xffffffffu, fmaxf(tm0, tm1) > st.thr)) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, o));
            tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, o));
        }
        // move each maximum up by d = max(tm, 0) (never down); everything accumulated so far shrinks by 2^-d
        // (the very first tile of an item sets the maximum outright: nothing has been accumulated yet)
        const bool fresh = st.thr == NEG_INF;
        const float d0 = (tm0 == NEG_INF) ? 0.0f : (fresh ? tm0 : fmaxf(tm0, 0.0f));
        const float d1 = (tm1 == NEG_INF) ? 0.0f : (fresh ? tm1 : fmaxf(tm1, 0.0f));
        const float f0 = fresh ? 1.0f : ex2_approx(-d0), f1 = fresh ? 1.0f : ex2_approx(-d1);
        st.m0 += d0; st.m1 += d1;
        st.l0 *= f0; st.l1 *= f1;
#pragma unroll
        for (int mt = 0; mt < C::MT; mt++) { st.O[mt][0] *= f0; st.O[mt][2] *= f0; st.O[mt][1] *= f1; st.O[mt][3] *= f1; }
#pragma unroll
        for (int i = 0; i < NT; i++) { s[i][0] -= d0; s[i][2] -= d0; s[i][1] -= d1; s[i][3] -= d1; }
        st.thr = RESCALE_SLACK;
    }
    uint32_t pb[NT][2];
#pragma unroll
    for (int i = 0; i < NT; i++) {
        const float p0 = ex2_approx(s[i][0]), p1 = ex2_approx(s[i][1]);
        const float p2 = ex2_approx(s[i][2]), p3 = ex2_approx(s[i][3]);
        st.l0 += p0 + p2; st.l1 += p1 + p3;
        // P^T as B operand: (k = tokens, col = head) through two 8x8 transposes
        pb[i][0] = movmatrix_trans(pack_half2_sat(p0 * nvg[i], p1 * nvg[i]));
        pb[i][1] = movmatrix_trans(pack_half2_sat(p2 * nvg8[i], p3 * nvg8[i]));
    }

    // ---- O^T += V^T P^T : (dims x tokens) x (tokens x heads) ----
    {
        uint32_t vw[NT][C::VL / 4];
#pragma unroll
        for (int i = 0; i < NT; i++) load_chunk<C::VL>(rec0 + i * C::REC + C::KSEC + lane * C::VL, vw[i]);
#pragma unroll
        for (int mt = 0; mt < C::MT; mt++) {
            uint32_t a[NT][4];
#pragma unroll
            for (int i = 0; i < NT; i++) {
                if (C::VQUAD) {
                    const uint2 e0 = lds64(entry_addr<true>(vw[i], tl_val_field_bit(VB, mt, 0, 0), 8, tabV));
                    const uint2 e1 = lds64(entry_addr<true>(vw[i], tl_val_field_bit(VB, mt, 1, 0), 8, tabV));
                    a[i][0] = e0.x; a[i][1] = e0.y; a[i][2] = e1.x; a[i][3] = e1.y;
                } else {
#pragma unroll
                    for (int half = 0; half < 2; half++)
#pragma unroll
                        for (int rs = 0; rs < 2; rs++)
                            a[i][2 * half + rs] = lds32(entry_addr<C::VBYTE>(vw[i], tl_val_field_bit(VB, mt, half, rs), 2 * VB, tabV));
                }
            }
#pragma unroll
            for (int i = 0; i < NT; i++) mma_f16(st.O[mt], a[i], pb[i][0], pb[i][1]);
        }
    }
}

template <int D, int KB, int VB, bool PAGED>
__global__ void __launch_bounds__(DecodeCfg<D, KB, VB>::THREADS, 1) decode_partial_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, KB, VB>;
    constexpr int WARPS = C::WARPS, NS = C::NS, SR = C::SR, RPW = C::RPW, GROUPS = C::GROUPS, WPG = C::WPG;
    constexpr uint32_t F_FIRST = 1u << 16, F_LAST = 1u << 17, F_END = 1u << 18;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    // ---- carve the shared window (see DecodeCfg): all positions are 32-bit shared addresses ----
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t end = base + C::DYN;
    uint32_t tabK_base, tabV_base, misc, ringA = base, ringB;
    int slotsA;
    if (C::NALIGNED) {
        const uint32_t al = (base + 65535u) & ~65535u;
        slotsA = (int)((al - base) / C::STAGE);
        tabK_base = C::KBYTE ? al : 0;
        tabV_base = C::VBYTE ? al + (C::KBYTE ? 128u : 0u) : 0;   // second half of every 256-byte entry block
        misc = al + 65536u;
    } else {
        slotsA = 0; tabK_base = tabV_base = 0; misc = base;
    }
    if (!C::KBYTE) { tabK_base = misc; misc += C::SMALL_K; }
    if (!C::VBYTE) { tabV_base = misc; misc += C::SMALL_V; }
    const uint32_t cent_addr = misc;                 // 32 floats
    const uint32_t full_addr = misc + 256;           // full[s]: the stage's bytes have landed
    const uint32_t empty_addr = full_addr + 8 * 8;   // empty[s]: every warp of the stage's group has finished with it
    const uint32_t meta_addr = empty_addr + 8 * 8;   // one uint4 per stage: {unit, chunk, tiles | flags, valid tokens}
    const uint32_t lens_addr = meta_addr + 8 * 16;   // sequence lengths of up to LENS_MAX sequences
    ringB = (lens_addr + C::LENS_MAX * 4 + 127u) & ~127u;
    const int slotsB = (int)((end - ringB) / C::STAGE);
    if (slotsA + slotsB < NS) {                      // cannot happen unless the window offset is unusually large
        if (threadIdx.x == 0) atomicExch(p.status, 2);
        return;
    }
    auto slot_addr = [&](int slot) -> uint32_t {
        return slot < slotsA ? ringA + slot * C::STAGE : ringB + (slot - slotsA) * C::STAGE;
    };
    uint8_t* const smem_gen = smem_raw - base;       // generic pointer of shared address 0
    pdl_trigger();

    const bool lens_in_smem = p.batch <= C::LENS_MAX;
    const int32_t* lens = lens_in_smem ? reinterpret_cast<const int32_t*>(smem_gen + lens_addr) : p.seq_lens;
    if (threadIdx.x < 16) {
        float* cf = reinterpret_cast<float*>(smem_gen + cent_addr);
        cf[threadIdx.x] = threadIdx.x < (1 << KB) ? p.cent_k[threadIdx.x] : 0.0f;
        cf[16 + threadIdx.x] = threadIdx.x < (1 << VB) ? p.cent_v[threadIdx.x] : 0.0f;
    }
    if (threadIdx.x < NS) {
        mbar_init(full_addr + threadIdx.x * 8, 1);
        mbar_init(empty_addr + threadIdx.x * 8, WPG);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // ---- lookup tables ----
    {
        const float* cf = reinterpret_cast<const float*>(smem_gen + cent_addr);
        constexpr int KSTR = C::KBYTE ? 256 : 128, VSTR = C::VBYTE ? 256 : 128;
        for (int x = warp; x < C::LUTK_ENTRIES; x += WARPS + 1) {
            int clo, chi;
            tl_key_field_codes((uint32_t)x, KB, clo, chi);
            *reinterpret_cast<uint32_t*>(smem_gen + tabK_base + x * KSTR + lane * 4) = pack_half2(cf[clo], cf[chi]);
        }
        for (int x = warp; x < C::LUTV_ENTRIES; x += WARPS + 1) {
            if (C::VQUAD) {
                int ag, bg, ag8, bg8;
                tl_val_quad_codes((uint32_t)x, ag, bg, ag8, bg8);
                *reinterpret_cast<uint2*>(smem_gen + tabV_base + x * VSTR + (lane & 15) * 8) =
                    make_uint2(pack_half2(cf[16 + ag], cf[16 + bg]), pack_half2(cf[16 + ag8], cf[16 + bg8]));
            } else {
                int ca, cb;
                tl_val_pair_codes((uint32_t)x, VB, ca, cb);
                *reinterpret_cast<uint32_t*>(smem_gen + tabV_base + x * VSTR + lane * 4) = pack_half2(cf[16 + ca], cf[16 + cb]);
            }
        }
    }
    // everything above depends on constants only; from here on the preparation kernel's output is read
    pdl_wait();
    if (lens_in_smem)
        for (int i = threadIdx.x; i < p.batch; i += blockDim.x)
            reinterpret_cast<int32_t*>(smem_gen + lens_addr)[i] = p.seq_lens[i];
    __syncthreads();
    const uint32_t tabK = tabK_base + lane * 4;                    // for BYTE tables "+" is "|": the low 16 bits of the base are 0
    const uint32_t tabV = tabV_base + (C::VQUAD ? (lane & 15) * 8 : lane * 4);

    // ---- producer warp: streams the CTA's items.  Lane 0 owns the barriers and the stage headers and
    // issues the one bulk copy of a stage of a contiguous cache; for a paged cache every record is its own
    // copy (pages are scattered), and the 32 lanes issue them side by side.  All lanes track the cursor.
    if (warp == WARPS) {
        StageCursor<SR, GROUPS> cur;
        cur.item = blockIdx.x;
        cur.total_items = p.batch * p.kv_heads * p.nchunks;
        cur.stride = gridDim.x;
        cur.tiles_left = 0;
        cur.open(p, lens);
        bool ok = true;
        int end_marks = 0;
        uint32_t n = 0;
        for (;; n++) {
            const int s = n % NS;
            // paged cache: this lane's page of the coming stage is looked up before the wait for the slot,
            // so that the table read's latency hides behind it
            int64_t my_rec = -1;
            if (PAGED && cur.valid() && lane < cur.tiles_here()) {
                const int rpb = p.block_size / TILE;   // records per page
                const int tile = cur.tile0 + lane;
                const int blk = p.block_tables[(int64_t)cur.b * p.max_blocks + tile / rpb];
                my_rec = ((int64_t)blk * p.kv_heads + cur.h) * rpb + tile % rpb;
            }
            if (n >= NS) {
                if (lane == 0) ok = mbar_wait(empty_addr + 8 * s, ((n / NS) - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (!ok) break;
            uint4* meta = reinterpret_cast<uint4*>(smem_gen + meta_addr + s * 16);
            if (!cur.valid()) {                     // end of stream: one marker stage per consumer group
                if (lane == 0) {
                    *meta = make_uint4(0, 0, F_END, 0);
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_addr + 8 * s) : "memory");
                }
                if (++end_marks == GROUPS) break;
                continue;
            }
            const int nt = cur.tiles_here();
            const int left = cur.tok_end - cur.tile0 * TILE;
            if (lane == 0)
                *meta = make_uint4((uint32_t)cur.unit, (uint32_t)cur.chunk_idx,
                                   (uint32_t)nt | (cur.stage_idx < GROUPS ? F_FIRST : 0u) |
                                       (cur.stage_idx >= cur.stages - GROUPS ? F_LAST : 0u),
                                   (uint32_t)left);
            if (nt == 0) {                          // padding stage of a short item: flags only
                if (lane == 0)
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(full_addr + 8 * s) : "memory");
                cur.next(p, lens);
                continue;
            }
            const uint32_t dst = slot_addr(s);
            // (the consumers' reads of this slot are ordered before this write by the empty barrier)
            if (lane == 0) mbar_expect_tx(full_addr + 8 * s, (uint32_t)(nt * C::REC));
            __syncwarp();
            if (PAGED) {                            // (a stage has at most 32 records: one per lane)
                if (lane < nt) bulk_g2s(dst + lane * C::REC, p.store + my_rec * C::REC, C::REC, full_addr + 8 * s);
            } else if (lane == 0) {
                const int64_t rec = (int64_t)cur.unit * (p.max_seq / TILE) + cur.tile0;
                bulk_g2s(dst, p.store + rec * C::REC, (uint32_t)(nt * C::REC), full_addr + 8 * s);
            }
            cur.next(p, lens);
        }
        if (!ok && lane == 0) {
            // The consumers stopped releasing stages.  Record it and give the copies still in flight a
            // bounded chance to land before this CTA's shared memory is released.
            atomicExch(p.status, 1);
            for (uint32_t i = (n > (uint32_t)NS ? n - NS : 0); i < n; i++)
                (void)mbar_wait(full_addr + 8 * (i % NS), (i / NS) & 1);   // (padding stages complete at once)
        }
        return;
    }

    // ---- consumers: group (warp / WPG) takes every GROUPS-th stage; its warp i takes records RPW*i .. RPW*i+RPW-1 ----
    WarpState<C::MT> st;
    int unit = 0, chunk_idx = 0;
    st.m0 = st.m1 = st.l0 = st.l1 = 0.0f; st.thr = NEG_INF;
    const int r0 = RPW * (warp % WPG);
    for (uint32_t n = warp / WPG;; n += GROUPS) {
        const int s = n % NS;
        const bool ok = mbar_wait(full_addr + 8 * s, (n / NS) & 1);
        if (!__all_sync(0xffffffffu, ok)) {           // a copy never arrived: flag it and stop
            if (lane == 0) atomicExch(p.status, 1);
            break;
        }
        uint4 meta;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(meta.x), "=r"(meta.y), "=r"(meta.z), "=r"(meta.w) : "r"(meta_addr + s * 16));
        if (meta.z & F_END) {                         // end of the stream (release the marker's slot as well)
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_addr + 8 * s) : "memory");
            break;
        }
        const int nt = meta.z & 0xffff;
        if (meta.z & F_FIRST) {                       // this group's first stage of an item
            unit = (int)meta.x; chunk_idx = (int)meta.y;
            st.m0 = st.m1 = 0.0f; st.l0 = st.l1 = 0.0f; st.thr = NEG_INF;
#pragma unroll
            for (int mt = 0; mt < C::MT; mt++) { st.O[mt][0] = st.O[mt][1] = st.O[mt][2] = st.O[mt][3] = 0.0f; }
            const uint2* qsrc = reinterpret_cast<const uint2*>(p.qfrag) + ((int64_t)unit * C::MT) * 32 + lane;
#pragma unroll
            for (int ks = 0; ks < C::MT; ks++) { const uint2 v = qsrc[ks * 32]; st.qf[ks][0] = v.x; st.qf[ks][1] = v.y; }
        }
        if (r0 < nt) {
            const uint32_t rec = slot_addr(s) + r0 * C::REC;
            const int lv = (int)meta.w - r0 * TILE;   // valid tokens from this warp's first record on
            const int mine = min(RPW, nt - r0);
            if (C::NTMAX == 4 && mine == 4 && lv >= 4 * TILE) {
                process_tiles<D, KB, VB, 4, false>(st, rec, tabK, tabV, lane, g, 4 * TILE);
            } else {
                for (int i0 = 0; i0 < mine; i0 += 2) {
                    const uint32_t r = rec + i0 * C::REC;
                    const int v = lv - i0 * TILE;
                    if (mine - i0 >= 2) {
                        if (v >= 2 * TILE) process_tiles<D, KB, VB, 2, false>(st, r, tabK, tabV, lane, g, 2 * TILE);
                        else process_tiles<D, KB, VB, 2, true>(st, r, tabK, tabV, lane, g, v);
                    } else {
                        process_tiles<D, KB, VB, 1, true>(st, r, tabK, tabV, lane, g, v);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_addr + 8 * s) : "memory");

        if (meta.z & F_LAST) {                        // this group's last stage of the item: the warp's partial
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                st.l0 += __shfl_xor_sync(0xffffffffu, st.l0, o);
                st.l1 += __shfl_xor_sync(0xffffffffu, st.l1, o);
            }
            const bool none = st.thr == NEG_INF;      // this warp saw no token of the item
            const int64_t pbase = (((int64_t)unit * p.nchunks + chunk_idx) * WARPS + warp) * p.group;
            const int h0 = 2 * t, h1 = 2 * t + 1;
            if (g == 0) {
                if (h0 < p.group) { p.part_m[pbase + h0] = none ? NEG_INF : st.m0; p.part_l[pbase + h0] = st.l0; }
                if (h1 < p.group) { p.part_m[pbase + h1] = none ? NEG_INF : st.m1; p.part_l[pbase + h1] = st.l1; }
            }
#pragma unroll
            for (int mt = 0; mt < C::MT; mt++) {
                const int dg = 16 * mt + g, dg8 = dg + 8;
                if (h0 < p.group) {
                    p.part_acc[(pbase + h0) * D + dg] = st.O[mt][0];
                    p.part_acc[(pbase + h0) * D + dg8] = st.O[mt][2];
                }
                if (h1 < p.group) {
                    p.part_acc[(pbase + h1) * D + dg] = st.O[mt][1];
                    p.part_acc[(pbase + h1) * D + dg8] = st.O[mt][3];
                }
            }
        }
    }
}

// =================================================================================================
// 3. merge of the chunks + inverse value rotation
// =================================================================================================
// One CTA per (unit, query head of the group).  Threads are (chunk group cg) x (dimension j).  Every
// global load that does not depend on another one is issued up front (chunk maxima and sums, the first
// eight accumulator rows of the thread, its rows of R_v), so the kernel costs about one memory round
// trip.
// 256 threads for head_dim 64 (all CTAs of the benchmark shape are then resident at once), else 512.
constexpr int MERGE_MAX_CHUNKS = 1024;
constexpr int MERGE_BATCH = 16;

template <typename OutT, int MERGE_THREADS>
__global__ void __launch_bounds__(MERGE_THREADS) decode_merge_kernel(const DecodeParams p, int dim,
                                                                     const float* __restrict__ Rv,
                                                                     OutT* __restrict__ out,
                                                                     int32_t* __restrict__ advance) {
    __shared__ float sm_m[MERGE_MAX_CHUNKS];
    __shared__ float sm_l[MERGE_MAX_CHUNKS];
    __shared__ float red[MERGE_THREADS];
    __shared__ float y[128];
    const int u = blockIdx.x / p.group, n = blockIdx.x - u * p.group;
    const int b = u / p.kv_heads, h = u - b * p.kv_heads;
    const int tid = threadIdx.x, groups = MERGE_THREADS / dim, cg = tid / dim, j = tid - cg * dim;
    const int rows = dim / groups;                       // rows of R_v per thread (8, 16 or 32)
    pdl_trigger();
    constexpr int RVN = MERGE_THREADS == 256 ? 16 : 8;
    float rv[RVN];                                       // first RVN of this thread's R_v rows (a constant input:
#pragma unroll                                           // fetched while the streaming kernel may still be running)
    for (int k = 0; k < RVN; k++) rv[k] = k < rows ? Rv[(int64_t)(cg + k * groups) * dim + j] : 0.0f;
    pdl_wait();
    const int S = p.seq_lens[b];
    // a fused step publishes the new length once nothing of this call reads the caller's array any more
    if (advance && h == 0 && n == 0 && threadIdx.x == 0) advance[b] = S;
    // every chunk contributes one partial per consumer warp of the streaming kernel
    const int nch = min(((S + p.chunk - 1) / p.chunk) * p.sets, MERGE_MAX_CHUNKS);
    const int64_t pbase = (int64_t)u * p.nchunks * p.sets * p.group + n;

    for (int c = tid; c < nch; c += MERGE_THREADS) {
        sm_m[c] = p.part_m[pbase + (int64_t)c * p.group];
        sm_l[c] = p.part_l[pbase + (int64_t)c * p.group];
    }
    float raw[MERGE_BATCH];
#pragma unroll
    for (int k = 0; k < MERGE_BATCH; k++) {
        const int c = cg + k * groups;
        raw[k] = c < nch ? p.part_acc[(pbase + (int64_t)c * p.group) * dim + j] : 0.0f;
    }
    __syncthreads();

    float M = NEG_INF;
    for (int c = 0; c < nch; c++) M = fmaxf(M, sm_m[c]);
    __syncthreads();
    // the chunk weights 2^(m_c - M) are computed once (by the threads that loaded the chunk's m and l)
    for (int c = tid; c < nch; c += MERGE_THREADS) {
        const float w = exp2f(sm_m[c] - M);
        sm_m[c] = w;
        sm_l[c] *= w;
    }
    __syncthreads();
    float L = 0.0f;
    for (int c = 0; c < nch; c++) L += sm_l[c];
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < MERGE_BATCH; k++) {
        const int c = cg + k * groups;
        if (c < nch) acc = fmaf(sm_m[c], raw[k], acc);
    }
    for (int c = cg + MERGE_BATCH * groups; c < nch; c += groups)     // very long contexts only
        acc = fmaf(sm_m[c], p.part_acc[(pbase + (int64_t)c * p.group) * dim + j], acc);
    red[tid] = acc;
    __syncthreads();
    if (tid < dim) {
        float a = 0.0f;
        for (int gg = 0; gg < groups; gg++) a += red[gg * dim + tid];
        y[tid] = (nch > 0 && L > 0.0f) ? a / L : 0.0f;
    }
    __syncthreads();
    // out_k = sum_j y_j Rv[j][k]: this thread takes rows cg, cg + groups, ...
    float o = 0.0f;
#pragma unroll
    for (int k = 0; k < RVN; k++) if (k < rows) o = fmaf(y[cg + k * groups], rv[k], o);
    for (int k = RVN; k < rows; k++) o = fmaf(y[cg + k * groups], Rv[(int64_t)(cg + k * groups) * dim + j], o);
    __syncthreads();
    red[tid] = o;
    __syncthreads();
    if (tid < dim) {
        float a = 0.0f;
        for (int gg = 0; gg < groups; gg++) a += red[gg * dim + tid];
        out[((int64_t)b * p.q_heads + h * p.group + n) * dim + tid] = from_f32<OutT>(a);
    }
}

// ---- host side -------------------------------------------------------------------------------------

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tokens per work item: small enough that every warp of the grid gets several items, large enough
// that the per-item partial (group x (D+2) floats) stays a few percent of the streamed bytes.
// Tokens per (unit, chunk) work item of the streaming kernel.  Work items are dealt round-robin to the
// CTAs (one per SM); every item yields one partial per consumer warp, so the chunk count per unit is
// bounded by what the merge kernel keeps in shared memory.
static int choose_chunk(int64_t units, int64_t max_len, int64_t ctas, int stage_tokens, int sets) {
    int best = 0;
    double best_cost = 1e300;
    for (int64_t L = stage_tokens; L <= (int64_t)1 << 24; L *= 2) {
        const int64_t nch = (max_len + L - 1) / L;
        if (nch * sets <= 1024) {
            const int64_t rounds = (units * nch + ctas - 1) / ctas;
            const double cost = (double)rounds * ((double)std::min<int64_t>(L, max_len) + stage_tokens);
            if (cost <= best_cost) { best_cost = cost; best = (int)L; }
        }
        if (L >= max_len && best) break;
    }
    return best;
}

static DecodeWorkspace plan_workspace(int batch, int q_heads, int kv_heads, int dim, int64_t max_len) {
    DecodeWorkspace w{};
    const int64_t units = (int64_t)batch * kv_heads;
    const int group = q_heads / kv_heads;
    const int sets = dim == 64 ? 16 : 8;
    w.chunk = choose_chunk(units, std::max<int64_t>(max_len, 1), sm_count(), sets * 32, sets);
    w.nchunks = (int)std::max<int64_t>(1, (max_len + w.chunk - 1) / w.chunk);
    size_t off = 0;
    w.off_status = off; off = align_up(off + 256, 256);
    w.off_lens = off;   off = align_up(off + (size_t)batch * 4, 256);    // sequence lengths of a fused step
    w.off_qfrag = off;  off = align_up(off + (size_t)units * dim * 16, 256);   // (dim/16) x 64 words
    const size_t parts = (size_t)units * w.nchunks * sets * group;
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
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::DYN));
    const int64_t items = (int64_t)p.batch * p.kv_heads * p.nchunks;
    if (items + sm_count() >= 0x7fffffff)
        return fail(TQB_ERR_UNSUPPORTED, "decode_attention: too many (sequence, head, chunk) work items");
    const int grid = (int)std::min<int64_t>(sm_count(), items);
    TQB_CUDA(launch_pdl(pdl_mask() & 2, kern, dim3(grid), dim3(C::THREADS), C::DYN, st, p));
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

namespace tqb {
static int g_phases = 7;   // launches a decode call makes: 1 = preparation, 2 = streaming kernel, 4 = merge

// Shared by tqb_decode_attention (key == nullptr) and tqb_decode_step (key, value: the new token of every
// unit; lens_mut: the caller's sequence lengths, advanced by one at the end of the call).
static int decode_common(const void* query, int q_dtype, const void* key, const void* value, int64_t kv_stride,
                         const float* bnd_k, const float* bnd_v, int32_t* lens_mut,
                         int batch, int q_heads, int kv_heads,
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
    p.store = store; p.sets = dim == 64 ? 16 : 8;
    p.seq_lens = seq_lens; p.block_tables = block_tables; p.max_seq = max_seq;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = group;
    p.max_blocks = max_blocks; p.block_size = block_size; p.chunk = w.chunk; p.nchunks = w.nchunks;
    p.cent_k = cent_k; p.cent_v = cent_v;
    p.status = reinterpret_cast<int*>(ws + w.off_status);
    uint32_t* qfrag = reinterpret_cast<uint32_t*>(ws + w.off_qfrag);
    p.qfrag = qfrag;
    p.part_m = reinterpret_cast<float*>(ws + w.off_m);
    p.part_l = reinterpret_cast<float*>(ws + w.off_l);
    p.part_acc = reinterpret_cast<float*>(ws + w.off_acc);
    cudaStream_t st = (cudaStream_t)stream;
    const int units = batch * kv_heads;

    int32_t* lens_now = reinterpret_cast<int32_t*>(ws + w.off_lens);
    if (key) p.seq_lens = lens_now;
    cudaError_t launch_err = cudaSuccess;
    if (g_phases & 1) {
#define TQB_PREP(T, NQ) launch_err = launch_pdl(pdl_mask() & 1, decode_prepare_kernel<T, NQ>, dim3(units), dim3(256), 0, st,            \
        (const T*)query, (const T*)key, (const T*)value, kv_stride, q_heads, kv_heads, group, dim, rot_k, rot_v, \
        bnd_k, bnd_v, kbits, vbits, scale, const_cast<uint8_t*>(store), max_seq, seq_lens, lens_now, qfrag, p.status)
        switch (q_dtype) {
            case TQB_F32: if (dim == 64) TQB_PREP(float, 2); else TQB_PREP(float, 4); break;
            case TQB_F16: if (dim == 64) TQB_PREP(__half, 2); else TQB_PREP(__half, 4); break;
            case TQB_BF16: if (dim == 64) TQB_PREP(__nv_bfloat16, 2); else TQB_PREP(__nv_bfloat16, 4); break;
            default: return fail(TQB_ERR_INVALID, "decode_attention: unknown query dtype %d", q_dtype);
        }
#undef TQB_PREP
        TQB_CUDA(launch_err);
        if (int e = check_launch("decode_prepare")) return e;
    }

    if (max_len > 0 && (g_phases & 2)) {
        int e;
        if (dim == 64) e = paged ? dispatch_bits<64, true>(kbits, vbits, p, st) : dispatch_bits<64, false>(kbits, vbits, p, st);
        else e = paged ? dispatch_bits<128, true>(kbits, vbits, p, st) : dispatch_bits<128, false>(kbits, vbits, p, st);
        if (e) return e;
    }

    if (!(g_phases & 4)) return TQB_OK;
#define TQB_MERGE(T, TH) launch_err = launch_pdl(pdl_mask() & 4, decode_merge_kernel<T, TH>, dim3(units * group), dim3(TH), 0, st, p, dim, rot_v, (T*)out, lens_mut)
    switch (out_dtype) {
        case TQB_F32: if (dim == 64) TQB_MERGE(float, 256); else TQB_MERGE(float, 512); break;
        case TQB_F16: if (dim == 64) TQB_MERGE(__half, 256); else TQB_MERGE(__half, 512); break;
        case TQB_BF16: if (dim == 64) TQB_MERGE(__nv_bfloat16, 256); else TQB_MERGE(__nv_bfloat16, 512); break;
        default: return fail(TQB_ERR_INVALID, "decode_attention: unknown output dtype %d", out_dtype);
    }
#undef TQB_MERGE
    TQB_CUDA(launch_err);
    return check_launch("decode_merge");
}
}  // namespace tqb

extern "C" int tqb_decode_attention(const void* query, int q_dtype, int batch, int q_heads, int kv_heads,
                                    int dim, const uint8_t* store, int64_t max_seq,
                                    const int32_t* seq_lens, int64_t max_len, const int32_t* block_tables,
                                    int max_blocks, int block_size, const float* rot_k, const float* cent_k,
                                    int kbits, const float* rot_v, const float* cent_v, int vbits, float scale,
                                    void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                                    void* stream) {
    return tqb::decode_common(query, q_dtype, nullptr, nullptr, 0, nullptr, nullptr, nullptr, batch, q_heads,
                              kv_heads, dim, store, max_seq, seq_lens, max_len, block_tables, max_blocks,
                              block_size, rot_k, cent_k, kbits, rot_v, cent_v, vbits, scale, workspace,
                              workspace_bytes, out, out_dtype, stream);
}

extern "C" void tqb_debug_decode_phases(int mask) { tqb::g_phases = mask & 7; }

extern "C" int tqb_decode_step(const void* query, const void* key, const void* value, int dtype,
                               int64_t kv_stride, int batch, int q_heads, int kv_heads, int dim, uint8_t* store,
                               int64_t max_seq, int32_t* seq_lens, int64_t max_len, const float* rot_k,
                               const float* bnd_k, const float* cent_k, int kbits, const float* rot_v,
                               const float* bnd_v, const float* cent_v, int vbits, float scale, void* workspace,
                               size_t workspace_bytes, void* out, int out_dtype, void* stream) {
    TQB_REQUIRE(batch == 0 || (key && value && bnd_k && bnd_v), "decode_step: null pointer");
    TQB_REQUIRE(kv_stride >= dim, "decode_step: kv_stride (%lld) smaller than head_dim", (long long)kv_stride);
    TQB_REQUIRE(max_len >= 1, "decode_step: max_len counts the new token, so it is at least 1");
    return tqb::decode_common(query, dtype, key, value, kv_stride, bnd_k, bnd_v, seq_lens, batch, q_heads,
                              kv_heads, dim, store, max_seq, seq_lens, max_len, nullptr, 0, 0, rot_k, cent_k,
                              kbits, rot_v, cent_v, vbits, scale, workspace, workspace_bytes, out, out_dtype,
                              stream);
}
