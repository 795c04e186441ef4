// decode_attn.cu -- fused decode attention over a packed KV cache (one new token per sequence).
//
// Replaces "dequantise every cached key and value, then attend" (upstream
// turboquant_kv/cache.py:216-339) by ONE launch per layer call that never materialises dense K/V.
//
// decode_fused_kernel: one persistent CTA per SM.  A work item is (unit, chunk of the context); a unit
// is one (sequence, KV head), whose `group` query heads ride along as the N dimension of the MMA
// (grouped-query attention: decode cost is paid once per KV head).  Items are dealt round-robin to
// the CTAs.  Warp roles inside a CTA:
//
//   producer warp   streams the 16-token records of the CTA's items into a ring of shared-memory
//                   stages, one TMA bulk copy (cp.async.bulk + mbarrier) of up to 28 KB per stage.  It
//                   starts as soon as the sequence lengths are known: the ring fills while the other
//                   warps build the lookup tables and prepare the first item.
//   helper warp     prepares the items one ahead of the consumers: q_rot = R_k q per head, times
//                   scale * log2(e), written as mma.sync B fragments (fp16) into one of two
//                   shared-memory slots; for a fused step it also quantises the unit's new key and value
//                   and stores them into the record store before the producer copies that record (the
//                   item that holds the write position does this; the producer waits for it only before
//                   the stage with that record).  The CTA's first item is prepared before the roles
//                   split, by four warps while the others build the lookup tables.
//                   It also speaks for the consumer warps: once all of them have stored their partial
//                   of an item it counts the chunk into the unit's arrival counter (one fence for the lot).
//   consumer warps  two groups take alternate stages, four records per warp.  Per record: scores =
//                   K-codes x q on tensor cores (codes -> fp16 centroids through a 256-entry
//                   shared-memory table indexed by one byte = 2 codes), online softmax in the log2
//                   domain with a lazy running maximum, P^T via movmatrix, O^T += V^T-codes x P^T on
//                   tensor cores, all in ROTATED space.  One (m, l, acc) partial per (item, warp).
//   tail phase      once the CTA's own items are done its consumer warps take their share of ALL merges
//                   (task (unit, query head) number t -> CTA t % grid, warp (t / grid) % warps): wait,
//                   bounded, until the unit's chunks have been counted in, combine the partials, divide
//                   by l, apply the inverse value rotation acc @ R_v (reference.py:362) and write the
//                   output.  All CTAs are resident (grid <= SM count, one CTA per SM), so the wait is for
//                   work in progress.  The CTA that leaves last (exit counter) clears the arrival
//                   counters and publishes the advanced sequence lengths of a fused step.
//
// HBM traffic per token and KV head is the packed K row + packed V row + two float norms; everything
// else lives in L2 / shared memory.
//
// Every wait is bounded: a warp that gives up raises a bit of the status word at the start of the
// workspace and leaves, so a lost copy cannot hang the device.  The kernel only ever SETS bits of the
// status word (atomicOr, TQB_DECODE_* in tqb200.h); the arrival counters are returned to zero at the end
// of every call that ran to completion.  The caller zeroes the workspace once before its first
// use and after a status with TQB_DECODE_WAIT_EXPIRED or TQB_DECODE_NO_SMEM set.
#include "common.cuh"
#include "pipe.cuh"
#include "tiled_layout.cuh"


namespace tqb {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float NEG_INF = -__builtin_huge_valf();
constexpr float RESCALE_SLACK = 4.0f;   // lazy max: rescale only when a score exceeds m + 4 (log2)
constexpr int TILE = 16;                // tokens per MMA tile
constexpr int QSLOTS = 2;               // query-fragment slots (the helper warp works one item ahead)
constexpr int DSLOTS = 4;               // "every consumer warp has stored its partial" barriers, one per item in flight
constexpr int LEN_ROOM = 1 << 30;       // flag in an encoded length: this step appends a token to the sequence
constexpr int LEN_MASK = LEN_ROOM - 1;
constexpr int64_t MAX_LEN_LIMIT = (int64_t)1 << 30;
constexpr int MERGE_MAX_CHUNKS = 1024;  // partials per (unit, query head) the planner allows

// ---- launch parameters --------------------------------------------------------------------------
struct DecodeParams {
    uint8_t* store;                  // tiled records (tiled_layout.cuh)
    const int32_t* lens_in;          // the caller's sequence lengths
    int32_t* lens_out;               // fused step: the same array, advanced by the CTA that leaves last
    const int32_t* block_tables;
    int64_t max_seq;                 // token pitch of a unit (contiguous cache), multiple of 16
    int64_t max_len;                 // host bound of the attended lengths: the work plan covers [0, max_len)
    int batch, q_heads, kv_heads, group, max_blocks, block_size;
    int chunk, nchunks;              // tokens per (unit, chunk) work item
    int flat;                        // 1: the CTAs take equal pieces of the flattened tile range instead (see StageCursor)
    int step;                        // 1: append the new token of every unit first (tqb_decode_step)
    const void* query; const void* key; const void* value;
    int in_dtype; int64_t kv_stride;
    const float* rot_k; const float* rot_v; const float* bnd_k; const float* bnd_v;
    const float* cent_k; const float* cent_v;
    float scale;
    void* out; int out_dtype;
    // workspace views
    int* status; int* done;                           // header words: status bits, exit counter
    int* unit_cnt;                                    // per unit: arrivals of its chunks
    float* part_m; float* part_l; float* part_acc;
};

// Workspace layout shared by the size query and the launcher.
struct DecodeWorkspace {
    size_t off_status, off_cnt, off_m, off_l, off_acc, total;
    int chunk, nchunks;
    int flat;                           // the CTAs take equal pieces of the flattened tile range
};

__device__ __forceinline__ float load_in(const void* base, int dtype, int64_t idx) {
    if (dtype == TQB_F32) return reinterpret_cast<const float*>(base)[idx];
    if (dtype == TQB_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}
// Read-only 128-bit load that asks L1 to keep the line / not to allocate one.
__device__ __forceinline__ float4 ldg_keep(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::evict_last.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldg_stream(const float* p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
// Four consecutive elements (idx a multiple of 4, rows 8-byte aligned at least) as float4.
__device__ __forceinline__ float4 load_in4(const void* base, int dtype, int64_t idx) {
    if (dtype == TQB_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + idx);
    if (dtype == TQB_F16) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
        return make_float4(a.x, a.y, c.x, c.y);
    }
    return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u),
                       __uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
}
__device__ __forceinline__ void store_out(void* base, int dtype, int64_t idx, float v) {
    if (dtype == TQB_F32) reinterpret_cast<float*>(base)[idx] = v;
    else if (dtype == TQB_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ uint16_t half_bits_sat(float v) {   // fp16 with saturation to the largest finite value
    uint16_t r;
    asm("cvt.rn.satfinite.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
    return r;
}

// Encoded length of a sequence: bits 0..29 = tokens attended in this call, LEN_ROOM = a fused step stores
// its new token at position (attended - 1).  `flag` receives the status bits the length deserves:
// TQB_DECODE_UNIT_FULL (the step stores nothing) or TQB_DECODE_LEN_CLAMPED (the length lies outside what
// the host announced: negative, or beyond max_len).  The device never reads or writes beyond max_len / max_seq.
__device__ __forceinline__ int encode_len(const DecodeParams& p, int raw, int& flag) {
    flag = 0;
    const int cap = (int)min((int64_t)LEN_MASK, p.max_len);
    if (raw < 0) { flag = TQB_DECODE_LEN_CLAMPED; return 0; }
    if (!p.step) {
        if (raw > cap) { flag = TQB_DECODE_LEN_CLAMPED; return cap; }
        return raw;
    }
    if ((int64_t)raw >= p.max_seq) { flag = TQB_DECODE_UNIT_FULL; return (int)min((int64_t)cap, p.max_seq); }
    if (raw >= cap) { flag = TQB_DECODE_LEN_CLAMPED; return cap; }
    return (raw + 1) | LEN_ROOM;
}

// =================================================================================================
// streaming configuration
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
    static constexpr int THREADS = (WARPS + 2) * 32;                // consumer warps + producer warp + helper warp
    // head_dim 64: the first four warps prepare the CTA's first item while the others build the lookup tables
    // (one thread per row of R_k and R_v); head_dim 128 has too few warps for that and does one after the other.
    static constexpr int PREP_WARPS = D == 64 ? 4 : 0;
    // Shared-memory plan (dynamic, the whole opt-in maximum):  [ring A | aligned tables | misc | ring B]
    static constexpr int DYN = 227 * 1024;
    static constexpr int LENS_MAX = 256;
    static constexpr int QFRAG = MT * 256;                          // one slot of query fragments: MT x 32 lanes x 8 B
    // misc: centroids (256) | barriers and stage headers (8*(8+8+16) = 256) | helper barriers (64) |
    //       boundaries (128) | unit vectors of the new key / value (2*D*4) | their codes (2*D) and norms (16) |
    //       the unit's queries as float32 (8*D*4) | exit flags (16) | lengths |
    //       query-fragment slots | R_k, R_v (head_dim 64)
    static constexpr int OFF_BARS = 256, OFF_QBARS = OFF_BARS + 256, OFF_BND = OFF_QBARS + 128;
    static constexpr int OFF_UNIT = OFF_BND + 128, OFF_CODES = OFF_UNIT + 2 * D * 4, OFF_NRM = OFF_CODES + 2 * D;
    static constexpr int OFF_QVEC = OFF_NRM + 16, OFF_TODO = OFF_QVEC + 8 * D * 4, OFF_LENS = OFF_TODO + 16;
    static constexpr int OFF_TPRE = OFF_LENS + LENS_MAX * 4;        // flat partition: LENS_MAX + 1 prefix sums of tiles
    static constexpr int OFF_QFRAG = (OFF_TPRE + (LENS_MAX + 1) * 4 + 127) / 128 * 128;
    // head_dim 64: both rotation matrices live in shared memory (rows ROT_STRIDE floats apart: the 128-bit
    // loads of 32 lanes, one row each, then spread over all banks).  With the whole shared window in use the
    // L1 that is left (about 24 KB) cannot hold them, and under a saturated memory system every batch of row
    // loads from L2 took a microsecond or two: an item's preparation took 10-20 us, more than streaming it.
    // head_dim 128 has no room for 2 x 64 KB and keeps reading the rows from L2.
    static constexpr bool ROT_SMEM = D == 64;
    static constexpr int ROT_STRIDE = D + 4;
    static constexpr int ROT_BYTES = ROT_SMEM ? D * ROT_STRIDE * 4 : 0;      // one matrix
    static constexpr int OFF_ROT = OFF_QFRAG + QSLOTS * QFRAG;
    static constexpr int MISC_FIXED = OFF_ROT + 2 * ROT_BYTES;
    static constexpr int MISC = SMALL_K + SMALL_V + MISC_FIXED;
    static constexpr int BASE_MAX = 4096;                           // assumed upper bound of the window offset
    static constexpr int SLOTS_A = NALIGNED ? (65536 - BASE_MAX) / STAGE : 0;
    static constexpr int TAIL = NALIGNED ? DYN - 2 * 65536 : DYN - BASE_MAX;
    static constexpr int SLOTS_B = (TAIL - MISC - 128) / STAGE;
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

// Sequence lengths as the kernel sees them: encoded (encode_len), from a shared-memory copy when the
// batch fits, else recomputed from the caller's array.
struct Lens {
    const int32_t* sm;               // null: not cached
    const int32_t* tpre;             // flat partition: tpre[b] = 16-token tiles of all units of sequences < b; [batch] = total
    __device__ __forceinline__ int get(const DecodeParams& p, int b) const {
        if (sm) return sm[b];
        int flag;
        return encode_len(p, p.lens_in[b], flag);
    }
};

// Position of a CTA in its stream of pipeline stages.  Two ways of dealing the work:
//   chunks  items (unit, chunk of p.chunk tokens; a unit's last chunk takes the remainder too, so no item is
//           tiny) are dealt round-robin to the CTAs; the host chose the chunk from its bound on the lengths.
//           Partials of an item go to slot unit * nchunks + chunk.
//   flat    (p.flat) the tiles of all units, in unit order, form one range of T tiles (T from the lengths on
//           the device); CTA c takes tiles [c Q, (c+1) Q), Q = ceil(T / grid): a piece of a unit, whole units,
//           a piece of the next -- every CTA streams the same number of tokens whatever the number of units.
//           An item is the part of one unit inside the CTA's range; the pieces of unit u lie in consecutive
//           CTAs first(u) .. last(u), and the partials of (u, c) go to slot c + u (unique: first(u+1) >= last(u)).
// An item is streamed in stages of up to SR records, which the consumer warps share (RPW records each).
template <int SR, int GROUPS, bool FLAT>
struct StageCursor {
    int item, total_items, stride;     // (the host checks that the item count fits 31 bits)
    int seq;                            // items of this CTA opened so far, minus one
    int tiles_left, tile0;              // tiles of the item not yet taken; index of the next one in its unit
    int unit, b, h, slot, tok_end;
    bool append;                        // this item holds the position a fused step writes its new token to
    int stage_idx, stages;              // position in the item; an item takes at least GROUPS stages (empty ones
                                        // if need be) so that every consumer group sees its start and its end
    int gpos, gend;                     // flat: next global tile of this CTA, end of its range
    __device__ __forceinline__ static int flat_quota(const DecodeParams& p, const Lens& lens) {
        const int T = lens.tpre[p.batch];
        return max(1, (T + (int)gridDim.x - 1) / (int)gridDim.x);
    }
    __device__ __forceinline__ void start(const DecodeParams& p, const Lens& lens) {
        seq = -1;
        tiles_left = 0;
        if (FLAT) {
            const int T = lens.tpre[p.batch], Q = flat_quota(p, lens);
            const long long g0 = (long long)blockIdx.x * Q;
            gpos = (int)min((long long)T, g0);
            gend = (int)min((long long)T, g0 + Q);
            total_items = 1;
        } else {
            item = blockIdx.x;
            total_items = p.batch * p.kv_heads * p.nchunks;
            stride = gridDim.x;
        }
        open(p, lens);
    }
    __device__ __forceinline__ bool valid() const { return item < total_items; }
    __device__ __forceinline__ int tiles_here() const { return min(SR, tiles_left); }
    __device__ __forceinline__ void open(const DecodeParams& p, const Lens& lens) {
        if (FLAT) {
            item = 1;
            if (gpos >= gend) return;
            int lo = 0, hi = p.batch;                     // tpre[lo] <= gpos < tpre[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (lens.tpre[mid] <= gpos) lo = mid; else hi = mid;
            }
            b = lo;
            const int e = lens.get(p, b);
            const int S = e & LEN_MASK, tb = (S + TILE - 1) / TILE;      // (tb > 0: the sequence owns tile gpos)
            const int off = gpos - lens.tpre[b];
            h = off / tb;
            tile0 = off - h * tb;
            unit = b * p.kv_heads + h;
            tiles_left = min(tb - tile0, gend - gpos);
            tok_end = min(S, (tile0 + tiles_left) * TILE);
            stage_idx = 0;
            stages = max(GROUPS, (tiles_left + SR - 1) / SR);
            append = (e & LEN_ROOM) && tile0 + tiles_left == tb;
            slot = (int)blockIdx.x + unit;
            item = 0;
            seq++;
            return;
        } else {
        while (item < total_items) {
            unit = item / p.nchunks;
            const int chunk_idx = item - unit * p.nchunks;
            b = unit / p.kv_heads;
            h = unit - b * p.kv_heads;
            const int e = lens.get(p, b);
            const int S = e & LEN_MASK;
            const int tok0 = chunk_idx * p.chunk;
            tok_end = chunk_idx == p.nchunks - 1 ? S : min(S, tok0 + p.chunk);     // the last chunk takes the rest
            if (tok0 < tok_end) {
                tiles_left = (tok_end - tok0 + TILE - 1) / TILE;
                tile0 = tok0 / TILE;
                stage_idx = 0;
                stages = max(GROUPS, (tiles_left + SR - 1) / SR);
                append = (e & LEN_ROOM) && min(p.nchunks - 1, (S - 1) / p.chunk) == chunk_idx;
                slot = unit * p.nchunks + chunk_idx;
                seq++;
                return;
            }
            item += stride;
        }
        }
    }
    __device__ __forceinline__ void next(const DecodeParams& p, const Lens& lens) {
        const int n = tiles_here();
        tiles_left -= n; tile0 += n; stage_idx++;
        if (FLAT) gpos += n;
        if (stage_idx == stages) {
            if (!FLAT) item += stride;
            open(p, lens);
        }
    }
    __device__ __forceinline__ void next_item(const DecodeParams& p, const Lens& lens) {
        if (FLAT) gpos += tiles_left; else item += stride;
        open(p, lens);
    }
};

// Where the partials of a unit lie and how many items (arrivals) make it complete.
template <bool FLAT>
__device__ __forceinline__ void unit_pieces(const DecodeParams& p, const Lens& lens, int unit, int S, int& slot0, int& need) {
    if (FLAT) {
        const int b = unit / p.kv_heads, h = unit - b * p.kv_heads;
        const int tb = (S + TILE - 1) / TILE, Q = StageCursor<1, 1, true>::flat_quota(p, lens);
        const int a = lens.tpre[b] + h * tb;
        const int first = a / Q, last = (a + tb - 1) / Q;
        slot0 = first + unit;
        need = last - first + 1;
    } else {
        slot0 = unit * p.nchunks;
        need = min(p.nchunks, (S + p.chunk - 1) / p.chunk);
    }
}

// =================================================================================================
// item preparation: query fragments, and the new token of a fused step
// =================================================================================================
// Shared-memory scratch of the preparation (DecodeCfg::OFF_*).
struct PrepScratch {
    const float* bnd;                // [2][16] boundaries (keys, values), +inf beyond the last
    float* qvec;                     // [8][D]  the unit's queries as float32
    float* unit;                     // [2][D]  unit vector of the new key / value
    uint32_t qvec_addr, unit_addr;   //         shared addresses of qvec and unit
    uint8_t* codes;                  // [2][D]
    float* nrm;                      // [2]
    uint32_t rot_addr;               //         shared address of R_k, R_v behind it (DecodeCfg::ROT_SMEM)
};

// Prepares one item with `nthreads` threads (`tid` = 0..nthreads-1): one warp (barriers are __syncwarp), or a
// group of warps that meets on named barrier 2.  Writes the B fragments of the unit's rotated queries into
// `qslot`: element (ks, lane = 4n+t, half) of head n holds the rotated query coordinates (16ks + 8half + 2t,
// +1) times scale * log2(e) as fp16 (11 significant bits whatever the magnitude; the products stay far
// inside fp16's range); the columns of heads >= group stay zero.
//
// With `append` it first quantises the unit's new key and value and stores them at position `pos`.  The
// code selection repeats quantize.cu's arithmetic exactly (norm by per-lane partial sums over consecutive
// elements and a butterfly, unit = x / max(norm, 1e-10), y_j as one fused-multiply-add chain over k ascending,
// code = number of boundaries below y_j), so the stored codes are those tqb_kv_append would store.
// The stores are followed by a proxy fence: the producer copies that record with the TMA engine.
template <int D, int KB, int VB, bool ONE_WARP, bool DO_Q = true, bool DO_KV = true>
__device__ __forceinline__ void prepare_item(const DecodeParams& p, int unit, bool append_item, int pos,
                                             uint16_t* qslot, const PrepScratch& sc, int tid, int nthreads) {
    // DO_Q: the query fragments.  DO_KV: the new token of a fused step.  The two halves can be done by
    // different warps at the same time (they share no scratch), or one after the other.
    const bool append = DO_KV && append_item;
    if (!DO_Q && !append) return;
    constexpr int NQ = D / 32;
    const int b = unit / p.kv_heads, h = unit - b * p.kv_heads;
    const int warp = tid >> 5, lane = tid & 31;
    auto sync = [&]() {
        if (ONE_WARP) __syncwarp();
        else asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");
    };
    using C = DecodeCfg<D, KB, VB>;
    const int64_t q0 = ((int64_t)b * p.q_heads + h * p.group) * D;
    const float fold = p.scale * LOG2E;
    if (DO_Q)
        for (int e = 4 * tid; e < p.group * D; e += 4 * nthreads)  // the unit's queries -> float32 in shared memory
            *reinterpret_cast<float4*>(sc.qvec + e) = load_in4(p.query, p.in_dtype, q0 + e);
    if (append) {
        // norm and unit vector of the key (which = 0) and the value (1): one warp each, or one after the other
        for (int which = ONE_WARP ? 0 : warp; which < 2; which += ONE_WARP ? 1 : 2) {
            const void* x = which ? p.value : p.key;
            const int64_t x0 = (int64_t)unit * p.kv_stride;
            float v[NQ], ss = 0.0f;
#pragma unroll
            for (int qq = 0; qq < NQ; qq++) {
                v[qq] = load_in(x, p.in_dtype, x0 + lane * NQ + qq);         // (the norm's summation order of quantize.cu)
                ss = fmaf(v[qq], v[qq], ss);
            }
            const float n = sqrtf(warp_sum(ss));
            const float den = fmaxf(n, 1e-10f);
#pragma unroll
            for (int qq = 0; qq < NQ; qq++) sc.unit[which * D + lane * NQ + qq] = v[qq] / den;
            if (lane == 0) sc.nrm[which] = n;
        }
    }
    sync();
    // One thread per ROW of a rotation matrix: row j of R_k serves the unit's `group` queries and its new key
    // (the row is fetched once for all of them), row j of R_v the new value.  A row is fetched in batches of
    // eight 128-bit loads that are all in flight together -- from shared memory at head_dim 64, else from
    // global memory with a request to L1 to keep the lines (evict-last): under a saturated memory system a
    // round trip to L2 takes microseconds, and R_k is re-read for every item.  The sums run over k ascending.
    const int ntasks = append ? 2 * D : D;
    for (int task = tid; task < ntasks; task += nthreads) {
        const int which = task / D, j = task - which * D;           // 0: R_k row (queries, key), 1: R_v row (value)
        const float4* row = reinterpret_cast<const float4*>((which ? p.rot_v : p.rot_k) + (int64_t)j * D);
        const uint32_t srow = sc.rot_addr + which * C::ROT_BYTES + j * C::ROT_STRIDE * 4;   // (head_dim 64: the row in shared memory)
        float aq[8], ax = 0.0f;
#pragma unroll
        for (int n = 0; n < 8; n++) aq[n] = 0.0f;
#pragma unroll 1
        for (int kb = 0; kb < D / 4; kb += 8) {
            float4 r[8];
#pragma unroll
            for (int i = 0; i < 8; i++) r[i] = C::ROT_SMEM ? lds128f(srow + (kb + i) * 16) : ldg_keep(row + kb + i);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int k0 = 4 * (kb + i);
                if (DO_Q && which == 0) {
#pragma unroll
                    for (int n = 0; n < 8; n++) {
                        if (n < p.group) {
                            const float4 x = lds128f(sc.qvec_addr + (n * D + k0) * 4);
                            aq[n] = fmaf(x.x, r[i].x, aq[n]);
                            aq[n] = fmaf(x.y, r[i].y, aq[n]);
                            aq[n] = fmaf(x.z, r[i].z, aq[n]);
                            aq[n] = fmaf(x.w, r[i].w, aq[n]);
                        }
                    }
                }
                if (append) {
                    const float4 u = lds128f(sc.unit_addr + (which * D + k0) * 4);
                    ax = fmaf(u.x, r[i].x, ax);
                    ax = fmaf(u.y, r[i].y, ax);
                    ax = fmaf(u.z, r[i].z, ax);
                    ax = fmaf(u.w, r[i].w, ax);
                }
            }
        }
        if (DO_Q && which == 0) {
            const int ks = j >> 4, half = (j >> 3) & 1, t = (j & 7) >> 1, hi = j & 1;
#pragma unroll
            for (int n = 0; n < 8; n++)
                if (n < p.group) qslot[2 * (ks * 64 + (4 * n + t) * 2 + half) + hi] = half_bits_sat(aq[n] * fold);
        }
        if (append) {
            const float* bnd = sc.bnd + which * 16;
            uint32_t c = 0;
            for (int s = 1 << ((which ? VB : KB) - 1); s > 0; s >>= 1)
                if (bnd[c + s - 1] < ax) c += s;
            sc.codes[which * D + j] = (uint8_t)c;
        }
    }
    sync();
    if (append) {
        for (int which = ONE_WARP ? 0 : warp; which < 2; which += ONE_WARP ? 1 : 2) {
            uint32_t code[NQ];
#pragma unroll
            for (int qq = 0; qq < NQ; qq++) code[qq] = sc.codes[which * D + lane + 32 * qq];
            tiled_store_row<NQ>(p.store, which + 1, KB, VB, (int64_t)unit * p.max_seq + pos, code, sc.nrm[which], lane, D);
            // generic-proxy stores above, async-proxy (TMA) read of the same record below
            asm volatile("fence.proxy.async;" ::: "memory");
        }
        sync();
    }
}

// Per-warp softmax state of the item being processed.
template <int MT>
struct WarpState {
    float m0, m1, l0, l1;      // running maximum (log2 domain; 0 before the first token) and row sums
    float thr;                 // rescale when a shifted score exceeds this: -inf before the first token, then the slack
    float O[MT][4];
    uint32_t qf[MT][2];
};

// NT (1, 2 or 4) 16-token records at once: scores, online softmax, accumulation.  All records go through
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
        // the four norms this lane needs of the record: keys of tokens g, g+8, values of tokens g, g+8
        uint32_t nw[4];
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(nw[0]), "=r"(nw[1]), "=r"(nw[2]), "=r"(nw[3])
                     : "r"(rec0 + i * C::REC + C::KSEC + C::VSEC + 16 * g));
        const bool val_g = !MASKED || 16 * i + g < valid, val_g8 = !MASKED || 16 * i + g + 8 < valid;
        float nkg = __uint_as_float(nw[0]), nkg8 = __uint_as_float(nw[1]);
        nvg[i] = __uint_as_float(nw[2]);
        nvg8[i] = __uint_as_float(nw[3]);
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

// =================================================================================================
// tail phase: merge of a (unit, query head) + inverse value rotation, by one warp
// =================================================================================================
// Partial c (< nparts) of head n sits at part_*[pbase + c * group] (and * D for the accumulators).  The
// partials were written by other warps, possibly of other CTAs, before they bumped the unit's arrival
// counter: they are read past L1 (ld.global.cg).
template <int D>
__device__ __forceinline__ void merge_head(const DecodeParams& p, int unit, int slot0, int n, int nparts, int lane,
                                           const float* rot_v, int rot_stride) {
    constexpr int NQ = D / 32;
    const int b = unit / p.kv_heads, h = unit - b * p.kv_heads;
    const int64_t pbase = (int64_t)slot0 * (D == 64 ? 16 : 8) * p.group + n;
    // The kernel is a chain of round trips to L2; every phase keeps as many loads in flight as it can.
    float M = NEG_INF;
    for (int c0 = 0; c0 < nparts; c0 += 128) {
        float mv[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int c = c0 + 32 * k + lane;
            mv[k] = c < nparts ? __ldcg(p.part_m + pbase + (int64_t)c * p.group) : NEG_INF;
        }
#pragma unroll
        for (int k = 0; k < 4; k++) M = fmaxf(M, mv[k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.0f, acc[NQ];
#pragma unroll
    for (int i = 0; i < NQ; i++) acc[i] = 0.0f;
    for (int c0 = 0; c0 < nparts; c0 += 32) {
        const int c = c0 + lane;
        const int cn = min(32, nparts - c0);                        // (a multiple of 8: 8 or 16 partials per chunk)
        // the first sixteen partial rows of the block are requested together with its maxima and sums
        float v[16][NQ];
#pragma unroll
        for (int cc = 0; cc < 16; cc++) {
            const float* row = p.part_acc + (pbase + (int64_t)(c0 + cc) * p.group) * D + lane;
#pragma unroll
            for (int i = 0; i < NQ; i++) v[cc][i] = cc < cn ? __ldcg(row + 32 * i) : 0.0f;
        }
        float w = 0.0f;
        if (c < nparts) {
            const float m = __ldcg(p.part_m + pbase + (int64_t)c * p.group);
            const float l = __ldcg(p.part_l + pbase + (int64_t)c * p.group);
            w = (m == NEG_INF) ? 0.0f : exp2f(m - M);
            L = fmaf(l, w, L);
        }
#pragma unroll
        for (int cc = 0; cc < 16; cc++) {
            const float wc = __shfl_sync(0xffffffffu, w, cc);
#pragma unroll
            for (int i = 0; i < NQ; i++) acc[i] = fmaf(wc, v[cc][i], acc[i]);
        }
        if (cn > 16) {
#pragma unroll
            for (int cc = 0; cc < 16; cc++) {
                const float* row = p.part_acc + (pbase + (int64_t)(c0 + 16 + cc) * p.group) * D + lane;
#pragma unroll
                for (int i = 0; i < NQ; i++) v[cc][i] = 16 + cc < cn ? __ldcg(row + 32 * i) : 0.0f;
            }
#pragma unroll
            for (int cc = 0; cc < 16; cc++) {
                const float wc = __shfl_sync(0xffffffffu, w, 16 + cc);
#pragma unroll
                for (int i = 0; i < NQ; i++) acc[i] = fmaf(wc, v[cc][i], acc[i]);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    const float inv = (nparts > 0 && L > 0.0f) ? 1.0f / L : 0.0f;
    float y[NQ], out[NQ];
#pragma unroll
    for (int i = 0; i < NQ; i++) { y[i] = acc[i] * inv; out[i] = 0.0f; }
    // out_k = sum_j y_j Rv[j][k]  (x = y @ R, reference.py:362); lane holds k = lane + 32 i.  R_v is read
    // through L1: the warps of a CTA that merge at the same time share its lines.
#pragma unroll
    for (int ij = 0; ij < NQ; ij++) {
#pragma unroll 1
        for (int jb = 0; jb < 32; jb += 16) {                       // sixteen rows of R_v in flight together
            float r[16][NQ];
#pragma unroll
            for (int jj = 0; jj < 16; jj++) {
                const float* row = rot_v + (int64_t)(32 * ij + jb + jj) * rot_stride + lane;
#pragma unroll
                for (int i = 0; i < NQ; i++) r[jj][i] = row[32 * i];
            }
#pragma unroll
            for (int jj = 0; jj < 16; jj++) {
                const float yj = __shfl_sync(0xffffffffu, y[ij], jb + jj);
#pragma unroll
                for (int i = 0; i < NQ; i++) out[i] = fmaf(yj, r[jj][i], out[i]);
            }
        }
    }
    const int64_t o0 = ((int64_t)b * p.q_heads + h * p.group + n) * D + lane;
#pragma unroll
    for (int i = 0; i < NQ; i++) store_out(p.out, p.out_dtype, o0 + 32 * i, out[i]);
}

// =================================================================================================
// the kernel
// =================================================================================================
template <int D, int KB, int VB, bool PAGED, bool FLAT>
__global__ void __launch_bounds__(DecodeCfg<D, KB, VB>::THREADS, 1) decode_fused_kernel(const DecodeParams p) {
    using C = DecodeCfg<D, KB, VB>;
    constexpr int WARPS = C::WARPS, NS = C::NS, SR = C::SR, RPW = C::RPW, GROUPS = C::GROUPS, WPG = C::WPG;
    constexpr int PREP_WARPS = C::PREP_WARPS;
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
        slotsA = 0; tabK_base = tabV_base = 0; misc = (base + 127u) & ~127u;
    }
    if (!C::KBYTE) { tabK_base = misc; misc += C::SMALL_K; }
    if (!C::VBYTE) { tabV_base = misc; misc += C::SMALL_V; }
    const uint32_t cent_addr = misc;                             // 32 floats
    const uint32_t full_addr = misc + C::OFF_BARS;               // full[s]: the stage's bytes have landed
    const uint32_t empty_addr = full_addr + 8 * 8;               // empty[s]: every warp of the stage's group has finished with it
    const uint32_t meta_addr = empty_addr + 8 * 8;               // one uint4 per stage: {unit, chunk, tiles | flags, valid tokens}
    const uint32_t qfull_addr = misc + C::OFF_QBARS;             // qfull[q]: the item's query fragments are in slot q
    const uint32_t qempty_addr = qfull_addr + 8 * QSLOTS;        // qempty[q]: every consumer warp has taken them
    const uint32_t done_addr = qempty_addr + 8 * QSLOTS;         // done[d]: every consumer warp has stored its partial of the item
    const uint32_t qfrag_addr = misc + C::OFF_QFRAG;
    const uint32_t rot_addr = misc + C::OFF_ROT;
    ringB = (misc + C::MISC_FIXED + 127u) & ~127u;
    const int slotsB = ringB < end ? (int)((end - ringB) / C::STAGE) : 0;
    if (slotsA + slotsB < NS) {                      // cannot happen unless the window offset is unusually large
        if (threadIdx.x == 0) atomicOr(p.status, TQB_DECODE_NO_SMEM);
        return;
    }
    auto slot_addr = [&](int slot) -> uint32_t {
        return slot < slotsA ? ringA + slot * C::STAGE : ringB + (slot - slotsA) * C::STAGE;
    };
    uint8_t* const smem_gen = smem_raw - base;       // generic pointer of shared address 0
    // [1] this CTA leaves last  [2] items of this CTA whose new token (if any) has been stored
    volatile int* const todo = reinterpret_cast<volatile int*>(smem_gen + misc + C::OFF_TODO);
    PrepScratch scratch;
    scratch.bnd = reinterpret_cast<const float*>(smem_gen + misc + C::OFF_BND);
    scratch.unit = reinterpret_cast<float*>(smem_gen + misc + C::OFF_UNIT);
    scratch.qvec = reinterpret_cast<float*>(smem_gen + misc + C::OFF_QVEC);
    scratch.qvec_addr = misc + C::OFF_QVEC;
    scratch.unit_addr = misc + C::OFF_UNIT;
    scratch.codes = smem_gen + misc + C::OFF_CODES;
    scratch.nrm = reinterpret_cast<float*>(smem_gen + misc + C::OFF_NRM);
    scratch.rot_addr = rot_addr;
    pdl_trigger();

    // ---- constants: centroids, boundaries, barriers, empty query slots ----
    if (threadIdx.x < 16) {
        float* cf = reinterpret_cast<float*>(smem_gen + cent_addr);
        cf[threadIdx.x] = threadIdx.x < (1 << KB) ? p.cent_k[threadIdx.x] : 0.0f;
        cf[16 + threadIdx.x] = threadIdx.x < (1 << VB) ? p.cent_v[threadIdx.x] : 0.0f;
    } else if (threadIdx.x < 48 && p.step) {
        const int which = (threadIdx.x - 16) >> 4, i = threadIdx.x & 15;
        const int nb = (1 << (which ? VB : KB)) - 1;
        reinterpret_cast<float*>(smem_gen + misc + C::OFF_BND)[which * 16 + i] =
            i < nb ? (which ? p.bnd_v : p.bnd_k)[i] : __int_as_float(0x7f800000);
    }
    if (threadIdx.x < NS) {
        mbar_init(full_addr + threadIdx.x * 8, 1);
        mbar_init(empty_addr + threadIdx.x * 8, WPG);
    }
    if (threadIdx.x < QSLOTS) {
        mbar_init(qfull_addr + threadIdx.x * 8, 1);
        mbar_init(qempty_addr + threadIdx.x * 8, WARPS);
    }
    if (threadIdx.x < DSLOTS) mbar_init(done_addr + threadIdx.x * 8, WARPS);
    if (threadIdx.x == 0) { todo[0] = 0; todo[1] = 0; todo[2] = 0; }
    for (int i = threadIdx.x; i < QSLOTS * C::QFRAG / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem_gen + qfrag_addr)[i] = 0u;
    if (C::ROT_SMEM) {                               // (constants: no wait for the previous launch needed)
        constexpr int V4 = D / 4;                    // float4 per row
        for (int e = threadIdx.x; e < 2 * D * V4; e += blockDim.x) {
            const int which = e / (D * V4), rem = e - which * D * V4, j = rem / V4, c = rem - j * V4;
            const float4 v = __ldg(reinterpret_cast<const float4*>(which ? p.rot_v : p.rot_k) + rem);
            *reinterpret_cast<float4*>(smem_gen + rot_addr + which * C::ROT_BYTES + (j * C::ROT_STRIDE + 4 * c) * 4) = v;
        }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // ---- lookup tables (constants only), and -- by the first PREP_WARPS warps, at the same time, when
    // PREP_WARPS > 0 -- the sequence lengths and the CTA's first item (the caller's tensors) ----
    const bool lens_in_smem = p.batch <= C::LENS_MAX;
    Lens lens;
    lens.sm = lens_in_smem ? reinterpret_cast<const int32_t*>(smem_gen + misc + C::OFF_LENS) : nullptr;
    lens.tpre = reinterpret_cast<const int32_t*>(smem_gen + misc + C::OFF_TPRE);
    StageCursor<SR, GROUPS, FLAT> cur;
    // lengths clamped to what the host announced; CTA 0 reports and clears the outputs of empty sequences
    auto load_lens = [&](int tid, int nthreads) {
        if (!lens_in_smem && blockIdx.x != 0) return;
        for (int i = tid; i < p.batch; i += nthreads) {
            int flag;
            const int e = encode_len(p, p.lens_in[i], flag);
            if (lens_in_smem) reinterpret_cast<int32_t*>(smem_gen + misc + C::OFF_LENS)[i] = e;
            if (blockIdx.x == 0) {
                if (flag) atomicOr(p.status, flag);
                if ((e & LEN_MASK) == 0)            // nothing to attend to: the output rows are zero
                    for (int k = 0; k < p.q_heads * D; k++) store_out(p.out, p.out_dtype, (int64_t)i * p.q_heads * D + k, 0.0f);
            }
        }
    };
    auto first_item = [&](int tid, int nthreads) {   // (every thread of the preparing group takes the same path)
        cur.start(p, lens);
        if (cur.valid())
            prepare_item<D, KB, VB, false, true, PREP_WARPS == 0>(p, cur.unit, cur.append, (lens.get(p, cur.b) & LEN_MASK) - 1,
                                                                 reinterpret_cast<uint16_t*>(smem_gen + qfrag_addr), scratch, tid, nthreads);
    };
    // Roles of the prologue.  The PRODUCER loads the lengths (everybody's cursor needs them) and starts
    // streaming at once: records depend neither on the tables nor on the queries, so the ring fills while
    // the others work.  The first PREP_WARPS warps (all but the producer when PREP_WARPS == 0) prepare the
    // CTA's first item; the rest builds the lookup tables, which depend on constants only and so come
    // before the wait for the previous launch.  Consumers and helper meet on barrier 4 before the stream is
    // consumed; the producer is not held up by it.
    // SPLIT (head_dim 64): four consumer warps rotate the first item's queries, the helper warp stores its new
    // token at the same time, the other consumer warps build the tables.  Otherwise all warps but the
    // producer build the tables, then prepare the first item together.
    constexpr bool SPLIT = PREP_WARPS > 0;
    const bool prep_group = SPLIT ? warp < PREP_WARPS : warp != WARPS;
    constexpr int NPREP = SPLIT ? PREP_WARPS : WARPS + 1;
    constexpr int COUNT3 = (1 + NPREP + (SPLIT ? 1 : 0)) * 32;         // producer (arrives), preparing warps, helper
    constexpr int COUNT4 = (SPLIT ? WARPS : WARPS + 1) * 32;           // the warps that wait for tables and fragments
    if (warp == WARPS) {
        pdl_wait();
        load_lens(lane, 32);
        __syncwarp();
        if (FLAT) {
            // exclusive prefix sums of the units' tiles per sequence (p.flat implies batch <= LENS_MAX): each
            // lane takes a run of sequences, the runs are scanned across the warp
            int32_t* tpre = reinterpret_cast<int32_t*>(smem_gen + misc + C::OFF_TPRE);
            const int per = (p.batch + 31) / 32, b0 = lane * per;
            int run = 0;
            for (int i = 0; i < per; i++)
                if (b0 + i < p.batch) run += p.kv_heads * (((lens.sm[b0 + i] & LEN_MASK) + TILE - 1) / TILE);
            int incl = run;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            int acc = incl - run;
            for (int i = 0; i < per; i++)
                if (b0 + i < p.batch) {
                    tpre[b0 + i] = acc;
                    acc += p.kv_heads * (((lens.sm[b0 + i] & LEN_MASK) + TILE - 1) / TILE);
                }
            if (lane == 31) tpre[p.batch] = incl;
            __syncwarp();
        }
        asm volatile("bar.arrive 3, %0;" ::"n"(COUNT3) : "memory");   // the lengths are in shared memory
        cur.start(p, lens);
    } else if (SPLIT && warp == WARPS + 1) {
        pdl_wait();
        asm volatile("bar.sync 3, %0;" ::"n"(COUNT3) : "memory");
        cur.start(p, lens);
        if (cur.valid())
            prepare_item<D, KB, VB, true, false, true>(p, cur.unit, cur.append, (lens.get(p, cur.b) & LEN_MASK) - 1,
                                                       reinterpret_cast<uint16_t*>(smem_gen + qfrag_addr), scratch, lane, 32);
        __syncwarp();
        if (lane == 0) { __threadfence_block(); todo[2] = 1; }        // the first item's new token is in the store
    } else {
        if (!SPLIT || !prep_group) {
            const float* cf = reinterpret_cast<const float*>(smem_gen + cent_addr);
            constexpr int KSTR = C::KBYTE ? 256 : 128, VSTR = C::VBYTE ? 256 : 128;
            constexpr int TW = SPLIT ? WARPS - PREP_WARPS : WARPS + 1; // warps that build the tables
            const int tw = SPLIT ? warp - PREP_WARPS : (warp > WARPS ? WARPS : warp);
            for (int x = tw; x < C::LUTK_ENTRIES; x += TW) {
                int clo, chi;
                tl_key_field_codes((uint32_t)x, KB, clo, chi);
                *reinterpret_cast<uint32_t*>(smem_gen + tabK_base + x * KSTR + lane * 4) = pack_half2(cf[clo], cf[chi]);
            }
            for (int x = tw; x < C::LUTV_ENTRIES; x += TW) {
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
        // everything above depends on constants only; from here on the caller's tensors and the workspace are used
        pdl_wait();
        if (prep_group) {
            asm volatile("bar.sync 3, %0;" ::"n"(COUNT3) : "memory");
            first_item(warp > WARPS ? (int)threadIdx.x - 32 : (int)threadIdx.x, NPREP * 32);
        }
        asm volatile("bar.sync 4, %0;" ::"n"(COUNT4) : "memory");
        if (!prep_group) cur.start(p, lens);
    }
    if (threadIdx.x == 0) {
        if (!SPLIT) { __threadfence_block(); todo[2] = 1; }
        if (cur.valid()) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qfull_addr) : "memory");
    }
    const uint32_t tabK = tabK_base + lane * 4;                    // for BYTE tables "+" is "|": the low 16 bits of the base are 0
    const uint32_t tabV = tabV_base + (C::VQUAD ? (lane & 15) * 8 : lane * 4);

    if (warp == WARPS) {
        // ---- producer warp: streams the CTA's items.  Lane 0 owns the barriers and the stage headers and
        // issues the one bulk copy of a stage of a contiguous cache; for a paged cache every record is its own
        // copy (pages are scattered), and the 32 lanes issue them side by side.  All lanes track the cursor.
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
            if (ok && cur.valid() && cur.append && cur.tiles_left <= SR) {
                // the new token of this item's unit (its last position) must be in the record store before the
                // stage that holds its record is copied; the item's earlier stages do not wait for it.  (A
                // counter, not a barrier: the helper may be two items ahead of this point.)
                if (lane == 0) {
                    const unsigned long long t0 = wall_ns();
                    while (todo[2] <= cur.seq)
                        if (wall_ns() - t0 > WAIT_LIMIT_NS) { ok = false; break; }
                    __threadfence_block();
                }
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
                *meta = make_uint4((uint32_t)cur.unit, (uint32_t)cur.slot,
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
            atomicOr(p.status, TQB_DECODE_WAIT_EXPIRED);
            for (uint32_t i = (n > (uint32_t)NS ? n - NS : 0); i < n; i++)
                (void)mbar_wait(full_addr + 8 * (i % NS), (i / NS) & 1);   // (padding stages complete at once)
        }
    } else if (warp == WARPS + 1) {
        // ---- helper warp: prepares the CTA's second, third, ... item while earlier ones stream, and speaks
        // for the CTA's consumer warps: once all of them have stored their partial of an item (done barrier)
        // it counts the chunk into the unit's arrival counter, with one fence for the lot.  The merges wait
        // for these counters in the tail phase.
        StageCursor<SR, GROUPS, FLAT> told = cur;            // the next item to announce
        bool ok = true;
        auto announce = [&]() {
            if (lane == 0) ok = mbar_wait(done_addr + 8 * (told.seq % DSLOTS), (told.seq / DSLOTS) & 1);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) return;
            if (lane == 0) {
                __threadfence();                                  // the consumers' partials before the count
                atomicAdd(p.unit_cnt + told.unit, 1);
            }
            told.next_item(p, lens);
        };
        while (ok) {
            cur.next_item(p, lens);
            if (!cur.valid()) break;
            const int q = cur.seq % QSLOTS, use = cur.seq / QSLOTS;
            if (use >= 1) {                         // the slot's previous fragments have been taken by every consumer warp
                if (lane == 0) ok = mbar_wait(qempty_addr + 8 * q, (use - 1) & 1);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
            }
            uint16_t* const qdst = reinterpret_cast<uint16_t*>(smem_gen + qfrag_addr + q * C::QFRAG);
            const int pos = (lens.get(p, cur.b) & LEN_MASK) - 1;
            if (SPLIT) {
                // queries first: the consumers can start on the item while its new token is being stored
                if (cur.seq == 1) {                 // (the first item's queries were staged in the same scratch)
                    if (lane == 0) ok = mbar_wait(qfull_addr, 0);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                }
                prepare_item<D, KB, VB, true, true, false>(p, cur.unit, cur.append, pos, qdst, scratch, lane, 32);
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qfull_addr + 8 * q) : "memory");
                prepare_item<D, KB, VB, true, false, true>(p, cur.unit, cur.append, pos, qdst, scratch, lane, 32);
            } else {
                prepare_item<D, KB, VB, true>(p, cur.unit, cur.append, pos, qdst, scratch, lane, 32);
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qfull_addr + 8 * q) : "memory");
            }
            __syncwarp();
            if (lane == 0) { __threadfence_block(); todo[2] = cur.seq + 1; }
            // The item two behind the one just prepared was finished by the consumers before they could take
            // this slot's previous fragments, so its announcement never waits long; and because it comes before
            // the next item is handed over, the done barriers (DSLOTS in rotation) can never be lapped.
            if (cur.seq >= 2) announce();
        }
        while (ok && told.valid()) announce();
        if (!ok && lane == 0) atomicOr(p.status, TQB_DECODE_WAIT_EXPIRED);
    } else {
    // ---- consumers: group (warp / WPG) takes every GROUPS-th stage; its warp i takes records RPW*i .. RPW*i+RPW-1 ----
    WarpState<C::MT> st;
    int unit = 0, slot = 0, seq = -1;
    st.m0 = st.m1 = st.l0 = st.l1 = 0.0f; st.thr = NEG_INF;
    const int r0 = RPW * (warp % WPG);
    for (uint32_t n = warp / WPG;; n += GROUPS) {
        const int s = n % NS;
        bool ok = mbar_wait(full_addr + 8 * s, (n / NS) & 1);
        uint4 meta = make_uint4(0, 0, 0, 0);
        if (ok)
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(meta.x), "=r"(meta.y), "=r"(meta.z), "=r"(meta.w) : "r"(meta_addr + s * 16));
        if (ok && (meta.z & F_FIRST) && !(meta.z & F_END)) {      // this group's first stage of an item
            seq++;
            ok = mbar_wait(qfull_addr + 8 * (seq % QSLOTS), (seq / QSLOTS) & 1);
        }
        if (!__all_sync(0xffffffffu, ok)) {           // a copy or the helper warp never arrived: flag it and stop
            if (lane == 0) atomicOr(p.status, TQB_DECODE_WAIT_EXPIRED);
            break;
        }
        if (meta.z & F_END) {                         // end of the stream (release the marker's slot as well)
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_addr + 8 * s) : "memory");
            break;
        }
        const int nt = meta.z & 0xffff;
        if (meta.z & F_FIRST) {
            unit = (int)meta.x; slot = (int)meta.y;
            st.m0 = st.m1 = 0.0f; st.l0 = st.l1 = 0.0f; st.thr = NEG_INF;
#pragma unroll
            for (int mt = 0; mt < C::MT; mt++) { st.O[mt][0] = st.O[mt][1] = st.O[mt][2] = st.O[mt][3] = 0.0f; }
            const uint32_t qsrc = qfrag_addr + (seq % QSLOTS) * C::QFRAG + lane * 8;
#pragma unroll
            for (int ks = 0; ks < C::MT; ks++)
                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(st.qf[ks][0]), "=r"(st.qf[ks][1]) : "r"(qsrc + ks * 256));
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(qempty_addr + 8 * (seq % QSLOTS)) : "memory");
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
            const int64_t pbase = ((int64_t)slot * WARPS + warp) * p.group;
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
            // tell the helper warp (no fence, no wait: it publishes the CTA's partials of this item in one go)
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(done_addr + 8 * (seq % DSLOTS)) : "memory");
        }
    }

    // ---- tail phase: the merges of all units, dealt to the consumer warps of all CTAs ----
    // Task (unit, query head) number t goes to CTA t % grid, warp (t / grid) % WARPS: the CTAs finish their
    // streams at about the same time, so every warp gets at most a task or two whichever CTA streamed the
    // unit's chunks.  A warp waits (bounded) until the unit's chunks have all been counted in.
    {
        const int tasks = p.batch * p.kv_heads * p.group;
        bool ok = true;
        for (int task = (int)blockIdx.x + (int)gridDim.x * warp; task < tasks && ok; task += (int)gridDim.x * WARPS) {
            const int u = task / p.group, nh = task - u * p.group;
            const int S = lens.get(p, u / p.kv_heads) & LEN_MASK;
            if (S == 0) continue;                             // (CTA 0 zeroed the outputs of empty sequences)
            int slot0, need;
            unit_pieces<FLAT>(p, lens, u, S, slot0, need);
            if (lane == 0) {
                const unsigned long long t0 = wall_ns();
                int seen;
                for (;;) {
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.unit_cnt + u) : "memory");
                    if (seen >= need) break;
                    if (wall_ns() - t0 > WAIT_LIMIT_NS) { ok = false; break; }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) { if (lane == 0) atomicOr(p.status, TQB_DECODE_WAIT_EXPIRED); break; }
            merge_head<D>(p, u, slot0, nh, need * WARPS, lane,
                          C::ROT_SMEM ? reinterpret_cast<const float*>(smem_gen + rot_addr + C::ROT_BYTES) : p.rot_v,
                          C::ROT_SMEM ? C::ROT_STRIDE : D);
        }
    }
    }   // consumers

    // ---- the CTA that leaves last clears the arrival counters and publishes the new lengths of a fused step ----
    __syncthreads();                                  // every role of this CTA is done (no read of lengths or counters after this)
    if (threadIdx.x == 0) {
        __threadfence();
        const int last = atomicAdd(p.done, 1) == (int)gridDim.x - 1;
        if (last) atomicExch(p.done, 0);
        todo[1] = last;
    }
    __syncthreads();
    if (todo[1]) {
        for (int i = threadIdx.x; i < p.batch * p.kv_heads; i += blockDim.x) p.unit_cnt[i] = 0;
        if (p.step) {
            for (int i = threadIdx.x; i < p.batch; i += blockDim.x) {
                int flag;
                const int e = encode_len(p, __ldcg(p.lens_in + i), flag);
                if (e & LEN_ROOM) p.lens_out[i] = e & LEN_MASK;
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Tokens per (unit, chunk) work item of the streaming kernel.  A unit has floor(max_len / L) chunks of L
// tokens, the last of which takes the remainder too (an item of a few tokens would cost as much set-up as a
// long one).  Items are dealt round-robin to the CTAs (one per SM).  The estimate of a CTA's load, in tokens:
// its number of items times the longest item plus a fixed cost for switching items (preparation, partials,
// a pipeline bubble), taking every sequence at the host's bound max_len.  Small chunks balance the CTAs, large
// ones keep the partials (consumer warps x group x (D+2) floats per item) and the merge small; the planner
// keeps the partials per unit within MERGE_MAX_CHUNKS.
constexpr double ITEM_COST = 2048.0;      // measured: an extra item costs a CTA about 5 us, the time of 2,000 tokens
static int choose_chunk(int64_t units, int64_t max_len, int64_t ctas, int stage_tokens, int sets, double* cost_out) {
    int best = 0;
    double best_cost = 1e300;
    for (int64_t L = stage_tokens; L <= (int64_t)1 << 30; L *= 2) {
        const int64_t nch = std::max<int64_t>(1, max_len / L);
        if (nch * sets <= MERGE_MAX_CHUNKS) {
            const int64_t longest = max_len - (nch - 1) * L;
            const double cost = (double)((units * nch + ctas - 1) / ctas) * ((double)longest + ITEM_COST);
            if (cost < best_cost) { best_cost = cost; best = (int)L; }
        }
        if (L >= max_len && best) break;
    }
    *cost_out = best_cost;
    return best;
}

static DecodeWorkspace plan_workspace(int batch, int q_heads, int kv_heads, int dim, int64_t max_len) {
    DecodeWorkspace w{};
    const int64_t units = (int64_t)batch * kv_heads;
    const int group = q_heads / kv_heads;
    const int sets = dim == 64 ? 16 : 8;
    double chunk_cost = 0.0;
    w.chunk = choose_chunk(units, std::max<int64_t>(max_len, 1), sm_count(), sets * 32, sets, &chunk_cost);
    w.nchunks = (int)std::max<int64_t>(1, max_len / w.chunk);
    // The flat partition needs the lengths in shared memory (batch <= 256) and tile counts that fit an int.
    const int64_t max_tiles = units * ((std::max<int64_t>(max_len, 1) + TILE - 1) / TILE);
    // It streams the same number of tokens on every CTA but costs a CTA one more item and a fixed 4,600 tokens'
    // worth of set-up and merging (measured at two shapes): it is taken where the chunked deal leaves CTAs idle
    // for longer than that -- several units per CTA and a number of units that the CTAs do not divide.
    const double per_cta = (double)units / sm_count();
    const double flat_cost = per_cta * (double)std::max<int64_t>(max_len, 1) + (per_cta + 1.0) * ITEM_COST + 4608.0;
    w.flat = batch <= 256 && max_tiles + sm_count() < 0x7fffffff && flat_cost < 0.98 * chunk_cost;
    size_t off = 0;
    w.off_status = off; off = align_up(off + 256, 256);                    // status word, exit counter
    w.off_cnt = off;    off = align_up(off + (size_t)units * 4, 256);      // arrival counter per unit
    // partial slots: one per (unit, chunk), or one per (unit, CTA that streams a piece of it): slot = CTA + unit
    const size_t slots = w.flat ? (size_t)units + sm_count() : (size_t)units * w.nchunks;
    const size_t parts = slots * sets * group;
    w.off_m = off;   off = align_up(off + parts * 4, 256);
    w.off_l = off;   off = align_up(off + parts * 4, 256);
    w.off_acc = off; off = align_up(off + parts * dim * 4, 256);
    w.total = off;
    return w;
}

template <int D, int KB, int VB, bool PAGED, bool FLAT>
static int launch_fused(const DecodeParams& p, cudaStream_t st) {
    using C = DecodeCfg<D, KB, VB>;
    auto kern = decode_fused_kernel<D, KB, VB, PAGED, FLAT>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::DYN));
    const int64_t items = p.flat ? (int64_t)p.batch * p.kv_heads * ((p.max_len + TILE - 1) / TILE)
                                 : (int64_t)p.batch * p.kv_heads * p.nchunks;
    if (items + sm_count() >= 0x7fffffff)
        return fail(TQB_ERR_UNSUPPORTED, "decode_attention: too many (sequence, head, chunk) work items");
    const int grid = (int)std::min<int64_t>(sm_count(), std::max<int64_t>(items, 1));
    // programmatic dependent launch: the tables are built while the previous kernel of the stream drains
    TQB_CUDA(launch_pdl(1, kern, dim3(grid), dim3(C::THREADS), C::DYN, st, p));
    return check_launch("decode_fused");
}

template <int D, bool PAGED>
static int dispatch_bits(int kbits, int vbits, const DecodeParams& p, cudaStream_t st) {
#define TQB_CASE(kb, vb)                                                                               \
    if (kbits == kb && vbits == vb)                                                                    \
        return p.flat ? launch_fused<D, kb, vb, PAGED, true>(p, st) : launch_fused<D, kb, vb, PAGED, false>(p, st);
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
    if (max_len < 0 || max_len > tqb::MAX_LEN_LIMIT) return 0;
    return tqb::plan_workspace(batch, q_heads, kv_heads, dim, max_len).total;
}

namespace tqb {

// Shared by tqb_decode_attention (key == nullptr) and tqb_decode_step (key, value: the new token of every
// unit; lens_mut: the caller's sequence lengths, advanced by one at the end of the call).
static int decode_common(const void* query, int q_dtype, const void* key, const void* value, int64_t kv_stride,
                         const float* bnd_k, const float* bnd_v, int32_t* lens_mut,
                         int batch, int q_heads, int kv_heads, int dim, const uint8_t* store, int64_t max_seq,
                         const int32_t* seq_lens, int64_t max_len, const int32_t* block_tables,
                         int max_blocks, int block_size, const float* rot_k, const float* cent_k,
                         int kbits, const float* rot_v, const float* cent_v, int vbits, float scale,
                         void* workspace, size_t workspace_bytes, void* out, int out_dtype, void* stream) {
    using namespace tqb;
    TQB_REQUIRE(batch >= 0 && q_heads > 0 && kv_heads > 0, "decode_attention: bad head counts");
    TQB_REQUIRE(q_heads % kv_heads == 0, "decode_attention: q_heads (%d) must be a multiple of kv_heads (%d)",
                q_heads, kv_heads);
    const int group = q_heads / kv_heads;
    if (dim != 64 && dim != 128)
        return fail(TQB_ERR_UNSUPPORTED, "decode_attention: head_dim must be 64 or 128, got %d", dim);
    if (group > 8) return fail(TQB_ERR_UNSUPPORTED, "decode_attention: at most 8 query heads per KV head, got %d", group);
    // everything is validated before the first launch: a refused call has no side effects
    if (kbits < 2 || kbits > 4 || vbits < 2 || vbits > 4)
        return fail(TQB_ERR_UNSUPPORTED, "decode_attention: key/value bits must be 2..4, got %d/%d", kbits, vbits);
    if (q_dtype != TQB_F32 && q_dtype != TQB_F16 && q_dtype != TQB_BF16)
        return fail(TQB_ERR_INVALID, "decode_attention: unknown query dtype %d", q_dtype);
    if (out_dtype != TQB_F32 && out_dtype != TQB_F16 && out_dtype != TQB_BF16)
        return fail(TQB_ERR_INVALID, "decode_attention: unknown output dtype %d", out_dtype);
    TQB_REQUIRE(max_len >= 0, "decode_attention: negative max_len");
    if (max_len > MAX_LEN_LIMIT)
        return fail(TQB_ERR_UNSUPPORTED, "decode_attention: max_len %lld exceeds the limit of 2^30 tokens", (long long)max_len);
    if (batch == 0) return TQB_OK;
    TQB_REQUIRE(query && store && seq_lens && rot_k && cent_k && rot_v &&
                cent_v && workspace && out, "decode_attention: null pointer");
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
    p.store = const_cast<uint8_t*>(store);
    p.lens_in = seq_lens; p.lens_out = lens_mut; p.block_tables = block_tables;
    p.max_seq = paged ? (int64_t)max_blocks * block_size : max_seq; p.max_len = max_len;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = group;
    p.max_blocks = max_blocks; p.block_size = block_size; p.chunk = w.chunk; p.nchunks = w.nchunks; p.flat = w.flat;
    p.step = key != nullptr ? 1 : 0;
    p.query = query; p.key = key; p.value = value; p.in_dtype = q_dtype; p.kv_stride = kv_stride;
    p.rot_k = rot_k; p.rot_v = rot_v; p.bnd_k = bnd_k; p.bnd_v = bnd_v; p.cent_k = cent_k; p.cent_v = cent_v;
    p.scale = scale; p.out = out; p.out_dtype = out_dtype;
    p.status = reinterpret_cast<int*>(ws + w.off_status);
    p.done = p.status + 1;
    p.unit_cnt = reinterpret_cast<int*>(ws + w.off_cnt);
    p.part_m = reinterpret_cast<float*>(ws + w.off_m);
    p.part_l = reinterpret_cast<float*>(ws + w.off_l);
    p.part_acc = reinterpret_cast<float*>(ws + w.off_acc);
    cudaStream_t st = (cudaStream_t)stream;
    if (dim == 64) return paged ? dispatch_bits<64, true>(kbits, vbits, p, st) : dispatch_bits<64, false>(kbits, vbits, p, st);
    return paged ? dispatch_bits<128, true>(kbits, vbits, p, st) : dispatch_bits<128, false>(kbits, vbits, p, st);
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
