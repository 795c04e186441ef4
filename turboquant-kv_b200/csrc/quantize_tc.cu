// quantize_tc.cu -- Algorithm 1 quantisation (MSE mode) on the 5th-generation tensor cores.
//
//   norm -> rotation y = R x (tcgen05.mma, accumulators in tensor memory) -> y / ||x|| -> Lloyd-Max code
//   selection -> bit-plane pack (or the tiled KV-store layout), one pass over the input.
//
// Arithmetic contract (upstream turboquant_kv/reference.py:293-317): codes are those of the float32
// computation; a code may differ only where the rotated coordinate is an exact tie with a decision
// boundary.  Tensor cores multiply bf16, so both operands are split into bf16 terms whose sum is the
// float32 value (bf16 input: 1 term, fp16: 2, fp32: 3; the rotation: 3) and the products that matter are
// accumulated in float32 in tensor memory:
//      y = sum x_a R_b   over the term pairs with a + b <= 2 (counted from 0): every product whose weight
//      is above 2^-24 of the leading one -- 3, 5 or 6 MMAs per 16 elements of K
// Every product of two bf16 numbers is exact in float32; what is left is the accumulator's rounding (toward
// zero, after every MMA, by up to 2^-23 of its magnitude at that point).  The low-order products go first,
// while the accumulator is small, the leading product x_0 R_0 takes the last K/16 steps: the result is then
// within about 5e-8 * ||x|| of the FMA chain (measured: no code differs from the FFMA kernel's over 8e8
// coordinates with a guard half as wide as the one below, a handful with a sixth of it).  A GUARD BAND takes care of
// it: a coordinate closer to a decision boundary than guard(y) = GUARD_ABS + GUARD_REL * |y| is computed again
// with the float32 FMA chain of quantize.cu (same norm, same unit vector, same order of operations; about one
// coordinate in a thousand), and its code replaces the tensor-core one.  The result therefore carries exactly
// the codes of the FFMA kernel.
//
// One persistent CTA per SM, 128-row tiles, warp roles:
//   warp 0      producer: streams the tile's raw rows into a shared-memory staging ring with TMA bulk
//               copies (cp.async.bulk + mbarrier), 16 or 32 rows per stage
//   warp 1      issues the MMAs (one elected lane): tcgen05.mma kind::f16, M = 128, N = dim, K = 16 per
//               instruction, A and B from shared memory (K-major, 128-byte swizzle), D in tensor memory,
//               two accumulator buffers; tcgen05.commit signals "operands free" and "accumulator full"
//   warps 4-11  converters: staging -> norm, bf16 terms of the rows in the UMMA operand layout (two such
//               buffers where shared memory has room, so that conversion overlaps the previous tile's MMAs)
//   warps 12-19 epilogue: tcgen05.ld of their 32 accumulator rows (thread = half a row, eight columns per
//               load, the next load in flight), scaling, code selection through a 256-cell table with the
//               guard test, exact recomputation of the guarded coordinates pooled per warp, packing, stores
// The rotation's bf16 terms are built once per CTA.  Hot loops are rolled and the slow paths (polling, exact
// recomputation) are functions of their own: four roles share an SM's instruction cache.  Every wait is
// bounded in time; a warp that gives up raises the error flag word and the CTA drains and frees its tensor
// memory.
#include <type_traits>
#include "common.cuh"
#include "pipe.cuh"
#include "tiled_layout.cuh"

namespace tqb {

constexpr int TC_TILE = 128;            // rows per tile = TMEM lanes of the accumulator
constexpr int TC_CELLS = 256;           // cells of the code-selection table
#ifndef TQB_GUARD_SCALE
#define TQB_GUARD_SCALE 1.0f
#endif
constexpr float GUARD_ABS = 1.2e-7f * TQB_GUARD_SCALE;      // guard band around a decision boundary, in units of ||x|| ...
constexpr float GUARD_REL = 1.8e-6f * TQB_GUARD_SCALE;      // ... plus this fraction of |y|

struct TcArgs {
    const void* x; int64_t n, x_stride;      // rows, elements between rows
    const float* rot; const float* bnd;      // (dim, dim); 2^bits - 1 boundaries
    int bits;
    uint8_t* packed; float* norms;           // upstream rows (tiled == 0)
    RowMap map;
    int tiled, kb, vb;                       // 1 / 2: key / value section of the tiled KV store
    int heads;                               // tiled: units interleaved in the row order (row = token * heads + unit)
    int* error;                              // device word: set non-zero when a bounded wait expired
};

// ---- tcgen05 / TMEM wrappers ------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, float32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread i of the warp receives lane (base + i), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 lanes x 8 columns.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 8 columns, not waited for: the registers hold the values only after tmem_wait8 on them.
__device__ __forceinline__ void tmem_ld8_async(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(taddr) : "memory");
}
// Waits for the thread's tensor-memory loads; naming the registers keeps their uses behind the wait.
__device__ __forceinline__ void tmem_wait8(uint32_t (&v)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])
                 :: "memory");
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
// Four consecutive input elements as float4.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __half* p) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&w.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                       __uint_as_float(w.y & 0xffff0000u));
}

// Shared-memory operand descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart, groups of 8 rows
// 1024 bytes apart (the tile starts on a 1024-byte boundary).  Advancing by one MMA (16 bf16 = 32 bytes along
// K) adds 2 to the start-address field.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                              // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}
// Byte offset of element (row, k) inside a [rows][64 bf16] K-major block with 128-byte swizzle.
__device__ __forceinline__ uint32_t sw128_offset(int row, int k) {
    return (uint32_t)(row * 128 + ((((k >> 3) ^ row) & 7) << 4) + ((k & 7) << 1));
}

// The leading 8 significant bits of v as a bf16 (truncation): v - bf16_value(bf16_trunc(v)) is exact, so three
// such terms carry all 24 bits of a float32, with plain integer and add instructions.
__device__ __forceinline__ uint16_t bf16_trunc(float v) { return (uint16_t)(__float_as_uint(v) >> 16); }
__device__ __forceinline__ float bf16_value(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// The float32 chain of quantize.cu for one coordinate: unit_k = x_k / den, y = fma chain over k ascending,
// code = number of boundaries below y.  Called for the few coordinates inside the guard band only, so it is
// kept out of line (and out of the instruction cache of the main loops).
template <typename T, int D, int BITS>
static __device__ __noinline__ uint32_t exact_code(const T* xr, const float* rrow_f, float den, const float* bnd) {
    const float4* rrow = reinterpret_cast<const float4*>(rrow_f);
    float acc = 0.0f;
#pragma unroll 1
    for (int k8 = 0; k8 < D / 4; k8 += 8) {
        float4 rr[8], xv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { rr[i] = __ldg(rrow + k8 + i); xv[i] = load4(xr + 4 * (k8 + i)); }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            acc = fmaf(xv[i].x / den, rr[i].x, acc);
            acc = fmaf(xv[i].y / den, rr[i].y, acc);
            acc = fmaf(xv[i].z / den, rr[i].z, acc);
            acc = fmaf(xv[i].w / den, rr[i].w, acc);
        }
    }
    uint32_t c = 0;
#pragma unroll
    for (int sft = 1 << (BITS - 1); sft > 0; sft >>= 1)
        if (bnd[c + sft - 1] < acc) c += sft;
    return c;
}

// ---- whole records of the tiled store, assembled from a tile's code bytes -----------------------------
// A 128-row tile whose rows are 16 consecutive, aligned token slots of each of 8 units (one unit after the
// other, or `H` units interleaved row by row) holds exactly 8 records of the tiled layout.  Record w of the
// tile is then built by one warp: lane (g, t) gathers the codes of its chunk from the tile's code bytes in
// shared memory (cb: [128 rows][stride], one byte per code) and writes the chunk with wide stores, 512 or
// more contiguous bytes per warp instruction, instead of one bit field at a time.
__device__ __forceinline__ int tile_row(int w, int tok, int H) { return ((w / H) * 16 + tok) * H + (w % H); }

template <int NW>
__device__ __forceinline__ void put_bits(uint32_t (&W)[NW], int bit, int nbits, uint32_t v) {
    W[bit >> 5] |= v << (bit & 31);
    if ((bit & 31) + nbits > 32) W[(bit >> 5) + 1 < NW ? (bit >> 5) + 1 : NW - 1] |= v >> (32 - (bit & 31));
}
template <int NW>
__device__ __forceinline__ void store_chunk(uint8_t* dst, const uint32_t (&W)[NW]) {
    if (NW % 4 == 0) {
#pragma unroll
        for (int i = 0; i < NW / 4; i++) reinterpret_cast<uint4*>(dst)[i] = make_uint4(W[4 * i], W[4 * i + 1], W[4 * i + 2], W[4 * i + 3]);
    } else if (NW % 2 == 0) {
#pragma unroll
        for (int i = 0; i < NW / 2; i++) reinterpret_cast<uint2*>(dst)[i] = make_uint2(W[2 * i], W[2 * i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < NW; i++) reinterpret_cast<uint32_t*>(dst)[i] = W[i];
    }
}
// Key section (tl_key_slot): the lane's chunk = token g's fields, then token g+8's; field e = codes of the
// dims 8e + 2t and 8e + 2t + 1.
template <int D, int KB>
__device__ __forceinline__ void assemble_key_chunk(const uint8_t* cb, int stride, int w, int H, int lane, uint8_t* rec) {
    constexpr int KL = D * KB / 16, NW = KL / 4;
    const int g = lane >> 2, t = lane & 3;
    uint32_t W[NW];
#pragma unroll
    for (int i = 0; i < NW; i++) W[i] = 0;
#pragma unroll
    for (int second = 0; second < 2; second++) {
        const uint8_t* row = cb + tile_row(w, g + 8 * second, H) * stride + 2 * t;
#pragma unroll
        for (int e = 0; e < D / 8; e++) {
            const uint32_t x = *reinterpret_cast<const uint16_t*>(row + 8 * e);
            put_bits<NW>(W, second * KL * 4 + e * 2 * KB, 2 * KB, (x & 0xffu) | ((x >> 8) << KB));
        }
    }
    if (KL == 32) {              // two planes of 16-byte pieces (tl_key_piece_offset)
        reinterpret_cast<uint4*>(rec)[lane] = make_uint4(W[0], W[1], W[2 % NW], W[3 % NW]);
        reinterpret_cast<uint4*>(rec + 512)[lane] = make_uint4(W[4 % NW], W[5 % NW], W[6 % NW], W[7 % NW]);
    } else {
        store_chunk<NW>(rec + lane * KL, W);
    }
}
// Value section (tl_val_slot): the lane's chunk holds tokens {2t, 2t+1, 2t+8, 2t+9} x dims {16 mt + g, + 8}.
template <int D, int VB>
__device__ __forceinline__ void assemble_val_chunk(const uint8_t* cb, int stride, int w, int H, int lane, uint8_t* vsec) {
    constexpr int VL = D * VB / 16, NW = VL / 4;
    const int g = lane >> 2, t = lane & 3;
    uint32_t W[NW];
#pragma unroll
    for (int i = 0; i < NW; i++) W[i] = 0;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const uint8_t* ra = cb + tile_row(w, 2 * t + 8 * half, H) * stride + g;
        const uint8_t* rb = cb + tile_row(w, 2 * t + 8 * half + 1, H) * stride + g;
#pragma unroll
        for (int mt = 0; mt < D / 16; mt++) {
            if (VB == 2) {
                const uint32_t v = ra[16 * mt] | (rb[16 * mt] << 2) | (ra[16 * mt + 8] << 4) | (rb[16 * mt + 8] << 6);
                put_bits<NW>(W, (2 * mt + half) * 8, 8, v);
            } else {
#pragma unroll
                for (int sft = 0; sft < 2; sft++)
                    put_bits<NW>(W, (2 * (2 * mt + half) + sft) * 2 * VB, 2 * VB, ra[16 * mt + 8 * sft] | ((uint32_t)rb[16 * mt + 8 * sft] << VB));
            }
        }
    }
    store_chunk<NW>(vsec + lane * VL, W);
}

// ---- configuration ------------------------------------------------------------------------------------
template <typename T> struct TcTerms;                         // bf16 terms that add up to a value of type T
template <> struct TcTerms<__nv_bfloat16> { static constexpr int NA = 1; };
template <> struct TcTerms<__half> { static constexpr int NA = 2; };
template <> struct TcTerms<float> { static constexpr int NA = 3; };

template <typename T, int D, int ABUF_>
struct TcLayout {
    static constexpr int NA = TcTerms<T>::NA, NB = 3, ABUF = ABUF_;
    static constexpr int KBLK = D / 64;                       // 64-element (128-byte) blocks along K
    static constexpr int A_TERM = TC_TILE * D * 2, B_TERM = D * D * 2;
    static constexpr int A_BUF = NA * A_TERM;                                   // one tile's terms
    static constexpr int CHUNK = (NA == 3 && D == 128) ? 16 : 32;               // rows per staging stage
    static constexpr int STAGE = CHUNK * D * (int)sizeof(T);
    static constexpr int NSTAGE = (NA == 3 && D == 128) ? 3 : 4;
    static constexpr int OFF_B = 0, OFF_A = OFF_B + NB * B_TERM, OFF_STAGE = OFF_A + ABUF * A_BUF;
    static constexpr int OFF_NORM = OFF_STAGE + NSTAGE * STAGE;                 // [2][128] float
    static constexpr int OFF_BND = OFF_NORM + 2 * TC_TILE * 4;                  // 16 float
    static constexpr int OFF_CELLS = OFF_BND + 64;                              // TC_CELLS x {boundary, its index}
    static constexpr int OFF_BAR = OFF_CELLS + TC_CELLS * 8;                    // mbarriers
    static constexpr int NBAR = 2 * NSTAGE + 2 * ABUF + 4 + 1;                  // stage full/empty, a_ready/a_free, acc full/free x2, spare
    static constexpr int OFF_LIST = (OFF_BAR + NBAR * 8 + 8 + 15) / 16 * 16;    // [NEPI][32] guarded coordinates of a warp
    static constexpr int OFF_SLOTS = OFF_LIST + 8 * 32 * 4;                     // tiled output: the rows' slots (int64)
    static constexpr int OFF_CODES = OFF_SLOTS + TC_TILE * 8;                   // tiled output: [128 rows][D + 8]: code bytes, norm
    static constexpr int CODE_STRIDE = D + 8;                                   // padded: the 8-byte stores of 16 rows hit 16 bank pairs
    static constexpr int CODES = TC_TILE * CODE_STRIDE;
    static constexpr int TOTAL_ROWS = OFF_CODES + 1024;                         // + slack for the 1024-byte alignment
    static constexpr int TOTAL_TILED = OFF_CODES + CODES + 1024;
    static constexpr int TMEM_COLS = 2 * D;                                     // two accumulator buffers (power of two >= 32)
    static constexpr int CONV_WARP0 = 4, NCONV = 8, EPI_WARP0 = 12, NEPI = 8;    // EPI_WARP0 % 4 == 0 (TMEM lane quarters)
    static constexpr int THREADS = (EPI_WARP0 + NEPI) * 32;
};
// Two buffers for the tile's bf16 terms where shared memory has room for them (every case but fp16 / fp32
// rows of 128): the conversion of the next tile then overlaps the MMAs of this one.
template <typename T, int D>
struct TcCfg : TcLayout<T, D, (TcLayout<T, D, 2>::TOTAL_TILED <= 227 * 1024 ? 2 : 1)> {};

template <typename T, int D, int BITS>
__global__ void __launch_bounds__(TcCfg<T, D>::THREADS, 1) quantize_tc_kernel(const TcArgs a) {
    using C = TcCfg<T, D>;
    constexpr int NA = C::NA, NB = C::NB, KBLK = C::KBLK, NSTAGE = C::NSTAGE, TC_CHUNK = C::CHUNK, ABUF = C::ABUF;
    constexpr int NQ = D / 32;
    extern __shared__ uint8_t smem_unaligned[];
    const uint32_t raw = smem_u32(smem_unaligned);
    const uint32_t base = (raw + 1023u) & ~1023u;                    // operand tiles need 1024-byte alignment
    uint8_t* const sm = smem_unaligned + (base - raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t bar0 = base + C::OFF_BAR;
    auto stage_full = [&](int s) { return bar0 + 8 * s; };
    auto stage_empty = [&](int s) { return bar0 + 8 * (NSTAGE + s); };
    auto a_ready = [&](int b) { return bar0 + 8 * (2 * NSTAGE + b); };
    auto a_free = [&](int b) { return bar0 + 8 * (2 * NSTAGE + ABUF + b); };
    auto acc_full = [&](int b) { return bar0 + 8 * (2 * NSTAGE + 2 * ABUF + b); };
    auto acc_free = [&](int b) { return bar0 + 8 * (2 * NSTAGE + 2 * ABUF + 2 + b); };
    float* const norm_s = reinterpret_cast<float*>(sm + C::OFF_NORM);
    float* const bnd_s = reinterpret_cast<float*>(sm + C::OFF_BND);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(sm + C::OFF_BAR + C::NBAR * 8);

    const int64_t ntiles = (a.n + TC_TILE - 1) / TC_TILE;
    const T* const x = reinterpret_cast<const T*>(a.x);

    // ---- set-up: barriers, boundaries, tensor memory, the rotation's bf16 terms ----
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) { mbar_init(stage_full(s), 1); mbar_init(stage_empty(s), C::NCONV); }
        for (int b = 0; b < ABUF; b++) { mbar_init(a_ready(b), C::NCONV); mbar_init(a_free(b), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(acc_full(b), 1); mbar_init(acc_free(b), C::NEPI); }
    }
    if (threadIdx.x < 16) bnd_s[threadIdx.x] = threadIdx.x < (1 << BITS) - 1 ? a.bnd[threadIdx.x] : __int_as_float(0x7f800000);
    // Code-selection table: the range of the boundaries is cut into TC_CELLS equal cells (the outer two open
    // ended); a cell knows the boundary nearest to its centre and that boundary's index.  While cells are
    // narrower than 2/5 of the smallest gap between boundaries, no other boundary lies between a point of the
    // cell and that boundary, and none is nearer to the point by more than the cell's width allows: code(y) =
    // index + (boundary < y), and |y - boundary| decides the guard.  cell_inv == 0 says that the boundaries are
    // too dense for that (never the case for Lloyd-Max codebooks): the epilogue then takes the binary search.
    __shared__ float cell_off, cell_inv;
    {
        constexpr int NBND = (1 << BITS) - 1;
        const float b0 = a.bnd[0], b1 = a.bnd[NBND - 1];
        float gap = b1 - b0;
        for (int i = 1; i < NBND; i++) gap = fminf(gap, a.bnd[i] - a.bnd[i - 1]);
        const float w = (b1 - b0) / (float)(TC_CELLS - 2);            // one spare cell on either side
        const bool usable = w > 0.0f && 2.5f * w < gap;
        const float lo = b0 - w;
        if (threadIdx.x == 0) { cell_inv = usable ? 1.0f / w : 0.0f; cell_off = usable ? -lo / w : 0.0f; }
        if (usable && threadIdx.x < TC_CELLS) {
            const float centre = fmaf((float)threadIdx.x + 0.5f, w, lo);
            int best = 0;
            for (int i = 1; i < NBND; i++)
                if (fabsf(a.bnd[i] - centre) < fabsf(a.bnd[best] - centre)) best = i;
            reinterpret_cast<float2*>(sm + C::OFF_CELLS)[threadIdx.x] = make_float2(a.bnd[best], __int_as_float(best));
        }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    // R = R_0 + R_1 + R_2 (bf16 each), row j of R is row j of the B operand (K-major: y_j = sum_k x_k R[j][k])
    for (int e = threadIdx.x; e < D * D / 4; e += blockDim.x) {
        const int j = e / (D / 4), k = (e - j * (D / 4)) * 4;
        const float4 r = __ldg(reinterpret_cast<const float4*>(a.rot) + e);
        const float v[4] = {r.x, r.y, r.z, r.w};
        uint16_t t[NB][4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float rest = v[i];
#pragma unroll
            for (int b = 0; b < NB; b++) { t[b][i] = bf16_trunc(rest); rest -= bf16_value(t[b][i]); }
        }
        const uint32_t off = (uint32_t)(k >> 6) * (D * 128) + sw128_offset(j, k & 63);
#pragma unroll
        for (int b = 0; b < NB; b++)
            *reinterpret_cast<uint2*>(sm + C::OFF_B + b * C::B_TERM + off) =
                make_uint2(t[b][0] | ((uint32_t)t[b][1] << 16), t[b][2] | ((uint32_t)t[b][3] << 16));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes above, tensor-core reads below
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto give_up = [&]() { atomicExch(a.error, 1); };

    if (warp == 0) {
        // ================= producer: raw rows -> staging ring =================
        uint32_t n = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            for (int c = 0; c < TC_TILE / TC_CHUNK && ok; c++, n++) {
                const int s = n % NSTAGE;
                if (n >= (uint32_t)NSTAGE) {
                    if (lane == 0) ok = mbar_wait_compact(stage_empty(s), ((n / NSTAGE) - 1) & 1);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                }
                const int64_t r0 = tile * TC_TILE + c * TC_CHUNK;
                const int rows = (int)max((int64_t)0, min((int64_t)TC_CHUNK, a.n - r0));
                const uint32_t dst = base + C::OFF_STAGE + s * C::STAGE;
                constexpr uint32_t ROWB = D * sizeof(T);
                if (lane == 0) mbar_expect_tx(stage_full(s), rows * ROWB);   // (0 bytes: completes on the arrival alone)
                __syncwarp();
                if (a.x_stride == D) {                // contiguous rows: one copy
                    if (lane == 0 && rows > 0) bulk_g2s(dst, x + r0 * D, rows * ROWB, stage_full(s));
                } else if (lane < rows) {              // one copy per row
                    bulk_g2s(dst + lane * ROWB, x + (r0 + lane) * a.x_stride, ROWB, stage_full(s));
                }
            }
        }
        if (!ok && lane == 0) give_up();
    } else if (warp == 1) {
        // ================= MMA issuer =================
        constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(TC_TILE >> 4) << 24);
        bool ok = true;
        uint32_t it = 0;
        for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, it++) {
            const int buf = it & 1;
            if (lane == 0) {
                ok = mbar_wait_compact(a_ready(it % ABUF), (it / ABUF) & 1);
                if (ok && it >= 2) ok = mbar_wait_compact(acc_free(buf), ((it >> 1) - 1) & 1);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) {
                tc_fence_after();
                // The accumulator is rounded toward zero after every MMA, by up to 2^-23 of its magnitude at that
                // point.  The products of the low-order terms are 2^-8 and less of the leading one: they go first,
                // while the accumulator is small, and the leading product x_0 R_0 takes the last K/16 steps.
                uint32_t first = 1;
#pragma unroll
                for (int w = 2; w >= 0; w--)               // w = ta + tb
#pragma unroll
                    for (int ta = 0; ta < NA; ta++) {
                        const int tb = w - ta;
                        if (tb < 0 || tb >= NB) continue;
#pragma unroll
                        for (int kb = 0; kb < KBLK; kb++) {
                            const uint64_t ad = umma_desc(base + C::OFF_A + (it % ABUF) * C::A_BUF + ta * C::A_TERM + kb * (TC_TILE * 128));
                            const uint64_t bd = umma_desc(base + C::OFF_B + tb * C::B_TERM + kb * (D * 128));
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                umma_bf16(tmem_base + buf * D, ad + 2 * k, bd + 2 * k, IDESC, first ? 0u : 1u);
                                first = 0;
                            }
                        }
                    }
                umma_commit(a_free(it % ABUF));    // the A terms may be overwritten
                umma_commit(acc_full(buf));        // the accumulator may be read
            }
            __syncwarp();
        }
        if (!ok && lane == 0) give_up();
    } else if (warp >= C::CONV_WARP0 && warp < C::CONV_WARP0 + C::NCONV) {
        // ================= converters: staging -> norms and bf16 terms =================
        // Lane l of a converter takes the elements 4l .. 4l+3 of a row (D = 128) or 2l, 2l+1 (D = 64); a warp
        // takes RW rows of a chunk at once, as straight-line code, so that their shuffles and square roots
        // overlap.  Rows past the end of the input convert whatever the stage holds: their accumulator rows
        // are never read back.
        constexpr int EPL = D / 32;                                   // elements per lane
        constexpr int RW = TC_CHUNK / C::NCONV;                       // rows per warp and chunk
        const int cw = warp - C::CONV_WARP0;
        const int k = lane * EPL;
        bool ok = true;
        uint32_t n = 0, it = 0;
        for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, it++) {
            // the MMAs of the tile that used this A buffer have read it; the norms of two tiles ago have been used
            if (it >= (uint32_t)ABUF) ok = mbar_wait_compact(a_free(it % ABUF), ((it / ABUF) - 1) & 1);
            if (ok && it >= 2) ok = mbar_wait_compact(acc_free(it & 1), ((it >> 1) - 1) & 1);
            for (int c = 0; c < TC_TILE / TC_CHUNK; c++, n++) {
                const int s = n % NSTAGE;
                if (ok) ok = mbar_wait_compact(stage_full(s), (n / NSTAGE) & 1);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                const uint8_t* st = sm + C::OFF_STAGE + s * C::STAGE;
                float v[RW][EPL], ss[RW];
#pragma unroll
                for (int i = 0; i < RW; i++) {
                    const int rc = cw + C::NCONV * i;                 // row in the chunk
                    if (sizeof(T) == 4) {
                        if (EPL == 4) { const float4 f = *reinterpret_cast<const float4*>(st + rc * D * 4 + lane * 16); v[i][0] = f.x; v[i][1] = f.y; v[i][EPL - 2] = f.z; v[i][EPL - 1] = f.w; }
                        else { const float2 f = *reinterpret_cast<const float2*>(st + rc * D * 4 + lane * 8); v[i][0] = f.x; v[i][1] = f.y; }
                    } else {
                        const T* src = reinterpret_cast<const T*>(st + rc * D * 2) + lane * EPL;
                        if (EPL == 4) { const float4 f = load4(src); v[i][0] = f.x; v[i][1] = f.y; v[i][EPL - 2] = f.z; v[i][EPL - 1] = f.w; }
                        else { v[i][0] = to_f32<T>(src[0]); v[i][1] = to_f32<T>(src[1]); }
                    }
                    ss[i] = 0.0f;
#pragma unroll
                    for (int e = 0; e < EPL; e++) ss[i] = fmaf(v[i][e], v[i][e], ss[i]);
                }
                // the butterfly of warp_sum, over the RW rows at once
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                    for (int i = 0; i < RW; i++) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
#pragma unroll
                for (int i = 0; i < RW; i++) {
                    const int row = c * TC_CHUNK + cw + C::NCONV * i;  // row in the tile
                    const float nrm = sqrtf(ss[i]);
                    if (lane == 0) norm_s[(it & 1) * TC_TILE + row] = nrm;
                    // bf16 terms of the raw row: v = t_0 + t_1 + t_2 exactly (as far as float32 goes)
                    uint16_t t[NA][EPL];
#pragma unroll
                    for (int e = 0; e < EPL; e++) {
                        float rest = v[i][e];
#pragma unroll
                        for (int ta = 0; ta < NA; ta++) { t[ta][e] = bf16_trunc(rest); rest -= bf16_value(t[ta][e]); }
                    }
                    const uint32_t off = (uint32_t)(k >> 6) * (TC_TILE * 128) + sw128_offset(row, k & 63);
#pragma unroll
                    for (int ta = 0; ta < NA; ta++) {
                        uint8_t* dst = sm + C::OFF_A + (it % ABUF) * C::A_BUF + ta * C::A_TERM + off;
                        if (EPL == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(t[ta][0] | ((uint32_t)t[ta][1] << 16), t[ta][EPL - 2] | ((uint32_t)t[ta][EPL - 1] << 16));
                        else *reinterpret_cast<uint32_t*>(dst) = t[ta][0] | ((uint32_t)t[ta][1] << 16);
                    }
                }
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(stage_empty(s)) : "memory");
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");          // generic writes -> tensor-core reads
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_ready(it % ABUF)) : "memory");
        }
        if (!ok && lane == 0) give_up();
    } else if (warp >= C::EPI_WARP0) {
        // ================= epilogue: thread = one half of a row =================
        // The first four warps take the first half of the columns, the other four the second; warp % 4 selects
        // the 32 accumulator rows (TMEM lanes) a warp may read.  The columns come eight at a time, the next
        // eight in flight while these are turned into codes; sixteen columns make one turn of a rolled loop that
        // stays small in the instruction cache.
        const int ew = (warp - C::EPI_WARP0) & 3, half = (warp - C::EPI_WARP0) >> 2;
        const int row = ew * 32 + lane;
        const float coff = cell_off, cinv = cell_inv;
        const uint32_t cells_addr = base + C::OFF_CELLS;
        constexpr int BPP = D / 8, HQ = NQ / 2;                       // bytes per plane; 32-column words per half row
        constexpr int TURNS = D / 32;                                 // sixteen columns of the half row a turn
        const int col0 = half * (D / 2);
        bool ok = true;
        uint32_t it = 0;
        for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, it++) {
            const int buf = it & 1;
            ok = mbar_wait_compact(acc_full(buf), (it >> 1) & 1);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            tc_fence_after();
            const int64_t r = tile * TC_TILE + row;
            const float nrm = norm_s[buf * TC_TILE + row];
            const float inv = 1.0f / fmaxf(nrm, 1e-10f);
            uint32_t plane[BITS][HQ];
#pragma unroll
            for (int pl = 0; pl < BITS; pl++)
#pragma unroll
                for (int q = 0; q < HQ; q++) plane[pl][q] = 0;
            unsigned long long gmask = 0;                             // guarded columns of the half row
            uint8_t* const cbuf = sm + C::OFF_CODES + row * C::CODE_STRIDE + col0;   // (tiled output only)
            const uint32_t trow = tmem_base + ((uint32_t)(ew * 32) << 16) + buf * D + col0;

            // eight accumulators (columns 8 g8 ..) -> codes; the byte of every bit plane in out[pl]
            auto codes8 = [&](auto cells_tag, const uint32_t (&acc)[8], int g8, uint32_t (&out)[BITS]) {
                constexpr bool CELLS = decltype(cells_tag)::value;
                uint32_t nib = 0, gm = 0;                             // dimension j in nibble 7-j
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float y = __uint_as_float(acc[j]) * inv;
                    uint32_t c = 0;
                    float dmin;
                    if (CELLS) {
                        const float tc = fminf(fmaxf(fmaf(y, cinv, coff), 0.0f), (float)(TC_CELLS - 1));
                        const float2 e = lds64f(cells_addr + (uint32_t)__float2int_rz(tc) * 8u);
                        c = (uint32_t)__float_as_int(e.y) + (e.x < y ? 1u : 0u);
                        dmin = fabsf(y - e.x);
                    } else {
                        dmin = 1e30f;
#pragma unroll
                        for (int sft = 1 << (BITS - 1); sft > 0; sft >>= 1) {
                            const float bv = bnd_s[c + sft - 1];
                            dmin = fminf(dmin, fabsf(y - bv));
                            if (bv < y) c += sft;
                        }
                    }
                    if (dmin < fmaf(GUARD_REL, fabsf(y), GUARD_ABS)) gm |= 1u << j;
                    nib |= c << (4 * (7 - j));
                }
                if (gm) gmask |= (unsigned long long)gm << (8 * g8);
                if (a.tiled) {                                        // code bytes, dimension j in byte j
                    const uint32_t wlo = ((nib >> 28) & 0xfu) | ((nib >> 16) & 0xf00u) | ((nib >> 4) & 0xf0000u) | ((nib << 8) & 0xf000000u);
                    const uint32_t whi = ((nib >> 12) & 0xfu) | (nib & 0xf00u) | ((nib << 12) & 0xf0000u) | ((nib << 24) & 0xf000000u);
                    *reinterpret_cast<uint2*>(cbuf + 8 * g8) = make_uint2(wlo, whi);
                }
                // nibbles -> one byte per bit plane, most significant bit = first dimension
#pragma unroll
                for (int pl = 0; pl < BITS; pl++) {
                    const uint32_t xb = (nib >> pl) & 0x11111111u;
                    const uint32_t pr = (xb | (xb >> 3)) & 0x03030303u;
                    out[pl] = (pr * 0x01041040u) >> 24;
                }
            };
            auto half_row = [&](auto cells_tag) {
                uint32_t a0[8], a1[8];
                tmem_ld8_async(trow, a0);
#pragma unroll 1
                for (int g = 0; g < TURNS; g++) {
                    uint32_t b0[BITS], b1[BITS];
                    tmem_ld8_async(trow + 16 * g + 8, a1);            // (a wait covers every load issued so far)
                    tmem_wait8(a0);
                    codes8(cells_tag, a0, 2 * g, b0);
                    tmem_wait8(a1);
                    if (g + 1 < TURNS) tmem_ld8_async(trow + 16 * (g + 1), a0);
                    codes8(cells_tag, a1, 2 * g + 1, b1);
                    const int sh = 16 * (g & 1);
#pragma unroll
                    for (int pl = 0; pl < BITS; pl++) {
                        const uint32_t w = (b0[pl] | (b1[pl] << 8)) << sh;
#pragma unroll
                        for (int qq = 0; qq < HQ; qq++)
                            if (qq == (g >> 1)) plane[pl][qq] |= w;
                    }
                }
            };
            if (cinv != 0.0f) half_row(std::true_type{});
            else half_row(std::false_type{});
            // the accumulator buffer may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_free(buf)) : "memory");
            // The guarded coordinates again, with the float32 chain of quantize.cu.  The warp pools them, up to
            // 32 at a time: lane i computes the i-th, then the codes go back to the lanes that own the rows.
            if (r >= a.n) gmask = 0;
            uint32_t* const list = reinterpret_cast<uint32_t*>(sm + C::OFF_LIST) + (warp - C::EPI_WARP0) * 32;
            const float den = fmaxf(nrm, 1e-10f);
            while (__any_sync(0xffffffffu, gmask != 0)) {
                int cnt = 0;
                while (cnt < 32) {
                    const bool have = gmask != 0;
                    const uint32_t bal = __ballot_sync(0xffffffffu, have);
                    if (bal == 0) break;
                    const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
                    if (have && pos < 32) {
                        list[pos] = ((uint32_t)lane << 8) | (uint32_t)(__ffsll((long long)gmask) - 1);
                        gmask &= gmask - 1;
                    }
                    cnt = min(32, cnt + __popc(bal));
                }
                __syncwarp();
                const uint32_t mine = lane < cnt ? list[lane] : 0u;
                const int owner = (int)(mine >> 8), jr_mine = (int)(mine & 255u);       // column relative to col0
                const float den_o = __shfl_sync(0xffffffffu, den, owner);
                uint32_t c_mine = 0;
                if (lane < cnt)
                    c_mine = exact_code<T, D, BITS>(x + (tile * TC_TILE + ew * 32 + owner) * a.x_stride,
                                                    a.rot + (int64_t)(col0 + jr_mine) * D, den_o, bnd_s);
                for (int i = 0; i < cnt; i++) {
                    const uint32_t e = __shfl_sync(0xffffffffu, mine, i), c = __shfl_sync(0xffffffffu, c_mine, i);
                    if ((int)(e >> 8) != lane) continue;
                    // replace the coordinate's code: bit 7 - j%8 of byte (j%32)/8 of word j/32 of every plane
                    const int jr = (int)(e & 255u), w = jr >> 5, bit = 8 * ((jr & 31) >> 3) + 7 - (jr & 7);
#pragma unroll
                    for (int pl = 0; pl < BITS; pl++)
#pragma unroll
                        for (int q = 0; q < HQ; q++)
                            if (q == w) plane[pl][q] = (plane[pl][q] & ~(1u << bit)) | (((c >> pl) & 1u) << bit);
                    if (a.tiled) cbuf[jr] = (uint8_t)c;
                }
                __syncwarp();
            }
            if (r < a.n && !a.tiled) {
                const int64_t orow = a.map(r);
                if (orow >= 0) {
                    uint8_t* dst = a.packed + orow * (BITS * BPP) + half * (BPP / 2);
#pragma unroll
                    for (int pl = 0; pl < BITS; pl++) {
                        if (HQ == 2) *reinterpret_cast<uint2*>(dst + pl * BPP) = make_uint2(plane[pl][0], plane[pl][HQ - 1]);
                        else *reinterpret_cast<uint32_t*>(dst + pl * BPP) = plane[pl][0];
                    }
                    if (half == 0) a.norms[orow] = nrm;
                }
            }
            if (a.tiled) {
                // The tile's code bytes are in shared memory.  Warp w of the epilogue takes the w-th group of
                // sixteen rows that may form a record: written whole when their slots are sixteen consecutive,
                // aligned ones, else row by row.
                uint8_t* const cb0 = sm + C::OFF_CODES;
                int64_t* const slot_s = reinterpret_cast<int64_t*>(sm + C::OFF_SLOTS);
                if (half == 0) {
                    *reinterpret_cast<float*>(cb0 + row * C::CODE_STRIDE + D) = nrm;     // (the row's padding)
                    slot_s[row] = r < a.n ? a.map(r) : -1;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(C::NEPI * 32) : "memory");
                const int H = a.heads > 0 ? a.heads : 1, w = warp - C::EPI_WARP0;
                const int myrow = tile_row(w, lane & 15, H);
                const int64_t s_mine = slot_s[myrow], s_first = __shfl_sync(0xffffffffu, s_mine, 0);
                const bool whole = __all_sync(0xffffffffu, s_first >= 0 && (s_first & 15) == 0 && s_mine == s_first + (lane & 15));
                const int ksec = tl_key_section(D, a.kb), vsec = tl_val_section(D, a.vb);
                if (whole) {
                    uint8_t* rec = a.packed + (s_first >> 4) * (int64_t)tl_record_bytes(D, a.kb, a.vb);
                    if (a.tiled == 1) assemble_key_chunk<D, BITS>(cb0, C::CODE_STRIDE, w, H, lane, rec);
                    else assemble_val_chunk<D, BITS>(cb0, C::CODE_STRIDE, w, H, lane, rec + ksec);
                    if (lane < 16)
                        *reinterpret_cast<float*>(rec + ksec + vsec + tl_norm_offset(a.vb, a.tiled - 1, lane)) =
                            *reinterpret_cast<const float*>(cb0 + myrow * C::CODE_STRIDE + D);
                } else {
                    for (int tok = 0; tok < 16; tok++) {
                        const int rw = tile_row(w, tok, H);
                        const int64_t orow = slot_s[rw];
                        if (orow < 0) continue;
                        uint32_t code[NQ];
#pragma unroll
                        for (int q = 0; q < NQ; q++) code[q] = cb0[rw * C::CODE_STRIDE + lane + 32 * q];
                        tiled_store_row<NQ>(a.packed, a.tiled, a.kb, a.vb, orow, code,
                                            *reinterpret_cast<const float*>(cb0 + rw * C::CODE_STRIDE + D), lane, D);
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(C::NEPI * 32) : "memory");          // the code bytes may be overwritten
            }
        }
        if (!ok && lane == 0) give_up();
    }

    // ---- teardown: tensor memory is released by the warp that allocated it ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// Error word of the tensor-core quantiser: one per device, in the library's device image (the quantise entry
// points take no workspace).  Only ever set, by a kernel whose bounded wait expired; tqb_quantize_status reads
// and clears it.
static __device__ int g_tc_error;

template <typename T, int D, int BITS>
static int launch_tc(TcArgs a, cudaStream_t st) {
    using C = TcCfg<T, D>;
    const int smem = a.tiled ? C::TOTAL_TILED : C::TOTAL_ROWS;
    if (smem > 227 * 1024) return TQB_ERR_UNSUPPORTED;
    auto kern = quantize_tc_kernel<T, D, BITS>;
    TQB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    int* err = nullptr;
    TQB_CUDA(cudaGetSymbolAddress((void**)&err, g_tc_error));
    a.error = err;
    const int64_t ntiles = (a.n + TC_TILE - 1) / TC_TILE;
    const int grid = (int)std::min<int64_t>(sm_count(), ntiles);
    kern<<<grid, C::THREADS, smem, st>>>(a);
    return check_launch("quantize_tc");
}

template <typename T, int D>
static int tc_dispatch_bits(const TcArgs& a, cudaStream_t st) {
    switch (a.bits) {
        case 2: return launch_tc<T, D, 2>(a, st);
        case 3: return launch_tc<T, D, 3>(a, st);
        case 4: return launch_tc<T, D, 4>(a, st);
    }
    return TQB_ERR_UNSUPPORTED;
}

// Tries the tensor-core path.  Returns TQB_ERR_UNSUPPORTED (without touching the last-error text) when the
// call's shape is outside it: the caller then takes the FFMA kernel.
int quantize_tc_try(const void* x, int dtype, int64_t n, int dim, int64_t x_stride, const float* rot, const float* bnd,
                    int bits, uint8_t* packed, float* norms, const RowMap& map, int tiled, int kb, int vb, cudaStream_t st) {
    if ((dim != 64 && dim != 128) || bits < 2 || bits > 4 || n < 4 * TC_TILE) return TQB_ERR_UNSUPPORTED;
    const size_t esz = dtype == TQB_F32 ? 4 : 2;
    // TMA bulk copies need 16-byte aligned rows; plain rows need 16-byte aligned outputs for the vector stores
    if ((uintptr_t)x % 16 || (x_stride * esz) % 16 || (uintptr_t)rot % 16) return TQB_ERR_UNSUPPORTED;
    if (!tiled && (uintptr_t)packed % 16) return TQB_ERR_UNSUPPORTED;
    if (n >= 0x7fffffff) return TQB_ERR_UNSUPPORTED;
    TcArgs a{};
    a.x = x; a.n = n; a.x_stride = x_stride; a.rot = rot; a.bnd = bnd; a.bits = bits; a.packed = packed; a.norms = norms;
    a.map = map; a.tiled = tiled; a.kb = kb; a.vb = vb;
    const int64_t units = map.slots ? map.inner : 1;       // paged appends walk the heads of a token first
    a.heads = (units == 1 || units == 2 || units == 4 || units == 8) ? (int)units : 0;
#define TQB_TC(T) (dim == 64 ? tc_dispatch_bits<T, 64>(a, st) : tc_dispatch_bits<T, 128>(a, st))
    switch (dtype) {
        case TQB_F32: return TQB_TC(float);
        case TQB_F16: return TQB_TC(__half);
        case TQB_BF16: return TQB_TC(__nv_bfloat16);
    }
#undef TQB_TC
    return TQB_ERR_UNSUPPORTED;
}

}  // namespace tqb

// Reads and clears the error word of the tensor-core quantiser on the current device (synchronises `stream`).
extern "C" int tqb_quantize_status(void* stream) {
    int* err = nullptr;
    TQB_CUDA(cudaGetSymbolAddress((void**)&err, tqb::g_tc_error));
    int host = 0;
    TQB_CUDA(cudaMemcpyAsync(&host, err, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    TQB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (host) TQB_CUDA(cudaMemsetAsync(err, 0, sizeof(int), (cudaStream_t)stream));
    return host;
}
