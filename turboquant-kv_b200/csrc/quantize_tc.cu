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
// Every product of two bf16 numbers is exact in float32, so what is left is accumulation error of the order
// of 1e-7 * ||x||.  A GUARD BAND takes care of it: a coordinate closer to a decision boundary than
// guard(y) = GUARD_ABS + GUARD_REL * |y| is computed again by the thread that owns the row with the float32
// FMA chain of quantize.cu (same norm, same unit vector, same order of operations; a few coordinates in
// ten thousand), and its code replaces the tensor-core one.  The result therefore carries exactly the codes
// of the FFMA kernel.
//
// One persistent CTA per SM, 128-row tiles, warp roles:
//   warp 0      producer: streams the tile's raw rows into a shared-memory staging ring with TMA bulk
//               copies (cp.async.bulk + mbarrier), 32 rows per stage
//   warp 1      issues the MMAs (one elected lane): tcgen05.mma kind::f16, M = 128, N = dim, K = 16 per
//               instruction, A and B from shared memory (K-major, 128-byte swizzle), D in tensor memory,
//               two accumulator buffers; tcgen05.commit signals "operands free" and "accumulator full"
//   warps 4-7   converters: staging -> norm, bf16 terms of the rows in the UMMA operand layout
//   warps 8-15  epilogue: tcgen05.ld of their 32 accumulator rows (thread = half a row), scaling, binary
//               search with guard, exact recomputation of guarded coordinates, packing, stores
// The rotation's bf16 terms are built once per CTA.  Every wait is bounded in time; a warp that gives up
// raises the error flag word and the CTA drains and frees its tensor memory.
#include "common.cuh"
#include "pipe.cuh"
#include "tiled_layout.cuh"

namespace tqb {

constexpr int TC_TILE = 128;            // rows per tile = TMEM lanes of the accumulator
constexpr int TC_CHUNK = 32;            // rows per staging stage
constexpr float GUARD_ABS = 4e-7f;      // guard band around a decision boundary, in units of ||x|| ...
constexpr float GUARD_REL = 6e-6f;      // ... plus this fraction of |y|

struct TcArgs {
    const void* x; int64_t n, x_stride;      // rows, elements between rows
    const float* rot; const float* bnd;      // (dim, dim); 2^bits - 1 boundaries
    int bits;
    uint8_t* packed; float* norms;           // upstream rows (tiled == 0)
    RowMap map;
    int tiled, kb, vb;                       // 1 / 2: key / value section of the tiled KV store
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

__device__ __forceinline__ uint16_t bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf16_value(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// ---- configuration ------------------------------------------------------------------------------------
template <typename T> struct TcTerms;                         // bf16 terms that add up to a value of type T
template <> struct TcTerms<__nv_bfloat16> { static constexpr int NA = 1; };
template <> struct TcTerms<__half> { static constexpr int NA = 2; };
template <> struct TcTerms<float> { static constexpr int NA = 3; };

template <typename T, int D>
struct TcCfg {
    static constexpr int NA = TcTerms<T>::NA, NB = 3;
    static constexpr int KBLK = D / 64;                       // 64-element (128-byte) blocks along K
    static constexpr int A_TERM = TC_TILE * D * 2, B_TERM = D * D * 2;
    static constexpr int STAGE = TC_CHUNK * D * (int)sizeof(T);
    static constexpr int NSTAGE = (NA == 3 && D == 128) ? 2 : 4;
    static constexpr int OFF_B = 0, OFF_A = OFF_B + NB * B_TERM, OFF_STAGE = OFF_A + NA * A_TERM;
    static constexpr int OFF_NORM = OFF_STAGE + NSTAGE * STAGE;                 // [2][128] float
    static constexpr int OFF_BND = OFF_NORM + 2 * TC_TILE * 4;                  // 16 float
    static constexpr int OFF_BAR = OFF_BND + 64;                                // mbarriers
    static constexpr int NBAR = 2 * NSTAGE + 2 + 4 + 1;                         // stage full/empty, a_ready/a_free, acc full/free x2, spare
    static constexpr int OFF_CODES = (OFF_BAR + NBAR * 8 + 8 + 15) / 16 * 16;   // tiled output: [128 rows][D] code bytes
    static constexpr int CODES = TC_TILE * D;
    static constexpr int TOTAL_ROWS = OFF_CODES + 1024;                         // + slack for the 1024-byte alignment
    static constexpr int TOTAL_TILED = OFF_CODES + CODES + 1024;
    static constexpr int TMEM_COLS = 2 * D;                                     // two accumulator buffers (power of two >= 32)
    static constexpr int THREADS = 16 * 32;
};

template <typename T, int D, int BITS>
__global__ void __launch_bounds__(TcCfg<T, D>::THREADS, 1) quantize_tc_kernel(const TcArgs a) {
    using C = TcCfg<T, D>;
    constexpr int NA = C::NA, NB = C::NB, KBLK = C::KBLK, NSTAGE = C::NSTAGE;
    constexpr int NQ = D / 32;
    extern __shared__ uint8_t smem_unaligned[];
    const uint32_t raw = smem_u32(smem_unaligned);
    const uint32_t base = (raw + 1023u) & ~1023u;                    // operand tiles need 1024-byte alignment
    uint8_t* const sm = smem_unaligned + (base - raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const uint32_t bar0 = base + C::OFF_BAR;
    auto stage_full = [&](int s) { return bar0 + 8 * s; };
    auto stage_empty = [&](int s) { return bar0 + 8 * (NSTAGE + s); };
    const uint32_t a_ready = bar0 + 8 * (2 * NSTAGE), a_free = a_ready + 8;
    auto acc_full = [&](int b) { return a_free + 8 + 8 * b; };
    auto acc_free = [&](int b) { return a_free + 8 + 16 + 8 * b; };
    float* const norm_s = reinterpret_cast<float*>(sm + C::OFF_NORM);
    float* const bnd_s = reinterpret_cast<float*>(sm + C::OFF_BND);
    uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(sm + C::OFF_BAR + C::NBAR * 8);

    const int64_t ntiles = (a.n + TC_TILE - 1) / TC_TILE;
    const T* const x = reinterpret_cast<const T*>(a.x);

    // ---- set-up: barriers, boundaries, tensor memory, the rotation's bf16 terms ----
    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) { mbar_init(stage_full(s), 1); mbar_init(stage_empty(s), 4); }
        mbar_init(a_ready, 4); mbar_init(a_free, 1);
        for (int b = 0; b < 2; b++) { mbar_init(acc_full(b), 1); mbar_init(acc_free(b), 8); }
    }
    if (threadIdx.x < 16) bnd_s[threadIdx.x] = threadIdx.x < (1 << BITS) - 1 ? a.bnd[threadIdx.x] : __int_as_float(0x7f800000);
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
            for (int b = 0; b < NB; b++) { t[b][i] = bf16_bits(rest); rest -= bf16_value(t[b][i]); }
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
                    if (lane == 0) ok = mbar_wait(stage_empty(s), ((n / NSTAGE) - 1) & 1);
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
                ok = mbar_wait(a_ready, it & 1);
                if (ok && it >= 2) ok = mbar_wait(acc_free(buf), ((it >> 1) - 1) & 1);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) {
                tc_fence_after();
                uint32_t first = 1;
#pragma unroll
                for (int ta = 0; ta < NA; ta++)
#pragma unroll
                    for (int tb = 0; tb < NB; tb++) {
                        if (ta + tb > 2) continue;         // weights below 2^-24 of the leading product
#pragma unroll
                        for (int kb = 0; kb < KBLK; kb++) {
                            const uint64_t ad = umma_desc(base + C::OFF_A + ta * C::A_TERM + kb * (TC_TILE * 128));
                            const uint64_t bd = umma_desc(base + C::OFF_B + tb * C::B_TERM + kb * (D * 128));
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                umma_bf16(tmem_base + buf * D, ad + 2 * k, bd + 2 * k, IDESC, first ? 0u : 1u);
                                first = 0;
                            }
                        }
                    }
                umma_commit(a_free);               // the A terms may be overwritten
                umma_commit(acc_full(buf));        // the accumulator may be read
            }
            __syncwarp();
        }
        if (!ok && lane == 0) give_up();
    } else if (warp >= 4 && warp < 8) {
        // ================= converters: staging -> norms and bf16 terms =================
        // Lane l of a converter takes the elements 4l .. 4l+3 of a row (D = 128) or 2l, 2l+1 (D = 64).
        constexpr int EPL = D / 32;                                   // elements per lane
        const int cw = warp - 4;
        bool ok = true;
        uint32_t n = 0, it = 0;
        for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, it++) {
            // the previous tile's MMAs have read the A terms; the norms of two tiles ago have been used
            if (it >= 1) ok = mbar_wait(a_free, (it - 1) & 1);
            if (ok && it >= 2) ok = mbar_wait(acc_free(it & 1), ((it >> 1) - 1) & 1);
            for (int c = 0; c < TC_TILE / TC_CHUNK; c++, n++) {
                const int s = n % NSTAGE;
                if (ok) ok = mbar_wait(stage_full(s), (n / NSTAGE) & 1);
                if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
                const uint8_t* st = sm + C::OFF_STAGE + s * C::STAGE;
                const int64_t r0 = tile * TC_TILE + c * TC_CHUNK;
                // this warp converts rows cw, cw + 4, ... of the chunk: eight rows
#pragma unroll
                for (int i = 0; i < TC_CHUNK / 4; i++) {
                    const int rc = cw + 4 * i, row = c * TC_CHUNK + rc;           // row in the chunk / in the tile
                    float v[EPL];
                    if (r0 + rc < a.n) {
                        if (sizeof(T) == 4) {
                            if (EPL == 4) { const float4 f = *reinterpret_cast<const float4*>(st + rc * D * 4 + lane * 16); v[0] = f.x; v[1] = f.y; v[EPL - 2] = f.z; v[EPL - 1] = f.w; }
                            else { const float2 f = *reinterpret_cast<const float2*>(st + rc * D * 4 + lane * 8); v[0] = f.x; v[1] = f.y; }
                        } else {
                            const T* src = reinterpret_cast<const T*>(st + rc * D * 2) + lane * EPL;
#pragma unroll
                            for (int e = 0; e < EPL; e++) v[e] = to_f32<T>(src[e]);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < EPL; e++) v[e] = 0.0f;
                    }
                    float ss = 0.0f;
#pragma unroll
                    for (int e = 0; e < EPL; e++) ss = fmaf(v[e], v[e], ss);
                    const float nrm = sqrtf(warp_sum(ss));
                    if (lane == 0) norm_s[(it & 1) * TC_TILE + row] = nrm;
                    // bf16 terms of the raw row: v = t_0 + t_1 + t_2 exactly (as far as float32 goes)
                    uint16_t t[NA][EPL];
#pragma unroll
                    for (int e = 0; e < EPL; e++) {
                        float rest = v[e];
#pragma unroll
                        for (int ta = 0; ta < NA; ta++) { t[ta][e] = bf16_bits(rest); rest -= bf16_value(t[ta][e]); }
                    }
                    const int k = lane * EPL;
                    const uint32_t off = (uint32_t)(k >> 6) * (TC_TILE * 128) + sw128_offset(row, k & 63);
#pragma unroll
                    for (int ta = 0; ta < NA; ta++) {
                        uint8_t* dst = sm + C::OFF_A + ta * C::A_TERM + off;
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
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a_ready) : "memory");
        }
        if (!ok && lane == 0) give_up();
    } else if (warp >= 8) {
        // ================= epilogue: thread = one half of a row =================
        // Warps 8-11 take the first half of the columns, warps 12-15 the second; warp % 4 selects the 32
        // accumulator rows (TMEM lanes) a warp may read.  The columns are walked eight at a time in a rolled
        // loop: eight codes make one byte of every bit plane, and the loop body stays small enough for the
        // instruction cache.
        const int ew = (warp - 8) & 3, half = (warp - 8) >> 2;
        const int row = ew * 32 + lane;
        constexpr int BPP = D / 8, HQ = NQ / 2;                       // bytes per plane; 32-column words per half row
        const int col0 = half * (D / 2);
        bool ok = true;
        uint32_t it = 0;
        for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, it++) {
            const int buf = it & 1;
            ok = mbar_wait(acc_full(buf), (it >> 1) & 1);
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
            int nguard = 0;
            uint32_t guarded = 0;                                     // up to four guarded columns (relative to col0), a byte each
            uint8_t* const cbuf = sm + C::OFF_CODES + row * D + col0;            // (tiled output only)
            const uint32_t trow = tmem_base + ((uint32_t)(ew * 32) << 16) + buf * D + col0;
#pragma unroll
            for (int q = 0; q < HQ; q++) {
#pragma unroll 1
                for (int m = 0; m < 4; m++) {
                    uint32_t acc[8];
                    tmem_ld8(trow + 32 * q + 8 * m, acc);
                    uint32_t nib = 0;                                 // dimension 8m+t in nibble 7-t
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float y = __uint_as_float(acc[j]) * inv;
                        uint32_t c = 0;
                        float dmin = 1e30f;
#pragma unroll
                        for (int sft = 1 << (BITS - 1); sft > 0; sft >>= 1) {
                            const float bv = bnd_s[c + sft - 1];
                            dmin = fminf(dmin, fabsf(y - bv));
                            if (bv < y) c += sft;
                        }
                        if (dmin < fmaf(GUARD_REL, fabsf(y), GUARD_ABS)) {
                            if (nguard < 4) guarded |= (uint32_t)(32 * q + 8 * m + j) << (8 * nguard);
                            nguard++;
                        }
                        nib |= c << (4 * (7 - j));
                        if (a.tiled) cbuf[32 * q + 8 * m + j] = (uint8_t)c;
                    }
                    // nibbles -> one byte per bit plane, most significant bit = first dimension
#pragma unroll
                    for (int pl = 0; pl < BITS; pl++) {
                        const uint32_t xb = (nib >> pl) & 0x11111111u;
                        const uint32_t pr = (xb | (xb >> 3)) & 0x03030303u;
                        plane[pl][q] |= ((pr * 0x01041040u) >> 24) << (8 * m);
                    }
                }
            }
            // the accumulator buffer may be overwritten
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_free(buf)) : "memory");
            if (r < a.n && nguard > 0) {
                // The float32 chain of quantize.cu for the guarded coordinates (all of the half row when there
                // were more than four): unit_k = x_k / max(norm, 1e-10), y_j = fma chain over k ascending.
                const float den = fmaxf(nrm, 1e-10f);
                const T* xr = x + r * a.x_stride;
                const int todo = nguard > 4 ? D / 2 : nguard;
                for (int gi = 0; gi < todo; gi++) {
                    const int jr = nguard > 4 ? gi : (int)((guarded >> (8 * gi)) & 255u);   // column relative to col0
                    const float4* rrow = reinterpret_cast<const float4*>(a.rot + (int64_t)(col0 + jr) * D);
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
                        if (bnd_s[c + sft - 1] < acc) c += sft;
                    // replace the coordinate's code: bit 7 - j%8 of byte (j%32)/8 of word j/32 of every plane
                    const int w = jr >> 5, bit = 8 * ((jr & 31) >> 3) + 7 - (jr & 7);
#pragma unroll
                    for (int pl = 0; pl < BITS; pl++)
#pragma unroll
                        for (int q = 0; q < HQ; q++)
                            if (q == w) plane[pl][q] = (plane[pl][q] & ~(1u << bit)) | (((c >> pl) & 1u) << bit);
                    if (a.tiled) cbuf[jr] = (uint8_t)c;
                }
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
                // code bytes of the quarter's 32 rows (both halves) -> the record layout, one row at a time with
                // lane = dimension; the two warps of the quarter meet on a named barrier and share the rows
                asm volatile("bar.sync %0, 64;" ::"r"(1 + ew) : "memory");
                for (int i = half * 16; i < half * 16 + 16; i++) {
                    const int64_t ri = tile * TC_TILE + ew * 32 + i;
                    const float nrm_i = __shfl_sync(0xffffffffu, nrm, i);   // (the norm buffer may already belong to a later tile)
                    if (ri >= a.n) continue;
                    const int64_t orow = a.map(ri);
                    if (orow < 0) continue;
                    uint32_t code[NQ];
#pragma unroll
                    for (int q = 0; q < NQ; q++) code[q] = sm[C::OFF_CODES + (ew * 32 + i) * D + lane + 32 * q];
                    tiled_store_row<NQ>(a.packed, a.tiled, a.kb, a.vb, orow, code, nrm_i, lane, D);
                }
                asm volatile("bar.sync %0, 64;" ::"r"(1 + ew) : "memory");   // the code bytes may be overwritten
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
