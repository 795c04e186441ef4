// pipe.cuh -- device helpers shared by the streaming kernels (decode attention, record scan):
// mbarrier and TMA bulk-copy wrappers with bounded waits, shared-memory loads on 32-bit shared
// addresses, mma.sync, and the lookup-table addressing of packed code fields.
#pragma once
#include "common.cuh"

namespace tqb {

// One bounded mbarrier wait gives up after this much wall-clock time (a poll may itself block for a
// hardware-defined while, so the bound is kept in time, not in polls).
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
__device__ __forceinline__ unsigned long long wall_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

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
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = wall_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (wall_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
}
// try_wait that lets the hardware keep the thread suspended for up to `ns` nanoseconds (a hint; the thread
// resumes as soon as the phase completes).
__device__ __forceinline__ bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait for kernels with many wait sites and many waiting warps: the polling loop is a function of its
// own (one copy per kernel image instead of one per wait site, so the hot loops stay small in the instruction
// cache) and each poll may sleep in the barrier unit, so that waiting warps leave the issue slots to the others.
static __device__ __noinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = wall_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 8; i++)
            if (mbar_try_wait_for(bar, parity, 20000u)) return true;
        if (wall_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ bool mbar_wait_compact(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_poll(bar, parity);
}
// TMA bulk copy global -> this CTA's shared memory, completion counted on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm(
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

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Loads from the pipeline stages use explicit shared-space instructions on 32-bit shared addresses (the
// stage lives wherever the carve-up put it, so the compiler could not prove the address space itself).
// They are volatile so that they stay behind the mbarrier wait that makes the stage readable.
__device__ __forceinline__ uint32_t lds32v(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float ldsf(uint32_t addr) { return __uint_as_float(lds32v(addr)); }

// A lane's chunk of NB bytes -> 32-bit registers, with the widest loads the chunk's alignment allows.
template <int NB>
__device__ __forceinline__ void load_chunk(uint32_t addr, uint32_t (&w)[NB / 4]) {
    if (NB % 16 == 0) {
#pragma unroll
        for (int i = 0; i < NB / 16; i++)
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[4 * i]), "=r"(w[4 * i + 1]), "=r"(w[4 * i + 2]), "=r"(w[4 * i + 3]) : "r"(addr + 16 * i));
    } else if (NB % 8 == 0) {
#pragma unroll
        for (int i = 0; i < NB / 8; i++)
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w[2 * i]), "=r"(w[2 * i + 1]) : "r"(addr + 8 * i));
    } else {
#pragma unroll
        for (int i = 0; i < NB / 4; i++) w[i] = lds32v(addr + 4 * i);
    }
}

// A lane's KEY chunk (tiled_layout.cuh): one piece, or two 16-byte planes when the chunk has 32 bytes.
template <int KL>
__device__ __forceinline__ void load_key_chunk(uint32_t rec, int lane, uint32_t (&w)[KL / 4]) {
    if (KL == 32) {
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(rec + lane * 16));
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w[KL / 4 - 4]), "=r"(w[KL / 4 - 3]), "=r"(w[KL / 4 - 2]), "=r"(w[KL / 4 - 1])
                     : "r"(rec + 512 + lane * 16));
    } else {
        load_chunk<KL>(rec + lane * KL, w);
    }
}

// (field value) << SHIFT taken straight out of the chunk registers; `bit` and `bits` are compile-time
// constants after unrolling: one shift and one mask (a funnel shift when the field straddles registers).
template <int NW, int SHIFT>
__device__ __forceinline__ uint32_t lut_offset(const uint32_t (&w)[NW], int bit, int bits) {
    const int i = bit >> 5, s = bit & 31;
    uint32_t v;
    if (s + bits <= 32) v = (s >= SHIFT) ? (w[i] >> (s - SHIFT)) : (w[i] << (SHIFT - s));
    else v = __funnelshift_r(w[i], w[(i + 1) < NW ? (i + 1) : i], s) << SHIFT;
    return v & (((1u << bits) - 1u) << SHIFT);
}

// Shared address of the table entry selected by the field at `bit` of chunk registers w.
//   BYTE table: tab = (table base, 64 KB aligned) | lane offset  -> one byte permute
//   otherwise:  tab = table base + lane offset                   -> shift, mask, add
template <bool BYTE, int NW>
__device__ __forceinline__ uint32_t entry_addr(const uint32_t (&w)[NW], int bit, int bits, uint32_t tab) {
    if (BYTE) return __byte_perm(w[bit >> 5], tab, 0x7604u | (((bit >> 3) & 3) << 4));
    return lut_offset<NW, 7>(w, bit, bits) + tab;
}

// Programmatic dependent launch: the three kernels of a call are launched so that each may be set up
// while its predecessor still runs.  A kernel lets its successor launch early (pdl_trigger at its start) and
// waits (pdl_wait) for the complete predecessor -- all its memory writes included -- before it touches
// anything a predecessor writes or reads.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with (enable != 0) or without the programmatic-serialization attribute.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(int enable, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = enable ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace tqb
