// kv_store.cu -- conversions between the tiled KV store (tiled_layout.cuh) and upstream rows.
//
// tqb_kv_export gives the upstream view (bit-plane packed codes + norms per token, the contents of
// QuantizedKVCache._key_packed / _key_norms / _val_packed / _val_norms in upstream cache.py:89-106) of
// any set of token slots; tqb_kv_import writes such rows into slots.  One warp per token; lane l
// handles dims l + 32 q; bit planes are assembled with __ballot_sync exactly as in the quantise kernel.
#include "common.cuh"
#include "tiled_layout.cuh"

namespace tqb {

struct StoreArgs {
    uint8_t* store;
    int64_t n;
    int dim, kb, vb;
    RowMap map;
    uint8_t* k_packed; float* k_norms; uint8_t* v_packed; float* v_norms;
};

__device__ __forceinline__ void st_atomic_write(uint32_t* words, int absbit, int nbits, uint32_t v) {
    const int w = absbit >> 5, s = absbit & 31;
    const uint32_t mask = (1u << nbits) - 1u;
    atomicAnd(&words[w], ~(mask << s));
    atomicOr(&words[w], v << s);
    if (s + nbits > 32) {
        const int r = 32 - s;
        atomicAnd(&words[w + 1], ~(mask >> r));
        atomicOr(&words[w + 1], v >> r);
    }
}

template <bool IMPORT>
__global__ void __launch_bounds__(256) kv_convert_kernel(const StoreArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int dim = a.dim, bpp = dim >> 3, nq = dim >> 5;
    const int recb = tl_record_bytes(dim, a.kb, a.vb);
    const int ksec = tl_key_section(dim, a.kb), vsec = tl_val_section(dim, a.vb);
    for (int64_t row = warp; row < a.n; row += nwarps) {
        const int64_t slot = a.map(row);
        if (slot < 0) continue;
        uint8_t* rec = a.store + (slot >> 4) * (int64_t)recb;
        const int r = (int)(slot & 15);
        uint8_t* nsec = rec + ksec + vsec;
        for (int which = 0; which < (a.vb ? 2 : 1); which++) {   // 0 = keys, 1 = values
            const int bits = which ? a.vb : a.kb;
            uint8_t* packed = which ? a.v_packed : a.k_packed;
            float* norms = which ? a.v_norms : a.k_norms;
            uint8_t* sec = which ? rec + ksec : rec;
            if (packed) {
                uint8_t* prow = packed + row * (int64_t)(bits * bpp);
                for (int q = 0; q < nq; q++) {
                    const int d = lane + 32 * q;
                    int base, bit;
                    if (which) tl_val_slot(dim, bits, r, d, base, bit);
                    else tl_key_slot(dim, bits, r, d, base, bit);
                    if (IMPORT) {
                        uint32_t c = 0;
                        for (int p = 0; p < bits; p++) c |= ((prow[p * bpp + (d >> 3)] >> (7 - (d & 7))) & 1u) << p;
                        st_atomic_write(reinterpret_cast<uint32_t*>(sec), base * 8 + bit, bits, c);
                    } else {
                        const uint32_t c = tl_read_bits(sec + base, bit, bits);
                        for (int p = 0; p < bits; p++) {
                            const uint32_t w = ballot_to_plane_word(__ballot_sync(0xffffffffu, (c >> p) & 1u));
                            if (lane == 0) *reinterpret_cast<uint32_t*>(prow + p * bpp + 4 * q) = w;
                        }
                    }
                }
            }
            if (norms && lane == 0) {
                float* nrm = reinterpret_cast<float*>(nsec + tl_norm_offset(a.vb, which, r));
                if (IMPORT) *nrm = norms[row];
                else norms[row] = *nrm;
            }
        }
    }
}

static int check_geometry(const char* who, int dim, int kb, int vb) {
    if (dim != 64 && dim != 128) return fail(TQB_ERR_UNSUPPORTED, "%s: head_dim must be 64 or 128, got %d", who, dim);
    if (kb < 2 || kb > 4 || (vb != 0 && (vb < 2 || vb > 4)))
        return fail(TQB_ERR_UNSUPPORTED, "%s: key bits must be 2..4 and value bits 2..4 (or 0: key-only records), got %d/%d",
                    who, kb, vb);
    return TQB_OK;
}

template <bool IMPORT>
static int launch_convert(const char* who, uint8_t* store, int64_t n, int dim, int kb, int vb, const tqb_rowmap* map,
                          uint8_t* kp, float* kn, uint8_t* vp, float* vn, void* stream) {
    TQB_REQUIRE(n >= 0, "%s: negative row count", who);
    if (int e = check_geometry(who, dim, kb, vb)) return e;
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(store, "%s: null store", who);
    TQB_REQUIRE((uintptr_t)store % 16 == 0, "%s: the record store must be 16-byte aligned", who);
    TQB_REQUIRE(((uintptr_t)kp | (uintptr_t)vp) % 4 == 0, "%s: packed rows must be 4-byte aligned", who);
    TQB_REQUIRE(vb != 0 || (!vp && !vn), "%s: key-only records have no value rows", who);
    StoreArgs a{};
    a.store = store; a.n = n; a.dim = dim; a.kb = kb; a.vb = vb; a.map = make_rowmap(map);
    a.k_packed = kp; a.k_norms = kn; a.v_packed = vp; a.v_norms = vn;
    const int grid = (int)std::min<int64_t>(ceil_div(n, 8), (int64_t)sm_count() * 8);
    kv_convert_kernel<IMPORT><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    return check_launch(who);
}

}  // namespace tqb

extern "C" int64_t tqb_kv_record_bytes(int dim, int kbits, int vbits) {
    if ((dim != 64 && dim != 128) || kbits < 2 || kbits > 4 || (vbits != 0 && (vbits < 2 || vbits > 4))) return 0;
    return tqb::tl_record_bytes(dim, kbits, vbits);
}

extern "C" int tqb_kv_export(const uint8_t* store, int64_t n, int dim, int kbits, int vbits, const tqb_rowmap* map,
                             uint8_t* k_packed, float* k_norms, uint8_t* v_packed, float* v_norms, void* stream) {
    return tqb::launch_convert<false>("kv_export", const_cast<uint8_t*>(store), n, dim, kbits, vbits, map, k_packed,
                                      k_norms, v_packed, v_norms, stream);
}

extern "C" int tqb_kv_import(uint8_t* store, int64_t n, int dim, int kbits, int vbits, const tqb_rowmap* map,
                             const uint8_t* k_packed, const float* k_norms, const uint8_t* v_packed,
                             const float* v_norms, void* stream) {
    return tqb::launch_convert<true>("kv_import", store, n, dim, kbits, vbits, map, const_cast<uint8_t*>(k_packed),
                                     const_cast<float*>(k_norms), const_cast<uint8_t*>(v_packed),
                                     const_cast<float*>(v_norms), stream);
}
