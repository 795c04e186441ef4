// pack.cu -- bit-plane pack / unpack of quantisation codes.
//
// Layout (upstream turboquant_kv/reference.py:191-255): a packed row is `bits` planes of
// ceil(dim/8) bytes; plane i holds bit i of every code; dimension 8m+t is bit 7-t of byte m.
// Both kernels are pure streaming: one thread produces one output byte (pack) or eight codes of
// one byte column (unpack), consecutive threads touch consecutive bytes.
#include "common.cuh"

namespace tqb {

__global__ void pack_codes_kernel(const uint8_t* __restrict__ codes, int64_t n, int dim, int bits,
                                  int bpp, uint8_t* __restrict__ packed) {
    const int64_t pd = (int64_t)bits * bpp;
    const int64_t total = n * pd;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / pd;
        const int col = (int)(i - row * pd);
        const int plane = col / bpp, m = col - plane * bpp;
        const uint8_t* c = codes + row * dim + 8 * m;
        const int lim = min(8, dim - 8 * m);
        uint32_t byte = 0;
        for (int t = 0; t < lim; t++) byte |= ((c[t] >> plane) & 1u) << (7 - t);
        packed[i] = (uint8_t)byte;
    }
}

__global__ void unpack_codes_kernel(const uint8_t* __restrict__ packed, int64_t n, int dim, int bits,
                                    int bpp, uint8_t* __restrict__ codes) {
    const int64_t pd = (int64_t)bits * bpp;
    const int64_t total = n * bpp;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / bpp;
        const int m = (int)(i - row * bpp);
        const uint8_t* p = packed + row * pd + m;
        uint32_t planes[8];
        for (int b = 0; b < bits; b++) planes[b] = p[(int64_t)b * bpp];
        const int lim = min(8, dim - 8 * m);
        uint8_t* c = codes + row * dim + 8 * m;
        for (int t = 0; t < lim; t++) {
            uint32_t v = 0;
            for (int b = 0; b < bits; b++) v |= ((planes[b] >> (7 - t)) & 1u) << b;
            c[t] = (uint8_t)v;
        }
    }
}

}  // namespace tqb

extern "C" int tqb_pack_codes(const uint8_t* codes, int64_t n, int dim, int bits, uint8_t* packed,
                              void* stream) {
    TQB_REQUIRE(bits >= 1 && bits <= 8, "pack_codes: bit_width must be 1-8, got %d", bits);
    TQB_REQUIRE(dim >= 1 && n >= 0, "pack_codes: bad shape (%lld, %d)", (long long)n, dim);
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(codes && packed, "pack_codes: null pointer");
    const int bpp = tqb::bytes_per_plane(dim);
    const int64_t total = n * bits * bpp;
    const int grid = (int)std::min<int64_t>(tqb::ceil_div(total, 256), (int64_t)tqb::sm_count() * 16);
    tqb::pack_codes_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(codes, n, dim, bits, bpp, packed);
    return tqb::check_launch("pack_codes");
}

extern "C" int tqb_unpack_codes(const uint8_t* packed, int64_t n, int dim, int bits, uint8_t* codes,
                                void* stream) {
    TQB_REQUIRE(bits >= 1 && bits <= 8, "unpack_codes: bit_width must be 1-8, got %d", bits);
    TQB_REQUIRE(dim >= 1 && n >= 0, "unpack_codes: bad shape (%lld, %d)", (long long)n, dim);
    if (n == 0) return TQB_OK;
    TQB_REQUIRE(codes && packed, "unpack_codes: null pointer");
    const int bpp = tqb::bytes_per_plane(dim);
    const int64_t total = n * bpp;
    const int grid = (int)std::min<int64_t>(tqb::ceil_div(total, 256), (int64_t)tqb::sm_count() * 16);
    tqb::unpack_codes_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(packed, n, dim, bits, bpp, codes);
    return tqb::check_launch("unpack_codes");
}
