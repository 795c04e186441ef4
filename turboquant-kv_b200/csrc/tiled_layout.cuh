// tiled_layout.cuh -- the fragment-major storage layout of the packed KV cache.
//
// The upstream layout (bit planes per token, reference.py:206-224) costs ~1.4 integer instructions per
// code to turn into tensor-core operands, and the decode kernel is bound by instruction issue, not
// by HBM.  The cache is therefore stored in a layout from which operands fall out of one shared-memory
// load and a table lookup per TWO codes.  It holds exactly the same codes and the same number of
// bytes per token; tqb_kv_export / tqb_kv_import convert to and from the upstream layout.
//
// Tokens are grouped in tiles of 16.  One RECORD holds one tile of one (sequence, KV head):
//
//   [ key section : 32 lanes x KL bytes ][ value section : 32 lanes x VL bytes ][ norm section : 32 floats ]
//      KL = D*KB/16                          VL = D*VB/16                          record = 2*D*(KB+VB) + 128 bytes
//
// Norm section: 8 groups of 16 bytes, group g = { key norm of token g, key norm of token g+8, value norm
// of token g, value norm of token g+8 } -- what MMA lane 4g+t needs of the record's norms, in one
// 128-bit shared load (tl_norm_offset).
//
// The search index uses the same records without the value half (VB = 0): 16 database rows per record,
// [ key section ][ 16 norms: 8 pairs { row g, row g+8 } ], record = 2*D*KB + 64 bytes -- the upstream
// 68 bytes per row at D = 128, 4 bits.
//
// Lane = 4*g + t is the mma.sync lane that consumes the bytes (g = lane/4, t = lane%4).
//
// Key section, lane (g, t) [stored contiguously per lane, or as two planes when KL = 32, see
// tl_key_piece_offset]: the codes of tokens g (first KL/2 bytes) and g+8 (last KL/2 bytes) for the
// dims this lane feeds into the score MMA.  A token's half is D/8 FIELDS of 2*KB bits, field e at bit
// e*2*KB (little endian).  Field e = code[d] | code[d+1] << KB with d = 16*(e/2) + 8*(e%2) + 2*t, i.e.
// exactly the A-operand elements (k = 2t, 2t+1 | 2t+8, 2t+9) of k-step e/2.
//
// Value section, lane (g, t): the codes of tokens {2t, 2t+1, 2t+8, 2t+9} for dims 16*mt + g and
// 16*mt + g + 8 (mt < D/16): the A-operand of O^T += V^T P^T, whose contraction index is the token.
//   VB == 2: field f = 2*mt + half (8 bits): bits[1:0] = code(token A, dim 16mt+g), [3:2] = (B, 16mt+g),
//            [5:4] = (A, 16mt+g+8), [7:6] = (B, 16mt+g+8), with A = 2t + 8*half, B = A + 1.
//   VB  > 2: field f = 2*(2*mt + half) + s (2*VB bits): code(A, dim) | code(B, dim) << VB, dim = 16mt+g+8s.
//
// Everything below is host/device so that tests replay it on the CPU.
#pragma once
#include <stdint.h>

#include "decode_bits.cuh"

namespace tqb {

constexpr int TL_TILE = 16;

TQB_HD int tl_key_lane_bytes(int D, int KB) { return D * KB / 16; }
TQB_HD int tl_val_lane_bytes(int D, int VB) { return D * VB / 16; }
// VB == 0: key-only records (the search index: rows instead of tokens) carry the 16 key norms only.
TQB_HD int tl_record_bytes(int D, int KB, int VB) { return 2 * D * (KB + VB) + (VB ? 128 : 64); }
TQB_HD int tl_key_section(int D, int KB) { return 32 * tl_key_lane_bytes(D, KB); }
TQB_HD int tl_val_section(int D, int VB) { return 32 * tl_val_lane_bytes(D, VB); }

// Byte offset, inside the norm section, of the norm of token row r (which = 0: key, 1: value).
TQB_HD int tl_norm_offset(int VB, int which, int r) {
    return VB ? 16 * (r & 7) + 8 * which + 4 * (r >> 3) : 8 * (r & 7) + 4 * (r >> 3);
}

// A lane's key chunk is stored in one piece, except 32-byte chunks (D = 128, 4 bits), which are stored as
// two 16-byte planes (the token-g half of all 32 lanes, then the token-g+8 half) so that each of the two
// 128-bit shared loads of a warp is free of bank conflicts.  Piece p of lane l starts here:
TQB_HD int tl_key_pieces(int D, int KB) { return tl_key_lane_bytes(D, KB) == 32 ? 2 : 1; }
TQB_HD int tl_key_piece_offset(int D, int KB, int lane, int piece) {
    const int pb = tl_key_lane_bytes(D, KB) / tl_key_pieces(D, KB);
    return piece * 32 * pb + lane * pb;
}

// Where the code of (token row r of the tile, dim d) lives in the KEY section:
// byte offset of the lane's token half and the bit offset inside it.
TQB_HD void tl_key_slot(int D, int KB, int r, int d, int& byte_base, int& bit) {
    const int g = r & 7, second = r >> 3;
    const int ks = d >> 4, half = (d >> 3) & 1, t = (d & 7) >> 1, hi = d & 1;
    const int e = 2 * ks + half;
    const int KL = tl_key_lane_bytes(D, KB);
    byte_base = tl_key_pieces(D, KB) == 2 ? tl_key_piece_offset(D, KB, 4 * g + t, second)
                                          : (4 * g + t) * KL + second * (KL / 2);
    bit = e * 2 * KB + hi * KB;
}

// Same for the VALUE section (byte_base = start of the lane's chunk).
TQB_HD void tl_val_slot(int D, int VB, int r, int d, int& byte_base, int& bit) {
    const int half = r >> 3, t = (r & 7) >> 1, ab = r & 1;
    const int mt = d >> 4, g = d & 7, s = (d >> 3) & 1;
    const int VL = tl_val_lane_bytes(D, VB);
    byte_base = (4 * g + t) * VL;
    if (VB == 2) bit = (2 * mt + half) * 8 + 4 * s + 2 * ab;
    else bit = (2 * (2 * mt + half) + s) * 2 * VB + ab * VB;
}

// Read `bits` bits at bit offset `bit` of a little-endian byte string (plain memory).
TQB_HD uint32_t tl_read_bits(const uint8_t* p, int bit, int bits) {
    uint32_t v = 0;
    for (int i = 0; i < bits; i++) v |= (uint32_t)((p[(bit + i) >> 3] >> ((bit + i) & 7)) & 1) << i;
    return v;
}

// Field extraction from a lane's chunk held in 32-bit registers (w[0] = first 4 bytes).
template <int NW>
TQB_HD uint32_t tl_field(const uint32_t (&w)[NW], int bit, int bits) {
    const int i = bit >> 5, s = bit & 31;
    uint32_t v = w[i] >> s;
    if (s + bits > 32 && i + 1 < NW) v |= w[i + 1] << (32 - s);
    return v & ((1u << bits) - 1u);
}

// Codes addressed by a key field / a value field (the table builders use these).
TQB_HD void tl_key_field_codes(uint32_t x, int KB, int& c_lo, int& c_hi) {
    c_lo = x & ((1 << KB) - 1);
    c_hi = (x >> KB) & ((1 << KB) - 1);
}
TQB_HD void tl_val_quad_codes(uint32_t x, int& a_g, int& b_g, int& a_g8, int& b_g8) {
    a_g = x & 3; b_g = (x >> 2) & 3; a_g8 = (x >> 4) & 3; b_g8 = (x >> 6) & 3;
}
TQB_HD void tl_val_pair_codes(uint32_t x, int VB, int& c_a, int& c_b) {
    c_a = x & ((1 << VB) - 1);
    c_b = (x >> VB) & ((1 << VB) - 1);
}

}  // namespace tqb

// ---- consumer-side field positions (shared by the kernel and the host replay) ---------------------
namespace tqb {

// Bit offset, inside a lane's KEY chunk, of the field feeding A-operand element pair
// (k-step ks, half) of token g (second = 0) or g+8 (second = 1).
TQB_HD int tl_key_field_bit(int D, int KB, int ks, int half, int second) {
    return second * (tl_key_lane_bytes(D, KB) * 4) + (2 * ks + half) * 2 * KB;
}
// Bit offset, inside a lane's VALUE chunk, of the field for m-tile mt, token half, fragment row s.
// VB == 2: one 8-bit field serves both rows (s ignored).
TQB_HD int tl_val_field_bit(int VB, int mt, int half, int s) {
    return VB == 2 ? (2 * mt + half) * 8 : (2 * (2 * mt + half) + s) * 2 * VB;
}

#ifdef __CUDACC__
// Clear-then-set of a bit field in 32-bit words; safe against concurrent writers of OTHER bits of
// the same word (two tokens of a pair share value bytes, 3-bit fields straddle bytes).
__device__ __forceinline__ void tl_atomic_write(uint32_t* words, int absbit, int nbits, uint32_t v) {
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

// One quantised row -> its token slot in the tiled KV store (tiled_layout.cuh).  Lane l holds the codes
// of dims l + 32 q.  Called by all 32 lanes with the same `slot`.
// `which`: 1 = key section, 2 = value section.
template <int NQ>
__device__ __forceinline__ void tiled_store_row(uint8_t* store, int which, int kb, int vb, int64_t slot,
                                                const uint32_t (&code)[NQ], float nrm, int lane, int dim) {
    uint8_t* rec = store + (slot >> 4) * (int64_t)tl_record_bytes(dim, kb, vb);
    const int r = (int)(slot & 15);
    const int ksec = tl_key_section(dim, kb), vsec = tl_val_section(dim, vb);
#pragma unroll
    for (int q = 0; q < NQ; q++) {
        const int d = lane + 32 * q;
        const uint32_t partner = __shfl_down_sync(0xffffffffu, code[q], 1);
        if (d >= dim) continue;
        int base, bit;
        if (which == 1) {
            tl_key_slot(dim, kb, r, d, base, bit);
            if (kb == 4) {   // a field is one whole byte owned by this token: plain store from the even lane
                if ((lane & 1) == 0) rec[base + (bit >> 3)] = (uint8_t)(code[q] | (partner << 4));
            } else {
                tl_atomic_write(reinterpret_cast<uint32_t*>(rec), base * 8 + bit, kb, code[q]);
            }
        } else {
            tl_val_slot(dim, vb, r, d, base, bit);
            tl_atomic_write(reinterpret_cast<uint32_t*>(rec + ksec), base * 8 + bit, vb, code[q]);
        }
    }
    if (lane == 0) *reinterpret_cast<float*>(rec + ksec + vsec + tl_norm_offset(vb, which - 1, r)) = nrm;
}
#endif  // __CUDACC__

}  // namespace tqb
