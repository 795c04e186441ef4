// decode_bits.cuh -- bit-plane -> tensor-core-fragment index arithmetic, shared by the decode
// attention kernel and the index scan.  Everything here is plain integer code marked
// TQB_HD so that the same functions run on the host: tests/test_fragment_maps.py compiles this
// header with g++ and replays a whole warp tile on the CPU against a direct computation.
//
// Packed layout (upstream turboquant_kv/reference.py:206-224): plane p of a row holds bit p of
// every code; dimension 8m+t is bit 7-t of plane byte m.
//
// Fragment conventions are those of mma.sync.aligned.m16n8k16 (row.col, 16-bit inputs, f32
// accumulate), lane = 4*g + t:
//   A (16x16): a0a1 = (row g,   k 2t,2t+1)   a2a3 = (row g+8, k 2t,2t+1)
//              a4a5 = (row g,   k 2t+8,+9)   a6a7 = (row g+8, k 2t+8,+9)
//   B (16x8):  b0b1 = (k 2t,2t+1,   col g)   b2b3 = (k 2t+8,+9, col g)
//   C (16x8):  c0,c1 = (row g, cols 2t,2t+1) c2,c3 = (row g+8, cols 2t,2t+1)
// The contraction index k may be permuted freely as long as A and B agree, which is what makes a
// cheap decode possible: a lookup index is one byte holding, for TWO codes, one bit pair from each
// plane, and the 256-entry table returns both centroids as a half2.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define TQB_HD __host__ __device__ __forceinline__
#else
#define TQB_HD inline
#endif

namespace tqb {

// ------------------------------------------------------------------------------------------
// KEY side (and scan rows): A operand = codes of 16 rows x 16 dims, pairs along dims.
//
// A thread (g, t) owns, for rows g and g+8, the plane bytes [BT*t, BT*t + BT) with BT = D/32.
// `P[p]` is a 32-bit word whose four bytes are four plane-p bytes the thread owns (for D = 64 two
// bytes of row g and two of row g+8; for D >= 128 four consecutive bytes of one row).
// For bit pair u (bits 2u+1, 2u of every byte) the index word holds, per byte lane,
//   bits[1:0] = plane 0, bits[3:2] = plane 1, bits[5:4] = plane 2, bits[7:6] = plane 3.
// In each 2-bit field bit 1 belongs to dimension 8m+6-2u ("lo", first element of the pair) and
// bit 0 to dimension 8m+7-2u ("hi").
template <int BITS>
TQB_HD uint32_t pair_index_word(const uint32_t (&P)[4], int u) {
    uint32_t r = (P[0] >> (2 * u)) & 0x03030303u;
    if (BITS > 1) r |= ((P[1] >> (2 * u)) << 2) & 0x0C0C0C0Cu;
    if (BITS > 2) r |= ((P[2] >> (2 * u)) << 4) & 0x30303030u;
    if (BITS > 3) r |= ((P[3] >> (2 * u)) << 6) & 0xC0C0C0C0u;
    return r;
}

// The two codes addressed by one index byte of pair_index_word.
template <int BITS>
TQB_HD void pair_index_codes(uint32_t x, int& code_lo, int& code_hi) {
    code_lo = 0; code_hi = 0;
    for (int p = 0; p < BITS; p++) {
        code_hi |= ((x >> (2 * p)) & 1) << p;
        code_lo |= ((x >> (2 * p + 1)) & 1) << p;
    }
}

// Dimensions covered by fragment element pair e = 2*ks + half of thread t (ks = k-step of 16
// dims, half = 0 for a0a1/a2a3, 1 for a4a5/a6a7).  e -> (u, i): u = e / BT bit pair, i = e % BT byte
// within the thread's slice; plane byte m = BT*t + i.
TQB_HD void pair_dims(int D, int t, int e, int& d_lo, int& d_hi) {
    const int BT = D / 32;
    const int u = e / BT, i = e % BT;
    const int m = BT * t + i;
    d_lo = 8 * m + 6 - 2 * u;
    d_hi = 8 * m + 7 - 2 * u;
}

// ------------------------------------------------------------------------------------------
// VALUE side: A operand = V^T, 16 dims x 16 tokens, pairs along TOKENS (the contraction index).
//
// A thread (g, t) owns dims of plane byte column(s) c = BV*g + i (BV = D/64 columns, i < BV) and
// the tokens 2t, 2t+1 (a0..a3) and 2t+8, 2t+9 (a4..a7).  M-tile mt = 4*i + u covers bit pair u of
// column c: fragment row g is dimension 8c+6-2u (bit 2u+1), row g+8 is dimension 8c+7-2u (bit 2u).
//
// WA / WB: the column's plane bytes of token A / token B, byte lane p = plane p (0 if p >= BITS).
TQB_HD void value_dims(int D, int g, int mt, int& d_row_g, int& d_row_g8) {
    const int BV = D / 64;
    const int i = mt / 4, u = mt % 4;
    const int c = BV * g + i;
    d_row_g = 8 * c + 6 - 2 * u;
    d_row_g8 = 8 * c + 7 - 2 * u;
}

// 2-bit values: one index byte covers 2 dims x 2 tokens x 2 planes.  W = A.p0 | A.p1<<8 | B.p0<<16 |
// B.p1<<24.  Result X: fields f0..f3 (2 bits each, from A.p0, A.p1, B.p0, B.p1); in every field bit 1
// is the row-g dimension and bit 0 the row-(g+8) dimension.
TQB_HD uint32_t quad_index_v2(uint32_t W, int u) {
    const uint32_t x = (W >> (2 * u)) & 0x03030303u;
    return (x * 0x01041040u) >> 24;  // 2^24 + 2^18 + 2^12 + 2^6
}
TQB_HD void quad_index_codes_v2(uint32_t X, int& a_rowg, int& b_rowg, int& a_rowg8, int& b_rowg8) {
    a_rowg = ((X >> 1) & 1) | (((X >> 3) & 1) << 1);
    a_rowg8 = (X & 1) | (((X >> 2) & 1) << 1);
    b_rowg = ((X >> 5) & 1) | (((X >> 7) & 1) << 1);
    b_rowg8 = ((X >> 4) & 1) | (((X >> 6) & 1) << 1);
}

// 3- and 4-bit values: one index byte covers 1 dim x 2 tokens x BITS planes.  token_pair_words
// interleaves the two tokens once per column; token_pair_index then serves all 8 bit positions.
//   Ze: at every even bit position b: bit b = A's bit b, bit b+1 = B's bit b
//   Zo: at every even bit position b: bit b = A's bit b+1, bit b+1 = B's bit b+1
TQB_HD void token_pair_words(uint32_t WA, uint32_t WB, uint32_t& Ze, uint32_t& Zo) {
    Ze = (WA & 0x55555555u) | ((WB & 0x55555555u) << 1);
    Zo = ((WA >> 1) & 0x55555555u) | (WB & 0xAAAAAAAAu);
}
// beta = bit position inside the byte (odd: row-g dimension of bit pair beta/2, even: row g+8).
TQB_HD uint32_t token_pair_index(uint32_t Ze, uint32_t Zo, int beta) {
    const uint32_t z = (beta & 1) ? Zo : Ze;
    const uint32_t x = (z >> (beta & ~1)) & 0x03030303u;
    return (x * 0x01041040u) >> 24;
}
template <int BITS>
TQB_HD void token_pair_codes(uint32_t X, int& code_a, int& code_b) {
    code_a = 0; code_b = 0;
    for (int p = 0; p < BITS; p++) {
        code_a |= ((X >> (2 * p)) & 1) << p;
        code_b |= ((X >> (2 * p + 1)) & 1) << p;
    }
}

}  // namespace tqb

// ------------------------------------------------------------------------------------------
// Gathers from a 16-row tile of packed rows (shared memory on the device, plain memory in the host
// replay).  `tile` points at row 0 of the tile, rows are `pitch` bytes apart.
namespace tqb {

// Key / scan rows.  NW words per plane: D = 64 -> 1 (row g in the low half-word, row g+8 in the
// high one); D = 128 -> 2 (word 0 = row g, word 1 = row g+8).
template <int D> struct KeyWords { static constexpr int NW = D / 64; };

template <int D, int BITS>
TQB_HD void gather_key_words(const uint8_t* tile, int pitch, int g, int t, uint32_t (&P)[KeyWords<D>::NW][4]) {
    static_assert(D == 64 || D == 128, "key fragments are built for head_dim 64 and 128");
    const uint8_t* r0 = tile + g * pitch;
    const uint8_t* r1 = tile + (g + 8) * pitch;
    for (int p = 0; p < 4; p++) {
        if (D == 64) {
            uint32_t lo = 0, hi = 0;
            if (p < BITS) {
                lo = *reinterpret_cast<const uint16_t*>(r0 + p * 8 + 2 * t);
                hi = *reinterpret_cast<const uint16_t*>(r1 + p * 8 + 2 * t);
            }
            P[0][p] = lo | (hi << 16);
        } else {
            P[0][p] = p < BITS ? *reinterpret_cast<const uint32_t*>(r0 + p * 16 + 4 * t) : 0u;
            P[D / 64 - 1][p] = p < BITS ? *reinterpret_cast<const uint32_t*>(r1 + p * 16 + 4 * t) : 0u;
        }
    }
}

// Which (word, byte lane) of the index words holds fragment element pair e of row g (second = false)
// or row g+8 (second = true).  u = e / BT selects the bit pair (one index word per u), i = e % BT.
template <int D>
TQB_HD void key_element_slot(int e, bool second, int& u, int& word, int& lane) {
    constexpr int BT = D / 32;
    u = e / BT;
    const int i = e % BT;
    if (D == 64) { word = 0; lane = (second ? 2 : 0) + i; }
    else { word = second ? 1 : 0; lane = i; }
}

// Value rows: plane bytes of column c for one token, byte lane p = plane p.
template <int D, int BITS>
TQB_HD uint32_t gather_value_word(const uint8_t* tile, int pitch, int token, int c) {
    const uint8_t* r = tile + token * pitch + c;
    uint32_t w = 0;
    for (int p = 0; p < BITS; p++) w |= (uint32_t)r[p * (D / 8)] << (8 * p);
    return w;
}

}  // namespace tqb
