// fragment_harness.cpp -- host replay of one warp tile of the decode-attention / scan kernels.
//
// Compiled by tests/test_fragment_maps.py with g++ against csrc/decode_bits.cuh (the very header
// the CUDA kernels include).  For every one of the 32 lanes it performs the gathers, index-word
// arithmetic and table lookups the kernel performs, places the results in the A / B operand
// positions defined by mma.sync.m16n8k16, multiplies on the CPU, and returns the product so that
// the test can compare it with a direct evaluation on unpacked codes.
#include <cstdint>
#include <cstring>
#include <vector>

#include "decode_bits.cuh"
#include "tiled_layout.cuh"

using namespace tqb;

namespace {

// scores[row][col] += sum_k A[row][k] * B[k][col] with operands given per lane in fragment form.
struct Frag {
    float a[32][8];  // a0..a7 per lane
    float b[32][4];  // b0..b3 per lane
};

void mma_replay(const Frag& f, float (&C)[16][8]) {
    float A[16][16] = {}, B[16][8] = {};
    for (int lane = 0; lane < 32; lane++) {
        const int g = lane >> 2, t = lane & 3;
        A[g][2 * t] = f.a[lane][0];          A[g][2 * t + 1] = f.a[lane][1];
        A[g + 8][2 * t] = f.a[lane][2];      A[g + 8][2 * t + 1] = f.a[lane][3];
        A[g][2 * t + 8] = f.a[lane][4];      A[g][2 * t + 9] = f.a[lane][5];
        A[g + 8][2 * t + 8] = f.a[lane][6];  A[g + 8][2 * t + 9] = f.a[lane][7];
        B[2 * t][g] = f.b[lane][0];          B[2 * t + 1][g] = f.b[lane][1];
        B[2 * t + 8][g] = f.b[lane][2];      B[2 * t + 9][g] = f.b[lane][3];
    }
    for (int r = 0; r < 16; r++)
        for (int c = 0; c < 8; c++) {
            float s = 0.f;
            for (int k = 0; k < 16; k++) s += A[r][k] * B[k][c];
            C[r][c] += s;
        }
}

template <int D, int BITS>
void key_tile(const uint8_t* tile, const float* cent, const float* q /*[8][D]*/, float* out /*[16][8]*/) {
    constexpr int NW = KeyWords<D>::NW;
    const int pitch = BITS * D / 8;
    float C[16][8] = {};
    for (int ks = 0; ks < D / 16; ks++) {
        Frag f{};
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane >> 2, t = lane & 3;
            uint32_t P[NW][4];
            gather_key_words<D, BITS>(tile, pitch, g, t, P);
            for (int half = 0; half < 2; half++) {
                const int e = 2 * ks + half;
                for (int second = 0; second < 2; second++) {
                    int u, word, bl;
                    key_element_slot<D>(e, second != 0, u, word, bl);
                    const uint32_t iw = pair_index_word<BITS>(P[word], u);
                    const uint32_t x = (iw >> (8 * bl)) & 0xFF;
                    int clo, chi;
                    pair_index_codes<BITS>(x, clo, chi);
                    f.a[lane][4 * half + 2 * second + 0] = cent[clo];
                    f.a[lane][4 * half + 2 * second + 1] = cent[chi];
                }
                int dlo, dhi;
                pair_dims(D, t, e, dlo, dhi);
                f.b[lane][2 * half + 0] = q[g * D + dlo];
                f.b[lane][2 * half + 1] = q[g * D + dhi];
            }
        }
        mma_replay(f, C);
    }
    std::memcpy(out, C, sizeof(C));
}

// O^T[dim][head] = sum_token V^T[dim][token] * P^T[token][head]; out is [D][8].
template <int D, int BITS>
void value_tile(const uint8_t* tile, const float* cent, const float* pw /*[16 tokens][8 heads]*/, float* out) {
    const int pitch = BITS * D / 8;
    constexpr int BV = D / 64;
    for (int mt = 0; mt < D / 16; mt++) {
        Frag f{};
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane >> 2, t = lane & 3;
            const int i = mt / 4, u = mt % 4;
            const int c = BV * g + i;
            for (int half = 0; half < 2; half++) {
                const int ta = 2 * t + 8 * half, tb = ta + 1;
                const uint32_t WA = gather_value_word<D, BITS>(tile, pitch, ta, c);
                const uint32_t WB = gather_value_word<D, BITS>(tile, pitch, tb, c);
                if (BITS == 2) {
                    const uint32_t X = quad_index_v2(WA | (WB << 16), u);
                    int ag, bg, ag8, bg8;
                    quad_index_codes_v2(X, ag, bg, ag8, bg8);
                    f.a[lane][4 * half + 0] = cent[ag];  f.a[lane][4 * half + 1] = cent[bg];
                    f.a[lane][4 * half + 2] = cent[ag8]; f.a[lane][4 * half + 3] = cent[bg8];
                } else {
                    uint32_t Ze, Zo;
                    token_pair_words(WA, WB, Ze, Zo);
                    int ca, cb;
                    token_pair_codes<BITS>(token_pair_index(Ze, Zo, 2 * u + 1), ca, cb);
                    f.a[lane][4 * half + 0] = cent[ca];  f.a[lane][4 * half + 1] = cent[cb];
                    token_pair_codes<BITS>(token_pair_index(Ze, Zo, 2 * u), ca, cb);
                    f.a[lane][4 * half + 2] = cent[ca];  f.a[lane][4 * half + 3] = cent[cb];
                }
                // B = P^T: (k = tokens 2t+8*half, +1 ; col = head g)
                f.b[lane][2 * half + 0] = pw[ta * 8 + g];
                f.b[lane][2 * half + 1] = pw[tb * 8 + g];
            }
        }
        float C[16][8] = {};
        mma_replay(f, C);
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane >> 2, t = lane & 3;
            int dg, dg8;
            value_dims(D, g, mt, dg, dg8);
            for (int j = 0; j < 2; j++) {
                out[dg * 8 + 2 * t + j] = C[g][2 * t + j];
                out[dg8 * 8 + 2 * t + j] = C[g + 8][2 * t + j];
            }
        }
    }
}


// ---- tiled (fragment-major) layout: writer = tl_*_slot, reader = what the decode kernel does ----
void write_bits(uint8_t* p, int bit, int bits, uint32_t v) {
    for (int i = 0; i < bits; i++) {
        p[(bit + i) >> 3] &= (uint8_t)~(1u << ((bit + i) & 7));
        p[(bit + i) >> 3] |= (uint8_t)(((v >> i) & 1u) << ((bit + i) & 7));
    }
}

void tiled_build(int D, int KB, int VB, const uint8_t* kcodes /*[16][D]*/, const uint8_t* vcodes, uint8_t* rec) {
    std::memset(rec, 0, tl_record_bytes(D, KB, VB));
    uint8_t* ksec = rec;
    uint8_t* vsec = rec + tl_key_section(D, KB);
    for (int r = 0; r < 16; r++)
        for (int d = 0; d < D; d++) {
            int base, bit;
            tl_key_slot(D, KB, r, d, base, bit);
            write_bits(ksec + base, bit, KB, kcodes[r * D + d]);
            tl_val_slot(D, VB, r, d, base, bit);
            write_bits(vsec + base, bit, VB, vcodes[r * D + d]);
        }
}

template <int NW>
void load_words(const uint8_t* p, uint32_t (&w)[NW], int nbytes) {
    for (int i = 0; i < NW; i++) w[i] = 0;
    std::memcpy(w, p, nbytes);
}

void tiled_key_tile(int D, int KB, int VB, const uint8_t* rec, const float* cent, const float* q, float* out) {
    const int KL = tl_key_lane_bytes(D, KB);
    float C[16][8] = {};
    for (int ks = 0; ks < D / 16; ks++) {
        Frag f{};
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane >> 2, t = lane & 3;
            uint32_t kw[8] = {};
            {
                const int pieces = tl_key_pieces(D, KB), pb = KL / pieces;
                for (int pc = 0; pc < pieces; pc++)
                    std::memcpy(reinterpret_cast<uint8_t*>(kw) + pc * pb, rec + tl_key_piece_offset(D, KB, lane, pc), pb);
            }
            for (int half = 0; half < 2; half++) {
                for (int second = 0; second < 2; second++) {
                    const uint32_t x = tl_field(kw, tl_key_field_bit(D, KB, ks, half, second), 2 * KB);
                    int clo, chi;
                    tl_key_field_codes(x, KB, clo, chi);
                    f.a[lane][4 * half + 2 * second + 0] = cent[clo];
                    f.a[lane][4 * half + 2 * second + 1] = cent[chi];
                }
                const int d = 16 * ks + 8 * half + 2 * t;   // natural B fragment
                f.b[lane][2 * half + 0] = q[g * D + d];
                f.b[lane][2 * half + 1] = q[g * D + d + 1];
            }
        }
        mma_replay(f, C);
    }
    std::memcpy(out, C, sizeof(C));
}

void tiled_value_tile(int D, int KB, int VB, const uint8_t* rec, const float* cent, const float* pw, float* out) {
    const int VL = tl_val_lane_bytes(D, VB);
    const uint8_t* vsec = rec + tl_key_section(D, KB);
    for (int mt = 0; mt < D / 16; mt++) {
        Frag f{};
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane >> 2, t = lane & 3;
            uint32_t vw[8];
            load_words(vsec + lane * VL, vw, VL);
            for (int half = 0; half < 2; half++) {
                const int ta = 2 * t + 8 * half, tb = ta + 1;
                if (VB == 2) {
                    const uint32_t x = tl_field(vw, tl_val_field_bit(VB, mt, half, 0), 8);
                    int ag, bg, ag8, bg8;
                    tl_val_quad_codes(x, ag, bg, ag8, bg8);
                    f.a[lane][4 * half + 0] = cent[ag];  f.a[lane][4 * half + 1] = cent[bg];
                    f.a[lane][4 * half + 2] = cent[ag8]; f.a[lane][4 * half + 3] = cent[bg8];
                } else {
                    for (int s = 0; s < 2; s++) {
                        const uint32_t x = tl_field(vw, tl_val_field_bit(VB, mt, half, s), 2 * VB);
                        int ca, cb;
                        tl_val_pair_codes(x, VB, ca, cb);
                        f.a[lane][4 * half + 2 * s + 0] = cent[ca];
                        f.a[lane][4 * half + 2 * s + 1] = cent[cb];
                    }
                }
                f.b[lane][2 * half + 0] = pw[ta * 8 + g];
                f.b[lane][2 * half + 1] = pw[tb * 8 + g];
            }
        }
        float C[16][8] = {};
        mma_replay(f, C);
        for (int lane = 0; lane < 32; lane++) {
            const int g = lane >> 2, t = lane & 3;
            for (int j = 0; j < 2; j++) {
                out[(16 * mt + g) * 8 + 2 * t + j] = C[g][2 * t + j];
                out[(16 * mt + g + 8) * 8 + 2 * t + j] = C[g + 8][2 * t + j];
            }
        }
    }
}

}  // namespace

extern "C" {

int replay_key_tile(int D, int bits, const uint8_t* tile, const float* cent, const float* q, float* out) {
#define CASE(d, b) if (D == d && bits == b) { key_tile<d, b>(tile, cent, q, out); return 0; }
    CASE(64, 2) CASE(64, 3) CASE(64, 4) CASE(128, 2) CASE(128, 3) CASE(128, 4)
#undef CASE
    return -1;
}

int replay_value_tile(int D, int bits, const uint8_t* tile, const float* cent, const float* pw, float* out) {
#define CASE(d, b) if (D == d && bits == b) { value_tile<d, b>(tile, cent, pw, out); return 0; }
    CASE(64, 2) CASE(64, 3) CASE(64, 4) CASE(128, 2) CASE(128, 3) CASE(128, 4)
#undef CASE
    return -1;
}


int tiled_record_bytes(int D, int KB, int VB) { return tl_record_bytes(D, KB, VB); }

// Builds a record from codes with the writer-side slot functions, then replays the reader side.
int replay_tiled(int D, int KB, int VB, const uint8_t* kcodes, const uint8_t* vcodes, const float* ck,
                 const float* cv, const float* q, const float* pw, float* scores, float* outv, uint8_t* rec) {
    if (!(D == 64 || D == 128) || KB < 2 || KB > 4 || VB < 2 || VB > 4) return -1;
    tiled_build(D, KB, VB, kcodes, vcodes, rec);
    tiled_key_tile(D, KB, VB, rec, ck, q, scores);
    tiled_value_tile(D, KB, VB, rec, cv, pw, outv);
    return 0;
}

}  // extern "C"
