// CPU model of the FP64 GEMM kernel's index arithmetic (no GPU needed).
//
// For every operand-layout combination it (1) places a CTA tile of A and B in
// a byte buffer exactly where TMA with the 128-byte swizzle puts it
// (elem_off), (2) has 32 simulated lanes fetch their fragments with the same
// base/immediate offsets the kernel uses (frag_base and the recipe documented
// in tile_layout.h), (3) applies the m16n8k8 FP64 MMA lane->element maps, and
// (4) scatters the accumulators through c_row/c_col.  The result must equal
// the plain product.  It also checks that each 16-byte fragment load is free
// of shared-memory bank conflicts (8 lanes of a quarter-warp hit 8 distinct
// 16-byte bank groups).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <vector>
#include <set>
#include "../../ulmblas_b200/csrc/tile_layout.h"

using namespace ulmb200;

static int g_fail = 0;

static void ld128(const std::vector<unsigned char> &s, uint32_t off, double &x, double &y)
{
    if (off % 16 != 0 || off + 16 > s.size()) { printf("bad fragment address %u\n", off); g_fail++; x = y = 0; return; }
    memcpy(&x, &s[off], 8);
    memcpy(&y, &s[off + 8], 8);
}

static void check_conflicts(const uint32_t (&addr)[32], const char *what)
{
    for (int q = 0; q < 4; ++q) {
        std::set<uint32_t> banks;
        for (int l = 8 * q; l < 8 * q + 8; ++l) banks.insert((addr[l] >> 4) & 7);
        if (banks.size() != 8) { printf("bank conflict in %s (quarter %d)\n", what, q); g_fail++; }
    }
}

template <int MAJOR_A, int MAJOR_B>
static void run(int BM, int BN, int WM, int WN)
{
    const int MT = WM / 16, NT = WN / 8;
    std::vector<double> A(BM * kBK), B(kBK * BN), Cref(BM * BN, 0.0), C(BM * BN, 0.0);
    for (auto &v : A) v = (rand() % 2001 - 1000) / 1000.0;
    for (auto &v : B) v = (rand() % 2001 - 1000) / 1000.0;
    for (int i = 0; i < BM; ++i)
        for (int j = 0; j < BN; ++j)
            for (int k = 0; k < kBK; ++k) Cref[i + j * BM] += A[i + k * BM] * B[k + j * kBK];

    std::vector<unsigned char> sA(BM * 128), sB(BN * 128);
    for (int r = 0; r < BM; ++r)
        for (int k = 0; k < kBK; ++k) memcpy(&sA[elem_off<MAJOR_A>(r, k)], &A[r + k * BM], 8);
    for (int r = 0; r < BN; ++r)
        for (int k = 0; k < kBK; ++k) memcpy(&sB[elem_off<MAJOR_B>(r, k)], &B[k + r * kBK], 8);

    for (int wm0 = 0; wm0 < BM; wm0 += WM)
        for (int wn0 = 0; wn0 < BN; wn0 += WN) {
            std::vector<double> acc(32 * MT * NT * 4, 0.0);
            auto ACC = [&](int lane, int i, int j, int r) -> double & { return acc[((lane * MT + i) * NT + j) * 4 + r]; };
            for (int h = 0; h < 2; ++h) {
                // fragments of all lanes
                std::vector<double> a(32 * MT * 4), b(32 * NT * 2);
                for (int i = 0; i < MT; ++i) {
                    uint32_t ad0[32], ad1[32];
                    for (int lane = 0; lane < 32; ++lane) {
                        uint32_t ba[2];
                        frag_base<MAJOR_A>(wm0, lane, ba);
                        double *al = &a[(lane * MT + i) * 4];
                        if (MAJOR_A == K_MAJOR) {
                            ad0[lane] = ba[h] + i * 2048; ad1[lane] = ba[h] + i * 2048 + 1024;
                            ld128(sA, ad0[lane], al[0], al[2]);
                            ld128(sA, ad1[lane], al[1], al[3]);
                        } else {
                            ad0[lane] = ba[0] + i * 2048 + h * 1024; ad1[lane] = ba[1] + i * 2048 + h * 1024;
                            ld128(sA, ad0[lane], al[0], al[1]);
                            ld128(sA, ad1[lane], al[2], al[3]);
                        }
                    }
                    check_conflicts(ad0, "A load 0");
                    check_conflicts(ad1, "A load 1");
                }
                if (MAJOR_B == K_MAJOR) {
                    for (int j = 0; j < NT; ++j) {
                        uint32_t ad[32];
                        for (int lane = 0; lane < 32; ++lane) {
                            uint32_t bb[2];
                            frag_base<MAJOR_B>(wn0, lane, bb);
                            ad[lane] = bb[h] + j * 1024;
                            ld128(sB, ad[lane], b[(lane * NT + j) * 2], b[(lane * NT + j) * 2 + 1]);
                        }
                        check_conflicts(ad, "B load");
                    }
                } else {
                    for (int jj = 0; jj < NT / 2; ++jj) {
                        uint32_t ad0[32], ad1[32];
                        for (int lane = 0; lane < 32; ++lane) {
                            uint32_t bb[2];
                            frag_base<MAJOR_B>(wn0, lane, bb);
                            ad0[lane] = bb[0] + jj * 2048 + h * 1024; ad1[lane] = bb[1] + jj * 2048 + h * 1024;
                            ld128(sB, ad0[lane], b[(lane * NT + 2 * jj) * 2], b[(lane * NT + 2 * jj + 1) * 2]);
                            ld128(sB, ad1[lane], b[(lane * NT + 2 * jj) * 2 + 1], b[(lane * NT + 2 * jj + 1) * 2 + 1]);
                        }
                        check_conflicts(ad0, "B load 0");
                        check_conflicts(ad1, "B load 1");
                    }
                }
                // the tensor-core instruction: D(16x8) += A(16x8) * B(8x8) with the documented lane maps
                for (int i = 0; i < MT; ++i)
                    for (int j = 0; j < NT; ++j) {
                        double Am[16][8], Bm[8][8];
                        for (int lane = 0; lane < 32; ++lane) {
                            const int g = lane >> 2, t = lane & 3;
                            const double *al = &a[(lane * MT + i) * 4];
                            Am[g][t] = al[0]; Am[g + 8][t] = al[1]; Am[g][t + 4] = al[2]; Am[g + 8][t + 4] = al[3];
                            Bm[t][g] = b[(lane * NT + j) * 2]; Bm[t + 4][g] = b[(lane * NT + j) * 2 + 1];
                        }
                        for (int lane = 0; lane < 32; ++lane) {
                            const int g = lane >> 2, t = lane & 3;
                            for (int r = 0; r < 4; ++r) {
                                const int row = g + 8 * (r >> 1), col = 2 * t + (r & 1);
                                double s = 0;
                                for (int k = 0; k < 8; ++k) s += Am[row][k] * Bm[k][col];
                                ACC(lane, i, j, r) += s;
                            }
                        }
                    }
            }
            for (int lane = 0; lane < 32; ++lane)
                for (int i = 0; i < MT; ++i)
                    for (int j = 0; j < NT; ++j)
                        for (int r = 0; r < 4; ++r) {
                            const int row = c_row<MAJOR_A>(wm0 + 16 * i, lane, r >> 1);
                            const int col = c_col<MAJOR_B>(wn0 + 8 * j, lane, r & 1);
                            if (row < 0 || row >= BM || col < 0 || col >= BN) { g_fail++; continue; }
                            C[row + col * BM] += ACC(lane, i, j, r);
                        }
        }
    double worst = 0;
    for (int e = 0; e < BM * BN; ++e) worst = fmax(worst, fabs(C[e] - Cref[e]));
    printf("majorA=%d majorB=%d tile %dx%d warp %dx%d: max |C-Cref| = %.3e\n", MAJOR_A, MAJOR_B, BM, BN, WM, WN, worst);
    if (!(worst < 1e-12)) g_fail++;
}

int main()
{
    srand(1);
    // k permutation must cover 0..15 exactly once per stage
    bool seen[16] = {};
    for (int h = 0; h < 2; ++h)
        for (int s = 0; s < 8; ++s) seen[k_of_slot(h, s)] = true;
    for (bool b : seen) if (!b) { printf("k_of_slot is not a permutation\n"); g_fail++; }
    run<MN_MAJOR, K_MAJOR>(128, 128, 64, 32);
    run<MN_MAJOR, MN_MAJOR>(128, 128, 64, 32);
    run<K_MAJOR, K_MAJOR>(128, 128, 64, 32);
    run<K_MAJOR, MN_MAJOR>(128, 128, 64, 32);
    run<MN_MAJOR, K_MAJOR>(64, 64, 32, 32);
    run<MN_MAJOR, MN_MAJOR>(64, 64, 32, 32);
    run<K_MAJOR, K_MAJOR>(64, 64, 32, 32);
    run<K_MAJOR, MN_MAJOR>(64, 64, 32, 32);
    printf(g_fail ? "FAIL (%d)\n" : "OK\n", g_fail);
    return g_fail ? 1 : 0;
}
