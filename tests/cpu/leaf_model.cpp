// CPU model of the in-place triangular leaf of the persistent DGEMM kernel
// (ulmblas_b200/csrc/dgemm_schedule.h: leaf_decode, leaf_block_of).  X <- op(T) X (or X op(T)) overwrites
// the very rows (columns) other tiles of the same strip still read, so the kernel counts, per strip and
// block of k, the tiles that have read the block, and a tile's output thread stores only when every longer
// tile of its strip has counted.  The model runs the kernel's protocol as a discrete-event simulation --
// P CTAs take units in order from a counter, each CTA multiplies one stage per tick, its output thread
// holds at most one finished tile (the consumers stall when the buffer is still occupied) -- and checks,
// for the four modes, many shapes, ragged k and CTA counts below and above the unit count, with CTAs
// that start late or run at different speeds, that
//   * every unit terminates (no wait cycle),
//   * no block of a strip is written before all tiles that read it have read it,
//   * every tile reads exactly the blocks of its triangle, every block is written exactly once,
//   * all counters are back at zero at the end.
// Prints OK.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../ulmblas_b200/csrc/dgemm_schedule.h"

using namespace ulmb200;

struct Cta {
    int unit = -1;          // unit the consumers work on, -1 = none
    int stage = 0;          // stages of it done
    int pending = -1;       // unit whose tile sits in the output buffer
    int start = 0;          // first tick at which this CTA runs
    int period = 1;         // it multiplies a stage every period ticks
    bool done = false;
};

static int run(int leaf, int T, int S, int kt, int P, unsigned seed)
{
    const bool left = leaf <= 2;
    const int tiles_m = left ? T : S, tiles_n = left ? S : T;
    const int units = T * S;
    std::vector<int> cnt((size_t)S * T, 0);
    std::vector<int> reads_done((size_t)S * T, 0);      // tiles that have read block b of strip s
    std::vector<int> readers((size_t)S * T, 0);         // tiles that must read it before it is written
    std::vector<int> written((size_t)S * T, 0);
    for (int u = 0; u < units; ++u) {
        const LeafUnit lu = leaf_decode(leaf, tiles_m, tiles_n, u, kt);
        if (lu.T != T || lu.d < 0 || lu.d >= T || lu.strip < 0 || lu.strip >= S || lu.kc0 >= lu.kc1) {
            printf("bad unit %d\n", u);
            return 1;
        }
        const int b0 = lu.kc0 / kLeafBlockStages, b1 = (lu.kc1 - 1) / kLeafBlockStages;
        const bool low = leaf == 1 || leaf == 3;
        if ((low && (b0 != 0 || b1 != lu.d)) || (!low && (b0 != lu.d || b1 != T - 1))) {
            printf("unit %d of mode %d reads blocks %d..%d, place %d of %d\n", u, leaf, b0, b1, lu.d, T);
            return 1;
        }
        for (int b = b0; b <= b1; ++b)
            if (b != lu.d) readers[(size_t)lu.strip * T + b]++;
    }
    for (int s = 0; s < S; ++s)
        for (int d = 0; d < T; ++d) {
            const LeafUnit probe = leaf_decode(leaf, tiles_m, tiles_n, ((leaf == 1 || leaf == 3) ? T - 1 - d : d) * S + s, kt);
            if (probe.d != d || probe.strip != s || probe.expect != readers[(size_t)s * T + d]) {
                printf("expect %d but %d tiles read block %d of strip %d\n", probe.expect, readers[(size_t)s * T + d], d, s);
                return 1;
            }
        }
    std::vector<Cta> cta(P);
    unsigned rng = seed * 2654435761u + 12345u;
    auto rnd = [&]() { rng = rng * 1664525u + 1013904223u; return rng >> 16; };
    for (int c = 0; c < P; ++c) {
        cta[c].start = seed ? (int)(rnd() % 40) : 0;
        cta[c].period = seed ? 1 + (int)(rnd() % 3) : 1;
    }
    const int grid = P < units ? P : units;
    int next = grid, finished = 0;
    for (int c = 0; c < P; ++c) {
        if (c < grid) cta[c].unit = c;
        else cta[c].done = true;
    }
    const long long limit = 1000000;
    for (long long tick = 0; finished < grid; ++tick) {
        if (tick > limit) {
            printf("no progress: mode %d T %d S %d kt %d P %d seed %u\n", leaf, T, S, kt, P, seed);
            return 1;
        }
        for (int c = 0; c < grid; ++c) {
            Cta &x = cta[c];
            if (x.done || tick < x.start) continue;
            // output thread: store the buffered tile once its readers are through
            if (x.pending >= 0) {
                const LeafUnit lu = leaf_decode(leaf, tiles_m, tiles_n, x.pending, kt);
                const size_t at = (size_t)lu.strip * T + lu.d;
                if (cnt[at] == lu.expect) {
                    if (reads_done[at] != readers[at]) {
                        printf("block %d of strip %d written after %d of %d reads\n", lu.d, lu.strip, reads_done[at], readers[at]);
                        return 1;
                    }
                    cnt[at] = 0;
                    written[at]++;
                    x.pending = -1;
                }
            }
            if ((tick - x.start) % x.period) continue;
            if (x.unit < 0) {
                if (x.pending < 0) { x.done = true; ++finished; }
                continue;
            }
            const LeafUnit lu = leaf_decode(leaf, tiles_m, tiles_n, x.unit, kt);
            const int len = lu.kc1 - lu.kc0;
            if (x.stage < len) {
                bool last;
                const int blk = leaf_block_of(lu, x.stage, last);
                if (written[(size_t)lu.strip * T + blk] && blk != lu.d) {
                    printf("unit %d reads block %d of strip %d after it was written\n", x.unit, blk, lu.strip);
                    return 1;
                }
                if (last && blk != lu.d) {
                    cnt[(size_t)lu.strip * T + blk]++;
                    reads_done[(size_t)lu.strip * T + blk]++;
                }
                ++x.stage;
            }
            if (x.stage == len && x.pending < 0) {
                // the finished tile goes into the buffer, the consumers take the next unit
                x.pending = x.unit;
                x.stage = 0;
                x.unit = next < units ? next++ : -1;
            }
        }
    }
    for (size_t i = 0; i < cnt.size(); ++i)
        if (cnt[i] != 0 || written[i] != 1) {
            printf("counter %zu left at %d, block written %d times\n", i, cnt[i], written[i]);
            return 1;
        }
    return 0;
}

int main()
{
    int bad = 0, cases = 0;
    const int Ts[] = {1, 2, 3, 8, 16};
    const int Ss[] = {1, 2, 5, 33, 64};
    const int Ps[] = {1, 3, 148, 1000};
    for (int leaf = 1; leaf <= 4; ++leaf)
        for (int T : Ts)
            for (int S : Ss)
                for (int ragged = 0; ragged < 2; ++ragged)
                    for (int P : Ps)
                        for (unsigned seed = 0; seed < 3; ++seed) {
                            // the last block holds 1..8 stages
                            const int kt = T * kLeafBlockStages - (ragged ? 5 : 0);
                            bad += run(leaf, T, S, kt, P, seed);
                            ++cases;
                            if (bad) return 1;
                        }
    printf("OK %d cases\n", cases);
    return 0;
}
