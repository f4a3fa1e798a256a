// CPU model of how the persistent DGEMM kernel lets the pieces of shared tiles leave through each CTA's
// single tile buffer (ulmblas_b200/csrc/dgemm_sm100.cu: announce_piece / stash_tile / the output thread;
// schedule from ulmblas_b200/csrc/dgemm_schedule.h).
//
// A CTA's consumers multiply one piece after the other; a finished piece goes into the CTA's buffer as soon as
// the buffer is free, and the consumers go on.  The CTA's output thread takes the buffered pieces in that
// order: the head of a tile is stored at once, a later piece only when the tile's flag shows that the piece
// before it in k is completely in C; then the flag moves on and the buffer is free again.  Whole tiles pass
// through the same buffer without a flag.  The model runs this as a discrete-event simulation -- units handed
// out as in the kernel (first unit = CTA index, then a shared counter), CTAs of uneven speed that start late,
// stores and additions that take a few ticks -- and checks, for many plans, that
//   * everything terminates (no CTA waits for a buffer or a flag for ever),
//   * the pieces of every tile reach C in order of k, each exactly once, the head first,
//   * no piece is added before the store or addition before it is complete,
//   * every flag is back at zero at the end.
// Prints OK.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../ulmblas_b200/csrc/dgemm_schedule.h"

using namespace ulmb200;

struct Job {              // one piece or whole tile, as the consumers announce it
    int r;                // shared tile, -1 = whole tile outside the region
    int kc0, kc1;
};

struct Cta {
    // consumers
    std::vector<Job> todo;        // pieces of the unit being worked on, in the walk's order
    size_t at = 0;                // piece of todo being multiplied
    int stage = 0;                // stages of it done
    bool waiting_for_buffer = false;
    bool no_more_units = false;
    // output thread
    bool buffer_full = false;     // a finished piece sits in the buffer
    Job held = {0, 0, 0};
    int busy = 0;                 // ticks left of the store / addition under way
    bool writing = false;
    int start = 0, period = 1;
};

static int run(long long whole, int region_tiles, int nsu, int kt, int P, int write_ticks, unsigned seed)
{
    const long long units = whole + nsu;
    const int grid = (int)(units < P ? units : P);
    std::vector<Cta> cta(grid);
    unsigned rng = seed * 2654435761u + 99u;
    auto rnd = [&]() { rng = rng * 1664525u + 1013904223u; return rng >> 16; };
    for (auto &c : cta) {
        c.start = seed ? (int)(rnd() % 50) : 0;
        c.period = seed ? 1 + (int)(rnd() % 3) : 1;
    }
    std::vector<int> flag(region_tiles, 0), applied(region_tiles, 0), in_flight(region_tiles, 0);
    long long next = grid, whole_done = 0;
    auto take = [&](Cta &c, long long unit) {
        c.todo.clear();
        c.at = 0;
        c.stage = 0;
        if (unit < whole) {
            c.todo.push_back({-1, 0, kt});
        } else {
            StreamWalk w(region_tiles, nsu, (int)(unit - whole), kt);
            Piece pc;
            while (w.next(pc)) c.todo.push_back({pc.r, pc.kc0, pc.kc1});
        }
    };
    for (int i = 0; i < grid; ++i) take(cta[i], i);
    int finished = 0;
    std::vector<char> done(grid, 0);
    const long long limit = 4000000;
    for (long long tick = 0; finished < grid; ++tick) {
        if (tick > limit) {
            printf("no progress: whole %lld region %d nsu %d kt %d P %d seed %u\n", whole, region_tiles, nsu, kt, P, seed);
            return 1;
        }
        for (int i = 0; i < grid; ++i) {
            Cta &c = cta[i];
            if (done[i] || tick < c.start) continue;
            // ---- output thread ----
            if (c.writing) {
                if (--c.busy <= 0) {
                    c.writing = false;
                    if (c.held.r >= 0) {
                        const bool partial = !(c.held.kc0 == 0 && c.held.kc1 == kt);
                        in_flight[c.held.r] = 0;
                        if (partial) flag[c.held.r] = c.held.kc1 == kt ? 0 : c.held.kc1;       // complete: publish
                    } else {
                        ++whole_done;
                    }
                    c.buffer_full = false;                                                      // buffer free again
                }
            } else if (c.buffer_full) {
                const Job &j = c.held;
                const bool partial = j.r >= 0 && !(j.kc0 == 0 && j.kc1 == kt);
                if (!partial || j.kc0 == 0 || flag[j.r] == j.kc0) {
                    if (j.r >= 0) {
                        if (in_flight[j.r]) { printf("tile %d: a piece starts while another is still being written\n", j.r); return 1; }
                        if (applied[j.r] != j.kc0) {
                            printf("tile %d: piece [%d,%d) follows %d\n", j.r, j.kc0, j.kc1, applied[j.r]);
                            return 1;
                        }
                        if (j.kc0 == 0 && partial && flag[j.r] != 0) { printf("head of tile %d finds a used flag\n", j.r); return 1; }
                        applied[j.r] = j.kc1;
                        in_flight[j.r] = 1;
                    }
                    c.writing = true;
                    c.busy = write_ticks;
                }
            }
            // ---- consumers ----
            if ((tick - c.start) % c.period) continue;
            if (c.at >= c.todo.size()) {
                if (c.no_more_units) {
                    if (!c.buffer_full && !c.writing) { done[i] = 1; ++finished; }
                    continue;
                }
                if (next < units) take(c, next++);
                else c.no_more_units = true;
                continue;
            }
            const Job &j = c.todo[c.at];
            if (c.stage < j.kc1 - j.kc0) { ++c.stage; continue; }
            // piece multiplied: into the buffer once the piece before it has left
            if (c.buffer_full) continue;
            c.held = j;
            c.buffer_full = true;
            ++c.at;
            c.stage = 0;
        }
    }
    for (int r = 0; r < region_tiles; ++r)
        if (flag[r] != 0 || applied[r] != kt) { printf("tile %d: flag %d, folded up to %d of %d\n", r, flag[r], applied[r], kt); return 1; }
    if (whole_done != whole) { printf("%lld of %lld whole tiles stored\n", whole_done, whole); return 1; }
    return 0;
}

int main()
{
    int bad = 0, cases = 0;
    const int slot_list[] = {2, 3, 7, 16, 132, 148};
    for (int slots : slot_list)
        for (int kt : {2, 3, 8, 17, 33, 64})
            for (int waves = 0; waves < 3; ++waves)
                for (int rem = 1; rem < slots && rem <= kRegionMax; rem += (slots > 16 ? 13 : 1))
                    for (int epi : {kEpilogueStages, kBufferedEpilogueStages})
                        for (unsigned seed = 0; seed < 3; ++seed) {
                            const long long nreal = (long long)waves * slots + rem;
                            const SharePlan sp = plan_shared_tiles(nreal, kt, slots, true, epi);
                            if (sp.nsu == 0) continue;
                            bad += run(nreal - sp.region_tiles, sp.region_tiles, sp.nsu, kt, slots, 1 + (int)(seed * 2), seed);
                            // fewer CTAs than units in the last wave as well: a grid the GPU has partly taken away
                            if (slots > 3) bad += run(nreal - sp.region_tiles, sp.region_tiles, sp.nsu, kt, sp.nsu, 3, seed);
                            ++cases;
                            if (bad) return 1;
                        }
    // the two shapes the path was written for
    {
        const SharePlan a = plan_shared_tiles(64, 64, 148, false, kBufferedEpilogueStages);
        const SharePlan b = plan_shared_tiles(384, 33, 148, false, kBufferedEpilogueStages);
        if (a.nsu == 0 || b.nsu == 0) { printf("1024^3 or 3001 x 2047 x 513 is not shared\n"); return 1; }
        bad += run(64 - a.region_tiles, a.region_tiles, a.nsu, 64, 148, 2, 1);
        bad += run(384 - b.region_tiles, b.region_tiles, b.nsu, 33, 148, 2, 1);
    }
    if (bad) { printf("FAILED\n"); return 1; }
    printf("OK %d plans\n", cases);
    return 0;
}
