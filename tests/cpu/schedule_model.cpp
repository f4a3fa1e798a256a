// CPU model of the persistent DGEMM kernel's work schedule (ulmblas_b200/csrc/dgemm_schedule.h):
// for many (working tiles, stages per tile, CTAs) it checks that
//   * the stream units cover every pipeline stage of every shared tile exactly once,
//   * the pieces of a shared tile fold into C in order of k when the units run one after the
//     other in increasing order (so a unit only ever waits for a unit picked up before it, and
//     within that unit for its first pieces),
//   * every fold flag is back at zero when the launch ends (a CTA's output thread folds its pieces in
//     the order its consumers multiplied them, so the same order holds for pieces that leave through
//     the tile buffer), and
//   * no unit's share is more than one stage longer than any other's.
// Prints OK.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../ulmblas_b200/csrc/dgemm_schedule.h"

using namespace ulmb200;

static int check(long long nreal, int kt, int slots, bool force, int epi = kEpilogueStages)
{
    const SharePlan sp = plan_shared_tiles(nreal, kt, slots, force, epi);
    if (sp.nsu == 0) return 0;
    if (sp.region_tiles != nreal % slots || sp.region_tiles > kRegionMax || sp.nsu > slots || sp.nsu < 2) {
        printf("bad plan: nreal %lld kt %d slots %d -> region %d nsu %d\n", nreal, kt, slots, sp.region_tiles, sp.nsu);
        return 1;
    }
    std::vector<int> covered((size_t)sp.region_tiles * kt, 0);
    std::vector<int> flag(sp.region_tiles, 0);
    long long shortest = 1ll << 60, longest = 0;
    for (int j = 0; j < sp.nsu; ++j) {
        StreamWalk w(sp.region_tiles, sp.nsu, j, kt);
        Piece pc;
        long long mine = 0;
        int last_r = 1 << 30;
        while (w.next(pc)) {
            if (pc.r < 0 || pc.r >= sp.region_tiles || pc.kc0 < 0 || pc.kc1 > kt || pc.kc0 >= pc.kc1 || pc.r >= last_r) {
                printf("bad piece: unit %d tile %d [%d,%d)\n", j, pc.r, pc.kc0, pc.kc1);
                return 1;
            }
            last_r = pc.r;
            for (int kc = pc.kc0; kc < pc.kc1; ++kc) covered[(size_t)pc.r * kt + kc]++;
            mine += pc.kc1 - pc.kc0;
            if (pc.kc0 == 0 && pc.kc1 == kt) continue;            // whole tile: no folding
            if (pc.kc0 > 0 && flag[pc.r] != pc.kc0) {
                printf("unit %d would wait for a later unit: tile %d [%d,%d) flag %d (nreal %lld kt %d slots %d)\n", j,
                       pc.r, pc.kc0, pc.kc1, flag[pc.r], nreal, kt, slots);
                return 1;
            }
            if (pc.kc0 == 0 && flag[pc.r] != 0) { printf("head piece finds a used flag\n"); return 1; }
            flag[pc.r] = pc.kc1 == kt ? 0 : pc.kc1;
        }
        if (mine < shortest) shortest = mine;
        if (mine > longest) longest = mine;
    }
    for (size_t i = 0; i < covered.size(); ++i)
        if (covered[i] != 1) { printf("stage %zu covered %d times\n", i, covered[i]); return 1; }
    for (int f : flag)
        if (f != 0) { printf("a fold flag is left at %d\n", f); return 1; }
    if (longest - shortest > 1) { printf("uneven shares: %lld .. %lld\n", shortest, longest); return 1; }
    return 0;
}

int main()
{
    int bad = 0;
    long long plans = 0;
    const int slot_list[] = {2, 3, 7, 16, 100, 132, 140, 147, 148};
    for (int slots : slot_list)
        for (int kt : {1, 2, 3, 8, 16, 17, 33, 64, 256, 1024})
            for (long long nreal = 1; nreal <= 3 * slots + 5; ++nreal)
                for (int force = 0; force < 2; ++force)
                    for (int epi : {kEpilogueStages, kBufferedEpilogueStages, 1}) {      // the planner's two cost settings, and a lower one
                        bad += check(nreal, kt, slots, force != 0, epi);
                        ++plans;
                    }
    // the shapes the schedule was written for
    bad += check(64, 64, 148, false);        // 1024^3
    bad += check(384, 33, 148, false);       // 3001 x 2047 x 513
    bad += check(384, 33, 148, false, kBufferedEpilogueStages);
    bad += check(64, 64, 148, false, kBufferedEpilogueStages);
    bad += check(2080, 256, 148, false);     // triangle of order 8192, k = 4096
    bad += check(262144, 1024, 148, false);  // 65536 x 65536 x 16384
    if (plan_shared_tiles(64, 64, 148, false).nsu != 128) { printf("1024^3 is not cut into halves\n"); ++bad; }
    if (plan_shared_tiles(148, 64, 148, false).nsu != 0) { printf("a full wave is shared\n"); ++bad; }
    if (plan_shared_tiles(100, 4, 148, false).nsu != 0) { printf("a short inner dimension is shared\n"); ++bad; }
    if (plan_shared_tiles(4, 16, 148, false).nsu > 16) { printf("256^3 is cut into tiny pieces\n"); ++bad; }
    if (bad) { printf("FAILED (%d)\n", bad); return 1; }
    printf("%lld plans checked\nOK\n", plans);
    return 0;
}
