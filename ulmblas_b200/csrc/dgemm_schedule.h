// Work schedule of the persistent FP64 GEMM kernel, as plain integer functions usable from
// host and device code (the host copy also feeds a CPU model in the tests).
//
// A launch has `units` work units.  Unit u < split_first is tile u with all of its K.  The
// other units are "stream units": the region_tiles tiles that do work among the tile ids
// >= split_first are laid end to end, stage by stage (kt pipeline stages each), and stream
// unit j of nsu takes the j-th equal share [S*j/nsu, S*(j+1)/nsu) of those S = region_tiles*kt
// stages.  A share is walked from the top down, so a unit starts with the head [0, x) of the
// last tile it touches and ends with the tail [y, kt) of the first one.
//
// A tile whose stages are spread over several units is folded into C in order of k: the
// piece [0, x) applies beta and publishes x in the tile's flag; the piece starting at x waits
// for that value, adds its share, and publishes its own end; the piece ending at kt puts the
// flag back to zero.  The piece a unit may have to wait for always belongs to a unit with a
// lower index, and that unit works on it first -- units are picked up in increasing order, so
// the wait is for work that is already under way.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ULMB_SCHED_HD __host__ __device__ __forceinline__
#else
#define ULMB_SCHED_HD inline
#endif

namespace ulmb200 {

constexpr int kRegionMax = 160;           // most tiles the shared region of a launch may hold

// Cost of one epilogue (read-modify-write of a C tile) in units of one pipeline stage of the
// main loop; only used to decide whether sharing the last tiles pays.
constexpr int kEpilogueStages = 3;

struct Piece {
    int r;          // index of the tile within the region
    int kc0, kc1;   // pipeline stages [kc0, kc1) of that tile
};

struct StreamWalk {
    long long lo, f;
    int kt;
    ULMB_SCHED_HD StreamWalk(int region_tiles, int nsu, int j, int kt_) : kt(kt_)
    {
        const long long S = (long long)region_tiles * kt_;
        lo = S * j / nsu;
        f = S * (j + 1) / nsu;
    }
    ULMB_SCHED_HD bool next(Piece &pc)
    {
        if (f <= lo) return false;
        const int r = (int)((f - 1) / kt);
        const long long base = (long long)r * kt;
        pc.r = r;
        pc.kc1 = (int)(f - base);
        pc.kc0 = lo > base ? (int)(lo - base) : 0;
        f = base + pc.kc0;
        return true;
    }
};

// How many of the `nreal` working tiles form the shared region and how many stream units deal
// with them, for a grid of `slots` CTAs; {0, 0} when sharing does not pay.  force: share
// whenever possible (test hook).
struct SharePlan {
    int region_tiles, nsu;
};

inline SharePlan plan_shared_tiles(long long nreal, int kt, int slots, bool force)
{
    SharePlan none = {0, 0};
    if (slots < 2 || kt < 1) return none;
    const int rem = (int)(nreal % slots);
    if (rem == 0 || rem > kRegionMax) return none;
    const long long S = (long long)rem * kt;
    const int nsu = (int)(S < slots ? S : slots);
    if (nsu < 2) return none;
    const long long share = (S + nsu - 1) / nsu;
    // one more wave of whole tiles costs kt stages and an epilogue; sharing costs a share of the
    // stages and, for most CTAs, two partial epilogues and a short wait
    const bool pays = share + 2 * kEpilogueStages + 1 < kt + kEpilogueStages;
    if (!pays && !force) return none;
    SharePlan p = {rem, nsu};
    return p;
}

}  // namespace ulmb200
