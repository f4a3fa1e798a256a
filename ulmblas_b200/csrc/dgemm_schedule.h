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

// Cost of the epilogue of a piece of a shared tile (the consumers' own read-modify-write of the C
// tile, about 9 us) in units of one pipeline stage of the main loop (2.1 us); only used to decide
// whether sharing the last tiles pays.
constexpr int kEpilogueStages = 4;
// The same for a piece that leaves through the CTA's tile buffer: the consumers only write the buffer and go
// on; one thread stores the head piece, or adds a later piece to C, with bulk tensor copies.
constexpr int kBufferedEpilogueStages = 2;

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

// Estimated cost, in pipeline stages, of sharing `rem` tiles of kt stages among nsu stream units.
// A unit multiplies its share of the stages and writes one partial epilogue per piece it holds;
// the pieces of a tile fold into C one after the other, so every piece of a tile beyond the first
// adds one more epilogue at the end.  With unit boundaries on tile boundaries the pieces of a tile
// all finish computing at the same moment and the whole chain is exposed: measured, such plans run
// about 15 % over this count (1024^3 in two halves per tile, 200 x 3000 x 1000 in thirds).
inline long long shared_cost(int rem, int kt, int nsu, int epi = kEpilogueStages)
{
    const long long S = (long long)rem * kt;
    const long long share = (S + nsu - 1) / nsu;
    const bool aligned = nsu % rem == 0;                       // unit boundaries fall on tile boundaries
    const long long pieces = aligned ? nsu / rem : (kt + share - 1) / share + 1;
    const long long own = aligned ? 1 : 2;                     // epilogues in a unit's own time line
    const long long cost = share + (own + (pieces - 1)) * epi;
    return aligned ? (cost * 115 + 99) / 100 : cost;
}

inline SharePlan plan_shared_tiles(long long nreal, int kt, int slots, bool force, int epi = kEpilogueStages)
{
    SharePlan none = {0, 0};
    if (slots < 2 || kt < 2) return none;
    const int rem = (int)(nreal % slots);
    if (rem == 0 || rem > kRegionMax) return none;
    const long long S = (long long)rem * kt;
    // candidates: every CTA takes part, or each tile is cut into p equal pieces (p = 2, 3, ...)
    int best = (int)(S < slots ? S : slots);
    long long best_cost = best >= 2 ? shared_cost(rem, kt, best, epi) : (1ll << 60);
    for (int p = 2; p <= 16 && (long long)rem * p <= slots && p <= kt; ++p) {
        const long long c = shared_cost(rem, kt, rem * p, epi);
        if (c < best_cost) { best_cost = c; best = rem * p; }
    }
    if (best < 2) return none;
    // one more wave of whole tiles costs kt stages and an epilogue
    const bool pays = best_cost < kt + epi;
    if (!pays && !force) return none;
    SharePlan p = {rem, best};
    return p;
}

// In-place product with a triangular operand (leaf mode 1..4 of the GEMM kernel): unit -> tile
// coordinates, the range of pipeline stages it multiplies, and its place.  The triangular operand
// spans T tiles of 128; the other dimension is cut into strips of one tile.  The tile at place d of a
// strip multiplies blocks 0..d of k (low: modes 1 and 3) or d..T-1 (high: modes 2 and 4, taken from the
// last block down), and units go out longest first: all strips of the longest place, then the next.
constexpr int kLeafBlockStages = 8;       // pipeline stages per block of 128 k
struct LeafUnit {
    int tm, tn, kc0, kc1, d, strip, T, rev, expect;
};
ULMB_SCHED_HD LeafUnit leaf_decode(int leaf, int tiles_m, int tiles_n, int unit, int kt)
{
    constexpr int HB = kLeafBlockStages;
    LeafUnit u;
    const bool left = leaf <= 2;
    const bool low = leaf == 1 || leaf == 3;
    u.T = left ? tiles_m : tiles_n;
    const int S = left ? tiles_n : tiles_m;
    const int r = unit / S;
    u.strip = unit - r * S;
    u.d = low ? u.T - 1 - r : r;
    u.tm = left ? u.d : u.strip;
    u.tn = left ? u.strip : u.d;
    if (low) { u.kc0 = 0; u.kc1 = (u.d + 1) * HB < kt ? (u.d + 1) * HB : kt; }
    else     { u.kc0 = u.d * HB < kt ? u.d * HB : kt; u.kc1 = kt; }
    u.rev = low ? 0 : 1;
    u.expect = low ? u.T - 1 - u.d : u.d;            // longer tiles of the strip: they all read block d
    return u;
}
// The block of k that stage number i (0 = first taken) of a unit belongs to, and whether it is the last
// stage of that block the unit takes.
ULMB_SCHED_HD int leaf_block_of(const LeafUnit &u, int i, bool &last_of_block)
{
    constexpr int HB = kLeafBlockStages;
    const int kc = u.kc0 + i;
    const int kk = u.rev ? u.kc0 + u.kc1 - 1 - kc : kc;
    last_of_block = u.rev ? (kk % HB == 0 || kc + 1 == u.kc1) : (kk % HB == HB - 1 || kc + 1 == u.kc1);
    return kk / HB;
}

}  // namespace ulmb200
