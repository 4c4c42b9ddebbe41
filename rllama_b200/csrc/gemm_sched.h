// Work schedule of the persistent tensor-core GEMM (gemm_tc.cu): which CTA computes which k-blocks of which
// output tile, and where the partial tiles of a K-split tile lie. Plain C++ (no device intrinsics) so that a host
// program can check it: every (tile, k-block) unit is computed exactly once, whatever the shape and the grid.
#pragma once

#ifdef __CUDACC__
#define RLB_HD __host__ __device__
#else
#define RLB_HD
#endif

namespace gemm_sched {

constexpr int TM = 128;   // tokens per MMA block (a tile holds 1 or 2 of them)

struct Sched {
    int n_mt, n_nt, nkb;   // token tiles, weight-row tiles, k-blocks per tile
    int whole;             // tiles handed out whole, round-robin (a multiple of the grid size)
    int rest;              // remaining tiles, dealt out by k-block
};
RLB_HD inline Sched make_sched(int n, int M, int nkb, int grid, int TN, int tile_tokens) {
    Sched s;
    s.n_mt = (n + tile_tokens - 1) / tile_tokens; s.n_nt = (M + TN - 1) / TN; s.nkb = nkb;
    const int tiles = s.n_mt * s.n_nt;
    s.whole = tiles / grid * grid;
    s.rest = tiles - s.whole;
    return s;
}
// First k-block unit of CTA c's run over the remaining tiles (units are numbered tile-major).
RLB_HD inline long long rest_begin(const Sched& s, int c, int grid) { return (long long)c * s.rest * s.nkb / grid; }

// One piece of work: k-blocks [kb0, kb1) of a tile. `slot` < 0: the piece covers the whole K range and
// its result goes straight to the output; otherwise it is partial tile number `slot` (0 or 1) of this CTA.
struct Piece { int tile, kb0, kb1, slot; };
struct PieceIter {
    Sched s; int cta, grid;
    int t;                  // next whole tile
    long long u, u0, u1;    // position in, and bounds of, this CTA's run over the remaining tiles
    RLB_HD PieceIter(const Sched& s_, int cta_, int grid_) : s(s_), cta(cta_), grid(grid_) {
        t = cta;
        u0 = rest_begin(s, cta, grid); u1 = rest_begin(s, cta + 1, grid); u = u0;
    }
    RLB_HD bool next(Piece& p) {
        if (t < s.whole) { p.tile = t; p.kb0 = 0; p.kb1 = s.nkb; p.slot = -1; t += grid; return true; }
        if (u >= u1) return false;
        const int j = (int)(u / s.nkb);
        p.tile = s.whole + j;
        p.kb0 = (int)(u - (long long)j * s.nkb);
        const long long left = u1 - u;
        p.kb1 = (int)(p.kb0 + left < s.nkb ? p.kb0 + left : s.nkb);
        p.slot = (p.kb0 == 0 && p.kb1 == s.nkb) ? -1 : (u == u0 ? 0 : 1);
        u += p.kb1 - p.kb0;
        return true;
    }
};

// The fix-up's view: the partial tile (cta * 2 + slot) that CTA c left for remaining tile j, or -1 when c's run does
// not meet the tile. (When a single CTA's run covers the whole tile it stored the result itself: the caller sees one
// meeting CTA and has nothing to add up.)
RLB_HD inline int partial_of(const Sched& s, int grid, int j, int c) {
    const long long u_first = (long long)j * s.nkb, u_last = u_first + s.nkb;
    const long long b = rest_begin(s, c, grid), e = rest_begin(s, c + 1, grid);
    if (!(e > b && b < u_last && e > u_first)) return -1;
    return c * 2 + (b >= u_first ? 0 : 1);  // the piece starts the run, or follows a tile boundary inside it
}

}  // namespace gemm_sched
