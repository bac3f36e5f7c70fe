// Tile geometry of the fused forward kernels: which queries a work item holds, the key box of
// their neighbourhoods and how many chunks it takes; per-row windows inside that box.
#pragma once
#include "tc_plan.cuh"

namespace natten {
namespace fwdgeom {

using namespace tc;
using namespace tcplan;

// Geometry of one work item (a tile of 128 queries of one (batch, head)).
struct FwdTile {
    int b, h, hk;
    int rg[3], origin[3], Lp[3], lo[3], nc[3], x0[3], sx[3], nq[3], nqf[3];
    int nnb, nch;          // nch == 0 in a published header: no more tiles
    int active;
};

// Walks the work items of a lane (w0, w0 + step, ...) without divisions: tile index inside the
// (batch, head), head and batch are advanced incrementally.
struct Cursor {
    unsigned w, bx, dq, dr;
    int h, b;
    __device__ __forceinline__ void init(const TcParams& P, unsigned w0, unsigned step)
    {
        w = w0;
        const unsigned hb = w0 / P.per_head;
        bx = w0 - hb * P.per_head;
        b = (int)(hb / (unsigned)P.Hq);
        h = (int)(hb - (unsigned)b * (unsigned)P.Hq);
        dq = step / P.per_head;
        dr = step - dq * P.per_head;
    }
    __device__ __forceinline__ void advance(const TcParams& P, unsigned step)
    {
        w += step;
        bx += dr;
        int dh = (int)dq;
        if (bx >= P.per_head) { bx -= P.per_head; ++dh; }
        h += dh;
        while (h >= P.Hq) { h -= P.Hq; ++b; }
    }
};

// Geometry of the cursor's work item (tile bx of (batch, head)); the same for every role of a lane.
// origin[] counts queries of the dilation group; query i of an axis sits at sub-grid index
// x0 + sx * i (every index when the output stride is 1).
__device__ __forceinline__ void fwd_tile(const TcParams& P, const Cursor& cur, int chunk_log, FwdTile& T)
{
    const unsigned bx = cur.bx;
    T.b = cur.b;
    T.h = cur.h;
    T.hk = (int)fast_div((unsigned)cur.h, P.group_mul);
    bool active = cta_geometry(P, bx, T.b, T.rg, T.origin, T.Lp);
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        T.sx[a] = P.qstep[a];
        T.x0[a] = P.qx0[a][T.rg[a]];
        const int lpf = (int)fast_div((unsigned)(P.L[a] - T.rg[a] + P.dil[a] - 1), P.dil_mul[a]);   // sub-grid length of the whole tensor
        if (T.x0[a] < 0) {                       // no output position falls into this dilation group
            T.nq[a] = 0; T.nqf[a] = 0; T.x0[a] = 0;
        } else if (T.sx[a] == 1) {
            T.nq[a] = T.Lp[a];
            T.nqf[a] = T.rg[a] < P.L[a] ? lpf : 0;
        } else {
            T.nq[a] = T.x0[a] < T.Lp[a] ? (T.Lp[a] - T.x0[a] + T.sx[a] - 1) / T.sx[a] : 0;
            T.nqf[a] = T.x0[a] < lpf ? (lpf - T.x0[a] + T.sx[a] - 1) / T.sx[a] : 0;
        }
        if (T.origin[a] >= T.nq[a]) active = false;
    }
    T.nnb = 1;
    if (active) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int lastq = T.origin[a] + P.tile[a] - 1 < T.nq[a] - 1 ? T.origin[a] + P.tile[a] - 1 : T.nq[a] - 1;
            const int xf = T.x0[a] + T.sx[a] * T.origin[a], xl = T.x0[a] + T.sx[a] * lastq;
            T.lo[a] = P.causal[a] ? xf - (P.K[a] - 1) : window_start(xf, T.Lp[a], P.K[a], 1);
            const int hi = P.causal[a] ? xl : window_start(xl, T.Lp[a], P.K[a], 1) + P.K[a] - 1;
            T.nc[a] = chunks_along(P, a, hi - T.lo[a] + 1);       // chunks this tile really needs
            T.nnb *= T.nc[a];
        }
    }
    T.nch = T.nnb + ((P.n_extra + (1 << chunk_log) - 1) >> chunk_log);   // then the additional tokens, one chunk at a time
    T.active = active ? 1 : 0;
}

// Output row of tile row `row`, whether it is a query of the sample / a row of the tensor, and (active
// tiles) its window as a box-relative range [f, e) per axis.
__device__ __forceinline__ long long row_geometry(const TcParams& P, const FwdTile& T, int row, int (&f)[3], int (&e)[3],
                                                  bool& valid_q, bool& in_tensor)
{
    int qi[3];
    row_offsets(P, row, qi);
    valid_q = true;
    in_tensor = true;
    long long oflat = 0;
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const int qa = T.origin[a] + qi[a];               // query count along the axis
        const int xq = T.x0[a] + T.sx[a] * qa;            // its sub-grid index
        const int pa = T.rg[a] + P.dil[a] * xq;           // its position in the tensor
        if (qa >= T.nq[a]) valid_q = false;
        if (qa >= T.nqf[a]) in_tensor = false;
        oflat = oflat * P.O[a] + (P.st[a] == 1 ? pa : pa / P.st[a]);
        f[a] = 0;
        e[a] = 0;
        if (T.active) {
            const int first = P.causal[a] ? xq - (P.K[a] - 1) : window_start(xq, T.Lp[a], P.K[a], 1);
            f[a] = (first > 0 ? first : 0) - T.lo[a];
            e[a] = (first + P.K[a] < T.Lp[a] ? first + P.K[a] : T.Lp[a]) - T.lo[a];
        }
    }
    if (!valid_q) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
    return ((long long)T.b * P.otot + oflat) * P.Hq + T.h;
}

} // namespace fwdgeom
} // namespace natten
