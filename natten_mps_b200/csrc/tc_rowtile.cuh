// Row tiles of the persistent tensor-core kernels (fused backward, both sides; double-buffered fused forward):
// geometry of one work item (128 rows of one (batch, head) and the box of columns their windows or inverse
// windows cover) and the tables a helper warp publishes one tile ahead.
#pragma once
#include "tc_plan.cuh"

namespace natten {
namespace rowtile {

using namespace tc;
using namespace tcplan;

constexpr int kCols = 64;                   // columns per chunk
constexpr int kAxisEntries = 130;           // entries of a tile's axis table: tile[0] + tile[1] + tile[2] <= 128 + 1 + 1

__device__ __forceinline__ int ws1(int p, int L, int K) { return window_start(p, L, K, 1); }

// Geometry of one work item: a tile of 128 rows (queries | keys) of one (batch, head).
struct BwdTile {
    int b, hy;                 // batch; head of the row tensors (query head | kv head)
    int rg[3], origin[3], Lp[3], boxlo[3], nc[3];
    int nchunks;               // chunks of the column box
    int nbox, total;           // column passes: box chunks x query heads of the group, then additional tokens
    bool active;
};

// What a compute thread needs to know about its row of a tile is separable: along every axis the row's
// coordinate alone decides its position in the tensor, whether it exists, and its valid column range.  The
// helper warp writes one entry per (axis, coordinate of the tile) one tile ahead, tile[0] + tile[1] + tile[2]
// entries instead of 128 rows x 3 axes; a compute thread combines the three entries of its row.
struct __align__(16) AxisEntry {
    short f, e;                // valid column range along the axis, relative to the column box
    int pa;                    // position along the axis in the tensor
    int flags;                 // bit 0: inside the (sub-grid of the) sample, bit 1: inside the tensor
    int pad;
};
static_assert(sizeof(AxisEntry) == 16, "axis table entries are 16 bytes");
struct TileHead {
    int active, total, nbox, nc[3];
    int nchunks, boxlo[3], Lp[3];      // for the MMA warps: chunks of the column box, its origin, sub-grid extents
    int b, hy;                         // batch and head of the rows
    short rg0, rg1, rg2, origin0, origin1, origin2;   // dilation residues and origin of the row tile (for its store)
};
static_assert(sizeof(TileHead) <= 96, "the tile head has 96 bytes behind the axis table");

template <bool kKeySide>
__device__ __forceinline__ void bwd_tile_setup(const TcParams& P, unsigned work, BwdTile& T)
{
    const unsigned hb = work / P.per_head;
    const unsigned bx = work - hb * P.per_head;
    const unsigned H = (unsigned)(kKeySide ? P.Hkv : P.Hq);
    T.b = (int)(hb / H);
    T.hy = (int)(hb - (unsigned)T.b * H);
    T.active = cta_geometry(P, bx, T.b, T.rg, T.origin, T.Lp);
    T.nchunks = 1;
    if (T.active) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int last = T.origin[a] + P.tile[a] - 1 < T.Lp[a] - 1 ? T.origin[a] + P.tile[a] - 1 : T.Lp[a] - 1;
            int hi;
            if (kKeySide) {
                int t;
                inverse_range(T.origin[a], T.Lp[a], P.K[a], P.causal[a], T.boxlo[a], t, /*exact=*/false);
                inverse_range(last, T.Lp[a], P.K[a], P.causal[a], t, hi, /*exact=*/false);
            } else {
                T.boxlo[a] = P.causal[a] ? T.origin[a] - (P.K[a] - 1) : ws1(T.origin[a], T.Lp[a], P.K[a]);
                hi = P.causal[a] ? last : ws1(last, T.Lp[a], P.K[a]) + P.K[a] - 1;
            }
            T.nc[a] = chunks_along(P, a, hi - T.boxlo[a] + 1);
            T.nchunks *= T.nc[a];
        }
    }
    T.nbox = T.nchunks * (kKeySide ? P.group : 1);
    T.total = T.nbox + (kKeySide ? 0 : ((P.n_extra + kCols - 1) >> 6));
}

} // namespace rowtile
} // namespace natten
