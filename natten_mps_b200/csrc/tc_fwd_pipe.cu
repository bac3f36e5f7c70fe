// Fused neighbourhood-attention forward for head dim 64 on tcgen05 tensor cores (sm_100a):
// one persistent CTA per SM that keeps TWO query tiles in flight.
//
// A tile is a box of 128 queries of one (batch, head); the union of their neighbourhoods is a
// box of keys walked in chunks of 128 keys (the additional tokens follow as extra chunks):
//   S = Q K^T                    tcgen05.mma, Q / K tiles staged by TMA (128-byte swizzle), S in TMEM
//   P = exp2(S*scale*log2e - m)  one thread per query row reads its S row from TMEM in 32-column
//                                pieces (pieces that are empty for a whole warp are skipped), applies
//                                the window mask and writes P (16-bit) back to TMEM
//   O += P V                     tcgen05.mma with A = P from TMEM, V tile read MN-major, O in TMEM
// The CTA runs two independent "lanes", each with its own softmax warp group (128 threads), MMA
// issuing thread, TMA loading thread, Q tile, three-stage K/V ring and 256 TMEM columns; lane g
// takes the work items 2*blockIdx.x + g, + 2*gridDim.x, ...  While one lane's threads do their
// softmax arithmetic the other lane's matrix products run, and the loading threads run ahead of
// both across tile boundaries, so neither the products nor the loads sit on the threads' critical
// path.  A row's stabiliser m is fixed at the first valid columns it meets and only moves (O and
// the row sum are then rescaled in place and the chunk is redone) if a later score exceeds it by
// 2^60 (2^14 for fp16): the probabilities are floating point, so any stabiliser within that
// range loses nothing, and there is no per-chunk maximum pass.
//
// TMEM columns of lane g (base 256*g):  S [0,128)  P [128,192)  O [192,256).
// Shared memory: 2 x (Q 16 KB + 3 x (K 16 KB + V 16 KB)) = 224 KB + barriers.
#include "tc_kernels.cuh"

#include "tc_plan.cuh"

#include <type_traits>

namespace natten {

using namespace tc;
using namespace tcplan;

// Optional clock stamps of one CTA's pipeline events (development builds only: -DNATTEN_TRACE).
#ifdef NATTEN_TRACE
__device__ long long g_trace[16 * 512];
#define STAMP(id)                                                                                   \
    do {                                                                                            \
        if (blockIdx.x == 7 && lane == 0 && tn < 255) {                                             \
            g_trace[warp * 512 + 2 * tn] = (id);                                                    \
            g_trace[warp * 512 + 2 * tn + 1] = clock64();                                           \
            ++tn;                                                                                   \
        }                                                                                           \
    } while (0)
#else
#define STAMP(id) do { } while (0)
#endif

namespace {

constexpr int DH = 64;
constexpr int kStages = 3;
constexpr int kThreads = 384;               // 2 x 4 softmax warps, 2 issuing warps, 2 loading warps
constexpr int kTile = kTileRows * 128;      // bytes of one [128 x 64] 16-bit tile
constexpr int kLaneBytes = kTile * (1 + 2 * kStages);
constexpr int kOffQ = 0, kOffK = kTile, kOffV = kTile * (1 + kStages);
constexpr int kBar = 2 * kLaneBytes;
constexpr int kLaneBars = 128;              // bytes of barriers per lane
constexpr int kHdrSlots = 4;                // tile headers published by the loading warp, per lane
constexpr int kHdrBytes = 144;
constexpr int kHdr = kBar + 2 * kLaneBars + 64;
constexpr int kSmemTotal = kHdr + 2 * kHdrSlots * kHdrBytes;
static_assert(kSmemTotal <= 232448, "shared memory budget");
constexpr uint32_t kColS = 0, kColP = 128, kColO = 192, kLaneCols = 256, kTmemCols = 512;

// Geometry of one work item.  The loading warp works it out once per tile and publishes it in
// shared memory; the issuing thread and the softmax threads read it from there.
struct FwdTile {
    int b, h, hk;
    int rg[3], origin[3], Lp[3], lo[3], nc[3], x0[3], sx[3], nq[3], nqf[3];
    int nnb, nch;          // nch == 0 in a published header: no more tiles
    int active;
};
static_assert(sizeof(FwdTile) <= kHdrBytes, "header slot too small");

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
__device__ __forceinline__ void fwd_tile(const TcParams& P, const Cursor& cur, FwdTile& T)
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
    T.nch = T.nnb + ((P.n_extra + kChunk - 1) >> 7);   // then the additional tokens, 128 per chunk
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

// kInner: innermost chunk extent when it is 16 or 32 (separable row / column masks),
// 0 = any geometry (per-column validity words from piece_word).
template <bool BF16, int kInner>
__global__ void __launch_bounds__(kThreads, 1)
tc_fwd_pipe_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmEK,
                   const __grid_constant__ CUtensorMap tmEV, const __grid_constant__ TcParams P,
                   uint16_t* __restrict__ out, float* __restrict__ lse)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef NATTEN_TRACE
    int tn = 0;
#endif
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);
    // role and lane of this warp
    const int g = warp < 8 ? (warp >> 2) : (warp & 1);
    const bool is_softmax = warp < 8, is_issuer = warp == 8 || warp == 9, is_loader = warp >= 10;

    const uint32_t sbase = smem_u32(smem);
    const uint32_t lbase = sbase + g * kLaneBytes;
    uint8_t* lsmem = smem + g * kLaneBytes;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBar + 2 * kLaneBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kBar + 2 * kLaneBars + 8);
    const uint32_t bars = sbase + kBar + g * kLaneBars;
    const uint32_t bar_q = bars + 0;            // Q tile landed
    const uint32_t bar_qfree = bars + 8;        // last Q K^T of the tile finished: Q may be overwritten
    const uint32_t bar_kv = bars + 16;          // [3] K, V chunk landed
    const uint32_t bar_kvfree = bars + 40;      // [3] P V of the chunk finished: stage may be overwritten
    const uint32_t bar_s = bars + 64;           // S of the chunk is in TMEM
    const uint32_t bar_p = bars + 72;           // every thread consumed S and stored P
    const uint32_t bar_o = bars + 80;           // P V of the chunk finished
    const uint32_t bar_hdr = bars + 88;         // [4] header of the lane's t-th tile published
    FwdTile* hdr_ring = reinterpret_cast<FwdTile*>(smem + kHdr + g * kHdrSlots * kHdrBytes);
    auto hdr_slot = [&](unsigned t) { return reinterpret_cast<FwdTile*>(reinterpret_cast<uint8_t*>(hdr_ring) + (t % kHdrSlots) * kHdrBytes); };

    if (warp == 8) {
        if (lane == 0) {
            // swizzled tiles need a 1024-byte aligned base; once any CTA has given up, the rest bail out
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            for (int gg = 0; gg < 2; ++gg) {
                const uint32_t bb = sbase + kBar + gg * kLaneBars;
                mbar_init(bb + 0, 1);
                mbar_init(bb + 8, 1);
                for (int s = 0; s < kStages; ++s) { mbar_init(bb + 16 + 8 * s, 1); mbar_init(bb + 40 + 8 * s, 1); }
                mbar_init(bb + 64, 1);
                mbar_init(bb + 72, 128);
                mbar_init(bb + 80, 1);
                for (int i = 0; i < kHdrSlots; ++i) mbar_init(bb + 88 + 8 * i, 1);
            }
            mbar_init_fence();
            fence_async_smem();
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot + g * kLaneCols;
    const unsigned nwork = P.work_q;
    const unsigned w0 = 2u * blockIdx.x + (unsigned)g, wstep = 2u * gridDim.x;

    if (is_loader) {
        // =====================================================================
        // Loading warp of this lane: walks the lane's work items, works out each tile's geometry and
        // publishes it, issues the TMA loads (lane 0) as far ahead as the rings allow, and writes the
        // zero rows of tiles that have nothing to attend to (whole warp), so that the other roles
        // only ever see tiles with work.
        // =====================================================================
        if (!*abort_flag) {
            unsigned tiles = 0, loaded = 0;
            bool ok = true;
            FwdTile T;
            Cursor cur;
            for (cur.init(P, w0, wstep); cur.w < nwork && ok; cur.advance(P, wstep)) {
                fwd_tile(P, cur, T);
                if (!T.active) {                 // rows that exist in the output are zero
#pragma unroll 1
                    for (int r = lane; r < kTileRows; r += 32) {
                        int f[3], e[3];
                        bool valid_q, in_tensor;
                        const long long out_row = row_geometry(P, T, r, f, e, valid_q, in_tensor);
                        if (in_tensor) {
                            uint4* o4 = reinterpret_cast<uint4*>(out + out_row * DH);
#pragma unroll
                            for (int i = 0; i < DH / 8; ++i) o4[i] = make_uint4(0, 0, 0, 0);
                            lse[out_row] = 0.f;
                        }
                    }
                    continue;
                }
                STAMP(100);
                if (tiles > 0) ok = mbar_wait(bar_qfree, (tiles - 1) & 1, abort_flag, P.wait_budget);
                if (!ok) break;
                STAMP(101);
                if (lane == 0) {
                    *hdr_slot(tiles) = T;
                    mbar_arrive(bar_hdr + 8 * (tiles % kHdrSlots));
                    mbar_expect_tx(bar_q, kTile + ((P.inject == 1 && tiles == 0) ? 16u : 0u));
                    tma_load_5d(lbase + kOffQ, &tmQ, bar_q, T.h * DH,
                                T.rg[2] + P.dil[2] * (T.x0[2] + T.sx[2] * T.origin[2]),
                                T.rg[1] + P.dil[1] * (T.x0[1] + T.sx[1] * T.origin[1]),
                                T.rg[0] + P.dil[0] * (T.x0[0] + T.sx[0] * T.origin[0]), T.b);
                }
                ++tiles;
                int ld[3] = {0, 0, 0};
                for (int c = 0; c < T.nch && ok; ++c, ++loaded) {
                    const int s = loaded % kStages;
                    if (loaded >= (unsigned)kStages)
                        ok = mbar_wait(bar_kvfree + 8 * s, ((loaded / kStages) - 1) & 1, abort_flag, P.wait_budget);
                    if (!ok) break;
                    STAMP(110 + c);
                    const uint32_t bar = bar_kv + 8 * s;
                    if (lane == 0) {
                        mbar_expect_tx(bar, 2 * kTile);
                        if (c < T.nnb) {
                            const int X0 = T.rg[0] + P.dil[0] * (T.lo[0] + chunk_coord(P, 0, ld[0], 0));
                            const int X1 = T.rg[1] + P.dil[1] * (T.lo[1] + chunk_coord(P, 1, ld[1], 0));
                            const int X2 = T.rg[2] + P.dil[2] * (T.lo[2] + chunk_coord(P, 2, ld[2], 0));
                            tma_load_5d(lbase + kOffK + s * kTile, &tmK, bar, T.hk * DH, X2, X1, X0, T.b);
                            tma_load_5d(lbase + kOffV + s * kTile, &tmV, bar, T.hk * DH, X2, X1, X0, T.b);
                        } else {                 // additional tokens (rows past n_extra are zero-filled)
                            const int e0 = (c - T.nnb) * kChunk;
                            tma_load_5d(lbase + kOffK + s * kTile, &tmEK, bar, T.hk * DH, e0, 0, 0, T.b);
                            tma_load_5d(lbase + kOffV + s * kTile, &tmEV, bar, T.hk * DH, e0, 0, 0, T.b);
                        }
                    }
                    if (c < T.nnb) { if (++ld[2] == T.nc[2]) { ld[2] = 0; if (++ld[1] == T.nc[1]) { ld[1] = 0; ++ld[0]; } } }
                }
            }
            // end marker: a header without chunks (its slot is free once the last tile's scores are done)
            if (ok && tiles > 0) ok = mbar_wait(bar_qfree, (tiles - 1) & 1, abort_flag, P.wait_budget);
            if (ok && lane == 0) {
                hdr_slot(tiles)->nch = 0;
                mbar_arrive(bar_hdr + 8 * (tiles % kHdrSlots));
            }
        }
    } else if (is_issuer) {
        // =====================================================================
        // MMA issue of this lane (one thread)
        // =====================================================================
        if (lane == 0 && !*abort_flag) {
            constexpr uint32_t idesc_qk = instr_desc(BF16 ? 1 : 0, kChunk, 0, 0);
            constexpr uint32_t idesc_pv = instr_desc(BF16 ? 1 : 0, DH, 0, 1);
            const uint64_t dq0 = smem_desc(lbase + kOffQ, 16, 1024);
            unsigned tiles = 0, n = 0;           // tiles / chunks issued so far
            bool ok = true;
            FwdTile T;
            auto issue_qk = [&](int s) {
                const uint64_t dk0 = smem_desc(lbase + kOffK + s * kTile, 16, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks)            // 32 bytes per k-step
                    mma_ss(tmem + kColS, dq0 + 2 * ks, dk0 + 2 * ks, idesc_qk, ks > 0);
                mma_commit(bar_s);
            };
            auto issue_pv = [&](int s, bool accumulate) {
                // V read MN-major: 16 key rows per k-step.  O stays in TMEM for the whole tile.
                const uint64_t dv0 = smem_desc(lbase + kOffV + s * kTile, kTile, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kChunk / 16; ++ks)
                    mma_ts(tmem + kColO, tmem + kColP + 8 * ks, dv0 + 128 * ks, idesc_pv, (accumulate || ks > 0) ? 1u : 0u);
                mma_commit(bar_o);
                mma_commit(bar_kvfree + 8 * s);
            };
            // The scores run one chunk ahead of the accumulating products, across tile boundaries:
            // cursor of the next Q K^T (tile Tq, chunk cq) and what the product behind it needs.
            bool more = true;                    // the cursor's tile exists (its header has chunks)
            unsigned first_bits = 0u;            // bit (n & 31): chunk n is the first of its tile (its product overwrites O)
            int cq = 0, qc[3] = {0, 0, 0};
            auto seek = [&]() {                  // header of the lane's next tile
                ok = ok && mbar_wait(bar_hdr + 8 * (tiles % kHdrSlots), (tiles / kHdrSlots) & 1, abort_flag, P.wait_budget);
                if (ok) T = *hdr_slot(tiles);
                more = ok && T.nch > 0;
            };
            // Issue the next Q K^T.  `blocking` = wait for its operands; otherwise only if they have landed.
            auto next_qk = [&](bool blocking) -> bool {
                if (!more) return true;
                const int s = n % kStages;
                if (!blocking) {
                    if (cq == 0 && !mbar_try_wait(bar_q, tiles & 1)) return false;
                    if (!mbar_try_wait(bar_kv + 8 * s, (n / kStages) & 1)) return false;
                } else {
                    if (cq == 0) ok = ok && mbar_wait(bar_q, tiles & 1, abort_flag, P.wait_budget);
                    ok = ok && mbar_wait(bar_kv + 8 * s, (n / kStages) & 1, abort_flag, P.wait_budget);
                    if (!ok) return true;
                }
                if (P.extents && cq < T.nnb) {
                    const int box0[3] = {T.lo[0] + chunk_coord(P, 0, qc[0], 0), T.lo[1] + chunk_coord(P, 1, qc[1], 0),
                                         T.lo[2] + chunk_coord(P, 2, qc[2], 0)};
                    zero_rows_past_extent(P, box0, T.Lp, kChunk, 1, kTile, lsmem + kOffK + s * kTile, lsmem + kOffV + s * kTile);
                    if (++qc[2] == T.nc[2]) { qc[2] = 0; if (++qc[1] == T.nc[1]) { qc[1] = 0; ++qc[0]; } }
                }
                issue_qk(s);
                STAMP(200 + cq);
                first_bits = cq == 0 ? (first_bits | (1u << (n & 31))) : (first_bits & ~(1u << (n & 31)));
                ++n;
                if (++cq == T.nch) {             // last scores of the tile: Q may go once they are done
                    mma_commit(bar_qfree);
                    ++tiles;
                    cq = 0; qc[0] = qc[1] = qc[2] = 0;
                    seek();
                }
                return true;
            };
            seek();
            unsigned npv = 0;                    // accumulating products issued so far
            next_qk(true);
            while (npv < n && ok) {
                ok = mbar_wait(bar_p, npv & 1, abort_flag, P.wait_budget);       // S(npv) consumed, P(npv) stored
                if (!ok) break;
                STAMP(210);
                // S is free again: the next scores go first if their operands are there (the threads wait for them)
                const bool early = next_qk(false);
                issue_pv(npv % kStages, (first_bits >> (npv & 31)) & 1u ? false : true);
                STAMP(220 + (early ? 1 : 0));
                ++npv;
                if (!early) next_qk(true);
            }
        }
    } else {
        // =====================================================================
        // softmax warps: thread = one query row, all 128 columns of the chunk
        // =====================================================================
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        constexpr float kGrow = BF16 ? 60.f : 14.f;      // exponent headroom of the stored probabilities
        bool ok = true;
        unsigned n = 0;                                  // chunks processed so far (all tiles of this lane)
        FwdTile T;
        for (unsigned tiles = 0;; ++tiles) {
            ok = mbar_wait(bar_hdr + 8 * (tiles % kHdrSlots), (tiles / kHdrSlots) & 1, abort_flag, P.wait_budget) && ok;
            if (!ok) break;
            T = *hdr_slot(tiles);
            if (T.nch == 0) break;
            // ---- this thread's query row ----
            int f[3], e[3];
            bool valid_q, in_tensor;
            const long long out_row = row_geometry(P, T, row, f, e, valid_q, in_tensor);
            uint4* o4 = reinterpret_cast<uint4*>(out + out_row * DH);

            float m = -INFINITY, l = 0.f;
            int ci[3] = {0, 0, 0};
            for (int c = 0; c < T.nch; ++c, ++n) {
                // ---- what decides the validity of this row's columns in this chunk ----
                const bool extra = c >= T.nnb;   // additional tokens: every live row sees the first n_extra columns
                int jl[3] = {0, 0, 0}, jh[3] = {0, 0, 0};
                uint32_t rowbits = 0u, colbits = 0u;
                if (!extra) {
#pragma unroll
                    for (int a = 0; a < 3; ++a) chunk_range(P, a, ci[a], f[a], e[a], jl[a], jh[a]);
                    if constexpr (kInner > 0) {
                        // inner rows of the chunk (kInner columns each) are numbered r = j0 * cb1 + j1
                        const uint32_t m1 = jh[1] > jl[1] ? (low_bits(jh[1]) & ~low_bits(jl[1])) : 0u;
                        for (int j0 = jl[0]; j0 < jh[0]; ++j0) rowbits |= m1 << (j0 << P.cb1_log);
                        colbits = jh[2] > jl[2] ? (low_bits(jh[2]) & ~low_bits(jl[2])) : 0u;
                    }
                }
                auto piece_bits = [&](int pc) -> uint32_t {
                    if (extra) return valid_q ? low_bits(P.n_extra - ((c - T.nnb) * kChunk + 32 * pc)) : 0u;
                    if constexpr (kInner > 0) {
                        uint32_t wd = 0u;
#pragma unroll
                        for (int t = 0; t < 32 / kInner; ++t)
                            if ((rowbits >> (pc * (32 / kInner) + t)) & 1u) wd |= colbits << (t * kInner);
                        return wd;
                    } else {
                        return piece_word_ranges(P, pc, jl, jh);
                    }
                };

                STAMP(300 + c);
                ok = ok && mbar_wait(bar_s, n & 1, abort_flag, P.wait_budget);
                tc_fence_after();
                STAMP(310);

                // One 32-column piece at a time, in a rolled loop (the hot code stays small): scores in,
                // probabilities out.  P(n-1) V must have finished before the first store.
                float lsum = 0.f;
                bool p_free = n == 0;
#pragma unroll 1
                for (int attempt = 0; attempt < 2; ++attempt) {
                    float xmax = -INFINITY, r0 = 0.f, r1 = 0.f;
                    // scores of piece pc -> probabilities, row sum, TMEM store
                    auto do_piece = [&](int pc, uint32_t wd, bool active, uint32_t (&s)[32]) {
                        uint32_t pk[16];
                        if (active) {
                            if (m == -INFINITY && wd != 0u) {       // first valid columns of this row: fix the stabiliser
                                float mm = -INFINITY;
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if ((wd >> i) & 1u) mm = fmaxf(mm, __uint_as_float(s[i]));
                                m = mm;
                            }
                            const float mb = (m == -INFINITY) ? 0.f : m * P.scale_log2;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                float x0 = fmaf(__uint_as_float(s[2 * i]), P.scale_log2, -mb);
                                float x1 = fmaf(__uint_as_float(s[2 * i + 1]), P.scale_log2, -mb);
                                if (!((wd >> (2 * i)) & 1u)) x0 = -INFINITY;
                                if (!((wd >> (2 * i + 1)) & 1u)) x1 = -INFINITY;
                                xmax = fmaxf(xmax, fmaxf(x0, x1));
                                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                                r0 += p0;
                                r1 += p1;
                                pk[i] = cvt_pack<BF16>(p0, p1);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) pk[i] = 0u;
                        }
                        if (!p_free) {
                            STAMP(320);
                            ok = mbar_wait(bar_o, (n - 1) & 1, abort_flag, P.wait_budget) && ok;
                            tc_fence_after();
                            p_free = true;
                        }
                        tmem_st16(trow + kColP + 16 * pc, pk);
                    };
#pragma unroll 1
                    for (int pc = 0; pc < 4; ++pc) {
                        const uint32_t wd = ok ? piece_bits(pc) : 0u;
                        const bool active = __any_sync(0xffffffffu, wd != 0u) != 0;
                        uint32_t s[32];
                        if (active) { tmem_ld32(trow + kColS + 32 * pc, s); tmem_ld_wait(); }
                        do_piece(pc, wd, active, s);
                    }
                    lsum = r0 + r1;
                    const bool grow = xmax > kGrow;
                    if (!__any_sync(0xffffffffu, grow)) break;
                    // rare: a score far above the stabiliser.  Move it, rescale O and the row sum, redo the chunk.
                    const float fac = grow ? fast_exp2(-xmax) : 1.f;
                    if (c > 0) {
#pragma unroll 1
                        for (int part = 0; part < DH / 16; ++part) {
                            uint32_t o[16];
                            tmem_ld16(trow + kColO + 16 * part, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * fac);
                            tmem_st16(trow + kColO + 16 * part, o);
                        }
                    }
                    l *= fac;
                    if (grow) m += xmax / P.scale_log2;
                }
                l += ok ? lsum : 0.f;
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(bar_p);
                STAMP(330);
                if (++ci[2] == T.nc[2]) { ci[2] = 0; if (++ci[1] == T.nc[1]) { ci[1] = 0; ++ci[0]; } }
            }

            // ---- normalise and write out ----
            ok = mbar_wait(bar_o, (n - 1) & 1, abort_flag, P.wait_budget) && ok;
            tc_fence_after();
            STAMP(340);
            {
                const bool live = valid_q && ok;
                const float inv = (live && l > 0.f) ? 1.f / l : 0.f;
                uint32_t o[2][32];
                tmem_ld32(trow + kColO, o[0]);
                tmem_ld32(trow + kColO + 32, o[1]);
                tmem_ld_wait();
#pragma unroll
                for (int part = 0; part < DH / 32; ++part) {
                    if (in_tensor) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t wv[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                wv[j] = live ? cvt_pack<BF16>(__uint_as_float(o[part][8 * i + 2 * j]) * inv, __uint_as_float(o[part][8 * i + 2 * j + 1]) * inv) : 0u;
                            o4[4 * part + i] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
                        }
                    }
                }
                // natural-log lse of scale * logits
                if (in_tensor)
                    lse[out_row] = (live && l > 0.f) ? (m * P.scale_log2 + log2f(l)) * 0.6931471805599453f : 0.f;
            }
            // the next tile's first P V is issued only after this thread has stored its next P
            tc_fence_before();
            STAMP(350);
        }
    }

    if (*abort_flag) abort_grace_sleep();       // loads of a wait that gave up may still be landing
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(*tmem_slot, kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

} // namespace

int tc_fused_fwd_pipe(int dtype, const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                      const void* ev, void* out, void* lse, cudaStream_t s)
{
    if (g.D != 64) return -2;
    if (!tc_eligible(dtype, g, q, k, v, /*allow_stride=*/true)) return -2;
    if (g.n_extra > 0 && ((reinterpret_cast<uintptr_t>(ek) | reinterpret_cast<uintptr_t>(ev)) & 15u)) return -2;
    Plan plan;
    if (!make_plan(g, plan, kChunk, /*with_stride=*/true, /*interleave=*/true)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mq, mk, mv, mek, mev;
    if (!encode_map(&mq, q, bf16, plan.p, g.Hq, g.D, g.qs, plan.box_q, /*query_lattice=*/true) ||
        !encode_map(&mk, k, bf16, plan.p, g.Hkv, g.D, g.ks, plan.box_kv, false, /*interleaved=*/true) ||
        !encode_map(&mv, v, bf16, plan.p, g.Hkv, g.Dv, g.vs, plan.box_kv, false, /*interleaved=*/true))
        return -2;
    mek = mk; mev = mv;                      // placeholders when there are no additional tokens
    if (g.n_extra > 0 && (!encode_extra_map(&mek, ek, bf16, g.B, g.n_extra, g.Hkv, g.D, kChunk) ||
                          !encode_extra_map(&mev, ev, bf16, g.B, g.n_extra, g.Hkv, g.Dv, kChunk)))
        return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    if (plan.p.work_q == 0 || g.B == 0) return 0;
    const unsigned grid = persistent_grid((plan.p.work_q + 1) / 2, 1);
    cudaError_t err = cudaSuccess;
    auto launch = [&](auto bf, auto inner) {
        constexpr bool kBf = decltype(bf)::value;
        constexpr int kInner = decltype(inner)::value;
        err = ensure_dynamic_smem((const void*)tc_fwd_pipe_kernel<kBf, kInner>, kSmemTotal);
        if (err != cudaSuccess) return;
        tc_fwd_pipe_kernel<kBf, kInner><<<grid, kThreads, kSmemTotal, s>>>(mq, mk, mv, mek, mev, plan.p, (uint16_t*)out, (float*)lse);
    };
    auto by_inner = [&](auto bf) {
        if (plan.p.cb[2] == 16) launch(bf, std::integral_constant<int, 16>{});
        else if (plan.p.cb[2] == 32) launch(bf, std::integral_constant<int, 32>{});
        else launch(bf, std::integral_constant<int, 0>{});
    };
    if (bf16) by_inner(std::true_type{});
    else by_inner(std::false_type{});
    if (err == cudaSuccess) err = cudaGetLastError();
    tc_count_launch();
    return err == cudaSuccess ? 0 : (int)err;
}

#ifdef NATTEN_TRACE
extern "C" int natten_trace_read(long long* host, int clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace));
    if (e == cudaSuccess && clear) {
        static long long zeros[16 * 512] = {0};
        e = cudaMemcpyToSymbol(g_trace, zeros, sizeof(g_trace));
    }
    return (int)e;
}
#endif

} // namespace natten
