// Fused neighbourhood-attention forward for head dims up to 128 on tcgen05 tensor cores (sm_100a),
// built from small persistent CTAs: four of them share an SM up to head dim 64, two above it, each working
// on one tile of 128 queries at a time (tiles blockIdx.x, + gridDim.x, ...).
//
// Per tile the union of the queries' neighbourhoods is a box of keys walked in chunks of 64 keys
// (additional tokens follow as extra chunks):
//   S = Q K^T                    tcgen05.mma (N = 64), Q / K tiles staged by TMA, S in TMEM
//   P = exp2(S*scale*log2e - m)  one thread per query row; the row's 64 scores are read from TMEM in
//                                16-column pieces (a piece that is empty for the whole warp is skipped),
//                                masked, and written back as 16-bit P over the scores they came from
//   O += P V                     tcgen05.mma with A = P from TMEM, V tile read MN-major, O in TMEM
// The chunk rows are interleaved (chunk c holds the key rows c, c + n, c + 2n, ... of the box), so every
// chunk carries a share of every warp's window and the four warps of a tile finish a chunk together.
// A row's stabiliser m is fixed at the first valid columns it meets and only moves if a later score
// exceeds it by 2^60 (2^14 for fp16); O, the row sum and the probabilities already stored for the
// chunk are then rescaled.  Up to head dim 64 four independent CTAs per SM give the schedulers sixteen
// softmax warps in different phases of their tiles, which is what hides the TMEM / barrier / MMA latencies
// (128 TMEM columns and 49 KB of shared memory per CTA).  Above it only two CTAs fit (256 columns, 97 KB),
// so the scores get two buffers there: S(c + 1) is computed while the threads work on S(c).
//
// TMEM columns: head dim 64: S [0,64) (P over [0,32)), O [64,128);
//               head dim 128: S of even chunks [0,64), of odd chunks [64,128), O [128,256).
#include "tc_kernels.cuh"

#include "tc_fwd_geom.cuh"
#include "tc_plan.cuh"

#include <type_traits>

#ifndef NATTEN_ABL
#define NATTEN_ABL 0
#endif

namespace natten {

using namespace tc;
using namespace tcplan;
using namespace fwdgeom;

#ifdef NATTEN_TRACE
__device__ long long g_trace_small[8 * 512];
#define STAMP(id)                                                                                   \
    do {                                                                                            \
        if (blockIdx.x == 9 && lane == 0 && tn < 255) {       \
            g_trace_small[warp * 512 + 2 * tn] = (id);                                              \
            g_trace_small[warp * 512 + 2 * tn + 1] = clock64();                                     \
            ++tn;                                                                                   \
        }                                                                                           \
    } while (0)
#else
#define STAMP(id) do { } while (0)
#endif

namespace {

constexpr int kKeys = 64;                   // keys per chunk
constexpr int kKeysLog = 6;
constexpr int kStages = 2;
constexpr int kThreads = 160;               // 4 softmax warps + 1 warp that loads and issues
constexpr int kHdrSlots = 3;                // tile headers published by the issuing warp
constexpr int kHdrBytes = 144;
static_assert(sizeof(FwdTile) <= kHdrBytes, "header slot too small");
constexpr uint32_t kColS = 0;

// Shared memory and TMEM of one CTA for head dim DH (64: four CTAs per SM, 128 TMEM columns; 128: two CTAs per
// SM, 256 TMEM columns).  Tiles are stored as blocks of 64 channels (128-byte rows, 128-byte swizzle).
template <int DH>
struct FwdSmall {
    static constexpr int kHalves = DH / 64;
    static constexpr int kQHalf = kTileRows * 128;          // [128 x 64] 16-bit
    static constexpr int kKVHalf = kKeys * 128;             // [64 x 64] 16-bit
    static constexpr int kQBytes = kQHalf * kHalves;
    static constexpr int kKVBytes = kKVHalf * kHalves;
    static constexpr int kOffQ = 0, kOffK = kQBytes, kOffV = kQBytes + kStages * kKVBytes;
    static constexpr int kBar = kQBytes + 2 * kStages * kKVBytes;
    static constexpr int kHdr = kBar + 160;
    static constexpr int kSmemTotal = kHdr + kHdrSlots * kHdrBytes;
    static constexpr uint32_t kTmemCols = DH == 64 ? 128 : 256;     // S 64 + O DH, rounded up to a power of two
    static constexpr int kPerSm = DH == 64 ? 4 : 2;
    // At head dim 128 the 256 TMEM columns hold two score buffers: S(c + 1) is computed while the threads turn
    // S(c) into probabilities (at 64 the four CTAs of an SM fill each other's gaps instead).
    static constexpr bool kTwoS = DH == 128;
    static constexpr uint32_t kColO = kTwoS ? 128 : 64;
};

template <int DH, bool BF16, int kInner>
__global__ void __launch_bounds__(kThreads, FwdSmall<DH>::kPerSm)
tc_fwd_small_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmEK,
                    const __grid_constant__ CUtensorMap tmEV, const __grid_constant__ TcParams P,
                    uint16_t* __restrict__ out, float* __restrict__ lse)
{
    using FS = FwdSmall<DH>;
    constexpr int kHalves = FS::kHalves, kQHalf = FS::kQHalf, kKVHalf = FS::kKVHalf, kQBytes = FS::kQBytes, kKVBytes = FS::kKVBytes;
    constexpr int kOffQ = FS::kOffQ, kOffK = FS::kOffK, kOffV = FS::kOffV, kBar = FS::kBar, kHdr = FS::kHdr;
    constexpr uint32_t kTmemCols = FS::kTmemCols, kColO = FS::kColO;
    constexpr bool kTwoS = FS::kTwoS;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef NATTEN_TRACE
    int tn = 0;
#endif
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);

    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kBar + 112);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kBar + 120);
    const uint32_t bar_q = sbase + kBar + 0;            // Q tile landed
    const uint32_t bar_qfree = sbase + kBar + 8;        // last Q K^T of the tile finished: Q may be overwritten
    const uint32_t bar_kv = sbase + kBar + 16;          // [2] K, V chunk landed
    const uint32_t bar_kvfree = sbase + kBar + 32;      // [2] P V of the chunk finished: stage may be overwritten
    const uint32_t bar_s = sbase + kBar + 48;           // S of the chunk is in TMEM (and every earlier product is done)
    const uint32_t bar_p = sbase + kBar + 56;           // every thread stored its P
    const uint32_t bar_o = sbase + kBar + 64;           // last P V of the tile finished
    const uint32_t bar_hdr = sbase + kBar + 72;         // [3] geometry of the CTA's t-th tile published
    const uint32_t bar_s1 = sbase + kBar + 96;          // two score buffers: bar_s / bar_p of the odd chunks
    const uint32_t bar_p1 = sbase + kBar + 104;
    const uint32_t bar_pv = sbase + kBar + 128;         // [2] two score buffers: P V of the chunk finished (by chunk parity)
    // chunk n (counted over the CTA's whole run) -> its score columns, barriers and wait parity
    auto s_cols = [&](unsigned n) -> uint32_t { return kTwoS ? 64u * (n & 1u) : 0u; };
    auto bar_s_of = [&](unsigned n) -> uint32_t { return (kTwoS && (n & 1u)) ? bar_s1 : bar_s; };
    auto bar_p_of = [&](unsigned n) -> uint32_t { return (kTwoS && (n & 1u)) ? bar_p1 : bar_p; };
    auto par_of = [&](unsigned n) -> uint32_t { return kTwoS ? ((n >> 1) & 1u) : (n & 1u); };
    auto hdr_slot = [&](unsigned t) { return reinterpret_cast<FwdTile*>(smem + kHdr + (t % kHdrSlots) * kHdrBytes); };

    if (warp == 4) {
        if (lane == 0) {
            // swizzled tiles need a 1024-byte aligned base; once any CTA has given up, the rest bail out
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            mbar_init(bar_q, 1);
            mbar_init(bar_qfree, 1);
            for (int s = 0; s < kStages; ++s) { mbar_init(bar_kv + 8 * s, 1); mbar_init(bar_kvfree + 8 * s, 1); }
            mbar_init(bar_s, 1);
            mbar_init(bar_p, 128);
            mbar_init(bar_s1, 1);
            mbar_init(bar_p1, 128);
            mbar_init(bar_pv, 1);
            mbar_init(bar_pv + 8, 1);
            mbar_init(bar_o, 1);
            for (int i = 0; i < kHdrSlots; ++i) mbar_init(bar_hdr + 8 * i, 1);
            mbar_init_fence();
            fence_async_smem();
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const unsigned nwork = P.work_q;

    if (warp == 4) {
        // =====================================================================
        // Geometry, TMA loads and MMA issue.  The whole warp walks the CTA's work items (blockIdx.x,
        // + gridDim.x, ...): it works out each tile's geometry and publishes it for the softmax warps,
        // writes the zero rows of tiles that have nothing to attend to, and lane 0 issues the loads (Q of
        // the next tile and the K/V ring run ahead across tile boundaries) and the matrix products.
        // =====================================================================
        if (!*abort_flag) {
            constexpr uint32_t idesc_qk = instr_desc(BF16 ? 1 : 0, kKeys, 0, 0);
            constexpr uint32_t idesc_pv = instr_desc(BF16 ? 1 : 0, DH, 0, 1);
            const uint64_t dq0 = smem_desc(sbase + kOffQ, 16, 1024);
            const uint32_t leader = elect_one();
            bool ok = true;
            Cursor cur;
            cur.init(P, blockIdx.x, gridDim.x);
            unsigned pub = 0;                    // headers published (the last one may be the end marker)
            bool exhausted = false;
            auto discover = [&]() {              // next tile with work -> header ring
                if (exhausted) return;
                FwdTile Tn;
                bool found = false;
                while (cur.w < nwork) {
                    fwd_tile(P, cur, kKeysLog, Tn);
                    cur.advance(P, gridDim.x);
                    if (Tn.active) { found = true; break; }
#pragma unroll 1
                    for (int r = lane; r < kTileRows; r += 32) {         // rows that exist in the output are zero
                        int f[3], e[3];
                        bool valid_q, in_tensor;
                        const long long out_row = row_geometry(P, Tn, r, f, e, valid_q, in_tensor);
                        if (in_tensor) {
                            uint4* o4 = reinterpret_cast<uint4*>(out + out_row * P.dreal);
#pragma unroll
                            for (int i = 0; i < DH / 8; ++i)
                                if (8 * i < P.dreal) o4[i] = make_uint4(0, 0, 0, 0);
                            lse[out_row] = 0.f;
                        }
                    }
                }
                if (!found) { exhausted = true; Tn.nch = 0; }
                if (lane == 0) {
                    *hdr_slot(pub) = Tn;
                    mbar_arrive(bar_hdr + 8 * (pub % kHdrSlots));
                }
                __syncwarp();
                ++pub;
            };

            // ---- loads: tile tl, its Q, then its chunks; never waits for work that has not been issued ----
            unsigned tl = 0, n_load = 0, n_pv = 0, n_qk = 0, qk_done_tiles = 0;
            int cl = 0, ldc[3] = {0, 0, 0};
            bool q_loaded = false;
            auto refill = [&]() -> bool {
                if (!ok || tl >= pub) return false;
                const FwdTile* H = hdr_slot(tl);
                if (H->nch == 0) return false;
                if (!q_loaded) {
                    if (tl > qk_done_tiles) return false;                // the previous tile still needs its Q
                    if (tl > 0) ok = mbar_wait(bar_qfree, (tl - 1) & 1, abort_flag, P.wait_budget);
                    if (!ok) return false;
                    if (lane == 0) {
                        mbar_expect_tx(bar_q, kQBytes + ((P.inject == 1 && tl == 0) ? 16u : 0u));
#pragma unroll
                        for (int hf = 0; hf < kHalves; ++hf)
                            tma_load_heads(sbase + kOffQ + hf * kQHalf, &tmQ, bar_q, P, DH, H->h * DH + 64 * hf,
                                        H->rg[2] + P.dil[2] * (H->x0[2] + H->sx[2] * H->origin[2]),
                                        H->rg[1] + P.dil[1] * (H->x0[1] + H->sx[1] * H->origin[1]),
                                        H->rg[0] + P.dil[0] * (H->x0[0] + H->sx[0] * H->origin[0]), H->b);
                    }
                    q_loaded = true;
                    return true;
                }
                if (n_load >= n_pv + kStages) return false;              // both stages wait for products not issued yet
                const int s = n_load % kStages;
                if (n_load >= (unsigned)kStages)
                    ok = mbar_wait(bar_kvfree + 8 * s, ((n_load / kStages) - 1) & 1, abort_flag, P.wait_budget);
                if (!ok) return false;
                if (lane == 0) {
                    const uint32_t bar = bar_kv + 8 * s;
                    mbar_expect_tx(bar, 2 * kKVBytes);
                    if (cl < H->nnb) {
                        const int X0 = H->rg[0] + P.dil[0] * (H->lo[0] + chunk_coord(P, 0, ldc[0], 0));
                        const int X1 = H->rg[1] + P.dil[1] * (H->lo[1] + chunk_coord(P, 1, ldc[1], 0));
                        const int X2 = H->rg[2] + P.dil[2] * (H->lo[2] + chunk_coord(P, 2, ldc[2], 0));
#pragma unroll
                        for (int hf = 0; hf < kHalves; ++hf) {
                            tma_load_heads(sbase + kOffK + s * kKVBytes + hf * kKVHalf, &tmK, bar, P, DH, H->hk * DH + 64 * hf, X2, X1, X0, H->b);
                            tma_load_heads(sbase + kOffV + s * kKVBytes + hf * kKVHalf, &tmV, bar, P, DH, H->hk * DH + 64 * hf, X2, X1, X0, H->b);
                        }
                    } else {                     // additional tokens (rows past n_extra are zero-filled)
                        const int e0 = (cl - H->nnb) * kKeys;
#pragma unroll
                        for (int hf = 0; hf < kHalves; ++hf) {
                            tma_load_heads(sbase + kOffK + s * kKVBytes + hf * kKVHalf, &tmEK, bar, P, DH, H->hk * DH + 64 * hf, e0, 0, 0, H->b);
                            tma_load_heads(sbase + kOffV + s * kKVBytes + hf * kKVHalf, &tmEV, bar, P, DH, H->hk * DH + 64 * hf, e0, 0, 0, H->b);
                        }
                    }
                }
                if (cl < H->nnb) { if (++ldc[2] == H->nc[2]) { ldc[2] = 0; if (++ldc[1] == H->nc[1]) { ldc[1] = 0; ++ldc[0]; } } }
                ++n_load;
                if (++cl == H->nch) { ++tl; cl = 0; ldc[0] = ldc[1] = ldc[2] = 0; q_loaded = false; }
                return true;
            };

            int qc[3] = {0, 0, 0};
            auto issue_qk = [&](const FwdTile* H, int c) {
                const int s = n_qk % kStages;
                ok = ok && mbar_wait(bar_kv + 8 * s, (n_qk / kStages) & 1, abort_flag, P.wait_budget);
                if (!ok) return;
                if (P.extents && c < H->nnb) {
                    const int box0[3] = {H->lo[0] + chunk_coord(P, 0, qc[0], 0), H->lo[1] + chunk_coord(P, 1, qc[1], 0),
                                         H->lo[2] + chunk_coord(P, 2, qc[2], 0)};
                    if (lane == 0)
                        zero_rows_past_extent(P, box0, H->Lp, kKeys, kHalves, kKVHalf, smem + kOffK + s * kKVBytes, smem + kOffV + s * kKVBytes);
                    __syncwarp();
                }
                {   // warp-uniform code; the tensor-core instructions execute on the elected lane
                    const uint64_t dk0 = smem_desc(sbase + kOffK + s * kKVBytes, 16, 1024);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < DH / 16; ++ks)            // 32 bytes per k-step inside a 64-channel block
                        mma_ss_e(tmem + kColS + s_cols(n_qk), dq0 + ((((ks / 4) * kQHalf) + (ks % 4) * 32) >> 4),
                                 dk0 + ((((ks / 4) * kKVHalf) + (ks % 4) * 32) >> 4), idesc_qk, ks > 0, leader);
                    mma_commit_e(bar_s_of(n_qk), leader);
                    if (c + 1 == H->nch) mma_commit_e(bar_qfree, leader);     // last scores of the tile: Q may go once they are done
                }
                if (c < H->nnb) { if (++qc[2] == H->nc[2]) { qc[2] = 0; if (++qc[1] == H->nc[1]) { qc[1] = 0; ++qc[0]; } } }
                ++n_qk;
                if (c + 1 == H->nch) { ++qk_done_tiles; qc[0] = qc[1] = qc[2] = 0; }
            };
            auto issue_pv = [&](int c, bool last) {
                // V read MN-major: 16 key rows per k-step; P sits as 16-bit pairs in the first 32 S columns
                const int s = n_pv % kStages;
                {
                    const uint64_t dv0 = smem_desc(sbase + kOffV + s * kKVBytes, kKVHalf, 1024);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < kKeys / 16; ++ks)
                        mma_ts_e(tmem + kColO, tmem + kColS + s_cols(n_pv) + 8 * ks, dv0 + 128 * ks, idesc_pv, (c > 0 || ks > 0) ? 1u : 0u, leader);
                    mma_commit_e(bar_kvfree + 8 * s, leader);
                    if (kTwoS) mma_commit_e(bar_pv + 8 * (n_pv & 1u), leader);
                    if (last) mma_commit_e(bar_o, leader);
                }
                ++n_pv;
            };

            discover();
            while (refill()) {}
            for (unsigned ti = 0; ok; ++ti) {
                const FwdTile* H = hdr_slot(ti);
                const int nch = H->nch;
                if (nch == 0) break;
                ok = mbar_wait(bar_q, ti & 1, abort_flag, P.wait_budget);
                issue_qk(H, 0);
                STAMP(200);
                discover();                      // the next tile's geometry, while the threads work on this chunk
                while (refill()) {}
                for (int c = 0; c < nch && ok; ++c) {
                    // two score buffers: S(c + 1) goes into the other buffer while the threads work on S(c); that
                    // buffer's P(c - 1) is read by a product issued earlier from this warp, so the order holds
                    if (kTwoS && c + 1 < nch) issue_qk(H, c + 1);
                    if (!ok) break;
                    ok = mbar_wait(bar_p_of(n_pv), par_of(n_pv), abort_flag, P.wait_budget);      // P(c) stored over S(c)
                    if (!ok) break;
                    STAMP(210);
                    issue_pv(c, c + 1 == nch);       // reads P(c) ...
                    if (!kTwoS && c + 1 < nch) issue_qk(H, c + 1);   // ... before the next scores overwrite it (issue order)
                    STAMP(220);
                    while (refill()) {}
                }
            }
        }
    } else {
        // =====================================================================
        // softmax warps: thread = one query row, the chunk's 64 columns in 16-column pieces
        // =====================================================================
        const uint32_t trow = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        constexpr float kGrow = BF16 ? 60.f : 14.f;      // exponent headroom of the stored probabilities
        constexpr float kGrowSum = BF16 ? 1.152921504606847e18f : 16384.f;      // 2^kGrow: a piece's row sum below it has no probability above it
        // With 16-column inner rows every piece is one inner row of the chunk: a piece is either inside the
        // row's window along the outer axes or not (one bit), and which of its 16 columns are valid is the
        // same for every piece.  The column mask then lives in the addends of the scale-and-shift, one
        // register per column: -m*scale*log2e inside the window, -inf outside.
        constexpr bool kRows16 = kInner == 16;
        bool ok = true;
        unsigned n = 0;                      // chunks processed so far (all tiles of this CTA)
        uint32_t scol = trow + kColS;        // TMEM address of this row's scores of the current chunk
        float m = -INFINITY, l = 0.f;
        float add[16];
        uint32_t add_cols = 0u;              // column mask the addends were built for
#pragma unroll
        for (int i = 0; i < 16; ++i) add[i] = -INFINITY;
        auto refresh_add = [&](uint32_t cols) {
            const float nmb = (m == -INFINITY) ? 0.f : -m * P.scale_log2;
#pragma unroll
            for (int i = 0; i < 16; ++i) add[i] = ((cols >> i) & 1u) ? nmb : -INFINITY;
            add_cols = cols;
        };
        // rare: a score far above the stabiliser.  Move it; rescale O, the row sum and the probabilities this
        // chunk has stored so far (every earlier product has finished).  `grow`: this row is the cause.
        auto rescale = [&](bool grow, float xmax, int c, int pc, uint32_t stored) {
            const float fac = grow ? fast_exp2(-xmax) : 1.f;
            if (c > 0) {
                // with two score buffers S(c) was issued before P V of chunk c - 1: wait for that product itself
                if (kTwoS) {
                    ok = mbar_wait(bar_pv + 8 * ((n - 1) & 1u), par_of(n - 1), abort_flag, P.wait_budget) && ok;
                    tc_fence_after();
                }
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
#pragma unroll 1
            for (int pp = 0; pp < pc; ++pp) {
                if (!((stored >> pp) & 1u)) continue;
                uint32_t old[8];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                             : "=r"(old[0]), "=r"(old[1]), "=r"(old[2]), "=r"(old[3]), "=r"(old[4]), "=r"(old[5]),
                               "=r"(old[6]), "=r"(old[7])
                             : "r"(scol + 8 * pp) : "memory");
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float lo, hi;
                    if (BF16) {
                        lo = __uint_as_float(old[i] << 16);
                        hi = __uint_as_float(old[i] & 0xFFFF0000u);
                    } else {
                        const __half2 h2 = *reinterpret_cast<const __half2*>(&old[i]);
                        lo = __low2float(h2);
                        hi = __high2float(h2);
                    }
                    old[i] = cvt_pack<BF16>(lo * fac, hi * fac);
                }
                tmem_st8(scol + 8 * pp, old);
            }
            l *= fac;
            if (grow) m += xmax / P.scale_log2;
        };

        for (unsigned t = 0;; ++t) {
        ok = mbar_wait(bar_hdr + 8 * (t % kHdrSlots), (t / kHdrSlots) & 1, abort_flag, P.wait_budget) && ok;
        if (!ok) break;
        const FwdTile T = *hdr_slot(t);
        if (T.nch == 0) break;
        STAMP(290);
        // ---- this thread's query row ----
        int f[3], e[3];
        bool valid_q, in_tensor;
        const long long out_row = row_geometry(P, T, warp * 32 + lane, f, e, valid_q, in_tensor);
        m = -INFINITY;
        l = 0.f;
        add_cols = 0xffffffffu;              // the addends belong to the previous tile's stabiliser
        int ci[3] = {0, 0, 0};
        const bool line = line_chunks(P);    // chunks are runs of the innermost axis (1-D windows): cheap validity words
        int jl[3] = {0, 0, 0}, jh[3] = {0, 0, 0};
        uint32_t rowbits = 0u, colbits = 0u, dirty = 7u;     // 16-column rows: one bit per piece, one per column
        // 16-column rows with a single chunk along the innermost axis and at most 16 chunks: which pieces of
        // which chunk lie inside the row's window is worked out once per tile from the row's side (a loop over
        // the window's rows, each of which lands in one piece of one chunk), four bits per chunk.
        bool mapped = false;
        unsigned long long rowmap = 0ull;
        if constexpr (kRows16) {
            if (T.nc[2] == 1 && T.nnb <= 16) {
                mapped = true;
                for (int x0 = f[0]; x0 < e[0]; ++x0) {
                    int c0, j0;
                    if (P.il[0] == 1) { c0 = x0 >> P.cb0_log; j0 = x0 & (P.cb[0] - 1); }
                    else { j0 = (int)fast_div((unsigned)x0, P.il_mul[0]); c0 = x0 - j0 * P.il[0]; }
                    for (int x1 = f[1]; x1 < e[1]; ++x1) {
                        int c1, j1;
                        if (P.il[1] == 1) { c1 = x1 >> P.cb1_log; j1 = x1 & (P.cb[1] - 1); }
                        else { j1 = (int)fast_div((unsigned)x1, P.il_mul[1]); c1 = x1 - j1 * P.il[1]; }
                        rowmap |= 1ull << (4 * (c0 * T.nc[1] + c1) + (j0 << P.cb1_log) + j1);
                    }
                }
                int l2, h2;
                chunk_range(P, 2, 0, f[2], e[2], l2, h2);
                colbits = h2 > l2 ? (low_bits(h2) & ~low_bits(l2)) : 0u;
            }
        }
        for (int c = 0; c < T.nch; ++c, ++n) {
            // ---- validity of this row's columns in this chunk ----
            // jl/jh (columns of the chunk inside the row's window, per axis) only change along the axes whose
            // chunk index moved since the last chunk: `dirty` has a bit per axis.
            const bool extra = c >= T.nnb;   // additional tokens: every live row sees the first n_extra columns
            uint32_t words[2] = {0u, 0u};    // generic form: one bit per column
            if (extra) {
#pragma unroll
                for (int pc = 0; pc < 2; ++pc)
                    words[pc] = valid_q ? low_bits(P.n_extra - ((c - T.nnb) * kKeys + 32 * pc)) : 0u;
            } else if (mapped) {
                rowbits = (uint32_t)(rowmap >> (4 * c)) & 15u;
            } else {
                if (kInner == 0 && line) {
#pragma unroll
                    for (int pc = 0; pc < 2; ++pc) words[pc] = line_word(P, pc, ci, f, e);
                } else {
#pragma unroll
                for (int a = 0; a < 3; ++a)
                    if ((dirty >> a) & 1u) chunk_range(P, a, ci[a], f[a], e[a], jl[a], jh[a]);
                if constexpr (kInner > 0) {
                    // inner rows of the chunk (kInner columns each) are numbered r = j0 * cb1 + j1
                    if (dirty & 3u) {
                        const uint32_t m1 = jh[1] > jl[1] ? (low_bits(jh[1]) & ~low_bits(jl[1])) : 0u;
                        rowbits = 0u;
                        for (int j0 = jl[0]; j0 < jh[0]; ++j0) rowbits |= m1 << (j0 << P.cb1_log);
                    }
                    if (dirty & 4u) colbits = jh[2] > jl[2] ? (low_bits(jh[2]) & ~low_bits(jl[2])) : 0u;
                    if constexpr (!kRows16) {
#pragma unroll
                        for (int pc = 0; pc < 2; ++pc) words[pc] = ((rowbits >> pc) & 1u) ? colbits : 0u;
                    }
                } else {
#pragma unroll
                    for (int pc = 0; pc < 2; ++pc) words[pc] = piece_word_ranges(P, pc, jl, jh);
                }
                }
                dirty = 0u;
            }
            const bool fast = kRows16 && !extra;
            if (fast && colbits != add_cols) refresh_add(colbits);

            STAMP(300 + c);
            scol = trow + kColS + s_cols(n);
            ok = ok && mbar_wait(bar_s_of(n), par_of(n), abort_flag, P.wait_budget);     // one score buffer: every earlier product has finished, too
            tc_fence_after();
            STAMP(310);
            if (!ok) { words[0] = 0u; words[1] = 0u; rowbits = 0u; dirty = 7u; }

            uint32_t stored = 0u;            // pieces of this chunk that hold probabilities (bit per piece)
            // one 16-column piece on the general path: scores s, validity bits wd -> probabilities pk
            auto generic_piece = [&](int pc, uint32_t (&s)[16], uint32_t wd, uint32_t (&pk)[8]) {
                if (m == -INFINITY && wd != 0u) {           // first valid columns of this row: fix the stabiliser
                    float mm = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if ((wd >> i) & 1u) mm = fmaxf(mm, __uint_as_float(s[i]));
                    m = mm;
                    add_cols = 0xffffffffu;                 // the addends of the fast path are stale now
                }
                const float mb = (m == -INFINITY) ? 0.f : m * P.scale_log2;
                // A piece that lies inside every row's window (most pieces of a long 1-D window) needs no
                // masks and no running maximum: two columns per packed instruction, and the row sum tells
                // whether any probability may have outgrown its stabiliser (then the general form redoes it).
                bool done = false;
                if (__all_sync(0xffffffffu, wd == 0xFFFFu)) {
                    const uint64_t sc2 = pack2(P.scale_log2, P.scale_log2), nb2 = pack2(-mb, -mb);
                    uint64_t rr = 0ull;
                    uint32_t pq[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint64_t xx = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), sc2, nb2);
                        const float p0 = fast_exp2(lo_of(xx)), p1 = fast_exp2(hi_of(xx));
                        rr = add2(rr, pack2(p0, p1));
                        pq[i] = cvt_pack<BF16>(p0, p1);
                    }
                    const float rs = lo_of(rr) + hi_of(rr);
                    if (!__any_sync(0xffffffffu, !(rs <= kGrowSum))) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) pk[i] = pq[i];
                        l += rs;
                        stored |= 1u << pc;
                        done = true;
                    }
                }
                if (!done) {
                float x[16], xmax = -INFINITY;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    x[i] = fmaf(__uint_as_float(s[i]), P.scale_log2, -mb);
                    if (!((wd >> i) & 1u)) x[i] = -INFINITY;
                    xmax = fmaxf(xmax, x[i]);
                }
                const bool grow = xmax > kGrow;
                if (__any_sync(0xffffffffu, grow)) {
                    rescale(grow, xmax, c, pc, stored);
                    if (grow) {
                        add_cols = 0xffffffffu;
#pragma unroll
                        for (int i = 0; i < 16; ++i) x[i] -= xmax;
                    }
                }
                float r0 = 0.f, r1 = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float p0 = fast_exp2(x[2 * i]), p1 = fast_exp2(x[2 * i + 1]);
                    r0 += p0;
                    r1 += p1;
                    pk[i] = cvt_pack<BF16>(p0, p1);
                }
                l += r0 + r1;
                stored |= 1u << pc;
                }
            };
#pragma unroll 1
            for (int pc = 0; pc < 4; ++pc) {
                uint32_t pk[8];
                if (fast) {
#if NATTEN_ABL == 2
                    const bool rowok = false;
#else
                    const bool rowok = ((rowbits >> pc) & 1u) && colbits != 0u;
#endif
                    if (__any_sync(0xffffffffu, rowok)) {
                        uint32_t s[16];
                        tmem_ld16(scol + 16 * pc, s);
                        tmem_ld_wait();
#if NATTEN_ABL == 3
#pragma unroll
                        for (int i = 0; i < 8; ++i) pk[i] = s[2 * i] & 1u;
                        stored |= 1u << pc;
#else
                        if (m == -INFINITY && rowok) {           // first valid columns of this row: fix the stabiliser
                            float mm = -INFINITY;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if ((colbits >> i) & 1u) mm = fmaxf(mm, __uint_as_float(s[i]));
                            m = mm;
                            refresh_add(colbits);
                        }
                        // No running maximum in the common case: the probabilities are formed at once and their
                        // row sum tells whether one of them may have outgrown the stabiliser; only then are the
                        // exponents looked at one by one (and, if it is so, everything rescaled and redone).
                        const uint64_t sc2 = pack2(P.scale_log2, P.scale_log2);
                        const uint32_t keep = rowok ? 0xffffffffu : 0u;     // rows outside their window store zeros
                        uint64_t rr = 0ull;                                 // two partial row sums
#pragma unroll
                        for (int i = 0; i < 8; ++i) {                       // two columns per packed fp32 fma
                            const uint64_t xx = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), sc2, pack2(add[2 * i], add[2 * i + 1]));
                            const float p0 = fast_exp2(lo_of(xx)), p1 = fast_exp2(hi_of(xx));
                            rr = add2(rr, pack2(p0, p1));
                            pk[i] = cvt_pack<BF16>(p0, p1) & keep;
                        }
                        if (__any_sync(0xffffffffu, rowok && !(lo_of(rr) + hi_of(rr) <= kGrowSum))) {
                            float x[16], xmax = -INFINITY;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                x[i] = fmaf(__uint_as_float(s[i]), P.scale_log2, add[i]);
                                xmax = fmaxf(xmax, x[i]);
                            }
                            const bool grow = rowok && xmax > kGrow;
                            if (__any_sync(0xffffffffu, grow)) {
                                rescale(grow, xmax, c, pc, stored);
                                if (grow) {
                                    refresh_add(colbits);
#pragma unroll
                                    for (int i = 0; i < 16; ++i) x[i] -= xmax;
                                }
                            }
                            rr = 0ull;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float p0 = fast_exp2(x[2 * i]), p1 = fast_exp2(x[2 * i + 1]);
                                rr = add2(rr, pack2(p0, p1));
                                pk[i] = cvt_pack<BF16>(p0, p1) & keep;
                            }
                        }
                        if (rowok) l += lo_of(rr) + hi_of(rr);
                        stored |= 1u << pc;
#endif
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) pk[i] = 0u;
                    }
                } else {
                    const uint32_t wd = ((pc & 2) ? words[1] : words[0]) >> (16 * (pc & 1)) & 0xFFFFu;
                    if (__any_sync(0xffffffffu, wd != 0u)) {
                        uint32_t s[16];
                        tmem_ld16(scol + 16 * pc, s);
                        tmem_ld_wait();
                        generic_piece(pc, s, wd, pk);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) pk[i] = 0u;
                    }
                }
                // P over the scores it came from: piece pc lands in columns this thread has already read
                tmem_st8(scol + 8 * pc, pk);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_p_of(n));
            STAMP(330);
            if (!mapped) {
                ++ci[2];
                dirty = 4u;
                if (ci[2] == T.nc[2]) {
                    ci[2] = 0; ++ci[1]; dirty = T.nc[2] > 1 ? 6u : 2u;
                    if (ci[1] == T.nc[1]) { ci[1] = 0; ++ci[0]; dirty = 1u | (T.nc[1] > 1 ? 2u : 0u) | (T.nc[2] > 1 ? 4u : 0u); }
                }
            }
        }

        // ---- normalise and write out ----
        ok = mbar_wait(bar_o, t & 1, abort_flag, P.wait_budget) && ok;
        tc_fence_after();
        STAMP(340);
        {
            const bool live = valid_q && ok;
            const float inv = (live && l > 0.f) ? 1.f / l : 0.f;
            uint4* o4 = reinterpret_cast<uint4*>(out + out_row * P.dreal);
#pragma unroll
            for (int part = 0; part < DH / 32; ++part) {
                if (32 * part >= P.dreal) break;             // padded channels are not part of the output
                uint32_t o[32];
                tmem_ld32(trow + kColO + 32 * part, o);
                tmem_ld_wait();
                if (in_tensor && NATTEN_ABL != 1) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (32 * part + 8 * i >= P.dreal) break;
                        uint32_t wv[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            wv[j] = live ? cvt_pack<BF16>(__uint_as_float(o[8 * i + 2 * j]) * inv, __uint_as_float(o[8 * i + 2 * j + 1]) * inv) : 0u;
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
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

} // namespace

int tc_fused_fwd_small(int dtype, const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                       const void* ev, void* out, void* lse, cudaStream_t s)
{
    if (g.D > 128) return -2;
    if (!tc_eligible(dtype, g, q, k, v, /*allow_stride=*/true)) return -2;
    if (g.n_extra > 0 && ((reinterpret_cast<uintptr_t>(ek) | reinterpret_cast<uintptr_t>(ev)) & 15u)) return -2;
    Plan plan;
    if (!make_plan(g, plan, kKeys, /*with_stride=*/true, /*interleave=*/true)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mq, mk, mv, mek, mev;
    if (!encode_map(&mq, q, bf16, plan.p, g.Hq, g.D, g.qs, plan.box_q, /*query_lattice=*/true) ||
        !encode_map(&mk, k, bf16, plan.p, g.Hkv, g.D, g.ks, plan.box_kv, false, /*interleaved=*/true) ||
        !encode_map(&mv, v, bf16, plan.p, g.Hkv, g.Dv, g.vs, plan.box_kv, false, /*interleaved=*/true))
        return -2;
    mek = mk; mev = mv;                      // placeholders when there are no additional tokens
    if (g.n_extra > 0 && (!encode_extra_map(&mek, ek, bf16, g.B, g.n_extra, g.Hkv, g.D, kKeys, plan.p.split_heads) ||
                          !encode_extra_map(&mev, ev, bf16, g.B, g.n_extra, g.Hkv, g.Dv, kKeys, plan.p.split_heads)))
        return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    if (plan.p.work_q == 0 || g.B == 0) return 0;
    cudaError_t err = cudaSuccess;
    auto launch = [&](auto dh, auto bf, auto inner) {
        constexpr int kDh = decltype(dh)::value;
        constexpr bool kBf = decltype(bf)::value;
        constexpr int kInner = decltype(inner)::value;
        using FS = FwdSmall<kDh>;
        const unsigned grid = persistent_grid(plan.p.work_q, FS::kPerSm);
        err = ensure_dynamic_smem((const void*)tc_fwd_small_kernel<kDh, kBf, kInner>, FS::kSmemTotal);
        if (err != cudaSuccess) return;
        tc_fwd_small_kernel<kDh, kBf, kInner><<<grid, kThreads, FS::kSmemTotal, s>>>(mq, mk, mv, mek, mev, plan.p, (uint16_t*)out, (float*)lse);
    };
    auto by_inner = [&](auto dh, auto bf) {
        if (plan.p.cb[2] == 16) launch(dh, bf, std::integral_constant<int, 16>{});
        else if (plan.p.cb[2] == 32) launch(dh, bf, std::integral_constant<int, 32>{});
        else launch(dh, bf, std::integral_constant<int, 0>{});
    };
    auto by_type = [&](auto dh) {
        if (bf16) by_inner(dh, std::true_type{});
        else by_inner(dh, std::false_type{});
    };
    if (g.D <= 64) by_type(std::integral_constant<int, 64>{});
    else by_type(std::integral_constant<int, 128>{});
    if (err == cudaSuccess) err = cudaGetLastError();
    tc_count_launch();
    return err == cudaSuccess ? 0 : (int)err;
}

// launches of the tensor-core kernels, counted on the host by every launcher
static unsigned long long g_tc_launches = 0;
void tc_count_launch() { ++g_tc_launches; }
unsigned long long tc_launch_count() { return g_tc_launches; }

#ifdef NATTEN_TRACE
extern "C" int natten_trace_read_small(long long* host, int clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(host, g_trace_small, sizeof(g_trace_small));
    if (e == cudaSuccess && clear) {
        static long long zeros[8 * 512] = {0};
        e = cudaMemcpyToSymbol(g_trace_small, zeros, sizeof(g_trace_small));
    }
    return (int)e;
}
#endif

} // namespace natten
